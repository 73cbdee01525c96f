// A run of Conv2 -> Relu -> MaxPool2 (2 x 2, stride 2) stages of a gradient-recording bf16 pass,
// kept channels-last from the first convolution's input to the last pool's output.
//
// The tensor-core convolution kernels work on channels-last data; run layer by layer, every
// convolution converts its input, its output and both operands of its weight gradient between
// NCHW and channels-last, and Relu and the pool each read and write the full activation.  Here
// the activations of the whole run stay channels-last: per stage the forward pass is the
// convolution and one Relu + pool kernel, the backward pass one kernel for the gradient at the
// convolution's output (written straight into the zero frame the input-gradient kernel wants)
// and the two gradient convolutions.  A first layer with few input channels (3 x 3 x 3 = 27 <= 64)
// is run as a 1 x 1 convolution over its patches (the patch is the channel axis), which puts it on
// the tensor cores too and makes its weight gradient a plain [oc][27] product.
//
// The values are those of the separate layers (Conv2 layer.rs:842-948, Relu layer.rs:1254-1298,
// MaxPool2 layer.rs:1193-1216 and their backward edges): the same roundings at the same places,
// the pool's first-maximum rule and its treatment of cells no window covers.  The run is one
// node of the graph with edges to the input (when it records a gradient) and to every
// parameter; the gradients inside the run are computed on demand and shared between the edges.
#pragma once

#include <memory>
#include <vector>

#include "../conv_tc.cuh"
#include "../nhwc_ops.cuh"
#include "nn.hpp"

namespace autograph {

struct StageDesc {
    Conv2 *conv = nullptr;
    int64_t ic = 0, ih = 0, iw = 0;   // the layer's input
    int64_t oc = 0, oh = 0, ow = 0;   // the convolution's output
    int64_t ph = 0, pw = 0;           // pooled
    int fh = 0, fw = 0;
    bool patches = false;             // few input channels: a 1 x 1 convolution over the patches
    // the convolution as the kernels see it
    int64_t k_ic = 0, k_ih = 0, k_iw = 0;
    int k_fh = 0, k_fw = 0;
    int64_t cp = 0, ocp = 0;          // channel pitches of its input and output
};

inline int64_t round_up_64(int64_t v) { return (v + 63) / 64 * 64; }

inline bool conv_stages_enabled() {
    static const bool on = [] {
        const char *e = getenv("AG_NHWC_STAGES");
        return !(e && e[0] == '0');
    }();
    return on;
}

// Fills `d` when the stage (conv on an input of [bs, ic, ih, iw], Relu, 2 x 2 pool) can be part of
// a channels-last run.  needs_dx: the gradient at the stage's input is wanted.
inline bool plan_stage(Conv2 &conv, const MaxPool2 &mp, ag_dtype dtype, int64_t bs, int64_t ic,
                       int64_t ih, int64_t iw, bool needs_dx, StageDesc *d) {
    if (dtype != AG_BF16 || !::ag::convtc::tc_conv_enabled()) return false;
    if (mp.filter[0] != 2 || mp.filter[1] != 2 || mp.stride[0] != 2 || mp.stride[1] != 2) return false;
    const Tensor &w = conv.weight.value;
    if (w.ndim() != 4 || w.dim(1) != ic || !w.is_standard_layout()) return false;
    const ConvOptions &o = conv.options;
    for (int i = 0; i < 2; ++i)
        if (o.padding[i] != 0 || o.stride[i] != 1 || o.dilation[i] != 1) return false;
    d->conv = &conv;
    d->ic = ic; d->ih = ih; d->iw = iw;
    d->oc = w.dim(0);
    d->fh = (int)w.dim(2); d->fw = (int)w.dim(3);
    d->oh = ih - d->fh + 1; d->ow = iw - d->fw + 1;
    if (d->oh < 2 || d->ow < 2) return false;
    d->ph = d->oh / 2; d->pw = d->ow / 2;
    d->ocp = round_up_64(d->oc);
    if (d->ocp != d->oc) return false;   // whole 64-channel blocks only (also: the bias gradient is a column sum)
    d->patches = ic < 16 && ic * d->fh * d->fw <= 64 && !needs_dx;
    if (d->patches) {
        d->k_ic = ic * d->fh * d->fw; d->k_ih = d->oh; d->k_iw = d->ow;
        d->k_fh = d->k_fw = 1;
    } else {
        d->k_ic = ic; d->k_ih = ih; d->k_iw = iw;
        d->k_fh = d->fh; d->k_fw = d->fw;
    }
    d->cp = round_up_64(d->k_ic);
    ag_conv2_options ko;
    ko.filter[0] = d->k_fh; ko.filter[1] = d->k_fw;
    for (int i = 0; i < 2; ++i) { ko.padding[i] = 0; ko.stride[i] = 1; ko.dilation[i] = 1; }
    using namespace ::ag::convtc;
    if (!eligible_forward(bs, d->k_ic, d->k_ih, d->k_iw, d->oc, &ko)) return false;
    if (!eligible_backward_weight(bs, d->k_ic, d->k_ih, d->k_iw, d->oc, &ko)) return false;
    if (needs_dx && !eligible_backward_input(bs, d->k_ic, d->k_ih, d->k_iw, d->oc, &ko)) return false;
    return true;
}

class StageRun : public std::enable_shared_from_this<StageRun> {
   public:
    Pool *pool = nullptr;
    ag_device *dev = nullptr;
    int64_t bs = 0;
    bool input_grad = false;
    std::vector<StageDesc> st;
    std::vector<Tensor> act, pre;     // per stage: the kernels' input and the convolution's output
    std::vector<Tensor> dpre;         // per stage: gradient at the convolution's output (maybe framed)
    std::vector<char> have, framed;

    using bf16 = __nv_bfloat16;
    static const bf16 *cptr(const Tensor &t) { return reinterpret_cast<const bf16 *>(t.data()); }
    static bf16 *ptr(const Tensor &t) { return reinterpret_cast<bf16 *>(t.data()); }
    Tensor make(const Shape &shape) { return Tensor::uninit(*pool, shape, AG_BF16); }

    ::ag::convtc::NhwcConv forward_conv(const StageDesc &d) const {
        ::ag::convtc::NhwcConv c;
        c.bs = bs; c.c_in = d.k_ic; c.in_h = d.k_ih; c.in_w = d.k_iw;
        c.c_out = d.oc; c.out_h = d.oh; c.out_w = d.ow;
        c.fh = d.k_fh; c.fw = d.k_fw; c.pad_h = c.pad_w = 0;
        c.transposed = false;
        return c;
    }
    // the input gradient: dy correlated with the reversed, transposed filter bank over a frame
    // of filter - 1 zeros
    ::ag::convtc::NhwcConv backward_conv(const StageDesc &d) const {
        ::ag::convtc::NhwcConv c;
        c.bs = bs; c.c_in = d.oc; c.in_h = d.oh; c.in_w = d.ow;
        c.c_out = d.k_ic; c.out_h = d.k_ih; c.out_w = d.k_iw;
        c.fh = d.k_fh; c.fw = d.k_fw; c.pad_h = d.k_fh - 1; c.pad_w = d.k_fw - 1;
        c.transposed = true;
        return c;
    }
    ag_conv2_options kernel_options(const StageDesc &d) const {
        ag_conv2_options ko;
        ko.filter[0] = d.k_fh; ko.filter[1] = d.k_fw;
        for (int i = 0; i < 2; ++i) { ko.padding[i] = 0; ko.stride[i] = 1; ko.dilation[i] = 1; }
        return ko;
    }

    // x: the run's input, NCHW.  Returns the last pool's output, NCHW.
    Tensor forward(const Tensor &x) {
        ::ag::DeviceGuard guard(dev);
        Tensor pooled;
        for (size_t s = 0; s < st.size(); ++s) {
            const StageDesc &d = st[s];
            Tensor a;
            if (s == 0) {
                if (d.patches) {
                    a = make({bs, d.oh, d.ow, d.cp});
                    check(::ag::nhwc::im2col_channels(dev, cptr(x), bs, d.ic, d.ih, d.iw, d.fh, d.fw, d.oh,
                                                      d.ow, d.cp, ptr(a)));
                } else {
                    a = make({bs, d.ih, d.iw, d.cp});
                    check(::ag::convtc::to_nhwc(dev, cptr(x), bs, d.ic, d.ih * d.iw, d.cp, ptr(a)));
                }
            } else {
                a = pooled;   // the previous stage's output is this stage's input as it is
            }
            const ::ag::convtc::NhwcConv c = forward_conv(d);
            Tensor wk = make({::ag::convtc::nhwc_filter_scratch_bytes(c) / 2});
            Tensor p = make({bs, d.oh, d.ow, d.ocp});
            const Tensor &wv = d.conv->weight.value;
            check(::ag::convtc::correlate_nhwc(
                dev, c, cptr(a), ::ag::convtc::nhwc_wants_frame(c), cptr(wv), d.oc, d.k_ic,
                d.conv->has_bias ? cptr(d.conv->bias.value) : nullptr, false, ptr(wk), ptr(p)));
            Tensor y = make({bs, d.ph, d.pw, d.ocp});
            check(::ag::nhwc::relu_pool(dev, cptr(p), bs, d.oh, d.ow, d.ocp, ptr(y)));
            act.push_back(a);
            pre.push_back(p);
            pooled = y;
        }
        const StageDesc &l = st.back();
        Tensor out = make({bs, l.oc, l.ph, l.pw});
        check(::ag::convtc::from_nhwc(dev, cptr(pooled), bs, l.oc, l.ph * l.pw, l.ocp, ptr(out)));
        dpre.resize(st.size());
        have.assign(st.size(), 0);
        framed.assign(st.size(), 0);
        return out;
    }

    bool wants_dx(size_t s) const { return s > 0 || input_grad; }

    // interior of stage s's gradient buffer and its pitches in elements
    struct View { bf16 *p; int64_t row_pitch, image_pitch; };
    View interior(size_t s) const {
        const StageDesc &d = st[s];
        if (!framed[s]) return View{ptr(dpre[s]), d.ow * d.ocp, d.oh * d.ow * d.ocp};
        const int64_t fy = d.k_fh - 1, fx = d.k_fw - 1;
        const int64_t hp = d.oh + 2 * fy, wp = d.ow + 2 * fx;
        return View{ptr(dpre[s]) + (fy * wp + fx) * d.ocp, wp * d.ocp, hp * wp * d.ocp};
    }

    // The gradient at the input of stage s, channels-last [bs][ih][iw][cp].
    Tensor input_gradient(size_t s, const Tensor &dy_out) {
        ensure(s, dy_out);
        const StageDesc &d = st[s];
        const ::ag::convtc::NhwcConv c = backward_conv(d);
        Tensor wk = make({::ag::convtc::nhwc_filter_scratch_bytes(c) / 2});
        Tensor dx = make({bs, d.k_ih, d.k_iw, d.cp});
        check(::ag::convtc::correlate_nhwc(dev, c, cptr(dpre[s]), framed[s] != 0,
                                           cptr(d.conv->weight.value), d.oc, d.k_ic, nullptr, false,
                                           ptr(wk), ptr(dx)));
        return dx;
    }

    // Makes dpre[s]; dy_out is the gradient at the run's output (NCHW).
    void ensure(size_t s, const Tensor &dy_out) {
        if (have[s]) return;
        ::ag::DeviceGuard guard(dev);
        const StageDesc &d = st[s];
        Tensor dpool;
        if (s + 1 == st.size()) {
            dpool = make({bs, d.ph, d.pw, d.ocp});
            check(::ag::convtc::to_nhwc(dev, cptr(dy_out), bs, d.oc, d.ph * d.pw, d.ocp, ptr(dpool)));
        } else {
            dpool = input_gradient(s + 1, dy_out);
        }
        const bool fr = wants_dx(s) && ::ag::convtc::nhwc_wants_frame(backward_conv(d));
        framed[s] = fr ? 1 : 0;
        if (fr) {
            const int fy = d.k_fh - 1, fx = d.k_fw - 1;
            const int64_t hp = d.oh + 2 * fy, wp = d.ow + 2 * fx;
            dpre[s] = make({bs, hp, wp, d.ocp});
            check(::ag::nhwc::zero_frame(dev, ptr(dpre[s]), bs, hp, wp, fy, fx, d.ocp));
        } else {
            dpre[s] = make({bs, d.oh, d.ow, d.ocp});
        }
        const View v = interior(s);
        check(::ag::nhwc::relu_pool_backward(dev, cptr(pre[s]), cptr(dpool), bs, d.oh, d.ow, d.ocp, v.p,
                                            v.row_pitch, v.image_pitch));
        have[s] = 1;
    }

    void weight_gradient(size_t s, const Tensor &dy_out, Tensor &dw) {
        ensure(s, dy_out);
        ::ag::DeviceGuard guard(dev);
        const StageDesc &d = st[s];
        const View v = interior(s);
        const ag_conv2_options ko = kernel_options(d);
        check(::ag::convtc::backward_weight_nhwc(dev, cptr(act[s]), bs, d.k_ic, d.k_ih, d.k_iw, v.p,
                                                 v.row_pitch, v.image_pitch, d.oc, &ko, 0.f, ptr(dw)));
    }

    void bias_gradient(size_t s, const Tensor &dy_out, Tensor &db) {
        ensure(s, dy_out);
        const StageDesc &d = st[s];
        // column sums of the whole buffer: the frame, when there is one, holds zeros
        const int64_t rows = dpre[s].len() / d.ocp;
        check(ag_bias_grad(dev, AG_BF16, dpre[s].data(), rows, d.ocp, 1, 0.f, db.data()));
    }

    Tensor run_input_gradient(const Tensor &dy_out) {
        Tensor dx_nhwc = input_gradient(0, dy_out);
        ::ag::DeviceGuard guard(dev);
        const StageDesc &d = st[0];
        Tensor dx = make({bs, d.ic, d.ih, d.iw});
        check(::ag::convtc::from_nhwc(dev, cptr(dx_nhwc), bs, d.ic, d.ih * d.iw, d.cp, ptr(dx)));
        return dx;
    }
};

// The variable around the run's output: one node with an edge to the input and to every
// parameter of the run's convolutions.
inline Variable conv_stage_run_forward(Pool &pool, std::shared_ptr<StageRun> run, const Variable &input) {
    Tensor y = run->forward(input.value);
    VariableBuilder builder;
    Pool *pp = &pool;
    if (input.node)
        builder.edge(input.node, [run](const Tensor &dy, Tensor *) { return run->run_input_gradient(dy); });
    for (size_t s = 0; s < run->st.size(); ++s) {
        Conv2 *conv = run->st[s].conv;
        Variable w = conv->weight.to_variable();
        if (w.node) {
            Shape wshape = conv->weight.value.shape();
            builder.edge(w.node, [run, s, pp, wshape](const Tensor &dy, Tensor *into) {
                Tensor dw = into ? *into : Tensor::uninit(*pp, wshape, dy.dtype());
                run->weight_gradient(s, dy, dw);
                return dw;
            });
        }
        if (conv->has_bias) {
            Variable b = conv->bias.to_variable();
            if (b.node) {
                const int64_t oc = run->st[s].oc;
                builder.edge(b.node, [run, s, pp, oc](const Tensor &dy, Tensor *into) {
                    Tensor db = into ? *into : Tensor::uninit(*pp, {oc}, dy.dtype());
                    run->bias_gradient(s, dy, db);
                    return db;
                });
            }
        }
    }
    return builder.build(y);
}

}  // namespace autograph
