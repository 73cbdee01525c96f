// C ABI of the host-side neural-network layer: model construction, parameter
// access, inference and training steps (the counterpart of LeNet5Classifier in
// benches/neural-network-benches/src/autograph_backend.rs:16-85).
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cuda_bf16.h>

#include "../comm.cuh"
#include "../common.cuh"
#include "nn.hpp"
#include "conv_stages.hpp"

using namespace autograph;

// Captured inference passes for one input shape.  A graph holds the input copy
// (device -> staging, or pinned host -> staging), the kernels of the layer chain
// and the output copy; per call only the two copy nodes are re-pointed at the
// caller's buffers, so a whole step is one graph launch.  Replaying removes the
// per-kernel launch cost, which dominates at small batch.
struct CapturedPass {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaGraphNode_t in_node = nullptr, out_node = nullptr;
    const void *y_ptr = nullptr;  // the chain's output inside the graph
    Pool::Parked parked;          // intermediate buffers baked into the graph
    uint64_t kernels = 0;         // kernel launches recorded in the graph
    int seen = 0;                 // calls before a graph exists
};

// A pass captured for one particular pair of pinned host buffers: the first kernel
// reads the images straight from host memory (the transfer overlaps its arithmetic
// instead of preceding it), so the pointers are part of the graph.
struct ZeroCopyPass {
    const void *x = nullptr;
    void *out = nullptr;
    CapturedPass pass;
    uint64_t last_use = 0;
};

struct GraphEntry {
    int64_t bs = 0, c = 0, h = 0, w = 0;
    Tensor x_stage;               // the graphs' input
    size_t out_bytes = 0;
    CapturedPass from_device, from_host;
    std::vector<ZeroCopyPass> zero_copy;  // host callers that reuse a few pinned buffers
    int zero_copy_misses = 0;
    uint64_t last_use = 0;
};

// A captured training step (host images and labels -> loss, gradients, update) for one
// input shape and one set of optimizer scalars.
struct TrainEntry {
    int64_t bs = 0, c = 0, h = 0, w = 0;
    float lr = 0.f, momentum = 0.f, grad_scale = 1.f;
    bool use_momentum = false;
    bool with_update = true;   // the optimizer step is part of the graph
    bool from_device = false;  // inputs are device buffers (copied device to device)
    Tensor x_stage, t_stage;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaGraphNode_t x_node = nullptr, t_node = nullptr;
    const void *x_src = nullptr, *t_src = nullptr;  // what the two copy nodes read at present
    Pool::Parked parked;
    uint64_t kernels = 0;
    int seen = 0;
};

struct ag_model {
    ag_device *dev;
    ag_dtype dtype;
    Pool pool;  // declared before every tensor so that it is destroyed last
    std::vector<TrainEntry> train_graphs;
    Tensor loss_dev;             // one f32: the loss of the step in flight
    float *loss_pinned = nullptr;
    float loss_eager = 0.f;      // loss of the last step that did not go through a graph
    bool loss_in_flight = false; // the last step left its loss in loss_pinned, not yet read
    std::vector<GraphEntry> graphs;
    uint64_t tick = 0;
    bool graphs_enabled = true;
    bool zero_copy_enabled = true;
    // Two side streams (each behind its own device handle) and the events that fork
    // and join them: a host-input pass is captured as batch slices that alternate
    // between the two, so one slice's later layers run while the next slice's first
    // layer is still pulling its images over PCIe.
    ag_device *side[2] = {nullptr, nullptr};
    cudaEvent_t fork_event = nullptr, join_event[2] = {nullptr, nullptr};
    int slices = 0;  // 0: chosen from the batch size
    bool whole_network = true;  // try the one-kernel form of the network at inference
    // Pipelined host inference (ag_model_infer_enqueue / _wait): two slots, each with a device
    // copy of its batch; the copy engine fills one slot on its own stream while the network runs
    // on the other.
    struct InferSlot {
        Tensor x_stage;
        cudaEvent_t copied = nullptr, done = nullptr;
        bool busy = false;
    };
    InferSlot infer_slots[2];
    cudaStream_t copy_stream = nullptr;
    int next_slot = 0;
    std::vector<std::unique_ptr<Layer>> layers;
    std::vector<Parameter *> params;
    std::vector<int64_t> offsets;  // element offset of each parameter in the buckets
    int64_t bucket_len = 0;
    Tensor values, grads, velocity;  // flat buckets [bucket_len]
    bool use_momentum = false;
    float momentum = 0.f;
    float grad_scale = 1.f;
    ag_model(ag_device *d, ag_dtype t) : dev(d), dtype(t), pool(d) {
        const char *e = getenv("AG_GRAPH");
        graphs_enabled = !(e && e[0] == '0');
        const char *z = getenv("AG_ZERO_COPY");
        zero_copy_enabled = !(z && z[0] == '0');
        if (const char *c = getenv("AG_INFER_SLICES")) slices = std::max(1, std::min(16, atoi(c)));
        const char *f = getenv("AG_FUSE_NET");
        whole_network = !(f && f[0] == '0');
    }
    bool ensure_side_streams() {
        if (side[0]) return true;
        if (ag_device_create(ag_device_ordinal(dev), &side[0]) != AG_OK ||
            ag_device_create(ag_device_ordinal(dev), &side[1]) != AG_OK)
            return false;
        bool ok = cudaEventCreateWithFlags(&fork_event, cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; i < 2; ++i)
            ok = ok && cudaEventCreateWithFlags(&join_event[i], cudaEventDisableTiming) == cudaSuccess;
        return ok;
    }
    void drop(CapturedPass &p) {
        if (p.exec) cudaGraphExecDestroy(p.exec);
        if (p.graph) cudaGraphDestroy(p.graph);
        p.exec = nullptr;
        p.graph = nullptr;
        pool.unpark(p.parked);
    }
    void drop(GraphEntry &g) {
        drop(g.from_device);
        drop(g.from_host);
        for (auto &z : g.zero_copy) drop(z.pass);
        g.zero_copy.clear();
    }
    void drop(TrainEntry &t) {
        if (t.exec) cudaGraphExecDestroy(t.exec);
        if (t.graph) cudaGraphDestroy(t.graph);
        t.exec = nullptr;
        t.graph = nullptr;
        pool.unpark(t.parked);
    }
    ~ag_model() {
        for (auto &g : graphs) drop(g);
        for (auto &t : train_graphs) drop(t);
        if (loss_pinned) ag_host_free(loss_pinned);
        for (int i = 0; i < 2; ++i) {
            if (side[i]) ag_device_destroy(side[i]);
            if (join_event[i]) cudaEventDestroy(join_event[i]);
        }
        if (fork_event) cudaEventDestroy(fork_event);
        if (copy_stream) {
            // batches still in flight under a ticket: let their copies and network passes finish
            cudaStreamSynchronize(copy_stream);
            cudaStreamSynchronize((cudaStream_t)ag_device_stream(dev));
        }
        for (auto &sl : infer_slots) {
            if (sl.copied) cudaEventDestroy(sl.copied);
            if (sl.done) cudaEventDestroy(sl.done);
        }
        if (copy_stream) cudaStreamDestroy(copy_stream);
    }
};

namespace {

// splitmix64: the seeded stream behind the default initialiser.
struct Rng {
    uint64_t s;
    uint64_t next() {
        uint64_t z = (s += 0x9e3779b97f4a7c15ull);
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
        return z ^ (z >> 31);
    }
    float uniform(float a) {  // U[-a, a)
        float u = (float)(next() >> 40) * (1.0f / 16777216.0f);
        return -a + 2.f * a * u;
    }
};

void fill_uniform(ag_model *m, Tensor &dst, float a, Rng &rng) {
    const int64_t n = dst.len();
    if (m->dtype == AG_F32) {
        std::vector<float> h((size_t)n);
        for (auto &v : h) v = rng.uniform(a);
        check(ag_upload(m->dev, dst.data(), h.data(), h.size() * 4));
        check(ag_device_wait(m->dev));
    } else {
        std::vector<__nv_bfloat16> h((size_t)n);
        for (auto &v : h) v = __float2bfloat16_rn(rng.uniform(a));  // bf16::from_f32 of the f32 draw
        check(ag_upload(m->dev, dst.data(), h.data(), h.size() * 2));
        check(ag_device_wait(m->dev));
    }
}

int64_t round_up(int64_t v, int64_t to) { return (v + to - 1) / to * to; }

void build_model(ag_model *m, const ag_layer_spec *specs, int n, uint64_t seed) {
    struct Pending {
        Parameter *p;
        Shape shape;
        float a;
    };
    std::vector<Pending> pending;
    for (int i = 0; i < n; ++i) {
        const ag_layer_spec &s = specs[i];
        switch (s.kind) {
            case AG_LAYER_CONV2: {
                if (s.a <= 0 || s.b <= 0 || s.c <= 0 || s.d <= 0)
                    throw Error(AG_ERR_INVALID, "Conv2: inputs, outputs and filter must be positive");
                auto l = std::make_unique<Conv2>();
                // a = sqrt(2 / (inputs * filter size)) (layer.rs:345-349)
                float a = std::sqrt(2.f / (float)(s.a * s.c * s.d));
                l->has_bias = s.bias != 0;
                pending.push_back({&l->weight, {s.b, s.a, s.c, s.d}, a});
                if (l->has_bias) pending.push_back({&l->bias, {s.b}, a});
                m->layers.push_back(std::move(l));
                break;
            }
            case AG_LAYER_DENSE: {
                if (s.a <= 0 || s.b <= 0)
                    throw Error(AG_ERR_INVALID, "Dense: inputs and outputs must be positive");
                auto l = std::make_unique<Dense>();
                float a = std::sqrt(2.f / (float)s.a);  // layer.rs:463-467
                l->has_bias = s.bias != 0;
                if (s.c > 0) {
                    // c = 1 + index of an earlier Dense layer whose parameters this one shares
                    auto *owner = s.c - 1 < i ? dynamic_cast<Dense *>(m->layers[s.c - 1].get()) : nullptr;
                    if (!owner || owner->tied || owner->weight_shape != Shape{s.a, s.b} ||
                        owner->has_bias != l->has_bias)
                        throw Error(AG_ERR_INVALID, "Dense: c must name an earlier Dense layer of the same shape");
                    l->tied = owner;
                    m->layers.push_back(std::move(l));
                    break;
                }
                l->weight_shape = {s.a, s.b};
                pending.push_back({&l->weight, {s.a, s.b}, a});
                if (l->has_bias) pending.push_back({&l->bias, {s.b}, a});
                m->layers.push_back(std::move(l));
                break;
            }
            case AG_LAYER_RELU: m->layers.push_back(std::make_unique<Relu>()); break;
            case AG_LAYER_MAXPOOL2: {
                if (s.c <= 0 || s.d <= 0) throw Error(AG_ERR_INVALID, "MaxPool2: bad filter");
                auto l = std::make_unique<MaxPool2>();
                l->filter[0] = l->stride[0] = s.c;
                l->filter[1] = l->stride[1] = s.d;
                m->layers.push_back(std::move(l));
                break;
            }
            case AG_LAYER_FLATTEN: m->layers.push_back(std::make_unique<Flatten>()); break;
            default: throw Error(AG_ERR_INVALID, "unknown layer kind");
        }
    }
    // Buckets: every parameter starts on a 16-byte boundary.
    int64_t off = 0;
    for (auto &p : pending) {
        m->offsets.push_back(off);
        off += round_up(numel(p.shape), 8);
    }
    m->bucket_len = off;
    m->values = Tensor::zeros(m->pool, {off}, m->dtype);
    m->grads = Tensor::zeros(m->pool, {off}, m->dtype);
    m->velocity = Tensor::zeros(m->pool, {off}, m->dtype);
    Rng rng{seed};
    for (size_t i = 0; i < pending.size(); ++i) {
        Parameter *p = pending[i].p;
        int64_t len = numel(pending[i].shape);
        p->value = m->values.narrow0(m->offsets[i], len).into_shape(pending[i].shape);
        p->grad = m->grads.narrow0(m->offsets[i], len).into_shape(pending[i].shape);
        p->velocity = m->velocity.narrow0(m->offsets[i], len).into_shape(pending[i].shape);
        fill_uniform(m, p->value, pending[i].a, rng);
        m->params.push_back(p);
    }
}

// ≙ the derived Forward: input.forward(&self.f0)?...forward(&self.fN) (autograph_derive/src/lib.rs:291-340)
// When no gradient is recorded (inference), a Relu and a MaxPool2 that follow a
// Conv2, and a Relu that follows a Dense, are folded into the producing kernel.
// The whole network as one kernel when it has the shape
// (Conv2 [Relu] [MaxPool2]){1,2} Flatten (Dense [Relu]){1,4}, no gradient is
// recorded and the kernel takes its sizes.  Returns false when the layers have to
// run one by one.
// u8 images (device-visible) standing in for v's data, scaled by alpha inside the kernel.
struct U8Images {
    const uint8_t *ptr;
    float alpha;
};

bool forward_whole_network(ag_model *m, const Variable &v, Variable *out, void *out_ptr,
                           const U8Images *u8 = nullptr) {
    if (!m->whole_network || v.node || v.value.ndim() != 4 || !v.value.is_standard_layout())
        return false;
    const size_t n = m->layers.size();
    size_t i = 0;
    std::vector<ag_conv_stage> stages;
    while (i < n) {
        auto *conv = dynamic_cast<Conv2 *>(m->layers[i].get());
        if (!conv) break;
        if (conv->records_gradient(v)) return false;
        ag_conv_stage st;
        st.w = conv->weight.value.data();
        st.bias = conv->has_bias ? conv->bias.value.data() : nullptr;
        st.oc = conv->weight.value.dim(0);
        st.options = to_c_options({conv->weight.value.dim(2), conv->weight.value.dim(3)},
                                  conv->options);
        st.relu = 0;
        st.pool[0] = st.pool[1] = 0;
        ++i;
        if (i < n && dynamic_cast<Relu *>(m->layers[i].get())) {
            st.relu = 1;
            ++i;
        }
        if (i < n) {
            if (auto *mp = dynamic_cast<MaxPool2 *>(m->layers[i].get())) {
                if (mp->stride[0] != mp->filter[0] || mp->stride[1] != mp->filter[1]) return false;
                st.pool[0] = mp->filter[0];
                st.pool[1] = mp->filter[1];
                ++i;
            }
        }
        stages.push_back(st);
    }
    if (stages.empty() || i >= n || !dynamic_cast<Flatten *>(m->layers[i].get())) return false;
    ++i;
    std::vector<int64_t> dims;
    std::vector<const void *> ws, bs;
    std::vector<int32_t> relus;
    while (i < n) {
        auto *d = dynamic_cast<Dense *>(m->layers[i].get());
        if (!d || d->W().node || (d->has_bias && d->B().node)) return false;
        if (dims.empty()) dims.push_back(d->W().value.dim(0));
        if (d->W().value.dim(0) != dims.back()) return false;
        dims.push_back(d->W().value.dim(1));
        ws.push_back(d->W().value.data());
        bs.push_back(d->has_bias ? d->B().value.data() : nullptr);
        const bool r = i + 1 < n && dynamic_cast<Relu *>(m->layers[i + 1].get());
        relus.push_back(r ? 1 : 0);
        i += r ? 2 : 1;
    }
    if (ws.empty()) return false;
    const Tensor &x = v.value;
    if (x.dim(0) == 0) return false;
    // out_ptr: device-visible memory of the caller that receives the logits directly
    Tensor y = out_ptr ? Tensor::external(x.device(), out_ptr, {x.dim(0), dims.back()}, x.dtype())
                       : Tensor::uninit(m->pool, {x.dim(0), dims.back()}, x.dtype());
    const int status =
        u8 ? ag_conv_dense_chain_forward_u8(x.device(), x.dtype(), u8->ptr, u8->alpha, x.dim(0),
                                            x.dim(1), x.dim(2), x.dim(3), (int32_t)stages.size(),
                                            stages.data(), (int32_t)ws.size(), dims.data(),
                                            ws.data(), bs.data(), relus.data(), y.data())
           : ag_conv_dense_chain_forward(x.device(), x.dtype(), x.data(), x.dim(0), x.dim(1),
                                         x.dim(2), x.dim(3), (int32_t)stages.size(), stages.data(),
                                         (int32_t)ws.size(), dims.data(), ws.data(), bs.data(),
                                         relus.data(), y.data());
    if (status == AG_ERR_UNSUPPORTED) {
        m->whole_network = false;  // decided by the layer sizes: do not ask again
        return false;
    }
    check(status);
    *out = Variable{y, nullptr};
    return true;
}

// One autograd node for a run of Dense (+ Relu) layers whose values were kept: the first
// edge asked for its gradient computes all of them with one ag_dense_chain_backward call
// (parameter gradients straight into the parameters' gradient storage where that is still
// unset), the others hand out what it left.
struct DenseChainGrads {
    bool done = false;
    Tensor dx;
    std::vector<Tensor> dw, db;
};

Variable attach_dense_chain(Pool &pool, const Variable &input, const std::vector<Dense *> &run,
                            const std::vector<int32_t> &relus, const std::vector<Tensor> &pre,
                            const std::vector<Tensor> &act) {
    const size_t L = run.size();
    const Tensor x = input.value;
    const std::shared_ptr<Node> in_node = input.node;
    std::vector<Tensor> wv;
    std::vector<std::shared_ptr<Node>> wn, bn;
    for (Dense *d : run) {
        wv.push_back(d->W().value);
        wn.push_back(d->W().node);
        bn.push_back(d->has_bias ? d->B().node : nullptr);
    }
    auto st = std::make_shared<DenseChainGrads>();
    Pool *pp = &pool;
    auto ensure = [=](const Tensor &dy) {
        if (st->done) return;
        const int64_t bs = x.dim(0);
        // A parameter's own gradient storage is handed out once: a parameter shared by two
        // layers of the run gets its second gradient in a fresh tensor, which the backward
        // walk then adds to the first.
        std::vector<const Node *> handed;
        auto target = [&](const std::shared_ptr<Node> &n, const Shape &shape) {
            if (n && !n->has_grad && n->grad_storage.defined() &&
                std::find(handed.begin(), handed.end(), n.get()) == handed.end()) {
                handed.push_back(n.get());
                return n->grad_storage;
            }
            return Tensor::uninit(*pp, shape, x.dtype());
        };
        std::vector<int64_t> dims = {x.dim(1)};
        std::vector<const void *> lin, ws, gate;
        std::vector<Tensor> g;
        std::vector<void *> gp, dwp, dbp;
        for (size_t l = 0; l < L; ++l) {
            const int64_t ins = wv[l].dim(0), outs = wv[l].dim(1);
            dims.push_back(outs);
            lin.push_back(l == 0 ? x.data() : (relus[l - 1] ? act[l - 1].data() : pre[l - 1].data()));
            ws.push_back(wv[l].data());
            gate.push_back(relus[l] ? pre[l].data() : nullptr);
            const bool need_g = l + 1 < L || relus[l];
            g.push_back(need_g ? Tensor::uninit(*pp, {bs, outs}, x.dtype()) : Tensor{});
            gp.push_back(need_g ? g.back().data() : nullptr);
            st->dw.push_back(target(wn[l], Shape{ins, outs}));
            dwp.push_back(st->dw.back().data());
            st->db.push_back(bn[l] ? target(bn[l], Shape{outs}) : Tensor{});
            dbp.push_back(bn[l] ? st->db.back().data() : nullptr);
        }
        if (in_node) st->dx = Tensor::uninit(*pp, x.shape(), x.dtype());
        check(ag_dense_chain_backward(x.device(), x.dtype(), bs, (int32_t)L, dims.data(), lin.data(),
                                      ws.data(), gate.data(), dy.data(), gp.data(),
                                      in_node ? st->dx.data() : nullptr, dwp.data(), dbp.data()));
        st->done = true;
    };
    VariableBuilder builder;
    if (in_node)
        builder.edge(in_node, [=](const Tensor &dy, Tensor *) {
            ensure(dy);
            return st->dx;
        });
    for (size_t l = 0; l < L; ++l) {
        if (wn[l])
            builder.edge(wn[l], [=](const Tensor &dy, Tensor *) {
                ensure(dy);
                return st->dw[l];
            });
        if (bn[l])
            builder.edge(bn[l], [=](const Tensor &dy, Tensor *) {
                ensure(dy);
                return st->db[l];
            });
    }
    return builder.build(relus[L - 1] ? act[L - 1] : pre[L - 1]);
}

// out_ptr (optional): where the result should land when the network runs as one kernel;
// the caller compares the returned tensor's address to see whether it did.
Variable forward_chain(ag_model *m, Variable v, void *out_ptr = nullptr) {
    const size_t n = m->layers.size();
    {
        Variable whole;
        if (forward_whole_network(m, v, &whole, out_ptr)) return whole;
    }
    for (size_t i = 0; i < n; ++i) {
        Layer *l = m->layers[i].get();
        auto *relu1 = i + 1 < n ? dynamic_cast<Relu *>(m->layers[i + 1].get()) : nullptr;
        if (auto *conv = dynamic_cast<Conv2 *>(l)) {
            if (!conv->records_gradient(v) && relu1) {
                auto *mp = i + 2 < n ? dynamic_cast<MaxPool2 *>(m->layers[i + 2].get()) : nullptr;
                const bool pool_ok = mp && mp->stride[0] == mp->filter[0] &&
                                     mp->stride[1] == mp->filter[1];
                v = conv->forward_fused(m->pool, v, true, pool_ok ? mp->filter : nullptr);
                i += pool_ok ? 2 : 1;
                continue;
            }
            // Recording gradients in bf16 with shapes the tensor-core kernels take: this and the
            // following Conv2 -> Relu -> MaxPool2 stages run as one channels-last node.
            if (conv->records_gradient(v) && relu1 && conv_stages_enabled() && v.value.ndim() == 4 &&
                v.value.is_standard_layout() && v.value.dtype() == AG_BF16) {
                auto run = std::make_shared<StageRun>();
                int64_t c = v.value.dim(1), h = v.value.dim(2), w = v.value.dim(3);
                size_t j = i;
                while (j + 2 < n) {
                    auto *cj = dynamic_cast<Conv2 *>(m->layers[j].get());
                    auto *rj = dynamic_cast<Relu *>(m->layers[j + 1].get());
                    auto *pj = dynamic_cast<MaxPool2 *>(m->layers[j + 2].get());
                    StageDesc d;
                    const bool needs_dx = j > i || (bool)v.node;
                    if (!cj || !rj || !pj || !cj->weight.to_variable().node ||
                        !plan_stage(*cj, *pj, v.value.dtype(), v.value.dim(0), c, h, w, needs_dx, &d))
                        break;
                    run->st.push_back(d);
                    c = d.oc; h = d.ph; w = d.pw;
                    j += 3;
                }
                if (!run->st.empty()) {
                    run->pool = &m->pool;
                    run->dev = m->dev;
                    run->bs = v.value.dim(0);
                    run->input_grad = (bool)v.node;
                    v = conv_stage_run_forward(m->pool, run, v);
                    i = j - 1;
                    continue;
                }
            }
            // Recording gradients, Relu and an even 2x2 pool next: one forward call that keeps
            // the convolution's output for the backward edges.
            if (conv->records_gradient(v) && relu1 && i + 2 < n && v.value.ndim() == 4 &&
                v.value.is_standard_layout() && v.value.dim(1) == conv->weight.value.dim(1)) {
                auto *mp = dynamic_cast<MaxPool2 *>(m->layers[i + 2].get());
                const Shape f = {conv->weight.value.dim(2), conv->weight.value.dim(3)};
                const ag_conv2_options copt = to_c_options(f, conv->options);
                int64_t oh = 0, ow = 0;
                if (mp && mp->filter[0] == 2 && mp->filter[1] == 2 && mp->stride[0] == 2 &&
                    mp->stride[1] == 2 &&
                    ag_conv2_output_shape(v.value.dim(2), v.value.dim(3), &copt, &oh, &ow) == AG_OK &&
                    oh >= 2 && ow >= 2 && oh % 2 == 0 && ow % 2 == 0) {
                    v = conv_relu_pool_forward(m->pool, *conv, v);
                    i += 2;
                    continue;
                }
            }
        } else if (auto *dense = dynamic_cast<Dense *>(l)) {
            // A run of Dense (+ Relu) layers goes to one fused call.
            if (!dense->records_gradient(v) && v.value.ndim() == 2 && v.value.is_standard_layout()) {
                std::vector<Dense *> run;
                std::vector<int32_t> relus;
                size_t j = i;
                while (j < n && run.size() < 4) {
                    auto *d = dynamic_cast<Dense *>(m->layers[j].get());
                    if (!d || d->W().node || (d->has_bias && d->B().node)) break;
                    if (!run.empty() && d->W().value.dim(0) != run.back()->W().value.dim(1)) break;
                    const bool r = j + 1 < n && dynamic_cast<Relu *>(m->layers[j + 1].get());
                    run.push_back(d);
                    relus.push_back(r ? 1 : 0);
                    j += r ? 2 : 1;
                }
                if (run.size() >= 2 && v.value.dim(1) == run[0]->W().value.dim(0)) {
                    std::vector<int64_t> dims = {v.value.dim(1)};
                    std::vector<const void *> ws, bs;
                    for (Dense *d : run) {
                        dims.push_back(d->W().value.dim(1));
                        ws.push_back(d->W().value.data());
                        bs.push_back(d->has_bias ? d->B().value.data() : nullptr);
                    }
                    Tensor y = Tensor::uninit(m->pool, {v.value.dim(0), dims.back()}, v.value.dtype());
                    check(ag_dense_chain_forward(v.value.device(), v.value.dtype(), v.value.data(),
                                                 v.value.dim(0), (int32_t)run.size(), dims.data(),
                                                 ws.data(), bs.data(), relus.data(), y.data()));
                    v = Variable{y, nullptr};
                    i = j - 1;
                    continue;
                }
            }
            if (!dense->records_gradient(v) && relu1) {
                v = dense->forward_fused(m->pool, v, true);
                i += 1;
                continue;
            }
            // Recording gradients: the same run as one call that keeps every layer's values,
            // then the layers' own backward edges around those values.
            if (dense->records_gradient(v) && v.value.ndim() == 2 && v.value.is_standard_layout() &&
                v.value.dim(1) == dense->W().value.dim(0)) {
                std::vector<Dense *> run;
                std::vector<int32_t> relus;
                size_t j = i;
                while (j < n && run.size() < 4) {
                    auto *d = dynamic_cast<Dense *>(m->layers[j].get());
                    if (!d) break;
                    if (!run.empty() && d->W().value.dim(0) != run.back()->W().value.dim(1)) break;
                    const bool r = j + 1 < n && dynamic_cast<Relu *>(m->layers[j + 1].get());
                    run.push_back(d);
                    relus.push_back(r ? 1 : 0);
                    j += r ? 2 : 1;
                }
                if (run.size() >= 2) {
                    const int64_t bs = v.value.dim(0);
                    std::vector<int64_t> dims = {v.value.dim(1)};
                    std::vector<const void *> ws, bs_ptr;
                    std::vector<Tensor> pre, act;
                    std::vector<void *> pre_ptr, act_ptr;
                    for (size_t k = 0; k < run.size(); ++k) {
                        Dense *d = run[k];
                        const int64_t outs = d->W().value.dim(1);
                        dims.push_back(outs);
                        ws.push_back(d->W().value.data());
                        bs_ptr.push_back(d->has_bias ? d->B().value.data() : nullptr);
                        pre.push_back(Tensor::uninit(m->pool, {bs, outs}, v.value.dtype()));
                        act.push_back(relus[k] ? Tensor::uninit(m->pool, {bs, outs}, v.value.dtype())
                                               : Tensor{});
                        pre_ptr.push_back(pre.back().data());
                        act_ptr.push_back(relus[k] ? act.back().data() : nullptr);
                    }
                    check(ag_dense_chain_forward_keep(v.value.device(), v.value.dtype(), v.value.data(),
                                                      bs, (int32_t)run.size(), dims.data(), ws.data(),
                                                      bs_ptr.data(), relus.data(), pre_ptr.data(),
                                                      act_ptr.data()));
                    v = attach_dense_chain(m->pool, v, run, relus, pre, act);
                    i = j - 1;
                    continue;
                }
            }
        }
        if (dynamic_cast<Relu *>(l) && i + 1 < n) {
            auto *mp = dynamic_cast<MaxPool2 *>(m->layers[i + 1].get());
            if (mp && relu_pool_fusable(v, *mp)) {
                v = relu_pool_forward(m->pool, v);
                i += 1;
                continue;
            }
        }
        v = l->forward(m->pool, v);
    }
    return v;
}

constexpr size_t kMaxGraphs = 16;

GraphEntry *find_graph(ag_model *m, int64_t bs, int64_t c, int64_t h, int64_t w) {
    for (auto &g : m->graphs)
        if (g.bs == bs && g.c == c && g.h == h && g.w == w) return &g;
    if (m->graphs.size() >= kMaxGraphs) {
        size_t victim = 0;
        for (size_t i = 1; i < m->graphs.size(); ++i)
            if (m->graphs[i].last_use < m->graphs[victim].last_use) victim = i;
        m->drop(m->graphs[victim]);
        m->graphs.erase(m->graphs.begin() + victim);
    }
    m->graphs.emplace_back();
    GraphEntry &g = m->graphs.back();
    g.bs = bs; g.c = c; g.h = h; g.w = w;  // the staging tensor is made on first use
    return &g;
}

// Device-visible address of pinned host memory, or null when `p` is not pinned.
void *pinned_device_pointer(const void *p) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
}

bool is_pinned_host(const void *p) { return pinned_device_pointer(p) != nullptr; }

constexpr size_t kMaxZeroCopy = 8;
constexpr int kZeroCopyMissLimit = 64;

// Host path for callers that cycle through a few pinned buffers: one graph per
// (input, output) pair whose first kernel reads the host images directly.
// Returns false when the caller should use the copying path instead.
bool run_zero_copy(ag_model *m, GraphEntry *g, const void *x, void *out) {
    if (g->zero_copy_misses > kZeroCopyMissLimit) return false;  // too many distinct buffers
    void *x_dev = pinned_device_pointer(x);
    if (!x_dev || !is_pinned_host(out)) return false;
    cudaStream_t stream = (cudaStream_t)ag_device_stream(m->dev);
    ZeroCopyPass *z = nullptr;
    for (auto &e : g->zero_copy)
        if (e.x == x && e.out == out) z = &e;
    if (!z) {
        ++g->zero_copy_misses;
        if (g->zero_copy.size() >= kMaxZeroCopy) {
            size_t victim = 0;
            for (size_t i = 1; i < g->zero_copy.size(); ++i)
                if (g->zero_copy[i].last_use < g->zero_copy[victim].last_use) victim = i;
            m->drop(g->zero_copy[victim].pass);
            g->zero_copy.erase(g->zero_copy.begin() + victim);
        }
        g->zero_copy.emplace_back();
        z = &g->zero_copy.back();
        z->x = x;
        z->out = out;
    }
    z->last_use = ++m->tick;
    CapturedPass &cp = z->pass;
    auto cuda_ok = [](cudaError_t e, const char *what) {
        if (e != cudaSuccess)
            throw Error(AG_ERR_CUDA, std::string(what) + " failed: " + cudaGetErrorString(e));
    };
    if (cp.exec) {
        cuda_ok(cudaGraphLaunch(cp.exec, stream), "cudaGraphLaunch");
        ::ag::count_launches(cp.kernels);
        return true;
    }
    void *out_dev = pinned_device_pointer(out);
    auto pass = [&]() {
        // The one-kernel network writes its logits straight into the caller's pinned
        // buffer; any other network leaves them on the device and they are copied.
        Tensor xt = Tensor::external(m->dev, x_dev, {g->bs, g->c, g->h, g->w}, m->dtype);
        Variable y = forward_chain(m, Variable{xt, nullptr}, out_dev);
        if (y.value.data() != out_dev)
            cuda_ok(cudaMemcpyAsync(out, y.value.data(), y.value.nbytes(), cudaMemcpyDeviceToHost,
                                    stream), "output copy");
    };
    // The captured form: batch slices alternating between the two side streams.
    // Every slice adds graph nodes and cross-stream dependencies (a few microseconds
    // each), so only batches whose copy takes far longer than that are sliced.
    const int want = m->slices > 0 ? m->slices : (g->bs >= 16384 ? 4 : 1);
    const int64_t slices = (want > 1 && g->bs >= 64 * want && m->ensure_side_streams()) ? want : 1;
    auto sliced_pass = [&]() {
        if (slices == 1) return pass();
        struct Restore {
            Pool &p; ag_device *d;
            ~Restore() { p.set_device(d); }
        } restore{m->pool, m->dev};
        const int64_t per = (g->bs + slices - 1) / slices;
        const size_t image_bytes = (size_t)(g->c * g->h * g->w) * element_size(m->dtype);
        cuda_ok(cudaEventRecord(m->fork_event, stream), "fork");
        size_t out_off = 0;
        for (int64_t s = 0, first = 0; first < g->bs; ++s, first += per) {
            ag_device *d = m->side[s & 1];
            cudaStream_t st = (cudaStream_t)ag_device_stream(d);
            if (s < 2) cuda_ok(cudaStreamWaitEvent(st, m->fork_event, 0), "fork wait");
            const int64_t n = std::min(per, g->bs - first);
            m->pool.set_device(d);
            Tensor xt = Tensor::external(d, (char *)x_dev + (size_t)first * image_bytes,
                                         {n, g->c, g->h, g->w}, m->dtype);
            Variable y = forward_chain(m, Variable{xt, nullptr});
            cuda_ok(cudaMemcpyAsync((char *)out + out_off, y.value.data(), y.value.nbytes(),
                                    cudaMemcpyDeviceToHost, st), "output copy");
            out_off += y.value.nbytes();
        }
        for (int i = 0; i < 2; ++i) {
            cuda_ok(cudaEventRecord(m->join_event[i], (cudaStream_t)ag_device_stream(m->side[i])), "join");
            cuda_ok(cudaStreamWaitEvent(stream, m->join_event[i], 0), "join wait");
        }
    };
    if (++cp.seen < 2) {
        pass();
        return true;
    }
    m->pool.set_hold(&cp.parked);
    const uint64_t launches_before = ::ag::launch_count();
    bool ok = cudaStreamBeginCapture(stream, cudaStreamCaptureModeRelaxed) == cudaSuccess;
    if (ok) {
        try {
            sliced_pass();
        } catch (...) {
            ok = false;
        }
        ok = (cudaStreamEndCapture(stream, &cp.graph) == cudaSuccess) && ok && cp.graph != nullptr;
    }
    m->pool.set_hold(nullptr);
    cp.kernels = ::ag::launch_count() - launches_before;
    if (ok) ok = cudaGraphInstantiate(&cp.exec, cp.graph, 0) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        m->drop(cp);
        g->zero_copy_misses = kZeroCopyMissLimit + 1;  // stop trying for this shape
        pass();
        return true;
    }
    cuda_ok(cudaGraphLaunch(cp.exec, stream), "cudaGraphLaunch");
    ::ag::count_launches(cp.kernels);
    return true;
}

// One inference pass x -> out.  `host` selects host pointers (x and out in host
// memory: H2D, chain, D2H) or device pointers (D2D, chain, D2D).  The first call for
// a shape runs eagerly; the second captures the pass; later calls replay it.
void run_inference(ag_model *m, GraphEntry *g, bool host, const void *x, void *out) {
    g->last_use = ++m->tick;
    // A network that runs as one kernel needs neither staging copies nor a graph: the
    // kernel reads the caller's images and writes the caller's logits (device memory, or
    // pinned host memory through its device address).
    if (m->whole_network && g->bs > 0 && (!host || m->zero_copy_enabled)) {
        void *x_dev = host ? pinned_device_pointer(x) : const_cast<void *>(x);
        void *out_dev = host ? pinned_device_pointer(out) : out;
        if (x_dev && out_dev) {
            Tensor xt = Tensor::external(m->dev, x_dev, {g->bs, g->c, g->h, g->w}, m->dtype);
            Variable y = forward_chain(m, Variable{xt, nullptr}, out_dev);
            if (y.value.data() != out_dev) {
                // not a one-kernel network after all (remembered): hand this result over
                cudaStream_t st = (cudaStream_t)ag_device_stream(m->dev);
                if (cudaMemcpyAsync(out, y.value.data(), y.value.nbytes(),
                                    host ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice,
                                    st) != cudaSuccess)
                    throw Error(AG_ERR_CUDA, "output copy failed");
                // y's block returns to the pool; later work on this stream is ordered after
                // the copy, so reuse is safe
            }
            return;
        }
    }
    if (host && m->graphs_enabled && m->zero_copy_enabled && g->bs > 0 &&
        run_zero_copy(m, g, x, out))
        return;
    cudaStream_t stream = (cudaStream_t)ag_device_stream(m->dev);
    if (!g->x_stage.defined())
        g->x_stage = Tensor::uninit(m->pool, {g->bs, g->c, g->h, g->w}, m->dtype);
    CapturedPass &cp = host ? g->from_host : g->from_device;
    const cudaMemcpyKind kin = host ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
    const cudaMemcpyKind kout = host ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
    auto cuda_ok = [](cudaError_t e, const char *what) {
        if (e != cudaSuccess)
            throw Error(AG_ERR_CUDA, std::string(what) + " failed: " + cudaGetErrorString(e));
    };
    if (cp.exec) {
        cuda_ok(cudaGraphExecMemcpyNodeSetParams1D(cp.exec, cp.in_node, g->x_stage.data(), x,
                                                    g->x_stage.nbytes(), kin), "graph input update");
        cuda_ok(cudaGraphExecMemcpyNodeSetParams1D(cp.exec, cp.out_node, out, cp.y_ptr, g->out_bytes,
                                                    kout), "graph output update");
        cuda_ok(cudaGraphLaunch(cp.exec, stream), "cudaGraphLaunch");
        ::ag::count_launches(cp.kernels);  // the replay enqueues the captured kernels
        return;
    }
    const void *y_ptr = nullptr;
    auto pass = [&]() {
        cuda_ok(cudaMemcpyAsync(g->x_stage.data(), x, g->x_stage.nbytes(), kin, stream), "input copy");
        Variable y = forward_chain(m, Variable{g->x_stage, nullptr});
        g->out_bytes = y.value.nbytes();
        y_ptr = y.value.data();
        cuda_ok(cudaMemcpyAsync(out, y_ptr, g->out_bytes, kout, stream), "output copy");
    };
    const bool capturable = m->graphs_enabled && g->bs > 0 &&
                            (!host || (is_pinned_host(x) && is_pinned_host(out)));
    if (!capturable || ++cp.seen < 2) {
        pass();
        return;
    }
    // Capture.  Blocks released while capturing stay parked with the graph.
    m->pool.set_hold(&cp.parked);
    const uint64_t launches_before = ::ag::launch_count();
    bool ok = cudaStreamBeginCapture(stream, cudaStreamCaptureModeRelaxed) == cudaSuccess;
    if (ok) {
        try {
            pass();
        } catch (...) {
            ok = false;
        }
        ok = (cudaStreamEndCapture(stream, &cp.graph) == cudaSuccess) && ok && cp.graph != nullptr;
    }
    m->pool.set_hold(nullptr);
    cp.kernels = ::ag::launch_count() - launches_before;
    cp.y_ptr = y_ptr;
    if (ok) {
        // Find the two copy nodes by the buffers they touch.
        size_t n = 0;
        ok = cudaGraphGetNodes(cp.graph, nullptr, &n) == cudaSuccess && n > 0;
        std::vector<cudaGraphNode_t> nodes(n);
        if (ok) ok = cudaGraphGetNodes(cp.graph, nodes.data(), &n) == cudaSuccess;
        for (size_t i = 0; ok && i < n; ++i) {
            cudaGraphNodeType type;
            if (cudaGraphNodeGetType(nodes[i], &type) != cudaSuccess) { ok = false; break; }
            if (type != cudaGraphNodeTypeMemcpy) continue;
            cudaMemcpy3DParms mp;
            if (cudaGraphMemcpyNodeGetParams(nodes[i], &mp) != cudaSuccess) { ok = false; break; }
            if (mp.dstPtr.ptr == g->x_stage.data()) cp.in_node = nodes[i];
            if (mp.srcPtr.ptr == y_ptr) cp.out_node = nodes[i];
        }
        ok = ok && cp.in_node && cp.out_node;
    }
    if (ok) ok = cudaGraphInstantiate(&cp.exec, cp.graph, 0) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        m->drop(cp);
        m->graphs_enabled = false;  // this model runs eagerly from now on
        pass();
        return;
    }
    cuda_ok(cudaGraphLaunch(cp.exec, stream), "cudaGraphLaunch");
    ::ag::count_launches(cp.kernels);
}

Tensor input_tensor(ag_model *m, const void *x, bool on_host, int64_t bs, int64_t c, int64_t h,
                    int64_t w) {
    if (bs < 0 || c <= 0 || h <= 0 || w <= 0) throw Error(AG_ERR_SHAPE, "bad input shape");
    if (!x && bs > 0) throw Error(AG_ERR_INVALID, "input pointer is null");
    Shape shape = {bs, c, h, w};
    if (on_host) return Tensor::from_host(m->pool, shape, m->dtype, x);
    return Tensor::external(m->dev, const_cast<void *>(x), shape, m->dtype);
}

float forward_backward(ag_model *m, const Tensor &x, const Tensor &t, float *loss_dev = nullptr) {
    for (Parameter *p : m->params) p->init_grad();  // ≙ model.init_parameter_grads()
    Variable y = forward_chain(m, Variable{x, nullptr});
    Loss loss = cross_entropy_loss(m->pool, y, t, loss_dev);
    loss.backward();
    for (Parameter *p : m->params) {
        if (!p->has_grad()) throw Error(AG_ERR_INVALID, "a parameter received no gradient");
    }
    return loss.value;
}

// ≙ model.update(lr, &sgd) (layer.rs:656-658 -> SGD::update, optimizer.rs:389-428), over the
// flat buckets: element-wise identical to updating each parameter.
void apply_update(ag_model *m, float lr) {
    if (m->grad_scale != 1.f)
        check(ag_scaled_add(m->dev, m->dtype, m->grad_scale - 1.f, m->grads.data(), m->grads.data(),
                            m->bucket_len));
    if (m->use_momentum)
        check(ag_sgd_update_momentum(m->dev, m->dtype, m->values.data(), m->grads.data(),
                                     m->velocity.data(), m->bucket_len, lr, m->momentum));
    else
        check(ag_sgd_update(m->dev, m->dtype, m->values.data(), m->grads.data(), m->bucket_len, lr));
    for (Parameter *p : m->params) p->node.reset();  // ≙ take_grad consumed the gradient
}

// One training step from pinned host buffers, replayed from a CUDA graph from the second
// call with the same shape and optimizer scalars on.  Returns false when the step has to
// run eagerly (pageable host memory, graphs disabled, capture failed).
bool train_step_graph(ag_model *m, const void *x_host, const uint8_t *t_host, int64_t bs, int64_t c,
                      int64_t h, int64_t w, float lr, float *loss_host, bool with_update = true,
                      bool from_device = false) {
    // x_host / t_host are device pointers when from_device is set (the data-parallel path:
    // forward and backward only, the caller all-reduces the gradient bucket and updates).
    if (!m->graphs_enabled || bs <= 0) return false;
    if (!from_device && (!is_pinned_host(x_host) || !is_pinned_host(t_host))) return false;
    const cudaMemcpyKind kin = from_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    cudaStream_t stream = (cudaStream_t)ag_device_stream(m->dev);
    TrainEntry *e = nullptr;
    for (auto &t : m->train_graphs)
        if (t.bs == bs && t.c == c && t.h == h && t.w == w && t.lr == lr &&
            t.momentum == m->momentum && t.use_momentum == m->use_momentum &&
            t.grad_scale == m->grad_scale && t.with_update == with_update &&
            t.from_device == from_device)
            e = &t;
    if (!e && with_update) {
        // A learning rate this shape has not been captured with, while another one has: a
        // schedule.  One graph without the update then serves every rate and the update follows
        // as a plain launch, instead of one capture (and, past eight, one eviction) per rate.
        bool other_rate = false;
        for (auto &t : m->train_graphs)
            if (t.bs == bs && t.c == c && t.h == h && t.w == w && t.with_update &&
                t.from_device == from_device && t.lr != lr)
                other_rate = true;
        if (other_rate) {
            if (!train_step_graph(m, x_host, t_host, bs, c, h, w, 0.f, nullptr, false, from_device))
                return false;
            apply_update(m, lr);
            if (loss_host) {
                if (cudaStreamSynchronize(stream) != cudaSuccess)
                    throw Error(AG_ERR_CUDA, "cudaStreamSynchronize failed");
                *loss_host = *m->loss_pinned;
                m->loss_in_flight = false;
            }
            return true;
        }
    }
    if (!e) {
        if (m->train_graphs.size() >= 8) {
            m->drop(m->train_graphs.front());
            m->train_graphs.erase(m->train_graphs.begin());
        }
        m->train_graphs.emplace_back();
        e = &m->train_graphs.back();
        e->bs = bs; e->c = c; e->h = h; e->w = w;
        e->lr = lr; e->momentum = m->momentum; e->use_momentum = m->use_momentum;
        e->grad_scale = m->grad_scale;
        e->with_update = with_update;
        e->from_device = from_device;
        e->x_stage = Tensor::uninit(m->pool, {bs, c, h, w}, m->dtype);
        e->t_stage = Tensor::uninit(m->pool, {bs}, AG_U8);
    }
    if (!m->loss_dev.defined()) {
        m->loss_dev = Tensor::zeros(m->pool, {1}, AG_F32);
        void *hp = nullptr;
        check(ag_host_alloc(sizeof(float), &hp));
        m->loss_pinned = (float *)hp;
    }
    auto cuda_ok = [](cudaError_t err, const char *what) {
        if (err != cudaSuccess)
            throw Error(AG_ERR_CUDA, std::string(what) + " failed: " + cudaGetErrorString(err));
    };
    auto finish = [&]() {
        m->loss_in_flight = loss_host == nullptr;
        if (!loss_host) return;  // the caller reads the loss later (ag_model_last_loss)
        cuda_ok(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
        *loss_host = *m->loss_pinned;
    };
    if (e->exec) {
        // a loader that refills the same buffers needs no node update
        if (e->x_src != x_host) {
            cuda_ok(cudaGraphExecMemcpyNodeSetParams1D(e->exec, e->x_node, e->x_stage.data(), x_host,
                                                        e->x_stage.nbytes(), kin),
                    "graph input update");
            e->x_src = x_host;
        }
        if (e->t_src != t_host) {
            cuda_ok(cudaGraphExecMemcpyNodeSetParams1D(e->exec, e->t_node, e->t_stage.data(), t_host,
                                                        e->t_stage.nbytes(), kin),
                    "graph label update");
            e->t_src = t_host;
        }
        cuda_ok(cudaGraphLaunch(e->exec, stream), "cudaGraphLaunch");
        ::ag::count_launches(e->kernels);
        finish();
        return true;
    }
    auto pass = [&]() {
        cuda_ok(cudaMemcpyAsync(e->x_stage.data(), x_host, e->x_stage.nbytes(), kin, stream),
                "input copy");
        cuda_ok(cudaMemcpyAsync(e->t_stage.data(), t_host, e->t_stage.nbytes(), kin, stream),
                "label copy");
        forward_backward(m, e->x_stage, e->t_stage, (float *)m->loss_dev.data());
        if (with_update) apply_update(m, lr);
        cuda_ok(cudaMemcpyAsync(m->loss_pinned, m->loss_dev.data(), sizeof(float),
                                cudaMemcpyDeviceToHost, stream), "loss copy");
    };
    if (++e->seen < 2) {
        pass();
        finish();
        return true;
    }
    m->pool.set_hold(&e->parked);
    const uint64_t launches_before = ::ag::launch_count();
    bool ok = cudaStreamBeginCapture(stream, cudaStreamCaptureModeRelaxed) == cudaSuccess;
    if (ok) {
        try {
            pass();
        } catch (...) {
            ok = false;
        }
        ok = (cudaStreamEndCapture(stream, &e->graph) == cudaSuccess) && ok && e->graph != nullptr;
    }
    m->pool.set_hold(nullptr);
    e->kernels = ::ag::launch_count() - launches_before;
    if (ok) {
        size_t n = 0;
        ok = cudaGraphGetNodes(e->graph, nullptr, &n) == cudaSuccess && n > 0;
        std::vector<cudaGraphNode_t> nodes(n);
        if (ok) ok = cudaGraphGetNodes(e->graph, nodes.data(), &n) == cudaSuccess;
        for (size_t i = 0; ok && i < n; ++i) {
            cudaGraphNodeType type;
            if (cudaGraphNodeGetType(nodes[i], &type) != cudaSuccess) { ok = false; break; }
            if (type != cudaGraphNodeTypeMemcpy) continue;
            cudaMemcpy3DParms mp;
            if (cudaGraphMemcpyNodeGetParams(nodes[i], &mp) != cudaSuccess) { ok = false; break; }
            if (mp.dstPtr.ptr == e->x_stage.data()) e->x_node = nodes[i];
            if (mp.dstPtr.ptr == e->t_stage.data()) e->t_node = nodes[i];
        }
        ok = ok && e->x_node && e->t_node;
    }
    if (ok) ok = cudaGraphInstantiate(&e->exec, e->graph, 0) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        m->drop(*e);
        for (Parameter *p : m->params) p->node.reset();
        m->graphs_enabled = false;
        return false;
    }
    e->x_src = x_host;  // the copy nodes were captured with this call's buffers
    e->t_src = t_host;
    cuda_ok(cudaGraphLaunch(e->exec, stream), "cudaGraphLaunch");
    ::ag::count_launches(e->kernels);
    finish();
    return true;
}

}  // namespace

// u8 host images -> logits on the host (blocking); see ag_model_infer_u8.
void infer_u8(ag_model *m, const uint8_t *x_host, int64_t bs, int64_t c, int64_t h, int64_t w,
              float alpha, void *logits_host) {
    cudaStream_t stream = (cudaStream_t)ag_device_stream(m->dev);
    auto sync = [&]() {
        cudaError_t e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess)
            throw Error(AG_ERR_CUDA, std::string("cudaStreamSynchronize failed: ") + cudaGetErrorString(e));
    };
    const size_t n = (size_t)(bs * c * h * w);
    // One-kernel network on pinned buffers: the kernel reads the u8 images over PCIe,
    // scales them while staging, and writes the logits into the caller's buffer.
    void *x_dev = pinned_device_pointer(x_host);
    void *out_dev = pinned_device_pointer(logits_host);
    if (m->whole_network && m->zero_copy_enabled && x_dev && out_dev) {
        U8Images u8{(const uint8_t *)x_dev, alpha};
        Tensor shape_only = Tensor::external(m->dev, x_dev, {bs, c, h, w}, m->dtype);
        Variable y;
        if (forward_whole_network(m, Variable{shape_only, nullptr}, &y, out_dev, &u8)) {
            sync();
            return;
        }
    }
    // General path: upload the bytes, scaled_cast on the device, then the usual pass.
    Tensor raw = Tensor::uninit(m->pool, {(int64_t)n}, AG_U8);
    check(ag_upload(m->dev, raw.data(), x_host, n));
    Tensor x = Tensor::uninit(m->pool, {bs, c, h, w}, m->dtype);
    check(ag_scaled_cast_u8(m->dev, m->dtype, alpha, (const uint8_t *)raw.data(), x.data(),
                            (int64_t)n));
    Variable y = forward_chain(m, Variable{x, nullptr});
    check(ag_download(m->dev, logits_host, y.value.data(), y.value.nbytes()));
}

#define AG_HOST_GUARD(body)                                         \
    try {                                                           \
        body                                                        \
    } catch (const Error &e) {                                      \
        return ::ag::fail(e.status(), "%s", e.what());              \
    } catch (const std::exception &e) {                             \
        return ::ag::fail(AG_ERR_INVALID, "%s", e.what());          \
    }                                                               \
    return AG_OK;

extern "C" {

int ag_model_create(ag_device *dev, ag_dtype dtype, const ag_layer_spec *layers, int32_t n_layers,
                    uint64_t seed, ag_model **out) {
    AG_REQUIRE(dev && layers && out && n_layers > 0, AG_ERR_INVALID, "null or empty argument");
    AG_REQUIRE(dtype == AG_F32 || dtype == AG_BF16, AG_ERR_DTYPE, "model dtype %d not implemented",
               (int)dtype);
    *out = nullptr;
    ag_model *m = nullptr;
    try {
        m = new ag_model(dev, dtype);
        build_model(m, layers, n_layers, seed);
    } catch (const Error &e) {
        delete m;
        return ::ag::fail(e.status(), "%s", e.what());
    } catch (const std::exception &e) {
        delete m;
        return ::ag::fail(AG_ERR_INVALID, "%s", e.what());
    }
    *out = m;
    return AG_OK;
}

int ag_model_create_lenet5(ag_device *dev, ag_dtype dtype, uint64_t seed, ag_model **out) {
    // benches/neural-network-benches/src/autograph_backend.rs:104-163
    const ag_layer_spec spec[] = {
        {AG_LAYER_CONV2, 1, 6, 5, 5, 0},   {AG_LAYER_RELU, 0, 0, 0, 0, 0},
        {AG_LAYER_MAXPOOL2, 0, 0, 2, 2, 0}, {AG_LAYER_CONV2, 6, 16, 5, 5, 0},
        {AG_LAYER_RELU, 0, 0, 0, 0, 0},    {AG_LAYER_MAXPOOL2, 0, 0, 2, 2, 0},
        {AG_LAYER_FLATTEN, 0, 0, 0, 0, 0}, {AG_LAYER_DENSE, 256, 128, 0, 0, 0},
        {AG_LAYER_RELU, 0, 0, 0, 0, 0},    {AG_LAYER_DENSE, 128, 84, 0, 0, 0},
        {AG_LAYER_RELU, 0, 0, 0, 0, 0},    {AG_LAYER_DENSE, 84, 10, 0, 0, 1},
    };
    return ag_model_create(dev, dtype, spec, (int32_t)(sizeof(spec) / sizeof(spec[0])), seed, out);
}

int ag_model_destroy(ag_model *model) {
    if (!model) return AG_OK;
    ag_device_wait(model->dev);
    delete model;
    return AG_OK;
}

int ag_model_parameter_count(ag_model *model, int32_t *count) {
    AG_REQUIRE(model && count, AG_ERR_INVALID, "null argument");
    *count = (int32_t)model->params.size();
    return AG_OK;
}

int ag_model_parameter_len(ag_model *model, int32_t index, int64_t *len) {
    AG_REQUIRE(model && len, AG_ERR_INVALID, "null argument");
    AG_REQUIRE(index >= 0 && index < (int32_t)model->params.size(), AG_ERR_INVALID,
               "parameter index %d out of range", index);
    *len = model->params[index]->value.len();
    return AG_OK;
}

int ag_model_set_parameter(ag_model *model, int32_t index, const void *host) {
    AG_REQUIRE(model && host, AG_ERR_INVALID, "null argument");
    AG_REQUIRE(index >= 0 && index < (int32_t)model->params.size(), AG_ERR_INVALID,
               "parameter index %d out of range", index);
    Tensor &v = model->params[index]->value;
    AG_TRY(ag_upload(model->dev, v.data(), host, v.nbytes()));
    return ag_device_wait(model->dev);
}

int ag_model_get_parameter(ag_model *model, int32_t index, void *host) {
    AG_REQUIRE(model && host, AG_ERR_INVALID, "null argument");
    AG_REQUIRE(index >= 0 && index < (int32_t)model->params.size(), AG_ERR_INVALID,
               "parameter index %d out of range", index);
    Tensor &v = model->params[index]->value;
    return ag_download(model->dev, host, v.data(), v.nbytes());
}

int ag_model_get_gradient(ag_model *model, int32_t index, void *host) {
    AG_REQUIRE(model && host, AG_ERR_INVALID, "null argument");
    AG_REQUIRE(index >= 0 && index < (int32_t)model->params.size(), AG_ERR_INVALID,
               "parameter index %d out of range", index);
    Tensor &g = model->params[index]->grad;
    return ag_download(model->dev, host, g.data(), g.nbytes());
}

int ag_model_get_velocity(ag_model *model, int32_t index, void *host) {
    AG_REQUIRE(model && host, AG_ERR_INVALID, "null argument");
    AG_REQUIRE(index >= 0 && index < (int32_t)model->params.size(), AG_ERR_INVALID,
               "parameter index %d out of range", index);
    Tensor &v = model->params[index]->velocity;
    return ag_download(model->dev, host, v.data(), v.nbytes());
}

int ag_model_set_velocity(ag_model *model, int32_t index, const void *host) {
    AG_REQUIRE(model && host, AG_ERR_INVALID, "null argument");
    AG_REQUIRE(index >= 0 && index < (int32_t)model->params.size(), AG_ERR_INVALID,
               "parameter index %d out of range", index);
    Tensor &v = model->params[index]->velocity;
    AG_TRY(ag_upload(model->dev, v.data(), host, v.nbytes()));
    return ag_device_wait(model->dev);
}

int ag_model_set_sgd(ag_model *model, float momentum) {
    AG_REQUIRE(model != nullptr, AG_ERR_INVALID, "model is null");
    model->use_momentum = momentum >= 0.f;
    model->momentum = momentum >= 0.f ? momentum : 0.f;
    return ag_fill_zero(model->dev, model->velocity.data(), model->velocity.nbytes());
}

int ag_model_set_grad_scale(ag_model *model, float scale) {
    AG_REQUIRE(model != nullptr, AG_ERR_INVALID, "model is null");
    model->grad_scale = scale;
    return AG_OK;
}

int ag_model_infer(ag_model *model, const void *x_host, int64_t bs, int64_t c, int64_t h, int64_t w,
                   void *logits_host) {
    AG_REQUIRE(model && logits_host, AG_ERR_INVALID, "null argument");
    AG_ENTER(model->dev);
    AG_HOST_GUARD({
        if (bs < 0 || c <= 0 || h <= 0 || w <= 0) throw Error(AG_ERR_SHAPE, "bad input shape");
        if (!x_host && bs > 0) throw Error(AG_ERR_INVALID, "input pointer is null");
        GraphEntry *g = find_graph(model, bs, c, h, w);
        run_inference(model, g, true, x_host, logits_host);
        cudaError_t e = cudaStreamSynchronize((cudaStream_t)ag_device_stream(model->dev));
        if (e != cudaSuccess)
            throw Error(AG_ERR_CUDA, std::string("cudaStreamSynchronize failed: ") + cudaGetErrorString(e));
    })
}

static void infer_enqueue_impl(ag_model *model, const void *x_host, int64_t bs, int64_t c, int64_t h,
                               int64_t w, void *logits_host, int32_t *ticket) {
        if (bs <= 0 || c <= 0 || h <= 0 || w <= 0) throw Error(AG_ERR_SHAPE, "bad input shape");
        if (!x_host) throw Error(AG_ERR_INVALID, "input pointer is null");
        void *out_dev = pinned_device_pointer(logits_host);
        if (!is_pinned_host(x_host) || !out_dev)
            throw Error(AG_ERR_INVALID, "pipelined inference needs pinned host buffers");
        auto cuda_ok = [](cudaError_t e, const char *what) {
            if (e != cudaSuccess)
                throw Error(AG_ERR_CUDA, std::string(what) + " failed: " + cudaGetErrorString(e));
        };
        cudaStream_t stream = (cudaStream_t)ag_device_stream(model->dev);
        if (!model->copy_stream)
            cuda_ok(cudaStreamCreateWithFlags(&model->copy_stream, cudaStreamNonBlocking), "copy stream");
        const int idx = model->next_slot;
        ag_model::InferSlot &sl = model->infer_slots[idx];
        if (!sl.copied) {
            cuda_ok(cudaEventCreateWithFlags(&sl.copied, cudaEventDisableTiming), "event");
            cuda_ok(cudaEventCreateWithFlags(&sl.done, cudaEventDisableTiming), "event");
        }
        if (sl.busy) throw Error(AG_ERR_INVALID, "both inference slots are in flight: wait for a ticket first");
        const Shape shape = {bs, c, h, w};
        if (!sl.x_stage.defined() || sl.x_stage.shape() != shape)
            sl.x_stage = Tensor::uninit(model->pool, shape, model->dtype);
        // the slot's previous network pass has been waited for (busy is false), so its copy of
        // the batch may be overwritten; the copy runs on its own stream
        cuda_ok(cudaMemcpyAsync(sl.x_stage.data(), x_host, sl.x_stage.nbytes(), cudaMemcpyHostToDevice,
                                model->copy_stream), "input copy");
        cuda_ok(cudaEventRecord(sl.copied, model->copy_stream), "event record");
        cuda_ok(cudaStreamWaitEvent(stream, sl.copied, 0), "event wait");
        Variable y = forward_chain(model, Variable{sl.x_stage, nullptr}, out_dev);
        if (y.value.data() != out_dev)
            cuda_ok(cudaMemcpyAsync(logits_host, y.value.data(), y.value.nbytes(), cudaMemcpyDeviceToHost,
                                    stream), "output copy");
        cuda_ok(cudaEventRecord(sl.done, stream), "event record");
        sl.busy = true;
        model->next_slot = idx ^ 1;
        *ticket = idx;
    }

int ag_model_infer_enqueue(ag_model *model, const void *x_host, int64_t bs, int64_t c, int64_t h,
                           int64_t w, void *logits_host, int32_t *ticket) {
    AG_REQUIRE(model && logits_host && ticket, AG_ERR_INVALID, "null argument");
    AG_ENTER(model->dev);
    AG_HOST_GUARD({ infer_enqueue_impl(model, x_host, bs, c, h, w, logits_host, ticket); })
}

int ag_model_infer_wait(ag_model *model, int32_t ticket) {
    AG_REQUIRE(model && (ticket == 0 || ticket == 1), AG_ERR_INVALID, "bad ticket");
    AG_ENTER(model->dev);
    AG_HOST_GUARD({
        ag_model::InferSlot &sl = model->infer_slots[ticket];
        if (!sl.busy) throw Error(AG_ERR_INVALID, "nothing in flight under this ticket");
        cudaError_t e = cudaEventSynchronize(sl.done);
        sl.busy = false;
        if (e != cudaSuccess)
            throw Error(AG_ERR_CUDA, std::string("cudaEventSynchronize failed: ") + cudaGetErrorString(e));
    })
}

int ag_model_infer_u8(ag_model *model, const uint8_t *x_host, int64_t bs, int64_t c, int64_t h,
                      int64_t w, float alpha, void *logits_host) {
    AG_REQUIRE(model && logits_host, AG_ERR_INVALID, "null argument");
    AG_ENTER(model->dev);
    AG_HOST_GUARD({
        if (bs < 0 || c <= 0 || h <= 0 || w <= 0) throw Error(AG_ERR_SHAPE, "bad input shape");
        if (!x_host && bs > 0) throw Error(AG_ERR_INVALID, "input pointer is null");
        if (bs > 0) infer_u8(model, x_host, bs, c, h, w, alpha, logits_host);
    })
}

int ag_model_forward_device(ag_model *model, const void *x_dev, int64_t bs, int64_t c, int64_t h,
                            int64_t w, void *logits_dev) {
    AG_REQUIRE(model && logits_dev, AG_ERR_INVALID, "null argument");
    AG_ENTER(model->dev);
    AG_HOST_GUARD({
        if (bs < 0 || c <= 0 || h <= 0 || w <= 0) throw Error(AG_ERR_SHAPE, "bad input shape");
        if (!x_dev && bs > 0) throw Error(AG_ERR_INVALID, "input pointer is null");
        GraphEntry *g = find_graph(model, bs, c, h, w);
        run_inference(model, g, false, x_dev, logits_dev);
    })
}

int ag_model_train_step(ag_model *model, const void *x_host, const uint8_t *t_host, int64_t bs,
                        int64_t c, int64_t h, int64_t w, float lr, float *loss_host) {
    AG_REQUIRE(model && t_host && loss_host, AG_ERR_INVALID, "null argument");
    AG_ENTER(model->dev);
    AG_HOST_GUARD({
        if (bs < 0 || c <= 0 || h <= 0 || w <= 0) throw Error(AG_ERR_SHAPE, "bad input shape");
        if (!x_host && bs > 0) throw Error(AG_ERR_INVALID, "input pointer is null");
        if (!train_step_graph(model, x_host, t_host, bs, c, h, w, lr, loss_host)) {
            Tensor x = input_tensor(model, x_host, true, bs, c, h, w);
            Tensor t = Tensor::from_host(model->pool, {bs}, AG_U8, t_host);
            *loss_host = forward_backward(model, x, t);
            apply_update(model, lr);
        }
    })
}

int ag_model_train_forward_backward(ag_model *model, const void *x_dev, const uint8_t *t_dev,
                                    int64_t bs, int64_t c, int64_t h, int64_t w, float *loss_host,
                                    void **grad_bucket, int64_t *grad_len) {
    AG_REQUIRE(model && t_dev, AG_ERR_INVALID, "null argument");
    AG_ENTER(model->dev);
    AG_HOST_GUARD({
        if (bs < 0 || c <= 0 || h <= 0 || w <= 0) throw Error(AG_ERR_SHAPE, "bad input shape");
        if (!x_dev && bs > 0) throw Error(AG_ERR_INVALID, "input pointer is null");
        if (!train_step_graph(model, x_dev, t_dev, bs, c, h, w, 0.f, loss_host, false, true)) {
            Tensor x = input_tensor(model, x_dev, false, bs, c, h, w);
            Tensor t = Tensor::external(model->dev, const_cast<uint8_t *>(t_dev), {bs}, AG_U8);
            model->loss_eager = forward_backward(model, x, t);
            model->loss_in_flight = false;
            if (loss_host) *loss_host = model->loss_eager;
        }
        if (grad_bucket) *grad_bucket = model->grads.data();
        if (grad_len) *grad_len = model->bucket_len;
    })
}

int ag_model_last_loss(ag_model *model, float *loss_host) {
    AG_REQUIRE(model && loss_host, AG_ERR_INVALID, "null argument");
    AG_ENTER(model->dev);
    if (model->loss_in_flight) {
        AG_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)ag_device_stream(model->dev)));
        model->loss_eager = *model->loss_pinned;
        model->loss_in_flight = false;
    }
    *loss_host = model->loss_eager;
    return AG_OK;
}

int ag_model_allreduce_update(ag_model *model, ag_comm *comm, int rank, float lr) {
    AG_REQUIRE(model != nullptr && comm != nullptr, AG_ERR_INVALID, "null argument");
    AG_ENTER(model->dev);
    AG_TRY(::ag::comm_fused_update(comm, rank, model->dtype, model->grads.data(),
                                   model->values.data(), model->velocity.data(), model->bucket_len,
                                   model->grad_scale, lr, model->momentum, model->use_momentum));
    for (Parameter *p : model->params) p->node.reset();  // ≙ take_grad consumed the gradient
    return AG_OK;
}

int ag_model_apply_update(ag_model *model, float lr) {
    AG_REQUIRE(model != nullptr, AG_ERR_INVALID, "model is null");
    AG_ENTER(model->dev);
    AG_HOST_GUARD({ apply_update(model, lr); })
}

}  // extern "C"
