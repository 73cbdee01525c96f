// Convolution entry points: implicit-GEMM forward / backward-input /
// backward-weight on the SIMT tile engine (the patch matrix is never written to
// memory), plus the stand-alone im2col / col2im kernels.
#include "conv2_direct.cuh"
#include "conv_tc.cuh"
#include "gemm_simt_launch.cuh"

namespace ag {

struct ConvGeom {
    int bs, c, ih, iw;      // image tensor [bs, c, ih, iw]
    int oh, ow;             // patch grid
    int fh, fw, ph, pw, sh, sw, dh, dw;
    FastDiv div_ohw, div_ow, div_ff, div_fw;
};

static int make_geom(int64_t bs, int64_t c, int64_t ih, int64_t iw, const ag_conv2_options *o,
                     ConvGeom *g) {
    AG_REQUIRE(o != nullptr, AG_ERR_INVALID, "conv options are null");
    AG_REQUIRE(bs >= 0 && c >= 0 && ih > 0 && iw > 0, AG_ERR_SHAPE,
               "bad image shape [%lld,%lld,%lld,%lld]", (long long)bs, (long long)c, (long long)ih,
               (long long)iw);
    AG_REQUIRE(o->filter[0] > 0 && o->filter[1] > 0 && o->stride[0] > 0 && o->stride[1] > 0 &&
                   o->dilation[0] > 0 && o->dilation[1] > 0 && o->padding[0] >= 0 &&
                   o->padding[1] >= 0,
               AG_ERR_INVALID, "bad convolution options");
    int64_t oh = (ih + 2 * o->padding[0] - o->dilation[0] * (o->filter[0] - 1) - 1);
    int64_t ow = (iw + 2 * o->padding[1] - o->dilation[1] * (o->filter[1] - 1) - 1);
    AG_REQUIRE(oh >= 0 && ow >= 0, AG_ERR_SHAPE, "filter does not fit the input");
    oh = oh / o->stride[0] + 1;
    ow = ow / o->stride[1] + 1;
    AG_REQUIRE(bs * oh * ow < (1ll << 31) && bs * c * ih * iw < (1ll << 31) &&
                   c * o->filter[0] * o->filter[1] < (1ll << 31),
               AG_ERR_LIMIT, "convolution problem beyond 2^31 elements");
    g->bs = (int)bs; g->c = (int)c; g->ih = (int)ih; g->iw = (int)iw;
    g->oh = (int)oh; g->ow = (int)ow;
    g->fh = o->filter[0]; g->fw = o->filter[1];
    g->ph = o->padding[0]; g->pw = o->padding[1];
    g->sh = o->stride[0]; g->sw = o->stride[1];
    g->dh = o->dilation[0]; g->dw = o->dilation[1];
    g->div_ohw = FastDiv((uint32_t)(oh * ow));
    g->div_ow = FastDiv((uint32_t)ow);
    g->div_ff = FastDiv((uint32_t)(g->fh * g->fw));
    g->div_fw = FastDiv((uint32_t)g->fw);
    return AG_OK;
}

// Element (pos, col) of im2col(x): pos = (b, hy, wy), col = (ci, fi, fj); zero in the padding.
template <class T>
__device__ __forceinline__ float im2col_at(const T *x, const ConvGeom &g, int pos, int col) {
    uint32_t b, r, hy, wy, ci, f, fi, fj;
    g.div_ohw.divmod((uint32_t)pos, b, r);
    g.div_ow.divmod(r, hy, wy);
    g.div_ff.divmod((uint32_t)col, ci, f);
    g.div_fw.divmod(f, fi, fj);
    int hx = (int)(hy * g.sh + fi * g.dh) - g.ph;
    int wx = (int)(wy * g.sw + fj * g.dw) - g.pw;
    if ((unsigned)hx >= (unsigned)g.ih || (unsigned)wx >= (unsigned)g.iw) return 0.f;
    return to_f32(x[((int64_t)(b * g.c + ci) * g.ih + hx) * g.iw + wx]);
}

// im2col(x) as a GEMM operand. POS_IS_K = false: mn = patch position (forward A
// operand); true: k = patch position (backward-weight B operand).
template <class T, bool POS_IS_K>
struct Im2colOperand {
    static constexpr bool kFastK = POS_IS_K;  // memory is contiguous along the position
    const T *x;
    ConvGeom g;
    int mn_size, k_size;
    bool vec;
    __device__ __forceinline__ float at(int mn, int k) const {
        if (mn >= mn_size || k >= k_size) return 0.f;
        return POS_IS_K ? im2col_at(x, g, k, mn) : im2col_at(x, g, mn, k);
    }
    __device__ __forceinline__ bool in_range4(int, int) const { return false; }
    __device__ __forceinline__ void load4(int, int, float (&)[4]) const {}
};

// dy^T as the backward-weight A operand: (mn = output channel, k = (b, hy, wy)).
template <class T>
struct DyTransposedOperand {
    static constexpr bool kFastK = true;
    const T *dy;
    int oc, ohw;
    FastDiv div_ohw;
    int mn_size, k_size;
    bool vec;
    __device__ __forceinline__ float at(int mn, int k) const {
        if (mn >= mn_size || k >= k_size) return 0.f;
        uint32_t b, r;
        div_ohw.divmod((uint32_t)k, b, r);
        return to_f32(dy[((int64_t)b * oc + mn) * ohw + r]);
    }
    __device__ __forceinline__ bool in_range4(int, int) const { return false; }
    __device__ __forceinline__ void load4(int, int, float (&)[4]) const {}
};

// Backward-input A operand: (mn = (b, hx, wx) input position, k = (co, fi, fj)) ->
// dy[b, co, hy, wy] when (hx + ph - fi*dh) = hy*sh and (wx + pw - fj*dw) = wy*sw
// for an in-range (hy, wy); zero otherwise.  g describes the forward geometry
// (g.c = input channels), oc the number of output channels.
template <class T>
struct DyGatherOperand {
    static constexpr bool kFastK = false;
    const T *dy;
    ConvGeom g;
    int oc;
    FastDiv div_ihw, div_iw, div_sh, div_sw;
    int mn_size, k_size;
    bool vec;
    __device__ __forceinline__ float at(int mn, int k) const {
        if (mn >= mn_size || k >= k_size) return 0.f;
        uint32_t b, r, hx, wx, co, f, fi, fj;
        div_ihw.divmod((uint32_t)mn, b, r);
        div_iw.divmod(r, hx, wx);
        g.div_ff.divmod((uint32_t)k, co, f);
        g.div_fw.divmod(f, fi, fj);
        int th = (int)hx + g.ph - (int)(fi * g.dh);
        int tw = (int)wx + g.pw - (int)(fj * g.dw);
        if (th < 0 || tw < 0) return 0.f;
        uint32_t hy, rh, wy, rw;
        div_sh.divmod((uint32_t)th, hy, rh);
        div_sw.divmod((uint32_t)tw, wy, rw);
        if (rh != 0 || rw != 0 || hy >= (uint32_t)g.oh || wy >= (uint32_t)g.ow) return 0.f;
        return to_f32(dy[((int64_t)(b * oc + co) * g.oh + hy) * g.ow + wy]);
    }
    __device__ __forceinline__ bool in_range4(int, int) const { return false; }
    __device__ __forceinline__ void load4(int, int, float (&)[4]) const {}
};

// Backward-input B operand: (k = (co, fi, fj), mn = ci) -> w[co, ci, fi, fj].
template <class T>
struct WeightTransposedOperand {
    static constexpr bool kFastK = true;
    const T *w;
    int ic, ff;
    FastDiv div_ff;
    int mn_size, k_size;
    bool vec;
    __device__ __forceinline__ float at(int mn, int k) const {
        if (mn >= mn_size || k >= k_size) return 0.f;
        uint32_t co, f;
        div_ff.divmod((uint32_t)k, co, f);
        return to_f32(w[((int64_t)co * ic + mn) * ff + f]);
    }
    __device__ __forceinline__ bool in_range4(int, int) const { return false; }
    __device__ __forceinline__ void load4(int, int, float (&)[4]) const {}
};

// Writes GEMM element (m = (b, position), n = channel) into an NCHW tensor,
// with optional bias and relu.  For bf16 the accumulator is rounded before the
// bias is added, so the result equals the reference's unfused sequence
// (dot -> bf16, then scaled_add of the bias in bf16).
template <class T>
struct NchwEpilogue {
    T *y;
    const T *bias;
    int channels, hw;
    FastDiv div_hw;
    bool relu;
    __device__ __forceinline__ void store(int m, int n, float acc) const {
        uint32_t b, r;
        div_hw.divmod((uint32_t)m, b, r);
        float v = to_f32(from_f32<T>(acc));
        if (bias != nullptr) v = to_f32(from_f32<T>(v + to_f32(bias[n])));
        if (relu) v = (v >= 0.f) ? v : 0.f;
        y[((int64_t)b * channels + n) * hw + r] = from_f32<T>(v);
    }
    __device__ __forceinline__ bool can4(int, int) const { return false; }
    __device__ __forceinline__ void store4(int, int, const float (&)[4]) const {}
};

template <class T>
static bool aligned4(const T *p) {
    return (reinterpret_cast<uintptr_t>(p) % (4 * sizeof(T))) == 0;
}

template <class T>
static int conv2_forward_t(ag_device *dev, const ConvGeom &g, const T *x, const T *w, int oc,
                           const T *bias, bool relu, T *y) {
    const int M = g.bs * g.oh * g.ow, N = oc, K = g.c * g.fh * g.fw;
    Im2colOperand<T, false> A{x, g, M, K, false};
    simt::StridedOperand<T, true> B{w, (int64_t)K, 1, N, K, (K % 4 == 0) && aligned4(w)};
    NchwEpilogue<T> E{y, bias, oc, g.oh * g.ow, FastDiv((uint32_t)(g.oh * g.ow)), relu};
    return simt::gemm(dev, M, N, K, A, B, E, /*allow_split=*/false);
}

template <class T>
static int conv2_backward_input_t(ag_device *dev, const ConvGeom &g, const T *w, int oc,
                                  const T *dy, T *dx) {
    const int M = g.bs * g.ih * g.iw, N = g.c, K = oc * g.fh * g.fw;
    DyGatherOperand<T> A{dy, g, oc, FastDiv((uint32_t)(g.ih * g.iw)), FastDiv((uint32_t)g.iw),
                         FastDiv((uint32_t)g.sh), FastDiv((uint32_t)g.sw), M, K, false};
    WeightTransposedOperand<T> B{w, g.c, g.fh * g.fw, FastDiv((uint32_t)(g.fh * g.fw)), N, K,
                                 false};
    NchwEpilogue<T> E{dx, nullptr, g.c, g.ih * g.iw, FastDiv((uint32_t)(g.ih * g.iw)), false};
    return simt::gemm(dev, M, N, K, A, B, E, /*allow_split=*/false);
}

template <class T>
static int conv2_backward_weight_t(ag_device *dev, const ConvGeom &g, const T *x, const T *dy,
                                   int oc, float beta, T *dw) {
    const int M = oc, N = g.c * g.fh * g.fw, K = g.bs * g.oh * g.ow;
    DyTransposedOperand<T> A{dy, oc, g.oh * g.ow, FastDiv((uint32_t)(g.oh * g.ow)), M, K, false};
    Im2colOperand<T, true> B{x, g, N, K, false};
    simt::StridedEpilogue<T> E{dw, (int64_t)N, 1, 1.f, beta, false, N};
    return simt::gemm(dev, M, N, K, A, B, E, /*allow_split=*/true);
}

// ---- stand-alone im2col / col2im ------------------------------------------
template <class T>
__global__ void im2col_kernel(const T *__restrict__ x, T *__restrict__ y, ConvGeom g, int cols,
                              int64_t total, FastDiv div_cols) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        // i = pos * cols + col; rows are split so that i / cols stays below 2^31
        int64_t pos = i / cols;
        int col = (int)(i - pos * cols);
        y[i] = from_f32<T>(im2col_at(x, g, (int)pos, col));
    }
}

// Gather form of col2im: every image element sums the patch entries that were
// copied from it, in f32 (the reference's device kernel does the same).
template <class T>
__global__ void col2im_kernel(const T *__restrict__ x, T *__restrict__ y, ConvGeom g, int oh_img,
                              int ow_img, int64_t total) {
    // g.oh / g.ow = patch grid (gh, gw); the image is [bs, c, oh_img, ow_img].
    const int ff = g.fh * g.fw;
    const int64_t cols = (int64_t)g.c * ff;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int wy = (int)(i % ow_img);
        int64_t t = i / ow_img;
        int hy = (int)(t % oh_img);
        t /= oh_img;
        int ci = (int)(t % g.c);
        int b = (int)(t / g.c);
        float acc = 0.f;
        for (int fi = 0; fi < g.fh; ++fi) {
            int th = hy + g.ph - fi * g.dh;
            if (th < 0 || th % g.sh != 0) continue;
            int hid = th / g.sh;
            if (hid >= g.oh) continue;
            for (int fj = 0; fj < g.fw; ++fj) {
                int tw = wy + g.pw - fj * g.dw;
                if (tw < 0 || tw % g.sw != 0) continue;
                int wid = tw / g.sw;
                if (wid >= g.ow) continue;
                int64_t row = ((int64_t)b * g.oh + hid) * g.ow + wid;
                acc += to_f32(x[row * cols + (int64_t)ci * ff + fi * g.fw + fj]);
            }
        }
        y[i] = from_f32<T>(acc);
    }
}

static unsigned grid_for(int64_t total, int threads, int sms) {
    int64_t blocks = ceil_div(total, threads);
    int64_t cap = (int64_t)sms * 16;
    return (unsigned)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

}  // namespace ag

using namespace ag;

extern "C" {

int ag_conv2_output_shape(int64_t ih, int64_t iw, const ag_conv2_options *opt, int64_t *oh,
                          int64_t *ow) {
    AG_REQUIRE(opt && oh && ow, AG_ERR_INVALID, "null argument");
    ConvGeom g;
    AG_TRY(make_geom(1, 1, ih, iw, opt, &g));
    *oh = g.oh;
    *ow = g.ow;
    return AG_OK;
}

int ag_conv2_forward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs, int64_t ic,
                     int64_t ih, int64_t iw, const void *w, int64_t oc, const void *bias,
                     const ag_conv2_options *opt, int fuse_relu, void *y) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "Conv %d not implemented", (int)dtype);
    ConvGeom g;
    AG_TRY(make_geom(bs, ic, ih, iw, opt, &g));
    AG_REQUIRE(oc >= 0 && oc < (1 << 30), AG_ERR_SHAPE, "bad output channel count");
    if (bs == 0 || oc == 0) return AG_OK;
    AG_REQUIRE(x && w && y, AG_ERR_INVALID, "null tensor pointer");
    if (dtype == AG_BF16 && convtc::eligible_forward(bs, ic, ih, iw, oc, opt))
        return convtc::forward(dev, (const __nv_bfloat16 *)x, bs, ic, ih, iw,
                               (const __nv_bfloat16 *)w, oc, (const __nv_bfloat16 *)bias, opt,
                               fuse_relu != 0, (__nv_bfloat16 *)y);
    if (direct::eligible(bs, ic, ih, iw, oc, opt)) {
        if (dtype == AG_F32)
            return direct::forward<float>(dev, (const float *)x, bs, ic, ih, iw, (const float *)w,
                                          oc, (const float *)bias, opt, fuse_relu != 0, false,
                                          (float *)y);
        return direct::forward<__nv_bfloat16>(dev, (const __nv_bfloat16 *)x, bs, ic, ih, iw,
                                              (const __nv_bfloat16 *)w, oc,
                                              (const __nv_bfloat16 *)bias, opt, fuse_relu != 0,
                                              false, (__nv_bfloat16 *)y);
    }
    if (dtype == AG_F32)
        return conv2_forward_t<float>(dev, g, (const float *)x, (const float *)w, (int)oc,
                                      (const float *)bias, fuse_relu != 0, (float *)y);
    return conv2_forward_t<__nv_bfloat16>(dev, g, (const __nv_bfloat16 *)x,
                                          (const __nv_bfloat16 *)w, (int)oc,
                                          (const __nv_bfloat16 *)bias, fuse_relu != 0,
                                          (__nv_bfloat16 *)y);
}

int ag_conv2_relu_max_pool2_forward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                                    int64_t ic, int64_t ih, int64_t iw, const void *w, int64_t oc,
                                    const void *bias, const ag_conv2_options *opt, int fuse_relu,
                                    int32_t pool_h, int32_t pool_w, void *y) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "Conv %d not implemented", (int)dtype);
    AG_REQUIRE(pool_h > 0 && pool_w > 0, AG_ERR_INVALID, "bad pool window");
    ConvGeom g;
    AG_TRY(make_geom(bs, ic, ih, iw, opt, &g));
    AG_REQUIRE(g.oh >= pool_h && g.ow >= pool_w, AG_ERR_SHAPE,
               "pool window [%d,%d] does not fit the convolution output [%d,%d]", pool_h, pool_w,
               g.oh, g.ow);
    if (bs == 0 || oc == 0) return AG_OK;
    AG_REQUIRE(x && w && y, AG_ERR_INVALID, "null tensor pointer");
    // Same engine as ag_conv2_forward would pick, so that the fused call equals the
    // separate calls bit for bit.
    const bool tensor_core = dtype == AG_BF16 && convtc::eligible_forward(bs, ic, ih, iw, oc, opt);
    if (!tensor_core && pool_h == 2 && pool_w == 2 && direct::eligible(bs, ic, ih, iw, oc, opt)) {
        if (dtype == AG_F32)
            return direct::forward<float>(dev, (const float *)x, bs, ic, ih, iw, (const float *)w,
                                          oc, (const float *)bias, opt, fuse_relu != 0, true,
                                          (float *)y);
        return direct::forward<__nv_bfloat16>(dev, (const __nv_bfloat16 *)x, bs, ic, ih, iw,
                                              (const __nv_bfloat16 *)w, oc,
                                              (const __nv_bfloat16 *)bias, opt, fuse_relu != 0,
                                              true, (__nv_bfloat16 *)y);
    }
    // General shapes: convolution into the device workspace, then the pool kernel.
    // (neither of the two kernels below uses the workspace itself)
    void *tmp = nullptr;
    AG_TRY(workspace(dev, (size_t)bs * oc * g.oh * g.ow * dtype_size(dtype), &tmp));
    AG_TRY(ag_conv2_forward(dev, dtype, x, bs, ic, ih, iw, w, oc, bias, opt, fuse_relu, tmp));
    return ag_max_pool2(dev, dtype, tmp, bs, oc, g.oh, g.ow, pool_h, pool_w, pool_h, pool_w, y);
}

int ag_conv2_relu_max_pool2_forward_keep(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                                         int64_t ic, int64_t ih, int64_t iw, const void *w,
                                         int64_t oc, const void *bias, const ag_conv2_options *opt,
                                         void *pre, void *y) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "Conv %d not implemented", (int)dtype);
    ConvGeom g;
    AG_TRY(make_geom(bs, ic, ih, iw, opt, &g));
    AG_REQUIRE(g.oh >= 2 && g.ow >= 2, AG_ERR_SHAPE,
               "pool window [2,2] does not fit the convolution output [%d,%d]", g.oh, g.ow);
    if (bs == 0 || oc == 0) return AG_OK;
    AG_REQUIRE(x && w && pre && y, AG_ERR_INVALID, "null tensor pointer");
    const bool tensor_core = dtype == AG_BF16 && convtc::eligible_forward(bs, ic, ih, iw, oc, opt);
    if (!tensor_core && oc < 32 && direct::eligible(bs, ic, ih, iw, oc, opt)) {
        if (dtype == AG_F32)
            return direct::forward<float>(dev, (const float *)x, bs, ic, ih, iw, (const float *)w,
                                          oc, (const float *)bias, opt, true, true, (float *)y,
                                          (float *)pre);
        return direct::forward<__nv_bfloat16>(dev, (const __nv_bfloat16 *)x, bs, ic, ih, iw,
                                              (const __nv_bfloat16 *)w, oc,
                                              (const __nv_bfloat16 *)bias, opt, true, true,
                                              (__nv_bfloat16 *)y, (__nv_bfloat16 *)pre);
    }
    AG_TRY(ag_conv2_forward(dev, dtype, x, bs, ic, ih, iw, w, oc, bias, opt, 0, pre));
    if ((g.oh & 1) == 0 && (g.ow & 1) == 0)
        return ag_relu_max_pool2_forward(dev, dtype, pre, bs, oc, g.oh, g.ow, y);
    // odd planes: relu into the workspace, then the general pool
    void *tmp = nullptr;
    AG_TRY(workspace(dev, (size_t)bs * oc * g.oh * g.ow * dtype_size(dtype), &tmp));
    AG_TRY(ag_relu(dev, dtype, pre, tmp, bs * oc * g.oh * g.ow));
    return ag_max_pool2(dev, dtype, tmp, bs, oc, g.oh, g.ow, 2, 2, 2, 2, y);
}

int ag_conv2_backward_input(ag_device *dev, ag_dtype dtype, const void *w, int64_t oc, int64_t ic,
                            const void *dy, int64_t bs, int64_t ih, int64_t iw,
                            const ag_conv2_options *opt, void *dx) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "Conv %d not implemented", (int)dtype);
    ConvGeom g;
    AG_TRY(make_geom(bs, ic, ih, iw, opt, &g));
    AG_REQUIRE(oc >= 0 && oc * g.fh * g.fw < (1ll << 31), AG_ERR_SHAPE,
               "bad output channel count");
    if (bs == 0 || ic == 0) return AG_OK;
    AG_REQUIRE(w && dy && dx, AG_ERR_INVALID, "null tensor pointer");
    if (dtype == AG_BF16 && convtc::eligible_backward_input(bs, ic, ih, iw, oc, opt))
        return convtc::backward_input(dev, (const __nv_bfloat16 *)w, oc, ic,
                                      (const __nv_bfloat16 *)dy, bs, ih, iw, opt,
                                      (__nv_bfloat16 *)dx);
    if (direct::eligible_backward_input(bs, ic, ih, iw, oc, opt)) {
        if (dtype == AG_F32)
            return direct::backward_input<float>(dev, (const float *)w, oc, ic, (const float *)dy,
                                                 bs, ih, iw, opt, (float *)dx);
        return direct::backward_input<__nv_bfloat16>(dev, (const __nv_bfloat16 *)w, oc, ic,
                                                     (const __nv_bfloat16 *)dy, bs, ih, iw, opt,
                                                     (__nv_bfloat16 *)dx);
    }
    if (dtype == AG_F32)
        return conv2_backward_input_t<float>(dev, g, (const float *)w, (int)oc, (const float *)dy,
                                             (float *)dx);
    return conv2_backward_input_t<__nv_bfloat16>(dev, g, (const __nv_bfloat16 *)w, (int)oc,
                                                 (const __nv_bfloat16 *)dy, (__nv_bfloat16 *)dx);
}

int ag_conv2_backward_weight(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs, int64_t ic,
                             int64_t ih, int64_t iw, const void *dy, int64_t oc,
                             const ag_conv2_options *opt, float beta, void *dw) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "Conv %d not implemented", (int)dtype);
    ConvGeom g;
    AG_TRY(make_geom(bs, ic, ih, iw, opt, &g));
    AG_REQUIRE(oc >= 0 && oc < (1 << 30), AG_ERR_SHAPE, "bad output channel count");
    if (oc == 0 || ic == 0) return AG_OK;
    AG_REQUIRE(dw && (bs == 0 || (x && dy)), AG_ERR_INVALID, "null tensor pointer");
    if (dtype == AG_BF16 && convtc::eligible_backward_weight(bs, ic, ih, iw, oc, opt))
        return convtc::backward_weight(dev, (const __nv_bfloat16 *)x, bs, ic, ih, iw,
                                       (const __nv_bfloat16 *)dy, oc, opt, beta,
                                       (__nv_bfloat16 *)dw);
    if (direct::eligible_backward_weight(bs, ic, ih, iw, oc, opt)) {
        if (dtype == AG_F32)
            return direct::backward_weight<float>(dev, (const float *)x, bs, ic, ih, iw,
                                                  (const float *)dy, oc, opt, beta, (float *)dw);
        return direct::backward_weight<__nv_bfloat16>(dev, (const __nv_bfloat16 *)x, bs, ic, ih, iw,
                                                      (const __nv_bfloat16 *)dy, oc, opt, beta,
                                                      (__nv_bfloat16 *)dw);
    }
    if (dtype == AG_F32)
        return conv2_backward_weight_t<float>(dev, g, (const float *)x, (const float *)dy, (int)oc,
                                              beta, (float *)dw);
    return conv2_backward_weight_t<__nv_bfloat16>(dev, g, (const __nv_bfloat16 *)x,
                                                  (const __nv_bfloat16 *)dy, (int)oc, beta,
                                                  (__nv_bfloat16 *)dw);
}

int ag_im2col_conv2(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs, int64_t c,
                    int64_t ih, int64_t iw, const ag_conv2_options *opt, void *y) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "im2col_conv2 %d unimplemented", (int)dtype);
    ConvGeom g;
    AG_TRY(make_geom(bs, c, ih, iw, opt, &g));
    const int cols = g.c * g.fh * g.fw;
    const int64_t total = (int64_t)g.bs * g.oh * g.ow * cols;
    if (total == 0) return AG_OK;
    AG_REQUIRE(x && y, AG_ERR_INVALID, "null tensor pointer");
    const int threads = 256;
    const unsigned grid = grid_for(total, threads, dev->sm_count);
    if (dtype == AG_F32)
        im2col_kernel<float><<<grid, threads, 0, dev->stream>>>((const float *)x, (float *)y, g,
                                                                cols, total, FastDiv(cols));
    else
        im2col_kernel<__nv_bfloat16><<<grid, threads, 0, dev->stream>>>(
            (const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, g, cols, total, FastDiv(cols));
    AG_CHECK_LAUNCH();
    return AG_OK;
}

int ag_col2im_conv2(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs, int64_t c,
                    int64_t gh, int64_t gw, const ag_conv2_options *opt, void *y) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "col2im_conv2 %d unimplemented", (int)dtype);
    AG_REQUIRE(opt != nullptr, AG_ERR_INVALID, "conv options are null");
    AG_REQUIRE(gh > 0 && gw > 0 && bs >= 0 && c >= 0, AG_ERR_SHAPE, "bad patch grid");
    // Image size (src/ops.rs Col2ImConv2Options::output_shape).
    int64_t oh = (gh - 1) * opt->stride[0] + opt->dilation[0] * (opt->filter[0] - 1) + 1 -
                 2 * opt->padding[0];
    int64_t ow = (gw - 1) * opt->stride[1] + opt->dilation[1] * (opt->filter[1] - 1) + 1 -
                 2 * opt->padding[1];
    AG_REQUIRE(oh > 0 && ow > 0, AG_ERR_SHAPE, "col2im image shape is not positive");
    ConvGeom g;
    g.bs = (int)bs; g.c = (int)c; g.ih = (int)oh; g.iw = (int)ow;
    g.oh = (int)gh; g.ow = (int)gw;
    g.fh = opt->filter[0]; g.fw = opt->filter[1];
    g.ph = opt->padding[0]; g.pw = opt->padding[1];
    g.sh = opt->stride[0]; g.sw = opt->stride[1];
    g.dh = opt->dilation[0]; g.dw = opt->dilation[1];
    AG_REQUIRE(g.fh > 0 && g.fw > 0 && g.sh > 0 && g.sw > 0 && g.dh > 0 && g.dw > 0 && g.ph >= 0 &&
                   g.pw >= 0,
               AG_ERR_INVALID, "bad convolution options");
    const int64_t total = bs * c * oh * ow;
    AG_REQUIRE(total < (1ll << 40), AG_ERR_LIMIT, "image too large");
    if (total == 0) return AG_OK;
    AG_REQUIRE(x && y, AG_ERR_INVALID, "null tensor pointer");
    const int threads = 256;
    const unsigned grid = grid_for(total, threads, dev->sm_count);
    if (dtype == AG_F32)
        col2im_kernel<float><<<grid, threads, 0, dev->stream>>>((const float *)x, (float *)y, g,
                                                                (int)oh, (int)ow, total);
    else
        col2im_kernel<__nv_bfloat16><<<grid, threads, 0, dev->stream>>>(
            (const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, g, (int)oh, (int)ow, total);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

}  // extern "C"
