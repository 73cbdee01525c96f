// Direct convolution for small channel counts with default options (no
// padding, stride 1, dilation 1): the LeNet5 layers and the first layer of the
// wider stack.  A CTA stages a group of images and the whole filter bank in
// shared memory; every thread owns a 2x4 block of output pixels for two output
// channels and keeps the (FH+1) x (FW+3) input patch of the current input
// channel in registers, so each filter tap costs one 8-byte shared-memory load
// and 16 FFMAs.  Bias, ReLU and a 2x2 / stride-2 max pool are applied to the
// block in registers, which removes the separate ReLU and pool passes (and
// their HBM / L2 round trips) from inference.
//
// The sum for one output runs over (input channel, fi, fj) in that order with
// fused multiply-add, the order of the reference's naive convolution
// (tests/integration_tests.rs:1147-1171).
#include "conv2_direct.cuh"
#include "conv2_direct_device.cuh"

namespace ag {
namespace direct {

// Stores to global memory: y [bs][oc][ph][pw] (pooled) or [bs][oc][oh][ow].
template <class T>
struct GlobalOut {
    T *y;
    int b0, oc, h, w;  // first image of the CTA; channel count; height and width of y
    T *pre_y;          // optional [bs][oc][ph][pw]: the convolution's output before relu / pool
    int ph, pw;
    __device__ __forceinline__ void pre(int g, int c, int yy, int xx, float v) const {
        pre_y[(((int64_t)(b0 + g) * oc + c) * ph + yy) * pw + xx] = from_f32<T>(v);
    }
    __device__ __forceinline__ void pooled(int g, int c, int py, int px, float v) const {
        y[(((int64_t)(b0 + g) * oc + c) * h + py) * w + px] = from_f32<T>(v);
    }
    __device__ __forceinline__ void plain(int g, int c, int yy, int xx, float v) const {
        pooled(g, c, yy, xx, v);
    }
};

// grid.x = ceil(bs / group); dynamic shared memory:
//   float img[group][ic][ih][iw]; float wts[ic][FH][FW][ocp]; float bias[ocp]
template <class T, int FH, int FW, bool BWD>
__global__ void __launch_bounds__(256, 2)
    conv2_direct_kernel(const T *__restrict__ x, const T *__restrict__ w,
                        const T *__restrict__ bias, T *__restrict__ y, const Params p,
                        T *__restrict__ pre_y) {
    extern __shared__ __align__(16) float smem[];
    const int img_elems = p.ic * p.ih * p.iw;
    const int taps = p.ic * FH * FW;
    const int b0 = blockIdx.x * p.group;
    const int nimg = min(p.group, p.bs - b0);
    float *s_img = smem;
    float *s_w = smem + ((p.group * img_elems + 3) & ~3);
    float *s_bias = s_w + taps * p.ocp;

    if (BWD) {
        // dy [nimg][ic][ih-2(FH-1)][iw-2(FW-1)] into the middle of a zeroed frame
        const int sh = p.ih - 2 * (FH - 1), sw = p.iw - 2 * (FW - 1);
        const T *src = x + (int64_t)b0 * p.ic * sh * sw;
        const int total = nimg * img_elems;
        if ((sw & 3) == 0 && reinterpret_cast<uintptr_t>(src) % (4 * sizeof(T)) == 0) {
            // zero the frames with 16-byte stores, then copy dy four elements per load
            float4 *z = reinterpret_cast<float4 *>(s_img);
            for (int i = threadIdx.x; i < (total + 3) / 4; i += blockDim.x)
                z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            __syncthreads();
            const int qpr = sw / 4;  // loads per source row
            for (int i = threadIdx.x; i < nimg * p.ic * sh * qpr; i += blockDim.x) {
                const int q = i % qpr, row = i / qpr;
                const int r = row % sh, plane = row / sh;
                float v[4];
                load4_to_f32<T>(src + (int64_t)row * sw + 4 * q, v);
                float *dst = s_img + plane * (p.ih * p.iw) + (r + FH - 1) * p.iw + (FW - 1) + 4 * q;
                dst[0] = v[0]; dst[1] = v[1]; dst[2] = v[2]; dst[3] = v[3];
            }
        } else {
            for (int i = threadIdx.x; i < total; i += blockDim.x) {
                const int plane = i / (p.ih * p.iw), rem = i - plane * (p.ih * p.iw);
                const int r = rem / p.iw - (FH - 1), c = rem % p.iw - (FW - 1);
                const bool inside = r >= 0 && r < sh && c >= 0 && c < sw;
                s_img[i] = inside ? to_f32(src[(plane * sh + r) * sw + c]) : 0.f;
            }
        }
        // w is [p.ic][p.oc][FH][FW] in memory (dy's channels outermost); staged as
        // [ci][FH][FW][ocp] with both spatial axes reversed
        for (int i = threadIdx.x; i < p.oc * taps; i += blockDim.x) {
            const int ci = i / (p.oc * FH * FW);
            int r = i - ci * (p.oc * FH * FW);
            const int oc = r / (FH * FW);
            r -= oc * (FH * FW);
            s_w[(ci * FH * FW + (FH * FW - 1 - r)) * p.ocp + oc] = to_f32(w[i]);
        }
        if (p.ocp != p.oc)
            for (int tap = threadIdx.x; tap < taps; tap += blockDim.x) s_w[tap * p.ocp + p.oc] = 0.f;
        for (int i = threadIdx.x; i < p.ocp; i += blockDim.x) s_bias[i] = 0.f;
    } else {
        stage_contiguous<T>(x + (int64_t)b0 * img_elems, s_img, nimg * img_elems);
        stage_filters<T>(w, bias, s_w, s_bias, p.oc, p.ocp, taps);
    }
    __syncthreads();

    const int oh = p.ih - FH + 1, ow = p.iw - FW + 1;
    GlobalOut<T> out{y, b0, p.oc, p.pool ? oh / 2 : oh, p.pool ? ow / 2 : ow, pre_y, oh, ow};
    if (!BWD && p.keep_pre && p.fine)
        compute_items_fine<T, FH, FW, GlobalOut<T>, 2, true>(s_img, s_w, s_bias, bias != nullptr, p,
                                                            nimg, out);
    else if (!BWD && p.keep_pre)
        compute_items<T, FH, FW, GlobalOut<T>, true>(s_img, s_w, s_bias, bias != nullptr, p, nimg,
                                                     out);
    else if (p.split > 1)
        compute_items_split<T, FH, FW>(s_img, s_w, s_bias, bias != nullptr, p, nimg,
                                       s_bias + p.ocp + 4, p.split, out);
    else if (p.fine && p.pool)
        compute_items_fine<T, FH, FW, GlobalOut<T>, 2, false>(s_img, s_w, s_bias, bias != nullptr, p,
                                                             nimg, out);
    else if (p.fine)
        compute_items_fine<T, FH, FW, GlobalOut<T>, 1, false>(s_img, s_w, s_bias, bias != nullptr, p,
                                                             nimg, out);
    else
        compute_items<T, FH, FW>(s_img, s_w, s_bias, bias != nullptr, p, nimg, out);
}

// ---- many output channels: results staged per band of rows ------------------------
// With 32 or more output channels the lanes of a warp are 32 channel pairs of ONE pixel
// block, so a direct store scatters 2- or 4-byte values over 64 channel planes.  Here a CTA
// (one image) walks bands of PBH output rows: every thread computes its items of the band
// into a shared-memory buffer [oc][rows][width], and the band is then written out with
// consecutive threads on consecutive addresses (for one channel the rows of a band are one
// contiguous run of the NCHW output).
template <class T>
__device__ __forceinline__ void store4_from_f32(T *dst, const float4 &v);
template <>
__device__ __forceinline__ void store4_from_f32<float>(float *dst, const float4 &v) {
    *reinterpret_cast<float4 *>(dst) = v;
}
template <>
__device__ __forceinline__ void store4_from_f32<__nv_bfloat16>(__nv_bfloat16 *dst, const float4 &v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 q;
    q.x = *reinterpret_cast<uint32_t *>(&lo);
    q.y = *reinterpret_cast<uint32_t *>(&hi);
    *reinterpret_cast<uint2 *>(dst) = q;
}

struct BandOut {
    float *buf;   // [oc][rows][width] of the current band
    int rows, width, y0;  // band geometry in output (or pooled output) coordinates
    __device__ __forceinline__ void pooled(int, int c, int py, int px, float v) const {
        buf[(c * rows + (py - y0)) * width + px] = v;
    }
    __device__ __forceinline__ void plain(int g, int c, int yy, int xx, float v) const {
        pooled(g, c, yy, xx, v);
    }
};

// grid.x = bs; dynamic shared memory:
//   float img[ic][ih][iw]; float wts[ic][FH][FW][ocp]; float bias[ocp + 4]; float band[oc][rows][width]
template <class T, int FH, int FW>
__global__ void __launch_bounds__(256, 2)
    conv2_direct_banded_kernel(const T *__restrict__ x, const T *__restrict__ w,
                               const T *__restrict__ bias, T *__restrict__ y, const Params p) {
    extern __shared__ __align__(16) float smem[];
    const int img_elems = p.ic * p.ih * p.iw;
    const int taps = p.ic * FH * FW;
    const int b = blockIdx.x;
    float *s_img = smem;
    float *s_w = smem + ((img_elems + 3) & ~3);
    float *s_bias = s_w + taps * p.ocp;
    float *s_band = s_bias + p.ocp + 4;
    stage_contiguous<T>(x + (int64_t)b * img_elems, s_img, img_elems);
    stage_filters<T>(w, bias, s_w, s_bias, p.oc, p.ocp, taps);
    __syncthreads();

    const int oh = p.ih - FH + 1, ow = p.iw - FW + 1;
    const int nby = oh / PBH, nbx = (ow + PBW - 1) / PBW;
    const int n_ocg = p.ocp / OC_T;
    const int out_h = p.pool ? oh / 2 : oh, out_w = p.pool ? ow / 2 : ow;
    const int band_rows = p.pool ? PBH / 2 : PBH;
    const int band_items = nbx * n_ocg;
    const int band_elems = band_rows * out_w;  // per channel
    T *yb = y + (int64_t)b * p.oc * out_h * out_w;
    for (int by = 0; by < nby; ++by) {
        BandOut out{s_band, band_rows, out_w, by * band_rows};
        for (int i = threadIdx.x; i < band_items; i += blockDim.x) {
            Item it;
            it.g = 0;
            const int bx = i / n_ocg;
            it.oc0 = (i - bx * n_ocg) * OC_T;
            it.y0 = by * PBH;
            it.x0 = bx * PBW;
            float acc[PBH][PBW][OC_T];
#pragma unroll
            for (int a = 0; a < PBH; ++a)
#pragma unroll
                for (int c = 0; c < PBW; ++c)
#pragma unroll
                    for (int o = 0; o < OC_T; ++o) acc[a][c][o] = 0.f;
            accumulate_item<FH, FW>(acc, s_img, s_w, p, it, 0, p.ic);
            finish_item<T, FH, FW>(acc, s_bias, bias != nullptr, p, it, out);
        }
        __syncthreads();
        const int total = p.oc * band_elems;
        // four elements per thread when every channel's run starts on a 4-element boundary
        const bool vec4 = (band_elems & 3) == 0 && ((out_h * out_w) & 3) == 0 &&
                          (reinterpret_cast<uintptr_t>(yb) % (4 * sizeof(T))) == 0 &&
                          (reinterpret_cast<uintptr_t>(s_band) & 15) == 0;
        if (vec4) {
            for (int i = threadIdx.x * 4; i < total; i += blockDim.x * 4) {
                const int c = i / band_elems, r = i - c * band_elems;
                const float4 v = *reinterpret_cast<const float4 *>(s_band + i);
                store4_from_f32<T>(yb + ((int64_t)c * out_h + by * band_rows) * out_w + r, v);
            }
        } else {
            for (int i = threadIdx.x; i < total; i += blockDim.x) {
                const int c = i / band_elems, r = i - c * band_elems;
                yb[((int64_t)c * out_h + by * band_rows) * out_w + r] = from_f32<T>(s_band[i]);
            }
        }
        __syncthreads();
    }
}

template <class T, int FH, int FW>
static int launch_banded(ag_device *dev, const T *x, const T *w, const T *bias, T *y,
                         const Params &p, size_t smem) {
    auto kernel = conv2_direct_banded_kernel<T, FH, FW>;
    if (smem > 48 * 1024)
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    kernel<<<(unsigned)p.bs, 256, smem, dev->stream>>>(x, w, bias, y, p);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

static bool filter_supported(int fh, int fw) {
    return (fh == 5 && fw == 5) || (fh == 3 && fw == 3);
}

bool eligible(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
              const ag_conv2_options *o) {
    if (o->padding[0] || o->padding[1] || o->stride[0] != 1 || o->stride[1] != 1 ||
        o->dilation[0] != 1 || o->dilation[1] != 1)
        return false;
    const int fh = o->filter[0], fw = o->filter[1];
    if (!filter_supported(fh, fw)) return false;
    const int64_t oh = ih - fh + 1, ow = iw - fw + 1;
    if (oh <= 0 || ow <= 0 || (oh & 1) || (ow & 1)) return false;
    if (bs <= 0 || ic <= 0 || ic > 16 || oc <= 0 || oc > 64) return false;
    // one image plus the filter bank must fit in shared memory with room to spare
    const int64_t ocp = (oc + 1) & ~1;
    const int64_t bytes = (ic * ih * iw + ic * fh * fw * ocp + ocp + 4) * 4;
    return bytes <= 96 * 1024;
}

// One image per CTA and few work items (a small batch of a small layer): several threads
// share a work item, each taking a range of input channels.
static int channel_split(int group, int items_per_img, int ic) {
    if (group != 1 || ic < 2 || items_per_img * 2 > 256) return 1;
    int split = 256 / items_per_img;
    if (split > ic) split = ic;
    if (split > 8) split = 8;
    const int chunk = (ic + split - 1) / split;
    return (ic + chunk - 1) / chunk;  // no empty ranges
}

static size_t split_bytes(int split, int items_per_img) {
    return split > 1 ? (size_t)(split - 1) * items_per_img * (PBH * PBW * OC_T) * sizeof(float) : 0;
}

template <class T, int FH, int FW, bool BWD>
static int launch(ag_device *dev, const T *x, const T *w, const T *bias, T *y, const Params &p,
                  size_t smem, int items_per_img, T *pre_y = nullptr) {
    auto kernel = conv2_direct_kernel<T, FH, FW, BWD>;
    if (smem > 48 * 1024)
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    int threads = ((p.group * items_per_img * p.split + 31) / 32) * 32;
    if (p.fine) threads *= (p.pool || p.keep_pre) ? 4 : 8;
    if (threads > 256) threads = 256;
    if (threads < 64) threads = 64;
    const unsigned grid = (unsigned)ceil_div(p.bs, p.group);
    kernel<<<grid, threads, smem, dev->stream>>>(x, w, bias, y, p, pre_y);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

template <class T>
int forward(ag_device *dev, const T *x, int64_t bs, int64_t ic, int64_t ih, int64_t iw, const T *w,
            int64_t oc, const T *bias, const ag_conv2_options *o, bool relu, bool pool, T *y,
            T *pre) {
    Params p;
    p.keep_pre = pre != nullptr;  // callers pass it only with fewer than 32 output channels
    p.bs = (int)bs; p.ic = (int)ic; p.ih = (int)ih; p.iw = (int)iw; p.oc = (int)oc;
    p.ocp = ((int)oc + 1) & ~1;
    p.relu = relu;
    p.pool = pool;
    const int fh = o->filter[0], fw = o->filter[1];
    const int oh = p.ih - fh + 1, ow = p.iw - fw + 1;
    const int items_per_img = (p.ocp / OC_T) * (oh / PBH) * ((ow + PBW - 1) / PBW);
    // Images per CTA.  A small batch is spread as one CTA per SM when that fits in 256
    // threads; otherwise a CTA takes as many images as give it about 256 work items.
    const int img_bytes = p.ic * p.ih * p.iw * 4;
    const int w_bytes = (p.ic * fh * fw * p.ocp + p.ocp + 4) * 4;
    int group = (int)ceil_div(bs, dev->sm_count);
    if ((int64_t)group * items_per_img > 256) group = 256 / items_per_img;
    if (group < 1) group = 1;
    while (group > 1 && (int64_t)group * img_bytes + w_bytes > 100 * 1024) --group;
    p.group = group;
    // no channel split in the forward direction: its sums must keep the order of the
    // whole-network kernel and of the fused conv + pool call (bit-for-bit equality)
    p.split = 1;
    // One image per CTA with fewer than 128 work items: finer items instead (the same sums
    // in the same order on more threads).
    p.fine = group == 1 && items_per_img < 128 && (ow & 1) == 0 && (oh & 1) == 0;
    // Many output channels, one image per CTA anyway: the banded kernel (coalesced stores).
    if (oc >= 32 && group == 1 && bs <= 2147483647 && pre == nullptr) {
        const int out_w = pool ? ow / 2 : ow;
        const int band_rows = pool ? PBH / 2 : PBH;
        const size_t smem_b = (size_t)(((p.ic * p.ih * p.iw + 3) & ~3) * 4) + (size_t)w_bytes +
                              (size_t)p.oc * band_rows * out_w * 4;
        if (smem_b <= 100 * 1024) {
            if (fh == 5) return launch_banded<T, 5, 5>(dev, x, w, bias, y, p, smem_b);
            return launch_banded<T, 3, 3>(dev, x, w, bias, y, p, smem_b);
        }
    }
    const size_t smem = (size_t)(((group * p.ic * p.ih * p.iw + 3) & ~3) * 4) + (size_t)w_bytes;
    if (fh == 5) return launch<T, 5, 5, false>(dev, x, w, bias, y, p, smem, items_per_img, pre);
    return launch<T, 3, 3, false>(dev, x, w, bias, y, p, smem, items_per_img, pre);
}

bool eligible_backward_input(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
                             const ag_conv2_options *o) {
    if (o->padding[0] || o->padding[1] || o->stride[0] != 1 || o->stride[1] != 1 ||
        o->dilation[0] != 1 || o->dilation[1] != 1)
        return false;
    const int fh = o->filter[0], fw = o->filter[1];
    if (!filter_supported(fh, fw)) return false;
    if (ih < fh || iw < fw || (ih & 1) || (iw & 1)) return false;
    if (bs <= 0 || oc <= 0 || oc > 16 || ic <= 0 || ic > 64) return false;
    const int64_t icp = (ic + 1) & ~1;
    const int64_t bytes = (oc * (ih + fh - 1) * (iw + fw - 1) + oc * fh * fw * icp + icp + 4) * 4;
    return bytes <= 96 * 1024;
}

template <class T>
int backward_input(ag_device *dev, const T *w, int64_t oc, int64_t ic, const T *dy, int64_t bs,
                   int64_t ih, int64_t iw, const ag_conv2_options *o, T *dx) {
    const int fh = o->filter[0], fw = o->filter[1];
    Params p;
    p.bs = (int)bs;
    p.ic = (int)oc;                      // channels of the staged image (dy)
    p.ih = (int)ih + fh - 1;             // dy height + 2 (fh - 1)
    p.iw = (int)iw + fw - 1;
    p.oc = (int)ic;                      // channels produced (dx)
    p.ocp = ((int)ic + 1) & ~1;
    p.relu = false;
    p.pool = false;
    const int items_per_img = (p.ocp / OC_T) * ((int)ih / PBH) * (((int)iw + PBW - 1) / PBW);
    const int img_bytes = p.ic * p.ih * p.iw * 4;
    const int w_bytes = (p.ic * fh * fw * p.ocp + p.ocp + 4) * 4;
    int group = (int)ceil_div(bs, dev->sm_count);
    if ((int64_t)group * items_per_img > 256) group = 256 / items_per_img;
    if (group < 1) group = 1;
    while (group > 1 && (int64_t)group * img_bytes + w_bytes > 100 * 1024) --group;
    p.group = group;
    p.split = channel_split(group, items_per_img, p.ic);
    const size_t smem = (size_t)(((group * p.ic * p.ih * p.iw + 3) & ~3) * 4) + (size_t)w_bytes +
                        split_bytes(p.split, items_per_img);
    if (fh == 5) return launch<T, 5, 5, true>(dev, dy, w, nullptr, dx, p, smem, items_per_img);
    return launch<T, 3, 3, true>(dev, dy, w, nullptr, dx, p, smem, items_per_img);
}

template int backward_input<float>(ag_device *, const float *, int64_t, int64_t, const float *,
                                   int64_t, int64_t, int64_t, const ag_conv2_options *, float *);
template int backward_input<__nv_bfloat16>(ag_device *, const __nv_bfloat16 *, int64_t, int64_t,
                                           const __nv_bfloat16 *, int64_t, int64_t, int64_t,
                                           const ag_conv2_options *, __nv_bfloat16 *);

template int forward<float>(ag_device *, const float *, int64_t, int64_t, int64_t, int64_t,
                            const float *, int64_t, const float *, const ag_conv2_options *, bool,
                            bool, float *, float *);
template int forward<__nv_bfloat16>(ag_device *, const __nv_bfloat16 *, int64_t, int64_t, int64_t,
                                    int64_t, const __nv_bfloat16 *, int64_t, const __nv_bfloat16 *,
                                    const ag_conv2_options *, bool, bool, __nv_bfloat16 *,
                                    __nv_bfloat16 *);

}  // namespace direct
}  // namespace ag
