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

namespace ag {
namespace direct {

template <class T>
__device__ __forceinline__ void load4_to_f32(const T *p, float *dst);
template <>
__device__ __forceinline__ void load4_to_f32<float>(const float *p, float *dst) {
    *reinterpret_cast<float4 *>(dst) = *reinterpret_cast<const float4 *>(p);
}
template <>
__device__ __forceinline__ void load4_to_f32<__nv_bfloat16>(const __nv_bfloat16 *p, float *dst) {
    uint2 q = *reinterpret_cast<const uint2 *>(p);
    dst[0] = __uint_as_float(q.x << 16);
    dst[1] = __uint_as_float(q.x & 0xffff0000u);
    dst[2] = __uint_as_float(q.y << 16);
    dst[3] = __uint_as_float(q.y & 0xffff0000u);
}

struct Params {
    int bs, ic, ih, iw, oc;
    int group;       // images per CTA
    int ocp;         // oc rounded up to a multiple of 2 (weight row pitch in shared memory)
    bool relu, pool;
};

constexpr int OC_T = 2;  // output channels per thread
constexpr int PBH = 2;   // a thread owns a PBH x PBW block of output pixels
constexpr int PBW = 4;

// grid.x = ceil(bs / group); dynamic shared memory:
//   float img[group][ic][ih][iw]; float wts[ic][FH][FW][ocp]; float bias[ocp]
// Work item = (image, 2x4 pixel block, pair of output channels); consecutive
// threads take consecutive channel pairs of one block, so a filter tap is one
// 8-byte shared-memory load per thread (contiguous across the channel pairs)
// and the input patch loads broadcast.  Per input channel a thread keeps the
// (FH+1) x (FW+3) patch in registers: 16 FFMAs per weight load.
template <class T, int FH, int FW>
__global__ void __launch_bounds__(256, 2)
    conv2_direct_kernel(const T *__restrict__ x, const T *__restrict__ w,
                        const T *__restrict__ bias, T *__restrict__ y, const Params p) {
    extern __shared__ __align__(16) float smem[];
    const int img_elems = p.ic * p.ih * p.iw;
    const int taps = p.ic * FH * FW;
    const int b0 = blockIdx.x * p.group;
    const int nimg = min(p.group, p.bs - b0);
    float *s_img = smem;
    float *s_w = smem + ((p.group * img_elems + 3) & ~3);
    float *s_bias = s_w + taps * p.ocp;

    // ---- stage images (contiguous in global memory) --------------------------
    {
        const T *src = x + (int64_t)b0 * img_elems;
        const int total = nimg * img_elems;
        const bool vec = ((reinterpret_cast<uintptr_t>(src) % (4 * sizeof(T))) == 0);
        const int nvec = vec ? total / 4 : 0;
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) load4_to_f32<T>(src + 4 * i, s_img + 4 * i);
        for (int i = nvec * 4 + threadIdx.x; i < total; i += blockDim.x) s_img[i] = to_f32(src[i]);
    }
    // ---- stage weights as [ci][fi][fj][oc] (coalesced global reads) and the bias ----
    {
        for (int i = threadIdx.x; i < p.oc * taps; i += blockDim.x) {
            const int oc = i / taps, tap = i - oc * taps;
            s_w[tap * p.ocp + oc] = to_f32(w[i]);
        }
        if (p.ocp != p.oc)
            for (int tap = threadIdx.x; tap < taps; tap += blockDim.x) s_w[tap * p.ocp + p.oc] = 0.f;
        for (int i = threadIdx.x; i < p.ocp; i += blockDim.x)
            s_bias[i] = (bias != nullptr && i < p.oc) ? to_f32(bias[i]) : 0.f;
    }
    __syncthreads();

    const int oh = p.ih - FH + 1, ow = p.iw - FW + 1;  // both even
    const int nby = oh / PBH, nbx = (ow + PBW - 1) / PBW;
    const int n_ocg = p.ocp / OC_T;
    const int items_per_img = n_ocg * nby * nbx;
    const int items = nimg * items_per_img;

    for (int item = threadIdx.x; item < items; item += blockDim.x) {
        const int g = item / items_per_img;
        int r = item - g * items_per_img;
        const int blk = r / n_ocg, ocg = r - blk * n_ocg;
        const int by = blk / nbx, bx = blk - by * nbx;
        const int oc0 = ocg * OC_T;
        const int y0 = by * PBH, x0 = bx * PBW;
        // Blocks at the right edge may hang over by two pixels (ow is even but not always
        // a multiple of four): clamp their reads, drop their results.
        const int col_max = p.iw - 1 - x0;

        float acc[PBH][PBW][OC_T];
#pragma unroll
        for (int a = 0; a < PBH; ++a)
#pragma unroll
            for (int b = 0; b < PBW; ++b)
#pragma unroll
                for (int o = 0; o < OC_T; ++o) acc[a][b][o] = 0.f;

        const float *img = s_img + g * img_elems + y0 * p.iw + x0;
        for (int ci = 0; ci < p.ic; ++ci) {
            float patch[FH + PBH - 1][FW + PBW - 1];
            const float *pi = img + ci * p.ih * p.iw;
#pragma unroll
            for (int a = 0; a < FH + PBH - 1; ++a) {
                const float *prow = pi + a * p.iw;
#pragma unroll
                for (int b = 0; b < FW + PBW - 1; ++b) patch[a][b] = prow[min(b, col_max)];
            }
            const float *wc = s_w + ci * FH * FW * p.ocp + oc0;
#pragma unroll
            for (int fi = 0; fi < FH; ++fi)
#pragma unroll
                for (int fj = 0; fj < FW; ++fj) {
                    const float2 wv = *reinterpret_cast<const float2 *>(wc + (fi * FW + fj) * p.ocp);
#pragma unroll
                    for (int a = 0; a < PBH; ++a)
#pragma unroll
                        for (int b = 0; b < PBW; ++b) {
                            acc[a][b][0] = fmaf(patch[fi + a][fj + b], wv.x, acc[a][b][0]);
                            acc[a][b][1] = fmaf(patch[fi + a][fj + b], wv.y, acc[a][b][1]);
                        }
                }
        }

        // ---- epilogue: round to T, bias, relu, optional 2x2 max pool ---------------
        const int bimg = b0 + g;
#pragma unroll
        for (int o = 0; o < OC_T; ++o) {
            const int oc = oc0 + o;
            if (oc >= p.oc) break;
            float v[PBH][PBW];
#pragma unroll
            for (int a = 0; a < PBH; ++a)
#pragma unroll
                for (int b = 0; b < PBW; ++b) {
                    float t = to_f32(from_f32<T>(acc[a][b][o]));
                    if (bias != nullptr) t = to_f32(from_f32<T>(t + s_bias[oc]));
                    if (p.relu) t = (t >= 0.f) ? t : 0.f;
                    v[a][b] = t;
                }
            if (p.pool) {
                const int ph = oh / 2, pw = ow / 2;
                T *dst = y + ((int64_t)bimg * p.oc + oc) * ph * pw;
#pragma unroll
                for (int wy = 0; wy < PBH / 2; ++wy)
#pragma unroll
                    for (int wx = 0; wx < PBW / 2; ++wx) {
                        const int py = y0 / 2 + wy, px = x0 / 2 + wx;
                        if (py < ph && px < pw) {
                            // window order (0,0),(0,1),(1,0),(1,1); the first maximum wins
                            float m = v[2 * wy][2 * wx];
                            if (v[2 * wy][2 * wx + 1] > m) m = v[2 * wy][2 * wx + 1];
                            if (v[2 * wy + 1][2 * wx] > m) m = v[2 * wy + 1][2 * wx];
                            if (v[2 * wy + 1][2 * wx + 1] > m) m = v[2 * wy + 1][2 * wx + 1];
                            dst[py * pw + px] = from_f32<T>(m);
                        }
                    }
            } else {
                T *dst = y + ((int64_t)bimg * p.oc + oc) * oh * ow;
#pragma unroll
                for (int a = 0; a < PBH; ++a)
#pragma unroll
                    for (int b = 0; b < PBW; ++b)
                        if (y0 + a < oh && x0 + b < ow) dst[(y0 + a) * ow + x0 + b] = from_f32<T>(v[a][b]);
            }
        }
    }
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

template <class T, int FH, int FW>
static int launch(ag_device *dev, const T *x, const T *w, const T *bias, T *y, const Params &p,
                  size_t smem, int items_per_img) {
    auto kernel = conv2_direct_kernel<T, FH, FW>;
    if (smem > 48 * 1024)
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    int threads = ((p.group * items_per_img + 31) / 32) * 32;
    if (threads > 256) threads = 256;
    if (threads < 64) threads = 64;
    const unsigned grid = (unsigned)ceil_div(p.bs, p.group);
    kernel<<<grid, threads, smem, dev->stream>>>(x, w, bias, y, p);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

template <class T>
int forward(ag_device *dev, const T *x, int64_t bs, int64_t ic, int64_t ih, int64_t iw, const T *w,
            int64_t oc, const T *bias, const ag_conv2_options *o, bool relu, bool pool, T *y) {
    Params p;
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
    const size_t smem = (size_t)(((group * p.ic * p.ih * p.iw + 3) & ~3) * 4) + (size_t)w_bytes;
    if (fh == 5) return launch<T, 5, 5>(dev, x, w, bias, y, p, smem, items_per_img);
    return launch<T, 3, 3>(dev, x, w, bias, y, p, smem, items_per_img);
}

template int forward<float>(ag_device *, const float *, int64_t, int64_t, int64_t, int64_t,
                            const float *, int64_t, const float *, const ag_conv2_options *, bool,
                            bool, float *);
template int forward<__nv_bfloat16>(ag_device *, const __nv_bfloat16 *, int64_t, int64_t, int64_t,
                                    int64_t, const __nv_bfloat16 *, int64_t, const __nv_bfloat16 *,
                                    const ag_conv2_options *, bool, bool, __nv_bfloat16 *);

}  // namespace direct
}  // namespace ag
