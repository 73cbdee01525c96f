// Direct convolution for small channel counts with default options (no
// padding, stride 1, dilation 1): the LeNet5 layers and the first layer of the
// wider stack.  A CTA stages a group of images and the whole filter bank in
// shared memory; every thread owns a 2x2 block of output pixels for OC_T output
// channels and keeps the (FH+1) x (FW+1) input patch of the current input
// channel in registers, so each filter tap costs one broadcast shared-memory
// load of OC_T weights and 4*OC_T FFMAs.  Bias, ReLU and a 2x2 / stride-2 max
// pool are applied to the 2x2 block in registers, which removes the separate
// ReLU and pool passes (and their HBM / L2 round trips) from inference.
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
    int ocp;         // oc rounded up to a multiple of 4 (weight row pitch in shared memory)
    bool relu, pool;
};

// grid.x = ceil(bs / group); dynamic shared memory:
//   float img[group][ic][ih][iw]; float wts[ic][FH][FW][ocp]; float bias[ocp]
template <class T, int FH, int FW, int OC_T>
__global__ void __launch_bounds__(256)
    conv2_direct_kernel(const T *__restrict__ x, const T *__restrict__ w,
                        const T *__restrict__ bias, T *__restrict__ y, const Params p) {
    extern __shared__ __align__(16) float smem[];
    const int img_elems = p.ic * p.ih * p.iw;
    const int b0 = blockIdx.x * p.group;
    const int nimg = min(p.group, p.bs - b0);
    float *s_img = smem;
    float *s_w = smem + ((p.group * img_elems + 3) & ~3);
    float *s_bias = s_w + p.ic * FH * FW * p.ocp;

    // ---- stage images (contiguous in global memory) --------------------------
    {
        const T *src = x + (int64_t)b0 * img_elems;
        const int total = nimg * img_elems;
        const bool vec = ((reinterpret_cast<uintptr_t>(src) % (4 * sizeof(T))) == 0);
        const int nvec = vec ? total / 4 : 0;
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) load4_to_f32<T>(src + 4 * i, s_img + 4 * i);
        for (int i = nvec * 4 + threadIdx.x; i < total; i += blockDim.x) s_img[i] = to_f32(src[i]);
    }
    // ---- stage weights as [ci][fi][fj][oc] and the bias ---------------------------
    {
        const int taps = p.ic * FH * FW;
        for (int i = threadIdx.x; i < taps * p.ocp; i += blockDim.x) {
            const int oc = i % p.ocp, tap = i / p.ocp;
            s_w[i] = (oc < p.oc) ? to_f32(w[(int64_t)oc * taps + tap]) : 0.f;
        }
        for (int i = threadIdx.x; i < p.ocp; i += blockDim.x)
            s_bias[i] = (bias != nullptr && i < p.oc) ? to_f32(bias[i]) : 0.f;
    }
    __syncthreads();

    const int oh = p.ih - FH + 1, ow = p.iw - FW + 1;
    const int ph = oh / 2, pw = ow / 2;  // 2x2 blocks (oh, ow are even)
    const int n_ocg = (p.oc + OC_T - 1) / OC_T;
    const int items_per_img = n_ocg * ph * pw;
    const int items = nimg * items_per_img;

    for (int item = threadIdx.x; item < items; item += blockDim.x) {
        const int g = item / items_per_img;
        int r = item - g * items_per_img;
        const int ocg = r / (ph * pw);
        r -= ocg * ph * pw;
        const int by = r / pw, bx = r - by * pw;
        const int oc0 = ocg * OC_T;

        float acc[4][OC_T];
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int o = 0; o < OC_T; ++o) acc[q][o] = 0.f;

        const float *img = s_img + g * img_elems + (2 * by) * p.iw + 2 * bx;
        for (int ci = 0; ci < p.ic; ++ci) {
            float patch[FH + 1][FW + 1];
            const float *pi = img + ci * p.ih * p.iw;
#pragma unroll
            for (int a = 0; a < FH + 1; ++a)
#pragma unroll
                for (int b = 0; b < FW + 1; ++b) patch[a][b] = pi[a * p.iw + b];
            const float *wc = s_w + ci * FH * FW * p.ocp + oc0;
#pragma unroll
            for (int fi = 0; fi < FH; ++fi)
#pragma unroll
                for (int fj = 0; fj < FW; ++fj) {
                    float wv[OC_T];
                    const float *wp = wc + (fi * FW + fj) * p.ocp;
                    if (OC_T % 4 == 0) {
#pragma unroll
                        for (int o = 0; o < OC_T; o += 4) {
                            float4 v = *reinterpret_cast<const float4 *>(wp + o);
                            wv[o] = v.x; wv[o + 1] = v.y; wv[o + 2] = v.z; wv[o + 3] = v.w;
                        }
                    } else {
#pragma unroll
                        for (int o = 0; o < OC_T; o += 2) {
                            float2 v = *reinterpret_cast<const float2 *>(wp + o);
                            wv[o] = v.x; wv[o + 1] = v.y;
                        }
                    }
#pragma unroll
                    for (int o = 0; o < OC_T; ++o) {
                        acc[0][o] = fmaf(patch[fi][fj], wv[o], acc[0][o]);
                        acc[1][o] = fmaf(patch[fi][fj + 1], wv[o], acc[1][o]);
                        acc[2][o] = fmaf(patch[fi + 1][fj], wv[o], acc[2][o]);
                        acc[3][o] = fmaf(patch[fi + 1][fj + 1], wv[o], acc[3][o]);
                    }
                }
        }

        // ---- epilogue: round to T, bias, relu, optional 2x2 max pool ---------------
        const int b = b0 + g;
#pragma unroll
        for (int o = 0; o < OC_T; ++o) {
            const int oc = oc0 + o;
            if (oc >= p.oc) break;
            float v[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float t = to_f32(from_f32<T>(acc[q][o]));
                if (bias != nullptr) t = to_f32(from_f32<T>(t + s_bias[oc]));
                if (p.relu) t = (t >= 0.f) ? t : 0.f;
                v[q] = t;
            }
            if (p.pool) {
                // window order (0,0),(0,1),(1,0),(1,1); the first maximum wins
                float m = v[0];
                if (v[1] > m) m = v[1];
                if (v[2] > m) m = v[2];
                if (v[3] > m) m = v[3];
                y[(((int64_t)b * p.oc + oc) * ph + by) * pw + bx] = from_f32<T>(m);
            } else {
                T *dst = y + (((int64_t)b * p.oc + oc) * oh + 2 * by) * ow + 2 * bx;
                dst[0] = from_f32<T>(v[0]);
                dst[1] = from_f32<T>(v[1]);
                dst[ow] = from_f32<T>(v[2]);
                dst[ow + 1] = from_f32<T>(v[3]);
            }
        }
    }
}

static int pick_oc_t(int fh, int fw, int oc) {
    if (!((fh == 5 && fw == 5) || (fh == 3 && fw == 3))) return 0;
    if (oc % 8 == 0) return 8;
    if (oc == 6 && fh == 5) return 6;
    return 0;
}

bool eligible(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
              const ag_conv2_options *o) {
    if (o->padding[0] || o->padding[1] || o->stride[0] != 1 || o->stride[1] != 1 ||
        o->dilation[0] != 1 || o->dilation[1] != 1)
        return false;
    const int fh = o->filter[0], fw = o->filter[1];
    if (pick_oc_t(fh, fw, (int)oc) == 0) return false;
    const int64_t oh = ih - fh + 1, ow = iw - fw + 1;
    if (oh <= 0 || ow <= 0 || (oh & 1) || (ow & 1)) return false;
    if (bs <= 0 || ic <= 0 || ic > 16 || oc > 64) return false;
    // one image plus the filter bank must fit in shared memory with room to spare
    const int64_t ocp = (oc + 3) & ~3;
    const int64_t bytes = (ic * ih * iw + ic * fh * fw * ocp + ocp + 4) * 4;
    return bytes <= 96 * 1024;
}

template <class T, int FH, int FW, int OC_T>
static int launch(ag_device *dev, const T *x, const T *w, const T *bias, T *y, const Params &p,
                  size_t smem) {
    auto kernel = conv2_direct_kernel<T, FH, FW, OC_T>;
    if (smem > 48 * 1024)
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    const int oh = p.ih - FH + 1, ow = p.iw - FW + 1;
    const int items = p.group * ((p.oc + OC_T - 1) / OC_T) * (oh / 2) * (ow / 2);
    int threads = ((items + 31) / 32) * 32;
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
    p.ocp = ((int)oc + 3) & ~3;
    p.relu = relu;
    p.pool = pool;
    const int fh = o->filter[0], fw = o->filter[1];
    const int oc_t = pick_oc_t(fh, fw, (int)oc);
    const int oh = p.ih - fh + 1, ow = p.iw - fw + 1;
    const int items_per_img = ((p.oc + oc_t - 1) / oc_t) * (oh / 2) * (ow / 2);
    // Images per CTA: enough work items for 128..256 threads, but keep at least about
    // two CTAs per SM in flight and stay inside shared memory.
    const int img_bytes = p.ic * p.ih * p.iw * 4;
    const int w_bytes = (p.ic * fh * fw * p.ocp + p.ocp + 4) * 4;
    int group = (256 + items_per_img - 1) / items_per_img;
    if (group < 1) group = 1;
    while (group > 1 && ceil_div(bs, group) < 2 * dev->sm_count) --group;
    while (group > 1 && (int64_t)group * img_bytes + w_bytes > 100 * 1024) --group;
    p.group = group;
    const size_t smem = (size_t)(((group * p.ic * p.ih * p.iw + 3) & ~3) * 4) + (size_t)w_bytes;
    if (fh == 5 && oc_t == 8) return launch<T, 5, 5, 8>(dev, x, w, bias, y, p, smem);
    if (fh == 5 && oc_t == 6) return launch<T, 5, 5, 6>(dev, x, w, bias, y, p, smem);
    return launch<T, 3, 3, 8>(dev, x, w, bias, y, p, smem);
}

template int forward<float>(ag_device *, const float *, int64_t, int64_t, int64_t, int64_t,
                            const float *, int64_t, const float *, const ag_conv2_options *, bool,
                            bool, float *);
template int forward<__nv_bfloat16>(ag_device *, const __nv_bfloat16 *, int64_t, int64_t, int64_t,
                                    int64_t, const __nv_bfloat16 *, int64_t, const __nv_bfloat16 *,
                                    const ag_conv2_options *, bool, bool, __nv_bfloat16 *);

}  // namespace direct
}  // namespace ag
