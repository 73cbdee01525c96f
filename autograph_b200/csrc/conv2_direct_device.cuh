// Device-side pieces of the direct convolution, shared by the stand-alone
// kernels (conv2_direct.cu) and the fused conv -> dense chain (conv_chain.cu).
#pragma once

#include "common.cuh"

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

// In the kernel's view: ic channels of ih x iw (staged in shared memory) are
// correlated with an [oc][ic][FH][FW] filter bank into oc channels of
// (ih-FH+1) x (iw-FW+1).  For the gradient with respect to the input the view
// is the transposed problem: the staged image is dy with a zero border of
// FH-1 / FW-1 on every side, ic counts dy's channels, oc the input channels, and
// the filter bank is read with its two channel axes swapped and both spatial
// axes reversed.
struct Params {
    int bs, ic, ih, iw, oc;
    int group;       // images per CTA
    int ocp;         // oc rounded up to a multiple of 2 (weight row pitch in shared memory)
    bool relu, pool;
    int split;       // threads per work item (ranges of input channels), stand-alone kernel only
    bool fine = false;  // 1x2-pixel work items (compute_items_fine), stand-alone kernel only
    bool keep_pre = false;  // also store the values before the relu, stand-alone kernel only
};

constexpr int OC_T = 2;  // output channels per thread
constexpr int PBH = 2;   // a thread owns a PBH x PBW block of output pixels
constexpr int PBW = 4;

// Copies `total` contiguous elements to shared memory as f32.
template <class T>
__device__ __forceinline__ void stage_contiguous(const T *__restrict__ src, float *dst, int total) {
    const bool vec = ((reinterpret_cast<uintptr_t>(src) % (4 * sizeof(T))) == 0);
    const int nvec = vec ? total / 4 : 0;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) load4_to_f32<T>(src + 4 * i, dst + 4 * i);
    for (int i = nvec * 4 + threadIdx.x; i < total; i += blockDim.x) dst[i] = to_f32(src[i]);
}

// Filter bank [oc][taps] (taps = ic*FH*FW) to shared memory as [tap][ocp], and the
// bias (zero where absent) to s_bias[ocp].
template <class T>
__device__ __forceinline__ void stage_filters(const T *__restrict__ w, const T *__restrict__ bias,
                                              float *s_w, float *s_bias, int oc, int ocp, int taps) {
    for (int i = threadIdx.x; i < oc * taps; i += blockDim.x) {
        const int o = i / taps, tap = i - o * taps;
        s_w[tap * ocp + o] = to_f32(w[i]);
    }
    if (ocp != oc)
        for (int tap = threadIdx.x; tap < taps; tap += blockDim.x) s_w[tap * ocp + oc] = 0.f;
    for (int i = threadIdx.x; i < ocp; i += blockDim.x)
        s_bias[i] = (bias != nullptr && i < oc) ? to_f32(bias[i]) : 0.f;
}

// One work item = (image, 2x4 pixel block, pair of output channels).
struct Item {
    int g, oc0, y0, x0;
};

__device__ __forceinline__ Item decode_item(int item, int items_per_img, int n_ocg, int nbx) {
    Item it;
    it.g = item / items_per_img;
    const int r = item - it.g * items_per_img;
    const int blk = r / n_ocg, ocg = r - blk * n_ocg;
    const int by = blk / nbx, bx = blk - by * nbx;
    it.oc0 = ocg * OC_T;
    it.y0 = by * PBH;
    it.x0 = bx * PBW;
    return it;
}

// acc += the contribution of input channels [ci0, ci1) to the item's 2x4x2 outputs.
// Per input channel a thread keeps the (FH+1) x (FW+3) patch in registers: 16 FFMAs per
// 8-byte weight load; the patch rows are read with 16-byte loads when the row length
// allows it.
template <int FH, int FW>
__device__ __forceinline__ void accumulate_item(float (&acc)[PBH][PBW][OC_T], const float *s_img,
                                                const float *s_w, const Params &p, const Item &it,
                                                int ci0, int ci1) {
    const int img_elems = p.ic * p.ih * p.iw;
    // Blocks at the right edge may hang over by two pixels (ow is even but not always
    // a multiple of four): clamp their reads, drop their results.
    const int col_max = p.iw - 1 - it.x0;
    const float *img = s_img + it.g * img_elems + it.y0 * p.iw + it.x0;
    // Rows whose length is a multiple of four floats keep every patch row 16-byte
    // aligned (x0 is a multiple of four): two or three 16-byte loads per row.  A block
    // at the right edge may then read a few floats past its row (the next row, or the
    // buffer that follows the images); only outputs that are dropped use them.
    const bool vec_rows = (p.iw & 3) == 0;
    for (int ci = ci0; ci < ci1; ++ci) {
        constexpr int PW = FW + PBW - 1;
        float patch[FH + PBH - 1][PW];
        const float *pi = img + ci * p.ih * p.iw;
        if (vec_rows) {
#pragma unroll
            for (int a = 0; a < FH + PBH - 1; ++a) {
                const float4 *prow = reinterpret_cast<const float4 *>(pi + a * p.iw);
#pragma unroll
                for (int q = 0; q < (PW + 3) / 4; ++q) {
                    const float4 v = prow[q];
                    if (4 * q + 0 < PW) patch[a][4 * q + 0] = v.x;
                    if (4 * q + 1 < PW) patch[a][4 * q + 1] = v.y;
                    if (4 * q + 2 < PW) patch[a][4 * q + 2] = v.z;
                    if (4 * q + 3 < PW) patch[a][4 * q + 3] = v.w;
                }
            }
        } else {
#pragma unroll
            for (int a = 0; a < FH + PBH - 1; ++a) {
                const float *prow = pi + a * p.iw;
#pragma unroll
                for (int b = 0; b < PW; ++b) patch[a][b] = prow[min(b, col_max)];
            }
        }
        const float *wc = s_w + ci * FH * FW * p.ocp + it.oc0;
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
}

// Epilogue of one item: round to T, bias, relu, optional 2x2 max pool.
// Results leave through `out`:
//   out.pooled(g, oc, py, px, v)  one value of the 2x2 / stride-2 max pool (p.pool)
//   out.plain(g, oc, y, x, v)     one convolution output                  (!p.pool)
// v has been rounded to T (after the sum and again after the bias) like a
// store / reload of the layer's output would.
// KEEP: every value is also handed to out.pre(g, oc, y, x, v) before the relu (the
// convolution's own output, which the backward edges of a following Relu gate on).
template <class T, int FH, int FW, class Out, bool KEEP = false>
__device__ __forceinline__ void finish_item(const float (&acc)[PBH][PBW][OC_T],
                                            const float *s_bias, bool has_bias, const Params &p,
                                            const Item &it, Out out) {
    const int oh = p.ih - FH + 1, ow = p.iw - FW + 1;  // both even
#pragma unroll
    for (int o = 0; o < OC_T; ++o) {
        const int oc = it.oc0 + o;
        if (oc >= p.oc) break;
        float v[PBH][PBW];
#pragma unroll
        for (int a = 0; a < PBH; ++a)
#pragma unroll
            for (int b = 0; b < PBW; ++b) {
                float t = to_f32(from_f32<T>(acc[a][b][o]));
                if (has_bias) t = to_f32(from_f32<T>(t + s_bias[oc]));
                if constexpr (KEEP) {
                    if (it.y0 + a < oh && it.x0 + b < ow) out.pre(it.g, oc, it.y0 + a, it.x0 + b, t);
                }
                if (p.relu) t = (t >= 0.f) ? t : 0.f;
                v[a][b] = t;
            }
        if (p.pool) {
            const int ph = oh / 2, pw = ow / 2;
#pragma unroll
            for (int wy = 0; wy < PBH / 2; ++wy)
#pragma unroll
                for (int wx = 0; wx < PBW / 2; ++wx) {
                    const int py = it.y0 / 2 + wy, px = it.x0 / 2 + wx;
                    if (py < ph && px < pw) {
                        // window order (0,0),(0,1),(1,0),(1,1); the first maximum wins
                        float m = v[2 * wy][2 * wx];
                        if (v[2 * wy][2 * wx + 1] > m) m = v[2 * wy][2 * wx + 1];
                        if (v[2 * wy + 1][2 * wx] > m) m = v[2 * wy + 1][2 * wx];
                        if (v[2 * wy + 1][2 * wx + 1] > m) m = v[2 * wy + 1][2 * wx + 1];
                        out.pooled(it.g, oc, py, px, m);
                    }
                }
        } else {
#pragma unroll
            for (int a = 0; a < PBH; ++a)
#pragma unroll
                for (int b = 0; b < PBW; ++b)
                    if (it.y0 + a < oh && it.x0 + b < ow)
                        out.plain(it.g, oc, it.y0 + a, it.x0 + b, v[a][b]);
        }
    }
}

// The work of one CTA once images, filters and bias are in shared memory.
// Consecutive threads take consecutive channel pairs of one pixel block, so a filter
// tap is one 8-byte shared-memory load per thread (contiguous across the channel
// pairs) and the input patch loads broadcast.
template <class T, int FH, int FW, class Out, bool KEEP = false>
__device__ __forceinline__ void compute_items(const float *s_img, const float *s_w,
                                              const float *s_bias, bool has_bias, const Params &p,
                                              int nimg, Out out) {
    const int oh = p.ih - FH + 1, ow = p.iw - FW + 1;
    const int nby = oh / PBH, nbx = (ow + PBW - 1) / PBW;
    const int n_ocg = p.ocp / OC_T;
    const int items_per_img = n_ocg * nby * nbx;
    const int items = nimg * items_per_img;
    for (int item = threadIdx.x; item < items; item += blockDim.x) {
        const Item it = decode_item(item, items_per_img, n_ocg, nbx);
        float acc[PBH][PBW][OC_T];
#pragma unroll
        for (int a = 0; a < PBH; ++a)
#pragma unroll
            for (int b = 0; b < PBW; ++b)
#pragma unroll
                for (int o = 0; o < OC_T; ++o) acc[a][b][o] = 0.f;
        accumulate_item<FH, FW>(acc, s_img, s_w, p, it, 0, p.ic);
        finish_item<T, FH, FW, Out, KEEP>(acc, s_bias, has_bias, p, it, out);
    }
}

// A CTA with few work items (one image of a small layer): an item is BH x 2 pixels x OC_T
// channels (BH = 1 without a pool, 2 with one: the item is then exactly one pool window per
// channel), four to eight times as many threads as above.  Every output is the same chain of
// FFMAs in the same (channel, row, column) order as in accumulate_item and goes through the
// same epilogue, so the values are identical.  Needs an even output width (and height for
// BH = 2).
template <class T, int FH, int FW, class Out, int BH, bool KEEP>
__device__ __forceinline__ void compute_items_fine(const float *s_img, const float *s_w,
                                                   const float *s_bias, bool has_bias,
                                                   const Params &p, int nimg, Out out) {
    const int oh = p.ih - FH + 1, ow = p.iw - FW + 1;
    const int nbx = ow / 2, nby = oh / BH, n_ocg = p.ocp / OC_T;
    const int items_per_img = n_ocg * nby * nbx;
    const int img_elems = p.ic * p.ih * p.iw;
    for (int item = threadIdx.x; item < nimg * items_per_img; item += blockDim.x) {
        const int g = item / items_per_img;
        const int r = item - g * items_per_img;
        const int blk = r / n_ocg, oc0 = (r - blk * n_ocg) * OC_T;
        const int by = blk / nbx;
        const int y0 = by * BH, x0 = (blk - by * nbx) * 2;
        float acc[BH][2][OC_T];
#pragma unroll
        for (int a = 0; a < BH; ++a)
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int o = 0; o < OC_T; ++o) acc[a][b][o] = 0.f;
        const float *img = s_img + g * img_elems + y0 * p.iw + x0;
        for (int ci = 0; ci < p.ic; ++ci) {
            float patch[FH + BH - 1][FW + 1];
            const float *pi = img + ci * p.ih * p.iw;
#pragma unroll
            for (int a = 0; a < FH + BH - 1; ++a)
#pragma unroll
                for (int b = 0; b < FW + 1; ++b) patch[a][b] = pi[a * p.iw + b];
            const float *wc = s_w + ci * FH * FW * p.ocp + oc0;
#pragma unroll
            for (int fi = 0; fi < FH; ++fi)
#pragma unroll
                for (int fj = 0; fj < FW; ++fj) {
                    const float2 wv = *reinterpret_cast<const float2 *>(wc + (fi * FW + fj) * p.ocp);
#pragma unroll
                    for (int a = 0; a < BH; ++a)
#pragma unroll
                        for (int b = 0; b < 2; ++b) {
                            acc[a][b][0] = fmaf(patch[fi + a][fj + b], wv.x, acc[a][b][0]);
                            acc[a][b][1] = fmaf(patch[fi + a][fj + b], wv.y, acc[a][b][1]);
                        }
                }
        }
#pragma unroll
        for (int o = 0; o < OC_T; ++o) {
            const int oc = oc0 + o;
            if (oc >= p.oc) break;
            float v[BH][2];
#pragma unroll
            for (int a = 0; a < BH; ++a)
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    float t = to_f32(from_f32<T>(acc[a][b][o]));
                    if (has_bias) t = to_f32(from_f32<T>(t + s_bias[oc]));
                    if constexpr (KEEP) out.pre(g, oc, y0 + a, x0 + b, t);
                    if (p.relu) t = (t >= 0.f) ? t : 0.f;
                    v[a][b] = t;
                }
            if constexpr (BH == 2) {
                if (p.pool) {
                    // window order (0,0),(0,1),(1,0),(1,1); the first maximum wins
                    float m = v[0][0];
                    if (v[0][1] > m) m = v[0][1];
                    if (v[1][0] > m) m = v[1][0];
                    if (v[1][1] > m) m = v[1][1];
                    out.pooled(g, oc, y0 / 2, x0 / 2, m);
                    continue;
                }
            }
#pragma unroll
            for (int a = 0; a < BH; ++a)
#pragma unroll
                for (int b = 0; b < 2; ++b) out.plain(g, oc, y0 + a, x0 + b, v[a][b]);
        }
    }
}

// The same for a CTA with few work items (one image of a small layer): `split` threads
// share an item, each taking a contiguous range of input channels; the partial sums meet
// in shared memory (red: [split][items][16] floats) and are added in range order by the
// thread of the first range, which also runs the epilogue.  Needs items * split <= blockDim.x;
// all threads of the CTA must call it.
template <class T, int FH, int FW, class Out>
__device__ __forceinline__ void compute_items_split(const float *s_img, const float *s_w,
                                                    const float *s_bias, bool has_bias,
                                                    const Params &p, int nimg, float *red, int split,
                                                    Out out) {
    constexpr int NACC = PBH * PBW * OC_T;
    const int oh = p.ih - FH + 1, ow = p.iw - FW + 1;
    const int nby = oh / PBH, nbx = (ow + PBW - 1) / PBW;
    const int n_ocg = p.ocp / OC_T;
    const int items_per_img = n_ocg * nby * nbx;
    const int items = nimg * items_per_img;
    const int item = threadIdx.x % items, part = threadIdx.x / items;
    const bool active = part < split;
    const Item it = decode_item(item, items_per_img, n_ocg, nbx);
    float acc[PBH][PBW][OC_T];
#pragma unroll
    for (int a = 0; a < PBH; ++a)
#pragma unroll
        for (int b = 0; b < PBW; ++b)
#pragma unroll
            for (int o = 0; o < OC_T; ++o) acc[a][b][o] = 0.f;
    if (active) {
        const int chunk = (p.ic + split - 1) / split;
        const int ci0 = part * chunk, ci1 = min(p.ic, ci0 + chunk);
        accumulate_item<FH, FW>(acc, s_img, s_w, p, it, ci0, ci1);
        if (part > 0) {
            float *dst = red + ((part - 1) * items + item) * NACC;
#pragma unroll
            for (int a = 0; a < PBH; ++a)
#pragma unroll
                for (int b = 0; b < PBW; ++b)
#pragma unroll
                    for (int o = 0; o < OC_T; ++o) dst[(a * PBW + b) * OC_T + o] = acc[a][b][o];
        }
    }
    __syncthreads();
    if (active && part == 0) {
        for (int s = 1; s < split; ++s) {
            const float *src = red + ((s - 1) * items + item) * NACC;
#pragma unroll
            for (int a = 0; a < PBH; ++a)
#pragma unroll
                for (int b = 0; b < PBW; ++b)
#pragma unroll
                    for (int o = 0; o < OC_T; ++o) acc[a][b][o] += src[(a * PBW + b) * OC_T + o];
        }
        finish_item<T, FH, FW>(acc, s_bias, has_bias, p, it, out);
    }
}

}  // namespace direct
}  // namespace ag
