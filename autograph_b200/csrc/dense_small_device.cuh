// Device-side pieces of the dense layer chain, shared by the stand-alone kernel
// (dense_small.cu) and the fused conv -> dense chain (conv_chain.cu).
#pragma once

#include "dense_small.cuh"

namespace ag {
namespace dense_small {

constexpr int ROWS = 8;  // rows of x a CTA owns

struct ChainStep {
    const void *w, *bias;
    int K, N, np, slices, kchunk, relu;
    void *pre, *act;  // optional [M, N] copies of the output before / after the relu
    // Backward steps (dx = dy . w^T): w is read as [N][K] (the forward layer's [inputs, outputs])
    // and the result is zeroed where gate[m][n] < 0 (the Relu in front of the forward layer).
    int transposed;
    const void *gate;
};
struct ChainParams {
    ChainStep s[kMaxChain];
    int n_layers, M, max_k, red_floats;
    int threads;  // (column, k slice) pairs of the widest layer
};

// Split of one layer over up to 1024 (column, k slice) pairs.
inline void plan_step(int k, int n, int *np, int *slices, int *kchunk) {
    *np = ((n + 31) / 32) * 32;
    int sl = 1024 / *np;
    if (sl > 16) sl = 16;
    if (sl > k / 8) sl = k / 8;
    if (sl < 1) sl = 1;
    *kchunk = (k + sl - 1) / sl;
    *slices = (k + *kchunk - 1) / *kchunk;
}

// Fills the plan; returns the shared-memory floats the layers need
// (2 * max_k * ROWS for the two activation buffers + red_floats).
inline size_t plan_chain(ChainParams *p, int m, int n_layers, const ChainLayer *layers) {
    p->n_layers = n_layers;
    p->M = m;
    p->max_k = 0;
    p->red_floats = 0;
    p->threads = 32;
    for (int i = 0; i < n_layers; ++i) {
        ChainStep &st = p->s[i];
        st.w = layers[i].w;
        st.bias = layers[i].bias;
        st.K = layers[i].inputs;
        st.N = layers[i].outputs;
        st.relu = layers[i].relu;
        st.pre = layers[i].pre_out;
        st.act = layers[i].act_out;
        st.transposed = layers[i].transposed;
        st.gate = layers[i].gate;
        plan_step(st.K, st.N, &st.np, &st.slices, &st.kchunk);
        if (st.transposed && st.K % 4 == 0) {  // whole groups of four weights per slice
            st.kchunk = (st.kchunk + 3) & ~3;
            st.slices = (st.K + st.kchunk - 1) / st.kchunk;
        }
        if (st.K > p->max_k) p->max_k = st.K;
        if (st.N > p->max_k) p->max_k = st.N;  // a layer's output is the next layer's input
        if (st.slices * ROWS * st.np > p->red_floats) p->red_floats = st.slices * ROWS * st.np;
        if (st.np * st.slices > p->threads) p->threads = st.np * st.slices;
    }
    return (size_t)2 * p->max_k * ROWS + (size_t)p->red_floats;
}

__device__ __forceinline__ void load2_to_f32(const float *p, float &a, float &b) {
    const float2 v = *reinterpret_cast<const float2 *>(p);
    a = v.x;
    b = v.y;
}
__device__ __forceinline__ void load2_to_f32(const __nv_bfloat16 *p, float &a, float &b) {
    const uint32_t v = *reinterpret_cast<const uint32_t *>(p);
    a = __uint_as_float(v << 16);
    b = __uint_as_float(v & 0xffff0000u);
}

__device__ __forceinline__ void load4_w(const float *p, float (&v)[4]) {
    const float4 q = *reinterpret_cast<const float4 *>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
}
__device__ __forceinline__ void load4_w(const __nv_bfloat16 *p, float (&v)[4]) {
    const uint2 q = *reinterpret_cast<const uint2 *>(p);
    v[0] = __uint_as_float(q.x << 16); v[1] = __uint_as_float(q.x & 0xffff0000u);
    v[2] = __uint_as_float(q.y << 16); v[3] = __uint_as_float(q.y & 0xffff0000u);
}

// Weight loads from a known address space.  A pointer that may be global or shared compiles
// to a generic load, which takes the global-memory path even when it lands in shared memory;
// SMEM = true reads through ld.shared.
template <bool SMEM>
__device__ __forceinline__ void load4_w_as(const float *p, float (&v)[4]) {
    if constexpr (SMEM) {
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3])
                     : "r"((uint32_t)__cvta_generic_to_shared(p)));
    } else {
        load4_w(p, v);
    }
}
template <bool SMEM>
__device__ __forceinline__ void load4_w_as(const __nv_bfloat16 *p, float (&v)[4]) {
    if constexpr (SMEM) {
        uint32_t a, b;
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];"
                     : "=r"(a), "=r"(b)
                     : "r"((uint32_t)__cvta_generic_to_shared(p)));
        v[0] = __uint_as_float(a << 16); v[1] = __uint_as_float(a & 0xffff0000u);
        v[2] = __uint_as_float(b << 16); v[3] = __uint_as_float(b & 0xffff0000u);
    } else {
        load4_w(p, v);
    }
}
template <bool SMEM>
__device__ __forceinline__ void load2_as(const float *p, float &a, float &b) {
    if constexpr (SMEM) {
        asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];"
                     : "=f"(a), "=f"(b)
                     : "r"((uint32_t)__cvta_generic_to_shared(p)));
    } else {
        load2_to_f32(p, a, b);
    }
}
template <bool SMEM>
__device__ __forceinline__ void load2_as(const __nv_bfloat16 *p, float &a, float &b) {
    if constexpr (SMEM) {
        uint32_t v;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"((uint32_t)__cvta_generic_to_shared(p)));
        a = __uint_as_float(v << 16);
        b = __uint_as_float(v & 0xffff0000u);
    } else {
        load2_to_f32(p, a, b);
    }
}

template <bool SMEM>
__device__ __forceinline__ float load1_as(const float *p) {
    if constexpr (SMEM) {
        float v;
        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"((uint32_t)__cvta_generic_to_shared(p)));
        return v;
    } else {
        return *p;
    }
}
template <bool SMEM>
__device__ __forceinline__ float load1_as(const __nv_bfloat16 *p) {
    if constexpr (SMEM) {
        unsigned short v;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"((uint32_t)__cvta_generic_to_shared(p)));
        return __uint_as_float((uint32_t)v << 16);
    } else {
        return to_f32(*p);
    }
}

// A layer with few outputs (the 84 -> 10 classifier head): split over (column, k slice) it is
// all barriers and reduction.  Here every output (row, column) belongs to four adjacent lanes;
// lane q adds the products of k = q, q + 4, ... in k order and the four sums are added as
// (p0 + p1) + (p2 + p3) by two shuffles -- no scratch, one barrier.  The order does not depend
// on the CTA size, and every kernel that runs such a layer comes through here, so the bits are
// the same everywhere.
__device__ __forceinline__ bool narrow_step(const ChainStep &st) {
    return !st.transposed && st.gate == nullptr && st.N <= 16 && st.K <= 1024;
}

template <class T, bool SMEM>
__device__ __forceinline__ void narrow_layer(const ChainStep &st, const T *w, const float *xa, float *xb,
                                             int m0, int rows, bool last, T *__restrict__ y) {
    const T *bias = reinterpret_cast<const T *>(st.bias);
    const int total = ROWS * st.N * 4;
    const int padded = (total + 31) & ~31;   // whole warps take part in the shuffles
    for (int it = threadIdx.x; it < padded; it += blockDim.x) {
        const bool live = it < total;
        const int q = it & 3, o = it >> 2;
        const int c = live ? o % st.N : 0, r = live ? o / st.N : 0;
        float p = 0.f;
        float bv = 0.f;
        if (live) {
            if (bias != nullptr && q == 0) bv = to_f32(bias[c]);   // in flight during the sums
            const T *wp = w + c;
#pragma unroll 4
            for (int k = q; k < st.K; k += 4)
                p = fmaf(xa[k * ROWS + r], load1_as<SMEM>(wp + (int64_t)k * st.N), p);
        }
        p += __shfl_xor_sync(0xffffffffu, p, 1);
        p += __shfl_xor_sync(0xffffffffu, p, 2);
        if (!live || q != 0) continue;
        float v = to_f32(from_f32<T>(p));
        if (bias != nullptr) v = to_f32(from_f32<T>(__fadd_rn(v, bv)));
        if (st.pre != nullptr && r < rows)
            reinterpret_cast<T *>(st.pre)[(int64_t)(m0 + r) * st.N + c] = from_f32<T>(v);
        if (st.relu) v = (v >= 0.f) ? v : 0.f;
        if (st.act != nullptr && r < rows)
            reinterpret_cast<T *>(st.act)[(int64_t)(m0 + r) * st.N + c] = from_f32<T>(v);
        if (last) {
            if (y != nullptr && r < rows) y[(int64_t)(m0 + r) * st.N + c] = from_f32<T>(v);
        } else {
            xb[c * ROWS + r] = v;
        }
    }
    __syncthreads();
}

// One layer of the chain: xa [K][ROWS] -> xb [N][ROWS] (or y for the last layer).  `w` is the
// layer's weight matrix as the kernel should read it: st.w, or a copy of it in shared memory.
// QUADS: a work item is four adjacent columns x four rows (half of ROWS) where the layer allows
// it.  Shared memory delivers 128 bytes per clock to the register file whether a load is a
// broadcast or not, so the square tile (16 + 16 bytes per k step for 16 FFMAs) beats the
// 8 rows x 2 columns of the default path (32 + 8 bytes).  The k slices, and with them every
// sum, are unchanged.
template <class T, bool QUADS = false, bool SMEM = false>
__device__ __forceinline__ void chain_layer(const ChainStep &st, const T *w, const float *xa,
                                            float *xb, float *red, int m0, int rows, bool last,
                                            T *__restrict__ y) {
    if (narrow_step(st)) {
        narrow_layer<T, SMEM>(st, w, xa, xb, m0, rows, last, y);
        return;
    }
    {
        const T *bias = reinterpret_cast<const T *>(st.bias);
        const bool quads = QUADS && !st.transposed && (st.N % 4 == 0) &&
                           (reinterpret_cast<uintptr_t>(w) % (4 * sizeof(T)) == 0);
        // Two adjacent output columns per (column, k slice) work item when the weight rows
        // allow an aligned two-element load: twice the FFMAs per load instruction.  The sum
        // for every output is the same either way (same k slices, same order).
        const bool pairs = (st.N % 2 == 0) &&
                           (reinterpret_cast<uintptr_t>(w) % (2 * sizeof(T)) == 0);
        if (quads) {
            // item = (four columns, half of the rows, k slice)
            const int quarter = st.np / 4;
            for (int vt = threadIdx.x; vt < quarter * 2 * st.slices; vt += blockDim.x) {
                const int half = vt & 1, q = vt >> 1;
                const int n = 4 * (q % quarter), slice = q / quarter;
                float acc[4][4];
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int r = 0; r < 4; ++r) acc[c][r] = 0.f;
                if (n < st.N) {
                    const int k0 = slice * st.kchunk, k1 = min(st.K, k0 + st.kchunk);
                    const T *wp = w + (int64_t)k0 * st.N + n;
                    const float *xp = xa + 4 * half;
#pragma unroll 8
                    for (int k = k0; k < k1; ++k, wp += st.N) {
                        float wv[4];
                        load4_w_as<SMEM>(wp, wv);
                        const float4 a = *reinterpret_cast<const float4 *>(xp + k * ROWS);
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            acc[c][0] = fmaf(a.x, wv[c], acc[c][0]); acc[c][1] = fmaf(a.y, wv[c], acc[c][1]);
                            acc[c][2] = fmaf(a.z, wv[c], acc[c][2]); acc[c][3] = fmaf(a.w, wv[c], acc[c][3]);
                        }
                    }
                }
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    *reinterpret_cast<float4 *>(red + (slice * ROWS + 4 * half + r) * st.np + n) =
                        make_float4(acc[0][r], acc[1][r], acc[2][r], acc[3][r]);
            }
        } else if (st.transposed) {
            // Thread (n, k slice) walks row n of w, contiguous in k: four weights per load
            // when the rows keep 4-element alignment.
            const bool vec4 = (st.K % 4 == 0) && (st.kchunk % 4 == 0) &&
                              (reinterpret_cast<uintptr_t>(w) % (4 * sizeof(T)) == 0);
            for (int vt = threadIdx.x; vt < st.np * st.slices; vt += blockDim.x) {
                const int n = vt % st.np, slice = vt / st.np;
                float acc[ROWS];
#pragma unroll
                for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
                if (n < st.N) {
                    const int k0 = slice * st.kchunk, k1 = min(st.K, k0 + st.kchunk);
                    const T *wp = w + (int64_t)n * st.K;
                    if (vec4) {
#pragma unroll 4
                        for (int k = k0; k < k1; k += 4) {
                            float wv[4];
                            load4_w(wp + k, wv);
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const float4 a = *reinterpret_cast<const float4 *>(xa + (k + q) * ROWS);
                                const float4 b = *reinterpret_cast<const float4 *>(xa + (k + q) * ROWS + 4);
                                acc[0] = fmaf(a.x, wv[q], acc[0]); acc[1] = fmaf(a.y, wv[q], acc[1]);
                                acc[2] = fmaf(a.z, wv[q], acc[2]); acc[3] = fmaf(a.w, wv[q], acc[3]);
                                acc[4] = fmaf(b.x, wv[q], acc[4]); acc[5] = fmaf(b.y, wv[q], acc[5]);
                                acc[6] = fmaf(b.z, wv[q], acc[6]); acc[7] = fmaf(b.w, wv[q], acc[7]);
                            }
                        }
                    } else {
#pragma unroll 4
                        for (int k = k0; k < k1; ++k) {
                            const float wv = to_f32(wp[k]);
                            const float4 a = *reinterpret_cast<const float4 *>(xa + k * ROWS);
                            const float4 b = *reinterpret_cast<const float4 *>(xa + k * ROWS + 4);
                            acc[0] = fmaf(a.x, wv, acc[0]); acc[1] = fmaf(a.y, wv, acc[1]);
                            acc[2] = fmaf(a.z, wv, acc[2]); acc[3] = fmaf(a.w, wv, acc[3]);
                            acc[4] = fmaf(b.x, wv, acc[4]); acc[5] = fmaf(b.y, wv, acc[5]);
                            acc[6] = fmaf(b.z, wv, acc[6]); acc[7] = fmaf(b.w, wv, acc[7]);
                        }
                    }
                }
#pragma unroll
                for (int r = 0; r < ROWS; ++r) red[(slice * ROWS + r) * st.np + n] = acc[r];
            }
        } else if (pairs) {
            const int half = st.np / 2;
            for (int vt = threadIdx.x; vt < half * st.slices; vt += blockDim.x) {
                const int n = 2 * (vt % half), slice = vt / half;
                float acc0[ROWS], acc1[ROWS];
#pragma unroll
                for (int r = 0; r < ROWS; ++r) acc0[r] = acc1[r] = 0.f;
                if (n < st.N) {
                    const int k0 = slice * st.kchunk, k1 = min(st.K, k0 + st.kchunk);
                    const T *wp = w + (int64_t)k0 * st.N + n;
#pragma unroll 8
                    for (int k = k0; k < k1; ++k, wp += st.N) {
                        float w0, w1;
                        load2_as<SMEM>(wp, w0, w1);
                        const float4 a = *reinterpret_cast<const float4 *>(xa + k * ROWS);
                        const float4 b = *reinterpret_cast<const float4 *>(xa + k * ROWS + 4);
                        acc0[0] = fmaf(a.x, w0, acc0[0]); acc1[0] = fmaf(a.x, w1, acc1[0]);
                        acc0[1] = fmaf(a.y, w0, acc0[1]); acc1[1] = fmaf(a.y, w1, acc1[1]);
                        acc0[2] = fmaf(a.z, w0, acc0[2]); acc1[2] = fmaf(a.z, w1, acc1[2]);
                        acc0[3] = fmaf(a.w, w0, acc0[3]); acc1[3] = fmaf(a.w, w1, acc1[3]);
                        acc0[4] = fmaf(b.x, w0, acc0[4]); acc1[4] = fmaf(b.x, w1, acc1[4]);
                        acc0[5] = fmaf(b.y, w0, acc0[5]); acc1[5] = fmaf(b.y, w1, acc1[5]);
                        acc0[6] = fmaf(b.z, w0, acc0[6]); acc1[6] = fmaf(b.z, w1, acc1[6]);
                        acc0[7] = fmaf(b.w, w0, acc0[7]); acc1[7] = fmaf(b.w, w1, acc1[7]);
                    }
                }
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    *reinterpret_cast<float2 *>(red + (slice * ROWS + r) * st.np + n) =
                        make_float2(acc0[r], acc1[r]);
            }
        } else {
            for (int vt = threadIdx.x; vt < st.np * st.slices; vt += blockDim.x) {
                const int n = vt % st.np, slice = vt / st.np;
                float acc[ROWS];
#pragma unroll
                for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
                if (n < st.N) {
                    const int k0 = slice * st.kchunk, k1 = min(st.K, k0 + st.kchunk);
                    const T *wp = w + (int64_t)k0 * st.N + n;
#pragma unroll 8
                    for (int k = k0; k < k1; ++k, wp += st.N) {
                        const float wv = to_f32(*wp);
                        const float4 a = *reinterpret_cast<const float4 *>(xa + k * ROWS);
                        const float4 b = *reinterpret_cast<const float4 *>(xa + k * ROWS + 4);
                        acc[0] = fmaf(a.x, wv, acc[0]); acc[1] = fmaf(a.y, wv, acc[1]);
                        acc[2] = fmaf(a.z, wv, acc[2]); acc[3] = fmaf(a.w, wv, acc[3]);
                        acc[4] = fmaf(b.x, wv, acc[4]); acc[5] = fmaf(b.y, wv, acc[5]);
                        acc[6] = fmaf(b.z, wv, acc[6]); acc[7] = fmaf(b.w, wv, acc[7]);
                    }
                }
#pragma unroll
                for (int r = 0; r < ROWS; ++r) red[(slice * ROWS + r) * st.np + n] = acc[r];
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < ROWS * st.np; i += blockDim.x) {
            const int r = i / st.np, c = i - r * st.np;
            if (c >= st.N) continue;
            float s = 0.f;
            if constexpr (QUADS) {
                // the partial sums are fetched together and added in slice order
                float part[16];
#pragma unroll
                for (int sl = 0; sl < 16; ++sl)
                    part[sl] = sl < st.slices ? red[(sl * ROWS + r) * st.np + c] : 0.f;
#pragma unroll
                for (int sl = 0; sl < 16; ++sl)
                    if (sl < st.slices) s += part[sl];
            } else {
                for (int sl = 0; sl < st.slices; ++sl) s += red[(sl * ROWS + r) * st.np + c];
            }
            float v = to_f32(from_f32<T>(s));
            if (bias != nullptr) v = to_f32(from_f32<T>(__fadd_rn(v, to_f32(bias[c]))));
            if (st.gate != nullptr && r < rows &&
                !(to_f32(reinterpret_cast<const T *>(st.gate)[(int64_t)(m0 + r) * st.N + c]) >= 0.f))
                v = 0.f;
            if (st.pre != nullptr && r < rows)
                reinterpret_cast<T *>(st.pre)[(int64_t)(m0 + r) * st.N + c] = from_f32<T>(v);
            if (st.relu) v = (v >= 0.f) ? v : 0.f;
            if (st.act != nullptr && r < rows)
                reinterpret_cast<T *>(st.act)[(int64_t)(m0 + r) * st.N + c] = from_f32<T>(v);
            if (last) {
                if (y != nullptr && r < rows) y[(int64_t)(m0 + r) * st.N + c] = from_f32<T>(v);
            } else {
                xb[c * ROWS + r] = v;  // already rounded to T: equals storing and reloading it
            }
        }
        __syncthreads();
    }
}

// Runs every layer of the chain for the ROWS rows whose first-layer input is in
// xa as [k][ROWS] (f32).  xb is the second activation buffer, red the
// [slices][ROWS][np] scratch.  The plan's (column, k slice) pairs are spread over
// the CTA's threads (a CTA with fewer threads than pairs takes several each), so
// the sums and their order do not depend on the CTA size.  Rows >= rows are
// computed but not stored.  All threads of the CTA must call this.
template <class T>
__device__ __forceinline__ void chain_layers(float *xa, float *xb, float *red, const ChainParams &p,
                                             int m0, int rows, T *__restrict__ y) {
    for (int l = 0; l < p.n_layers; ++l) {
        chain_layer<T>(p.s[l], reinterpret_cast<const T *>(p.s[l].w), xa, xb, red, m0, rows,
                       l + 1 == p.n_layers, y);
        float *t = xa;
        xa = xb;
        xb = t;
    }
}

}  // namespace dense_small
}  // namespace ag
