// SIMT (FFMA) tile engine shared by the f32 GEMM, the small / unaligned bf16
// GEMM and the implicit-GEMM convolutions.
//
// One CTA computes a BM x BN tile of C = A.B with f32 accumulation. Operands are
// described by accessor objects ("element (mn, k) of the operand, or zero when
// outside"), so the same kernel serves strided matrices (all four transpose
// layouts), im2col gathers of an NCHW tensor (implicit GEMM) and their
// transposes. Tiles are staged through shared memory as S[k][mn] with a
// two-buffer software pipeline (global -> registers -> shared while the
// previous tile is being multiplied).
#pragma once

#include "common.cuh"

namespace ag {
namespace simt {

template <int BM_, int BN_, int BK_, int TM_, int TN_, int MIN_BLOCKS_>
struct TileCfg {
    static constexpr int BM = BM_, BN = BN_, BK = BK_, TM = TM_, TN = TN_;
    static constexpr int MIN_BLOCKS = MIN_BLOCKS_;  // resident CTAs per SM to compile for
    static constexpr int TX = BN / TN;  // threads along n
    static constexpr int TY = BM / TM;  // threads along m
    static constexpr int THREADS = TX * TY;
    static constexpr int PAD = 4;
    static_assert(TM % 4 == 0 && TN % 4 == 0, "micro tile is built from float4 fragments");
    static_assert((BM * BK) % THREADS == 0 && (BN * BK) % THREADS == 0, "tile loads must divide");
};

#ifndef AG_CFGL_BM
#define AG_CFGL_BM 128
#define AG_CFGL_BN 128
#define AG_CFGL_BK 16
#define AG_CFGL_TM 8
#define AG_CFGL_TN 8
#define AG_CFGL_MINB 2
#endif
using CfgL = TileCfg<AG_CFGL_BM, AG_CFGL_BN, AG_CFGL_BK, AG_CFGL_TM, AG_CFGL_TN, AG_CFGL_MINB>;  // large problems
using CfgM = TileCfg<64, 64, 16, 4, 4, 3>;   // 256 threads, medium problems
using CfgXS = TileCfg<32, 32, 32, 4, 4, 8>;   // 64 threads, small problems (more CTAs, fewer k steps)
using CfgS16 = TileCfg<128, 16, 16, 4, 4, 4>;  // 128 threads, n <= 16
using CfgS16s = TileCfg<32, 16, 32, 4, 4, 8>;  // 32 threads, n <= 16 and few rows
using CfgS8 = TileCfg<256, 8, 16, 4, 4, 4>;    // 128 threads, n <= 8

// ---------------------------------------------------------------- accessors
// Concept:
//   static constexpr bool kFastK   threads of a warp walk k fastest (operand contiguous in k)
//   float at(int mn, int k) const  element or 0 when outside
//   bool vec                       runtime: groups of 4 along the contiguous index may be
//                                  fetched with one vector load (alignment checked by host)
//   void load4(int mn, int k, float (&v)[4]) const   the 4 elements starting at (mn,k)
//                                  along the contiguous index; caller guarantees in-range

template <class T>
__device__ __forceinline__ void load_vec4(const T *p, float (&v)[4]);
template <>
__device__ __forceinline__ void load_vec4<float>(const float *p, float (&v)[4]) {
    float4 q = *reinterpret_cast<const float4 *>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
}
template <>
__device__ __forceinline__ void load_vec4<__nv_bfloat16>(const __nv_bfloat16 *p, float (&v)[4]) {
    uint2 q = *reinterpret_cast<const uint2 *>(p);
    v[0] = __uint_as_float(q.x << 16);
    v[1] = __uint_as_float(q.x & 0xffff0000u);
    v[2] = __uint_as_float(q.y << 16);
    v[3] = __uint_as_float(q.y & 0xffff0000u);
}

// Strided matrix operand. For A (m x k): smn = row stride, sk = column stride.
// For B (k x n): smn = column stride, sk = row stride.
template <class T, bool FAST_K>
struct StridedOperand {
    static constexpr bool kFastK = FAST_K;
    const T *p;
    int64_t smn, sk;
    int mn_size, k_size;
    bool vec;
    __device__ __forceinline__ float at(int mn, int k) const {
        if (mn >= mn_size || k >= k_size) return 0.f;
        return to_f32(p[(int64_t)mn * smn + (int64_t)k * sk]);
    }
    __device__ __forceinline__ bool in_range4(int mn, int k) const {
        return FAST_K ? (mn < mn_size && k + 3 < k_size) : (mn + 3 < mn_size && k < k_size);
    }
    __device__ __forceinline__ void load4(int mn, int k, float (&v)[4]) const {
        load_vec4<T>(p + (int64_t)mn * smn + (int64_t)k * sk, v);
    }
};

// ---------------------------------------------------------------- epilogues
// Concept: void store(int m, int n, float acc) const; m < M, n < N guaranteed.
//          static constexpr bool kRow4; if true: void store4(m, n, const float (&v)[4])
//          with bool can4(m, n) telling whether the 4 columns n..n+3 may be
//          written with one vector store.

// C = alpha*acc + beta*C on a strided view.
template <class T>
struct StridedEpilogue {
    T *c;
    int64_t rs, cs;
    float alpha, beta;
    bool vec;  // cs == 1, rows 16-byte (f32) / 8-byte (bf16) aligned
    int n_size;
    __device__ __forceinline__ void store(int m, int n, float acc) const {
        T *q = c + (int64_t)m * rs + (int64_t)n * cs;
        float v = alpha * acc;
        if (beta != 0.f) v += beta * to_f32(*q);
        *q = from_f32<T>(v);
    }
    __device__ __forceinline__ bool can4(int m, int n) const { return vec && n + 3 < n_size; }
    __device__ __forceinline__ void store4(int m, int n, const float (&a)[4]) const;
};
template <>
__device__ __forceinline__ void StridedEpilogue<float>::store4(int m, int n,
                                                               const float (&a)[4]) const {
    float4 *q = reinterpret_cast<float4 *>(c + (int64_t)m * rs + n);
    float4 v = make_float4(alpha * a[0], alpha * a[1], alpha * a[2], alpha * a[3]);
    if (beta != 0.f) {
        float4 o = *q;
        v.x += beta * o.x; v.y += beta * o.y; v.z += beta * o.z; v.w += beta * o.w;
    }
    *q = v;
}
template <>
__device__ __forceinline__ void StridedEpilogue<__nv_bfloat16>::store4(int m, int n,
                                                                       const float (&a)[4]) const {
    uint2 *q = reinterpret_cast<uint2 *>(c + (int64_t)m * rs + n);
    float v[4] = {alpha * a[0], alpha * a[1], alpha * a[2], alpha * a[3]};
    if (beta != 0.f) {
        float o[4];
        load_vec4<__nv_bfloat16>(c + (int64_t)m * rs + n, o);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] += beta * o[i];
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
    __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 out;
    out.x = *reinterpret_cast<uint32_t *>(&lo);
    out.y = *reinterpret_cast<uint32_t *>(&hi);
    *q = out;
}

// Row-major y = acc (+ bias[n]) (relu): the Dense layer.  The accumulator is
// rounded to T before the bias is added and again after, so the result equals
// the reference's unfused sequence dot -> add_assign(bias) -> relu bit for bit.
template <class T>
struct BiasReluEpilogue {
    T *c;
    int64_t rs;
    const T *bias;
    bool relu;
    __device__ __forceinline__ void store(int m, int n, float acc) const {
        float v = to_f32(from_f32<T>(acc));
        if (bias != nullptr) v = to_f32(from_f32<T>(__fadd_rn(v, to_f32(bias[n]))));
        if (relu) v = (v >= 0.f) ? v : 0.f;
        c[(int64_t)m * rs + n] = from_f32<T>(v);
    }
    __device__ __forceinline__ bool can4(int, int) const { return false; }
    __device__ __forceinline__ void store4(int, int, const float (&)[4]) const {}
};

// Split-k partial sums: plane blockIdx.z of a [splits][M*N] f32 workspace.
struct PartialEpilogue {
    float *ws;
    int64_t plane;  // M*N
    int n_size;
    __device__ __forceinline__ void store(int m, int n, float acc) const {
        ws[(int64_t)blockIdx.z * plane + (int64_t)m * n_size + n] = acc;
    }
    __device__ __forceinline__ bool can4(int, int) const { return false; }
    __device__ __forceinline__ void store4(int, int, const float (&)[4]) const {}
};

// ------------------------------------------------------------------- kernel
template <class Cfg, class AOp, class BOp>
struct Loader {
    // Number of elements each thread moves per tile.
    static constexpr int A_PER = Cfg::BM * Cfg::BK / Cfg::THREADS;
    static constexpr int B_PER = Cfg::BN * Cfg::BK / Cfg::THREADS;
};

// Loads one BMN x BK operand tile into registers (r[]), element order defined by
// the mapping below; store_tile writes them to S[k][mn].
template <int BMN, int BK, int THREADS, class Op>
__device__ __forceinline__ void load_tile(const Op &op, int mn0, int k0, int tid,
                                          float (&r)[BMN * BK / THREADS]) {
    constexpr int PER = BMN * BK / THREADS;
    if (op.vec && PER % 4 == 0) {
        constexpr int GROUPS = (PER / 4) > 0 ? (PER / 4) : 1;
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
            int idx = tid + g * THREADS;
            int mn, k;
            if (Op::kFastK) {
                k = (idx % (BK / 4)) * 4;
                mn = idx / (BK / 4);
            } else {
                mn = (idx % (BMN / 4)) * 4;
                k = idx / (BMN / 4);
            }
            float v[4];
            if (op.in_range4(mn0 + mn, k0 + k)) {
                op.load4(mn0 + mn, k0 + k, v);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    v[j] = Op::kFastK ? op.at(mn0 + mn, k0 + k + j) : op.at(mn0 + mn + j, k0 + k);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) r[g * 4 + j] = v[j];
        }
    } else {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            int idx = tid + i * THREADS;
            int mn, k;
            if (Op::kFastK) {
                k = idx % BK;
                mn = idx / BK;
            } else {
                mn = idx % BMN;
                k = idx / BMN;
            }
            r[i] = op.at(mn0 + mn, k0 + k);
        }
    }
}

template <int BMN, int BK, int THREADS, int PITCH, class Op>
__device__ __forceinline__ void store_tile(const Op &op, float *S, int tid,
                                           const float (&r)[BMN * BK / THREADS]) {
    constexpr int PER = BMN * BK / THREADS;
    if (op.vec && PER % 4 == 0) {
        constexpr int GROUPS = (PER / 4) > 0 ? (PER / 4) : 1;
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
            int idx = tid + g * THREADS;
            if (Op::kFastK) {
                int k = (idx % (BK / 4)) * 4;
                int mn = idx / (BK / 4);
#pragma unroll
                for (int j = 0; j < 4; ++j) S[(k + j) * PITCH + mn] = r[g * 4 + j];
            } else {
                int mn = (idx % (BMN / 4)) * 4;
                int k = idx / (BMN / 4);
                *reinterpret_cast<float4 *>(&S[k * PITCH + mn]) =
                    make_float4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            int idx = tid + i * THREADS;
            int mn, k;
            if (Op::kFastK) {
                k = idx % BK;
                mn = idx / BK;
            } else {
                mn = idx % BMN;
                k = idx / BMN;
            }
            S[k * PITCH + mn] = r[i];
        }
    }
}

// grid = (ceil(M/BM), ceil(N/BN), splits); blockIdx.z works on k in
// [z*k_chunk, min(K, (z+1)*k_chunk)), k_chunk a multiple of BK.
template <class Cfg, class AOp, class BOp, class Epi>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::MIN_BLOCKS)
    gemm_simt_kernel(int M, int N, int K, int k_chunk, AOp A, BOp B, Epi E) {
    constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, TM = Cfg::TM, TN = Cfg::TN;
    constexpr int THREADS = Cfg::THREADS;
    constexpr int PA = BM + Cfg::PAD, PB = BN + Cfg::PAD;
    constexpr int RM = TM / 4, RN = TN / 4;

    __shared__ __align__(16) float As[2][BK * PA];
    __shared__ __align__(16) float Bs[2][BK * PB];

    const int tid = threadIdx.x;
    const int tx = tid % Cfg::TX, ty = tid / Cfg::TX;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int k_begin = blockIdx.z * k_chunk;
    const int k_end = min(K, k_begin + k_chunk);
    const int tiles = (k_end - k_begin + BK - 1) / BK;

#ifndef AG_SIMT_F32X2
#define AG_SIMT_F32X2 1
#endif
    float acc[TM][TN];
#if AG_SIMT_F32X2
    unsigned long long acc2[TM][TN / 2];   // pairs (acc[i][2j], acc[i][2j + 1])
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN / 2; ++j) acc2[i][j] = 0ull;
#else
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
#endif

    float ra[BM * BK / THREADS], rb[BN * BK / THREADS];

    if (tiles > 0) {
        load_tile<BM, BK, THREADS>(A, m0, k_begin, tid, ra);
        load_tile<BN, BK, THREADS>(B, n0, k_begin, tid, rb);
        store_tile<BM, BK, THREADS, PA>(A, As[0], tid, ra);
        store_tile<BN, BK, THREADS, PB>(B, Bs[0], tid, rb);
    }
    __syncthreads();

    for (int t = 0; t < tiles; ++t) {
        const int cur = t & 1;
        if (t + 1 < tiles) {
            // The tile's k range may end before k_end is reached by the mask in at().
            load_tile<BM, BK, THREADS>(A, m0, k_begin + (t + 1) * BK, tid, ra);
            load_tile<BN, BK, THREADS>(B, n0, k_begin + (t + 1) * BK, tid, rb);
        }
        const float *as = As[cur], *bs = Bs[cur];
        // Fragments of k step kk + 1 are loaded before the FFMAs of step kk, and the FFMAs run
        // over the micro tile in a serpentine (row i left to right, row i + 1 right to left), so
        // that consecutive instructions share an operand: 4 - 6 % over the plain loops at 4096^3
        // (measured; the loop order changes the share of dispatch stalls, which is what keeps this
        // kernel near 60 % of the FP32 pipe).  Every accumulator still adds its products in k order.
        auto load_frag = [&](int kk, float (&a)[TM], float (&b)[TN]) {
#pragma unroll
            for (int i = 0; i < RM; ++i) {
                float4 v = *reinterpret_cast<const float4 *>(&as[kk * PA + i * (BM / RM) + ty * 4]);
                a[i * 4] = v.x; a[i * 4 + 1] = v.y; a[i * 4 + 2] = v.z; a[i * 4 + 3] = v.w;
            }
#pragma unroll
            for (int j = 0; j < RN; ++j) {
                float4 v = *reinterpret_cast<const float4 *>(&bs[kk * PB + j * (BN / RN) + tx * 4]);
                b[j * 4] = v.x; b[j * 4 + 1] = v.y; b[j * 4 + 2] = v.z; b[j * 4 + 3] = v.w;
            }
        };
#if AG_SIMT_F32X2
        // Two FMAs per instruction (fma.rn.f32x2 on 64-bit register pairs): the same roundings,
        // half the instructions to dispatch and half the register-file reads per FMA.
        auto load_frag2 = [&](int kk, float (&a)[TM], unsigned long long (&b2)[TN / 2]) {
#pragma unroll
            for (int i = 0; i < RM; ++i) {
                float4 v = *reinterpret_cast<const float4 *>(&as[kk * PA + i * (BM / RM) + ty * 4]);
                a[i * 4] = v.x; a[i * 4 + 1] = v.y; a[i * 4 + 2] = v.z; a[i * 4 + 3] = v.w;
            }
#pragma unroll
            for (int j = 0; j < RN; ++j) {
                const ulonglong2 v =
                    *reinterpret_cast<const ulonglong2 *>(&bs[kk * PB + j * (BN / RN) + tx * 4]);
                b2[j * 2] = v.x; b2[j * 2 + 1] = v.y;
            }
        };
        float a[2][TM];
        unsigned long long b2[2][TN / 2];
        load_frag2(0, a[0], b2[0]);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            if (kk + 1 < BK) load_frag2(kk + 1, a[(kk + 1) & 1], b2[(kk + 1) & 1]);
#pragma unroll
            for (int i = 0; i < TM; ++i) {
                unsigned long long a2;
                asm("mov.b64 %0, {%1, %1};" : "=l"(a2) : "f"(a[kk & 1][i]));
#pragma unroll
                for (int jj = 0; jj < TN / 2; ++jj) {
                    const int j = (i & 1) ? TN / 2 - 1 - jj : jj;
                    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc2[i][j]) : "l"(a2), "l"(b2[kk & 1][j]));
                }
            }
        }
#else
        float a[2][TM], b[2][TN];
        load_frag(0, a[0], b[0]);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            if (kk + 1 < BK) load_frag(kk + 1, a[(kk + 1) & 1], b[(kk + 1) & 1]);
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int jj = 0; jj < TN; ++jj) {
                    const int j = (i & 1) ? TN - 1 - jj : jj;
                    acc[i][j] = fmaf(a[kk & 1][i], b[kk & 1][j], acc[i][j]);
                }
        }
#endif
        if (t + 1 < tiles) {
            store_tile<BM, BK, THREADS, PA>(A, As[cur ^ 1], tid, ra);
            store_tile<BN, BK, THREADS, PB>(B, Bs[cur ^ 1], tid, rb);
        }
        __syncthreads();
    }

#if AG_SIMT_F32X2
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN / 2; ++j)
            asm("mov.b64 {%0, %1}, %2;" : "=f"(acc[i][2 * j]), "=f"(acc[i][2 * j + 1]) : "l"(acc2[i][j]));
#endif
    // The k range of a split must not read beyond k_end: at() masks on the
    // operand's own k_size, so splits other than the last rely on k_chunk being
    // a multiple of BK.
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + (i / 4) * (BM / RM) + ty * 4 + (i % 4);
        if (m >= M) continue;
#pragma unroll
        for (int j4 = 0; j4 < RN; ++j4) {
            const int n = n0 + j4 * (BN / RN) + tx * 4;
            if (n >= N) continue;
            if (E.can4(m, n)) {
                float v[4] = {acc[i][j4 * 4], acc[i][j4 * 4 + 1], acc[i][j4 * 4 + 2],
                              acc[i][j4 * 4 + 3]};
                E.store4(m, n, v);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (n + j < N) E.store(m, n + j, acc[i][j4 * 4 + j]);
            }
        }
    }
}

// ------------------------------------------------------- short reductions
// k <= kSmallK and few output tiles (the Dense gradients of a small batch): the
// tile engine above spends its time on the latency of one global -> shared round
// per k tile with two warps per CTA.  Here a CTA of 256 threads owns a 32 x 32 tile
// of C, stages the WHOLE k range of both operands with one round of loads, and its
// four groups of 64 threads each accumulate a quarter of the k range for the full
// tile (4 x 4 outputs per thread); the quarters are added in group order, so the
// result is reproducible.
constexpr int kSmallK = 128;
constexpr int kSmallPitch = 36;  // floats per staged k row: 16-byte rows, see small_k_slot

// Element of an 8-k slab (32 rows/columns x 8 k) this thread moves.  Contiguous-in-k
// operands: a warp takes 4 rows x 8 k (four 32-byte segments; with the pitch of 36 the
// 32 stores fall into 32 banks).  Otherwise a warp takes 32 consecutive rows of one k.
template <class Op>
__device__ __forceinline__ void small_k_slot(int tid, int &mn, int &kb) {
    if (Op::kFastK) {
        kb = tid & 7;
        mn = ((tid >> 3) & 3) + 4 * (tid >> 5);
    } else {
        mn = tid & 31;
        kb = tid >> 5;
    }
}

template <class AOp, class BOp, class Epi>
__global__ void __launch_bounds__(256)
    gemm_small_k_kernel(int M, int N, int K, AOp A, BOp B, Epi E) {
    __shared__ __align__(16) float As[kSmallK][kSmallPitch];
    __shared__ __align__(16) float Bs[kSmallK][kSmallPitch];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
    constexpr int SLABS = kSmallK / 8;

    int amn, akb, bmn, bkb;
    small_k_slot<AOp>(tid, amn, akb);
    small_k_slot<BOp>(tid, bmn, bkb);
    float ra[SLABS], rb[SLABS];
#pragma unroll
    for (int i = 0; i < SLABS; ++i)
        if (i * 8 < K) {
            ra[i] = A.at(m0 + amn, i * 8 + akb);
            rb[i] = B.at(n0 + bmn, i * 8 + bkb);
        }
#pragma unroll
    for (int i = 0; i < SLABS; ++i)
        if (i * 8 < K) {
            As[i * 8 + akb][amn] = ra[i];
            Bs[i * 8 + bkb][bmn] = rb[i];
        }
    __syncthreads();

    const int kg = tid >> 6, t = tid & 63, tx = t & 7, ty = t >> 3;
    const int kp = (K + 7) & ~7;           // staged rows (zeros beyond K)
    const int kq = (kp / 8 + 3) / 4 * 8;   // k per group: whole slabs
    const int k0 = min(kp, kg * kq), k1 = min(kp, k0 + kq);
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 4
    for (int k = k0; k < k1; ++k) {
        const float4 a4 = *reinterpret_cast<const float4 *>(&As[k][ty * 4]);
        const float4 b4 = *reinterpret_cast<const float4 *>(&Bs[k][tx * 4]);
        const float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();  // the staged operands are no longer read
    float *red = &As[0][0];  // [3 groups][16 values][64 threads]
    if (kg > 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) red[((kg - 1) * 16 + i) * 64 + t] = acc[i / 4][i % 4];
    }
    __syncthreads();
    if (kg > 0) return;
#pragma unroll
    for (int g = 0; g < 3; ++g)
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i / 4][i % 4] += red[(g * 16 + i) * 64 + t];

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i, n = n0 + tx * 4;
        if (m >= M || n >= N) continue;
        if (E.can4(m, n)) {
            E.store4(m, n, acc[i]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (n + j < N) E.store(m, n + j, acc[i][j]);
        }
    }
}

// out[i] = alpha * sum_z ws[z][i] + beta * out[i] written through an epilogue
// (fixed summation order: deterministic).
template <class Epi>
__global__ void splitk_reduce_kernel(const float *ws, int64_t plane, int splits, int M, int N,
                                     Epi E) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= plane) return;
    float s = 0.f;
    for (int z = 0; z < splits; ++z) s += ws[(int64_t)z * plane + i];
    int m = (int)(i / N), n = (int)(i % N);
    E.store(m, n, s);
}

// The same sum for small planes with many splits: a CTA takes 32 outputs, eight
// thread groups each add every eighth plane, and the eight partial sums are added
// in group order (again a fixed order, so the result is reproducible).
template <class Epi>
__global__ void __launch_bounds__(256)
    splitk_reduce_small_kernel(const float *ws, int64_t plane, int splits, int M, int N, Epi E) {
    __shared__ float part[8][32];
    const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int64_t i = (int64_t)blockIdx.x * 32 + lane;
    float s = 0.f;
    if (i < plane)
        for (int z = grp; z < splits; z += 8) s += ws[(int64_t)z * plane + i];
    part[grp][lane] = s;
    __syncthreads();
    if (grp == 0 && i < plane) {
        float t = part[0][lane];
#pragma unroll
        for (int g = 1; g < 8; ++g) t += part[g][lane];
        E.store((int)(i / N), (int)(i % N), t);
    }
}

}  // namespace simt
}  // namespace ag
