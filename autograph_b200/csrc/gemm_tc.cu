// bf16 GEMM on the Blackwell tensor cores: C = alpha * A.B + beta * C with f32
// accumulation in tensor memory (TMEM).
//
// One persistent CTA per SM walks 128 x 256 output tiles.  Warp roles:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of 128x64 (A) and
//               256x64 (B) bf16 tiles, 128-byte swizzled, into a 4-stage ring
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=256,
//               K=16) reading the ring through shared-memory descriptors and
//               accumulating into one of two 256-column TMEM buffers
//   warps 2..5  epilogue: tcgen05.ld of the finished accumulator, alpha/beta,
//               bf16 rounding, 16-byte global stores -- overlapped with the
//               main loop of the next tile through the second TMEM buffer
// All four transpose layouts are handled without copies: an operand that is
// contiguous along k is loaded as a K-major tile, one contiguous along m / n
// as an MN-major tile (64-element swizzle atoms, several TMA boxes per stage).
// Every mbarrier wait is bounded; on expiry the kernel raises a status word,
// releases TMEM and returns.
#include <cuda.h>

#include <cstdlib>

#include "gemm_simt.cuh"
#include "gemm_tc.cuh"
#include "tc_ptx.cuh"

namespace ag {
namespace tc {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_N = 256;
constexpr int BLOCK_K = 64;  // 128 bytes of bf16: one swizzle atom
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_TILE_BYTES = BLOCK_M * BLOCK_K * 2;  // 16 KiB
constexpr int B_TILE_BYTES = BLOCK_N * BLOCK_K * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int ATOM_BYTES = 64 * BLOCK_K * 2;  // one 64(mn) x 64(k) MN-major box: 8 KiB
constexpr int TMEM_COLS = 512;                // two 256-column f32 accumulators
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int GROUP_M = 8;

struct Params {
    int M, N, K;
    int64_t ldc;
    float alpha, beta;
    __nv_bfloat16 *C;
    int *status;       // device status word (0 = ok)
    uint32_t lbo_k;    // leading byte offset used for K-major operands
    // split-k: a work item is (output tile, k slice); slices write f32 partial tiles to
    // partial[slice][M][N] and a second kernel adds them in slice order
    float *partial;    // null: one slice, results go to C
    int splits;
    int kb_per_split;  // 64-wide k blocks per slice
    const __nv_bfloat16 *bias;  // fused Dense epilogue (alpha = 1, beta = 0): bias [N] or null, relu
    int relu;
};

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int &m_blk, int &n_blk) {
    const int group_size = GROUP_M * num_n;
    const int g = tile / group_size;
    const int first_m = g * GROUP_M;
    const int gm = min(num_m - first_m, GROUP_M);
    const int r = tile - g * group_size;
    m_blk = first_m + r % gm;
    n_blk = r / gm;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                        const __grid_constant__ CUtensorMap tmap_b, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzled tiles need 1024-byte alignment.
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + STAGES * A_TILE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES);
    uint64_t *full_bar = bars;                       // [STAGES] TMA -> MMA
    uint64_t *empty_bar = bars + STAGES;             // [STAGES] MMA -> TMA
    uint64_t *tmem_full_bar = bars + 2 * STAGES;     // [2] MMA -> epilogue
    uint64_t *tmem_empty_bar = bars + 2 * STAGES + 2;  // [2] epilogue -> MMA
    uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_base_slot + 1);

    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;

    const int num_m = (p.M + BLOCK_M - 1) / BLOCK_M;
    const int num_n = (p.N + BLOCK_N - 1) / BLOCK_N;
    const int out_tiles = num_m * num_n;
    const int num_tiles = out_tiles * p.splits;
    const int total_kb = (p.K + BLOCK_K - 1) / BLOCK_K;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&tmem_full_bar[s]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[s]), 128);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_base_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                int m_blk, n_blk;
                const int split = tile / out_tiles;
                tile_coords(tile - split * out_tiles, num_m, num_n, m_blk, n_blk);
                const int kb0 = split * p.kb_per_split;
                const int kb1 = min(total_kb, kb0 + p.kb_per_split);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag)) {
                        atomicExch(p.status, 101);
                        ok = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&full_bar[stage]);
                    mbar_arrive_expect_tx(bar, STAGE_BYTES);
                    const uint32_t a_dst = smem_u32(smem_a + stage * A_TILE_BYTES);
                    const uint32_t b_dst = smem_u32(smem_b + stage * B_TILE_BYTES);
                    if (A_MN) {
#pragma unroll
                        for (int i = 0; i < BLOCK_M / 64; ++i)
                            tma_load_2d(a_dst + i * ATOM_BYTES, &tmap_a, bar,
                                        m_blk * BLOCK_M + i * 64, kb * BLOCK_K);
                    } else {
                        tma_load_2d(a_dst, &tmap_a, bar, kb * BLOCK_K, m_blk * BLOCK_M);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int i = 0; i < BLOCK_N / 64; ++i)
                            tma_load_2d(b_dst + i * ATOM_BYTES, &tmap_b, bar,
                                        n_blk * BLOCK_N + i * 64, kb * BLOCK_K);
                    } else {
                        tma_load_2d(b_dst, &tmap_b, bar, kb * BLOCK_K, n_blk * BLOCK_N);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(A_MN, B_MN, BLOCK_M, BLOCK_N);
            const uint32_t a_lbo = A_MN ? (uint32_t)ATOM_BYTES : p.lbo_k;
            const uint32_t b_lbo = B_MN ? (uint32_t)ATOM_BYTES : p.lbo_k;
            const uint32_t a_kstep = A_MN ? UMMA_K * 128 : UMMA_K * 2;  // bytes per UMMA_K
            const uint32_t b_kstep = B_MN ? UMMA_K * 128 : UMMA_K * 2;
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag)) {
                    atomicExch(p.status, 102);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BLOCK_N);
                const int split = tile / out_tiles;
                const int num_kb = min(total_kb, (split + 1) * p.kb_per_split) - split * p.kb_per_split;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag)) {
                        atomicExch(p.status, 103);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_base = smem_u32(smem_a + stage * A_TILE_BYTES);
                    const uint32_t b_base = smem_u32(smem_b + stage * B_TILE_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t a_desc = make_smem_desc(a_base + k * a_kstep, a_lbo, 1024);
                        const uint64_t b_desc = make_smem_desc(b_base + k * b_kstep, b_lbo, 1024);
                        umma_bf16(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&empty_bar[stage]));  // stage reusable once read
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(smem_u32(&tmem_full_bar[acc]));  // accumulator complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------- epilogue
        const int quarter = warp % 4;  // TMEM lanes this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            int m_blk, n_blk;
            const int split = tile / out_tiles;
            tile_coords(tile - split * out_tiles, num_m, num_n, m_blk, n_blk);
            if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag)) {
                if (lane == 0) atomicExch(p.status, 104);
                break;
            }
            tc_fence_after();
            const int row = m_blk * BLOCK_M + quarter * 32 + lane;
            const uint32_t taddr =
                tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BLOCK_N);
            __nv_bfloat16 *crow = p.C + (int64_t)row * p.ldc;
#pragma unroll 1
            for (int chunk = 0; chunk < BLOCK_N / 32; ++chunk) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + chunk * 32, r);
                tmem_ld_wait();
                const int col0 = n_blk * BLOCK_N + chunk * 32;
                if (p.partial != nullptr) {
                    // raw f32 sums of this k slice
                    if (row < p.M && col0 < p.N) {
                        float *prow = p.partial + ((int64_t)split * p.M + row) * p.N + col0;
                        if (col0 + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<uint4 *>(prow)[j] =
                                    make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        } else {
                            for (int j = 0; j < 32 && col0 + j < p.N; ++j)
                                prow[j] = __uint_as_float(r[j]);
                        }
                    }
                } else if (row < p.M && col0 < p.N) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int col = col0 + g * 8;
                        if (col >= p.N) break;
                        float v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] = p.alpha * __uint_as_float(r[g * 8 + j]);
                        if (col + 8 <= p.N) {
                            uint4 *dst = reinterpret_cast<uint4 *>(crow + col);
                            if (p.beta != 0.f) {
                                uint4 old = *dst;
                                const uint32_t o[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    v[2 * j] += p.beta * __uint_as_float(o[j] << 16);
                                    v[2 * j + 1] += p.beta * __uint_as_float(o[j] & 0xffff0000u);
                                }
                            }
                            uint32_t o[4];
                            if (p.bias != nullptr || p.relu) {
                                float bv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                                if (p.bias != nullptr) {
                                    const uint4 b4 = *reinterpret_cast<const uint4 *>(p.bias + col);
                                    const uint32_t bw[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
                                    for (int j = 0; j < 4; ++j) {
                                        bv[2 * j] = __uint_as_float(bw[j] << 16);
                                        bv[2 * j + 1] = __uint_as_float(bw[j] & 0xffff0000u);
                                    }
                                }
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    o[j] = bf16_pair_epilogue(__float_as_uint(v[2 * j]),
                                                              __float_as_uint(v[2 * j + 1]), bv[2 * j],
                                                              bv[2 * j + 1], p.bias != nullptr,
                                                              p.relu != 0);
                            } else {
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                                    o[j] = *reinterpret_cast<uint32_t *>(&h);
                                }
                            }
                            *dst = make_uint4(o[0], o[1], o[2], o[3]);
                        } else {
                            for (int j = 0; j < 8 && col + j < p.N; ++j) {
                                float x = v[j];
                                if (p.beta != 0.f) x += p.beta * __bfloat162float(crow[col + j]);
                                __nv_bfloat16 h = __float2bfloat16_rn(x);
                                if (p.bias != nullptr)
                                    h = __float2bfloat16_rn(__bfloat162float(h) +
                                                            __bfloat162float(p.bias[col + j]));
                                if (p.relu && !(__bfloat162float(h) >= 0.f)) h = __float2bfloat16_rn(0.f);
                                crow[col + j] = h;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
    }

    // ------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // Loads that were issued before a wait expired may still be landing in
        // shared memory: give them time before the CTA's memory is released.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------ host side
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
                cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

int make_tmap_bf16(CUtensorMap *map, const void *base, int rank, const uint64_t *dims,
                   const uint64_t *strides, const uint32_t *box) {
    EncodeTiledFn fn = encode_tiled_fn();
    AG_REQUIRE(fn != nullptr, AG_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    AG_REQUIRE(rank >= 2 && rank <= 5, AG_ERR_INVALID, "tensor map rank %d", rank);
    cuuint64_t d[5], st[4];
    cuuint32_t bx[5], estr[5];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        bx[i] = box[i];
        estr[i] = 1;
        if (i > 0) st[i - 1] = strides[i - 1] * 2;
    }
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank,
                    const_cast<void *>(base), d, st, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    AG_REQUIRE(r == CUDA_SUCCESS, AG_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d)",
               (int)r);
    return AG_OK;
}

// 2-D bf16 tensor map: `inner` contiguous elements, `outer` rows of
// outer_stride elements; box = box_inner x box_outer.
static int make_tmap(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer,
                     uint64_t outer_stride, uint32_t box_inner, uint32_t box_outer) {
    const uint64_t dims[2] = {inner, outer};
    const uint64_t strides[1] = {outer_stride};
    const uint32_t box[2] = {box_inner, box_outer};
    return make_tmap_bf16(map, base, 2, dims, strides, box);
}

static bool tc_enabled() {
    static int v = []() {
        const char *e = getenv("AG_TC");
        return (e && e[0] == '0') ? 0 : 1;
    }();
    return v != 0;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

bool gemm_bf16_eligible(int64_t m, int64_t k, int64_t n, const __nv_bfloat16 *a, int64_t rsa,
                        int64_t csa, const __nv_bfloat16 *b, int64_t rsb, int64_t csb,
                        const __nv_bfloat16 *c, int64_t rsc, int64_t csc) {
    if (!tc_enabled()) return false;
    if (m < 128 || n < 128 || k < 64) return false;
    if (!aligned16(a) || !aligned16(b) || !aligned16(c)) return false;
    const bool a_k = (csa == 1 && rsa % 8 == 0 && rsa >= k);
    const bool a_m = (rsa == 1 && csa % 8 == 0 && csa >= m);
    const bool b_k = (rsb == 1 && csb % 8 == 0 && csb >= k);
    const bool b_n = (csb == 1 && rsb % 8 == 0 && rsb >= n);
    if (!(a_k || a_m) || !(b_k || b_n)) return false;
    if (!(csc == 1 && rsc % 8 == 0 && rsc >= n)) return false;
    return true;
}

template <bool A_MN, bool B_MN>
static int launch(ag_device *dev, const CUtensorMap &ta, const CUtensorMap &tb, const Params &p) {
    auto kernel = gemm_bf16_tc_kernel<A_MN, B_MN>;
    // the attribute belongs to the (kernel, GPU) pair: remembered per instantiation and GPU
    static bool configured_on[64] = {};
    bool &configured = configured_on[dev->ordinal & 63];
    if (!configured) {
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_BYTES));
        configured = true;
    }
    const int tiles = (int)(ceil_div(p.M, BLOCK_M) * ceil_div(p.N, BLOCK_N)) * p.splits;
    const int grid = tiles < dev->sm_count ? tiles : dev->sm_count;
    kernel<<<grid, NUM_THREADS, SMEM_BYTES, dev->stream>>>(ta, tb, p);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

int gemm_bf16(ag_device *dev, int m, int k, int n, float alpha, const __nv_bfloat16 *a,
              int64_t rsa, int64_t csa, const __nv_bfloat16 *b, int64_t rsb, int64_t csb,
              float beta, __nv_bfloat16 *c, int64_t rsc, int64_t csc, const Epilogue *epi) {
    (void)csc;
    if (epi && !epi->bias && !epi->relu) epi = nullptr;
    if (epi) AG_REQUIRE(alpha == 1.f && beta == 0.f, AG_ERR_INVALID, "fused epilogue needs alpha 1, beta 0");
    if (epi && epi->bias)
        AG_REQUIRE((reinterpret_cast<uintptr_t>(epi->bias) & 15) == 0, AG_ERR_INVALID, "bias not 16-byte aligned");
    // Few output tiles and a long k (a Dense layer with tens of thousands of inputs at a
    // small batch): slices of k become work items so that the whole GPU is used.
    const int out_tiles = (int)(ceil_div(m, BLOCK_M) * ceil_div(n, BLOCK_N));
    const int total_kb = (int)ceil_div(k, BLOCK_K);
    int splits = 1, kb_per_split = total_kb;
    if (out_tiles * 4 <= dev->sm_count && total_kb >= 64) {
        splits = dev->sm_count / out_tiles;
        if (splits > total_kb / 4) splits = total_kb / 4;  // at least four k blocks per slice
        if (splits < 1) splits = 1;
        kb_per_split = (int)ceil_div(total_kb, splits);
        splits = (int)ceil_div(total_kb, kb_per_split);
    }
    if (splits == 1 && gemm_bf16_pair_enabled() && m >= 256 && n >= 256)
        return gemm_bf16_pair(dev, m, k, n, alpha, a, rsa, csa, b, rsb, csb, beta, c, rsc, csc, epi);
    const bool a_mn = !(csa == 1 && rsa % 8 == 0 && rsa >= k);  // else contiguous along m
    const bool b_mn = !(rsb == 1 && csb % 8 == 0 && csb >= k);  // else contiguous along n
    CUtensorMap ta, tb;
    if (a_mn)
        AG_TRY(make_tmap(&ta, a, (uint64_t)m, (uint64_t)k, (uint64_t)csa, 64, BLOCK_K));
    else
        AG_TRY(make_tmap(&ta, a, (uint64_t)k, (uint64_t)m, (uint64_t)rsa, BLOCK_K, BLOCK_M));
    if (b_mn)
        AG_TRY(make_tmap(&tb, b, (uint64_t)n, (uint64_t)k, (uint64_t)rsb, 64, BLOCK_K));
    else
        AG_TRY(make_tmap(&tb, b, (uint64_t)k, (uint64_t)n, (uint64_t)csb, BLOCK_K, BLOCK_N));
    Params p;
    p.M = m;
    p.N = n;
    p.K = k;
    p.ldc = rsc;
    p.alpha = alpha;
    p.beta = beta;
    p.C = c;
    p.status = dev->status_dev;
    p.lbo_k = 0;
    p.partial = nullptr;
    p.bias = (epi && splits == 1) ? epi->bias : nullptr;   // slices keep raw sums; the reduction applies it
    p.relu = (epi && splits == 1 && epi->relu) ? 1 : 0;
    p.splits = splits;
    p.kb_per_split = kb_per_split;
    if (splits > 1) {
        void *ws = nullptr;
        AG_TRY(workspace(dev, sizeof(float) * (size_t)splits * (size_t)m * (size_t)n, &ws));
        p.partial = (float *)ws;
    }
    if (a_mn && b_mn)
        AG_TRY((launch<true, true>(dev, ta, tb, p)));
    else if (a_mn)
        AG_TRY((launch<true, false>(dev, ta, tb, p)));
    else if (b_mn)
        AG_TRY((launch<false, true>(dev, ta, tb, p)));
    else
        AG_TRY((launch<false, false>(dev, ta, tb, p)));
    if (splits > 1) {
        // fixed slice order: the result does not depend on scheduling
        const int64_t plane = (int64_t)m * n;
        if (epi) {
            using Epi = simt::BiasReluEpilogue<__nv_bfloat16>;
            Epi E{c, rsc, epi->bias, epi->relu};
            simt::splitk_reduce_kernel<Epi><<<(unsigned)ceil_div(plane, 256), 256, 0, dev->stream>>>(
                p.partial, plane, splits, m, n, E);
        } else {
            using Epi = simt::StridedEpilogue<__nv_bfloat16>;
            Epi E{c, rsc, 1, alpha, beta, false, n};
            simt::splitk_reduce_kernel<Epi><<<(unsigned)ceil_div(plane, 256), 256, 0, dev->stream>>>(
                p.partial, plane, splits, m, n, E);
        }
        AG_CHECK_LAUNCH();
    }
    return AG_OK;
}

}  // namespace tc
}  // namespace ag
