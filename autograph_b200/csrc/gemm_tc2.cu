// bf16 GEMM on paired SMs: C = alpha * A.B + beta * C, f32 accumulation in TMEM.
//
// Two CTAs of a cluster share one 256 x 256 output tile (tcgen05 cta_group::2):
// CTA r of the pair stages rows [128r, 128r+128) of the A tile and columns
// [128r, 128r+128) of the B tile, and holds rows [128r, 128r+128) of the
// accumulator in its own tensor memory.  One thread of the leader CTA issues
// every tcgen05.mma (M=256, N=256, K=16), which reads the A rows and the B
// halves from both CTAs' shared memory.  Compared with one CTA per tile this
// halves the B bytes each SM has to stage and read per flop, which is what the
// single-CTA kernel is limited by.
//
// Roles per CTA (192 threads): warp 0 = TMA producer (own halves; the loads of
// both CTAs signal the leader's "full" barrier), warp 1 = MMA issuer (leader
// only) and TMEM allocation, warps 2..5 = epilogue of the CTA's own 128 rows.
// Ring stages are released, and finished accumulators published, to both CTAs
// with one tcgen05.commit that arrives in both CTAs.  Every TMA load is a plain
// (single-destination) load into the issuing CTA's own shared memory.
//
// The PTX wrappers that do not depend on the CTA group (mbarriers with bounded waits,
// descriptors, tensor-memory loads) are those of tc_ptx.cuh; only the cta_group::2 and
// cluster forms live here.
// Every mbarrier wait is bounded (about 2 s) and reports through a status word.
// Tensor memory is allocated in two 256-column steps; after the first step the
// two CTAs compare the addresses they were given, and stop with an error if
// they differ, before anything could block on tensor memory.
#include <cuda.h>

#include <cstdlib>

#include "gemm_tc.cuh"
#include "tc_ptx.cuh"

namespace ag {
namespace tc {

namespace pair {

constexpr int TILE_M = 256;   // per pair; 128 rows per CTA
constexpr int TILE_N = 256;   // per pair; each CTA stages 128 columns of B
constexpr int BLOCK_K = 64;
constexpr int UMMA_K = 16;
// Ring depth.  Seven stages fill the CTA's shared memory; a profiler that adds to the launch's
// resources cannot launch that, so a build for profiling may lower it (-DAG_TC2_STAGES=6).
#ifndef AG_TC2_STAGES
#define AG_TC2_STAGES 7
#endif
constexpr int STAGES = AG_TC2_STAGES;
constexpr int A_BYTES = 128 * BLOCK_K * 2;  // 16 KiB
constexpr int B_BYTES = 128 * BLOCK_K * 2;  // 16 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int ATOM_BYTES = 64 * BLOCK_K * 2;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}
__device__ __forceinline__ uint32_t ld_shared_cluster(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on a barrier that may live in the peer CTA (cluster address).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
                 : "memory");
}
// TMA load whose completion may be signalled to a barrier in the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map,
                                                 uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival on the barrier at the same offset in every CTA of `mask`, once all
// tcgen05 operations issued so far by this thread have completed.
__device__ __forceinline__ void umma2_commit_multicast(uint32_t bar, uint16_t mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
        "[%0], %1;" ::"r"(bar),
        "h"(mask)
        : "memory");
}
struct Params {
    int M, N, K;
    int64_t ldc;
    float alpha, beta;
    __nv_bfloat16 *C;
    int *status;
    // Work list: items [0, t_full) are whole 256 x 256 tiles; the tiles of the last,
    // partial wave are cut along n into `tail_split` pieces so that they spread over
    // all CTA pairs instead of leaving most of them idle for a whole tile time.
    int t_full, tail_split, num_work;
    int group_m;  // m blocks per group of the tile order (tiles of a group share B columns in L2)
    const __nv_bfloat16 *bias;  // fused Dense epilogue (alpha = 1, beta = 0): bias [N] or null, relu
    int relu;
};

struct Work {
    int m_blk, n_blk;
    int n_off;    // column offset of this piece inside the tile
    int n_width;  // 256, or 128 for a piece of a tail tile
};

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int group_m, int &m_blk,
                                            int &n_blk) {
    const int group_size = group_m * num_n;
    const int g = tile / group_size;
    const int first_m = g * group_m;
    const int gm = min(num_m - first_m, group_m);
    const int r = tile - g * group_size;
    m_blk = first_m + r % gm;
    n_blk = r / gm;
}

__device__ __forceinline__ Work decode_work(int w, const Params &p, int num_m, int num_n) {
    Work k;
    int tile;
    if (w < p.t_full) {
        tile = w;
        k.n_off = 0;
        k.n_width = TILE_N;
    } else {
        const int j = w - p.t_full;
        tile = p.t_full + j / p.tail_split;
        k.n_width = TILE_N / p.tail_split;
        k.n_off = (j % p.tail_split) * k.n_width;
    }
    tile_coords(tile, num_m, num_n, p.group_m, k.m_blk, k.n_blk);
    return k;
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
    gemm_bf16_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_b_tail, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    // Both CTAs of the pair compute the same aligned offset (the dynamic shared memory
    // window starts at the same address in every CTA of a kernel).
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + STAGES * A_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES);
    uint64_t *full_bar = bars;                           // [STAGES] used in the leader only
    uint64_t *empty_bar = bars + STAGES;                 // [STAGES] per CTA
    uint64_t *tmem_full_bar = bars + 2 * STAGES;         // [2] per CTA
    uint64_t *tmem_empty_bar = bars + 2 * STAGES + 2;    // [2] used in the leader only
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);  // [2]
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 2);

    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    const int num_m = (p.M + TILE_M - 1) / TILE_M;
    const int num_n = (p.N + TILE_N - 1) / TILE_N;
    const int num_work = p.num_work;
    const int num_kb = (p.K + BLOCK_K - 1) / BLOCK_K;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        prefetch_tmap(&tmap_b_tail);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&tmem_full_bar[s]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[s]), 256);  // 128 epilogue threads of each CTA
        }
        tmem_slot[0] = 0xffffffffu;
        tmem_slot[1] = 0xffffffffu;
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // ---- tensor memory, step 1: 256 columns; the pair must agree on the address ----
    if (warp == 1) tmem_alloc2(smem_u32(&tmem_slot[0]), 256);
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // barriers of both CTAs initialised; both slot[0] written
    tc_fence_after();
    bool ok_alloc = true;
    {
        const uint32_t mine = tmem_slot[0];
        const uint32_t theirs = ld_shared_cluster(map_to_cta(smem_u32(&tmem_slot[0]), rank ^ 1u));
        if (mine != theirs) ok_alloc = false;
    }
    cluster_sync();  // both CTAs have read each other's slot
    if (!ok_alloc) {
        // The two CTAs were given different addresses: this build's assumption about paired
        // allocation does not hold.  Give back what this CTA holds and stop.
        if (threadIdx.x == 0) atomicExch(p.status, 110);
        if (warp == 1) {
            tmem_dealloc2(tmem_slot[0], 256);
            tmem_relinquish2();
        }
        return;
    }
    // ---- step 2: the second accumulator -----------------------------------------------
    if (warp == 1) {
        tmem_alloc2(smem_u32(&tmem_slot[1]), 256);
        tmem_relinquish2();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc[2] = {tmem_slot[0], tmem_slot[1]};

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int w = pair_id; ok && w < num_work; w += num_pairs) {
                const Work wk = decode_work(w, p, num_m, num_n);
                const int half_n = wk.n_width / 2;  // B columns staged by each CTA
                const int m0 = wk.m_blk * TILE_M + (int)rank * 128;
                const int n0 = wk.n_blk * TILE_N + wk.n_off + (int)rank * half_n;
                const uint32_t stage_tx = (uint32_t)(2 * (A_BYTES + half_n * BLOCK_K * 2));
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag)) {
                        atomicExch(p.status, 121);
                        ok = false;
                        break;
                    }
                    // Loads of both CTAs are counted by the leader's barrier.
                    const uint32_t local_full = smem_u32(&full_bar[stage]);
                    if (leader) mbar_arrive_expect_tx(local_full, stage_tx);
                    const uint32_t bar = map_to_cta(local_full, 0);
                    const uint32_t a_dst = smem_u32(smem_a + stage * A_BYTES);
                    const uint32_t b_dst = smem_u32(smem_b + stage * B_BYTES);
                    if (A_MN) {
#pragma unroll
                        for (int i = 0; i < 2; ++i)
                            tma_load_2d_pair(a_dst + i * ATOM_BYTES, &tmap_a, bar, m0 + i * 64,
                                             kb * BLOCK_K);
                    } else {
                        tma_load_2d_pair(a_dst, &tmap_a, bar, kb * BLOCK_K, m0);
                    }
                    if (B_MN) {
                        for (int i = 0; i < half_n / 64; ++i)
                            tma_load_2d_pair(b_dst + i * ATOM_BYTES, &tmap_b, bar, n0 + i * 64,
                                             kb * BLOCK_K);
                    } else if (half_n == 128) {
                        tma_load_2d_pair(b_dst, &tmap_b, bar, kb * BLOCK_K, n0);
                    } else {
                        // tail pieces: one 64-row box (tmap_b_tail) per stage
                        tma_load_2d_pair(b_dst, &tmap_b_tail, bar, kb * BLOCK_K, n0);
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
        // -------------------------------------------------------- MMA issuer (leader only)
        if (leader && lane == 0) {
            const uint32_t a_lbo = A_MN ? (uint32_t)ATOM_BYTES : 0u;
            const uint32_t b_lbo = B_MN ? (uint32_t)ATOM_BYTES : 0u;
            const uint32_t a_kstep = A_MN ? UMMA_K * 128 : UMMA_K * 2;
            const uint32_t b_kstep = B_MN ? UMMA_K * 128 : UMMA_K * 2;
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int w = pair_id; ok && w < num_work; w += num_pairs) {
                const Work wk = decode_work(w, p, num_m, num_n);
                const uint32_t idesc = make_idesc(A_MN, B_MN, TILE_M, wk.n_width);
                if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag)) {
                    atomicExch(p.status, 122);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_acc[acc];
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag)) {
                        atomicExch(p.status, 123);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_base = smem_u32(smem_a + stage * A_BYTES);
                    const uint32_t b_base = smem_u32(smem_b + stage * B_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t a_desc = make_smem_desc(a_base + k * a_kstep, a_lbo, 1024);
                        const uint64_t b_desc = make_smem_desc(b_base + k * b_kstep, b_lbo, 1024);
                        umma2_bf16(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma2_commit_multicast(smem_u32(&empty_bar[stage]), 3);  // both CTAs' rings
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma2_commit_multicast(smem_u32(&tmem_full_bar[acc]), 3);
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------- epilogue (both CTAs)
        const int quarter = warp % 4;
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int w = pair_id; w < num_work; w += num_pairs) {
            const Work wk = decode_work(w, p, num_m, num_n);
            const int m_blk = wk.m_blk;
            if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag)) {
                if (lane == 0) atomicExch(p.status, 124);
                break;
            }
            tc_fence_after();
            const int row = m_blk * TILE_M + (int)rank * 128 + quarter * 32 + lane;
            const uint32_t taddr = tmem_acc[acc] + ((uint32_t)(quarter * 32) << 16);
            __nv_bfloat16 *crow = p.C + (int64_t)row * p.ldc;
            // Each thread holds one row of the accumulator and stores it in 16-byte pieces.
            // (Passing the tile through shared memory to store whole 128-byte lines was measured
            // and is slower: the main loop already saturates the shared-memory data path, 1306
            // against 1342 TFLOP/s at 4096^3.)  Two tensor-memory loads are in flight per wait.
#pragma unroll 1
            for (int chunk = 0; chunk < wk.n_width / 64; ++chunk) {
                uint32_t r2[2][32];
                tmem_ld_32x32(taddr + chunk * 64, r2[0]);
                tmem_ld_32x32(taddr + chunk * 64 + 32, r2[1]);
                tmem_ld_wait();
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint32_t(&r)[32] = r2[half];
                    const int col0 = wk.n_blk * TILE_N + wk.n_off + chunk * 64 + half * 32;
                    if (row < p.M && col0 < p.N) {
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
            }
            tc_fence_before();
            // The leader's MMA thread waits for the epilogues of both CTAs.
            mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[acc]), 0));
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
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    cluster_sync();  // no MMA of the pair is in flight, no remote arrive is pending
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc2(tmem_acc[0], 256);
        tmem_dealloc2(tmem_acc[1], 256);
    }
}

}  // namespace pair

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn2() {
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

// Encoding a tensor map costs a driver call of a microsecond or two, three per product; a
// caller that multiplies the same buffers again (every layer of every step does) finds its
// maps in a small per-thread cache keyed by everything the encoding depends on.
struct TmapKey {
    const void *base;
    uint64_t inner, outer, outer_stride;
    uint32_t box_inner, box_outer;
    bool operator==(const TmapKey &o) const {
        return base == o.base && inner == o.inner && outer == o.outer &&
               outer_stride == o.outer_stride && box_inner == o.box_inner && box_outer == o.box_outer;
    }
};
struct TmapCache {
    static constexpr int N = 32;
    TmapKey key[N];
    CUtensorMap map[N];
    int used = 0, next = 0;
};

static int make_tmap2(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer,
                      uint64_t outer_stride, uint32_t box_inner, uint32_t box_outer) {
    static thread_local TmapCache cache;
    const TmapKey k{base, inner, outer, outer_stride, box_inner, box_outer};
    for (int i = 0; i < cache.used; ++i)
        if (cache.key[i] == k) {
            *map = cache.map[i];
            return AG_OK;
        }
    EncodeTiledFn fn = encode_fn2();
    AG_REQUIRE(fn != nullptr, AG_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {outer_stride * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    AG_REQUIRE(r == CUDA_SUCCESS, AG_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d)",
               (int)r);
    const int slot = cache.used < TmapCache::N ? cache.used++ : (cache.next++ % TmapCache::N);
    cache.key[slot] = k;
    cache.map[slot] = *map;
    return AG_OK;
}

template <bool A_MN, bool B_MN>
static int launch_pair(ag_device *dev, const CUtensorMap &ta, const CUtensorMap &tb,
                       const CUtensorMap &tb_tail, const pair::Params &p) {
    auto kernel = pair::gemm_bf16_tc2_kernel<A_MN, B_MN>;
    static bool attr_done[64] = {};   // per GPU: the attribute belongs to the GPU's copy of the kernel
    if (dev->ordinal >= 64 || !attr_done[dev->ordinal]) {
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         pair::SMEM_BYTES));
        if (dev->ordinal < 64) attr_done[dev->ordinal] = true;
    }
    const int tiles = (int)(ceil_div(p.M, pair::TILE_M) * ceil_div(p.N, pair::TILE_N));
    (void)tiles;
    int pairs = dev->sm_count / 2;
    if (p.num_work < pairs) pairs = p.num_work;
    kernel<<<2 * pairs, pair::NUM_THREADS, pair::SMEM_BYTES, dev->stream>>>(ta, tb, tb_tail, p);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

bool gemm_bf16_pair_enabled() {
    static int v = []() {
        const char *e = getenv("AG_TC2");
        return (e && e[0] == '0') ? 0 : 1;
    }();
    return v != 0;
}

int gemm_bf16_pair(ag_device *dev, int m, int k, int n, float alpha, const __nv_bfloat16 *a,
                   int64_t rsa, int64_t csa, const __nv_bfloat16 *b, int64_t rsb, int64_t csb,
                   float beta, __nv_bfloat16 *c, int64_t rsc, int64_t csc, const Epilogue *epi) {
    (void)csc;
    const bool a_mn = !(csa == 1 && rsa % 8 == 0 && rsa >= k);
    const bool b_mn = !(rsb == 1 && csb % 8 == 0 && csb >= k);
    CUtensorMap ta, tb, tb_tail;
    if (a_mn)
        AG_TRY(make_tmap2(&ta, a, (uint64_t)m, (uint64_t)k, (uint64_t)csa, 64, pair::BLOCK_K));
    else
        AG_TRY(make_tmap2(&ta, a, (uint64_t)k, (uint64_t)m, (uint64_t)rsa, pair::BLOCK_K, 128));
    if (b_mn)
        AG_TRY(make_tmap2(&tb, b, (uint64_t)n, (uint64_t)k, (uint64_t)rsb, 64, pair::BLOCK_K));
    else
        AG_TRY(make_tmap2(&tb, b, (uint64_t)k, (uint64_t)n, (uint64_t)csb, pair::BLOCK_K, 128));
    if (b_mn)
        tb_tail = tb;
    else
        AG_TRY(make_tmap2(&tb_tail, b, (uint64_t)k, (uint64_t)n, (uint64_t)csb, pair::BLOCK_K, 64));
    pair::Params p;
    p.M = m;
    p.N = n;
    p.K = k;
    p.ldc = rsc;
    p.alpha = alpha;
    p.beta = beta;
    p.C = c;
    p.status = dev->status_dev;
    p.bias = epi ? epi->bias : nullptr;
    p.relu = epi && epi->relu ? 1 : 0;
    {
        static const int group_m = []() {
            const char *e = getenv("AG_TC2_GROUP_M");
            const int v = e ? atoi(e) : 8;
            return v < 1 ? 1 : v;
        }();
        p.group_m = group_m;
    }
    {
        const int tiles = (int)(ceil_div(m, pair::TILE_M) * ceil_div(n, pair::TILE_N));
        int pairs = dev->sm_count / 2;
        if (tiles < pairs) pairs = tiles;
        const int rem = tiles % pairs;
        static const bool tail_enabled = []() {
            const char *e = getenv("AG_TC2_TAIL");
            return !(e && e[0] == '0');
        }();
        int split = 1;
        if (tail_enabled && rem > 0 && tiles > pairs) {
            if (2 * rem <= pairs) split = 2;
        }
        p.tail_split = split;
        p.t_full = split > 1 ? tiles - rem : tiles;
        p.num_work = p.t_full + (split > 1 ? split * rem : 0);
        // Fewer tiles than half the CTA pairs (1024^3: 16 tiles on 74 pairs): every tile is cut
        // in two along n, which halves the time of the one and only wave.
        if (tail_enabled && 2 * tiles <= dev->sm_count / 2) {
            p.tail_split = 2;
            p.t_full = 0;
            p.num_work = 2 * tiles;
        }
    }
    if (a_mn && b_mn) return launch_pair<true, true>(dev, ta, tb, tb_tail, p);
    if (a_mn) return launch_pair<true, false>(dev, ta, tb, tb_tail, p);
    if (b_mn) return launch_pair<false, true>(dev, ta, tb, tb_tail, p);
    return launch_pair<false, false>(dev, ta, tb, tb_tail, p);
}

}  // namespace tc
}  // namespace ag
