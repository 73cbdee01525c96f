// bf16 implicit-GEMM convolution on tcgen05 with the filter bank resident in
// shared memory and ONE activation load per pixel tile.
//
// The channels-last activation of a whole batch is a matrix of rows: row
// q = (b * Hp + y) * Wp + x holds the 64-channel blocks of pixel (b, y, x) of the
// (zero-framed) image, 128 bytes per block.  For output pixel q and filter tap
// (fi, fj) the input pixel is row q + fi * Wp + fj: the A operand of a tap is the
// A operand of tap (0, 0) moved down by a constant number of rows.  So a CTA
// loads, per channel block, one box of 128 + (FH-1) * Wp + (FW-1) consecutive rows
// and issues every tap's tcgen05.mma on that box with the shared-memory descriptor
// advanced by (fi * Wp + fj) rows.  Rows are 128 bytes, so an advanced start
// address is a multiple of 128 but not of the 1024-byte swizzle atom.  That is
// fine as it stands: the 128-byte swizzle is a function of the absolute
// shared-memory address (bits 4-6 xor bits 7-9), for the TMA write and for the
// tensor core's read alike, so a descriptor that starts mid-atom reads the rows it
// names (base-offset field 0; measured: setting it to the row phase gives wrong
// sums, leaving it 0 reproduces the oracle bit for bit).  The M index runs over all rows q,
// including the Wp - OW right-hand columns and Hp - OH bottom rows of every image
// that are not outputs: their results are computed and dropped (12 % of the work
// for a 31x31 image and a 3x3 filter), which buys a tile that never straddles
// anything and nine times less operand traffic from L2 than one box per tap.
// The filter bank [tap][channel block][oc][64] is loaded once per CTA and stays.
//
// Warp roles, the two TMEM accumulators, the channels-last epilogue and the
// bounded waits are those of conv2_bf16_tc_kernel (conv_tc.cu).
#include "conv_tc.cuh"
#include "tc_ptx.cuh"

namespace ag {
namespace convtc {

using namespace ::ag::tc;

namespace {

constexpr int HB_M = 128;
constexpr int HB_K = 64;
constexpr int H_UMMA_K = 16;
constexpr int H_THREADS = 192;
constexpr int H_MAX_STAGES = 4;

struct HaloParams {
    int R;             // rows of the activation matrix: B * Hp * Wp
    int Hp, Wp;        // framed image size
    int OH, OW, OC, OCp;
    int FH, FW, CB;    // filter taps; channel blocks of 64
    int halo_rows;     // rows per activation box: 128 + (FH-1) * Wp + FW - 1, rounded up to 8
    int stages;        // activation boxes in flight
    FastDiv div_w, div_hw;
    const __nv_bfloat16 *bias;
    int relu;
    __nv_bfloat16 *y;  // channels-last [B][OH][OW][OCp]
    int *status;
};

template <int BLOCK_N>
__global__ void __launch_bounds__(H_THREADS, 1)
    conv2_bf16_tc_halo_kernel(const __grid_constant__ CUtensorMap tmap_x,
                              const __grid_constant__ CUtensorMap tmap_w, const HaloParams p) {
    constexpr int W_TILE_BYTES = BLOCK_N * HB_K * 2;
    constexpr int TMEM_COLS = 2 * BLOCK_N;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~uintptr_t(1023));
    const int taps = p.FH * p.FW;
    const int w_tiles = taps * p.CB;
    const int stage_bytes = p.halo_rows * 128;
    uint8_t *smem_w = smem;
    uint8_t *smem_a = smem + w_tiles * W_TILE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_a + p.stages * stage_bytes);
    uint64_t *full_bar = bars;                          // [stages] TMA -> MMA
    uint64_t *empty_bar = bars + H_MAX_STAGES;          // [stages] MMA -> TMA
    uint64_t *tmem_full_bar = bars + 2 * H_MAX_STAGES;  // [2]
    uint64_t *tmem_empty_bar = tmem_full_bar + 2;       // [2]
    uint64_t *w_full_bar = tmem_empty_bar + 2;          // filter bank landed
    uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(w_full_bar + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_base_slot + 1);
    // bias of this CTA's output channels as f32 (zero where there is none): read from
    // shared memory in the epilogue instead of one global load per element
    __shared__ float s_bias[BLOCK_N];

    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int num_tiles = (p.R + HB_M - 1) / HB_M;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_x);
        prefetch_tmap(&tmap_w);
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&tmem_full_bar[s]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[s]), 128);
        }
        mbar_init(smem_u32(w_full_bar), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    for (int i = threadIdx.x; i < BLOCK_N; i += H_THREADS)
        s_bias[i] = (p.bias != nullptr && i < p.OC) ? __bfloat162float(p.bias[i]) : 0.f;
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
            // the filter bank, once
            const uint32_t wbar = smem_u32(w_full_bar);
            mbar_arrive_expect_tx(wbar, (uint32_t)(w_tiles * W_TILE_BYTES));
            for (int t = 0; t < w_tiles; ++t)
                tma_load_2d(smem_u32(smem_w + t * W_TILE_BYTES), &tmap_w, wbar, t * HB_K, 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                for (int cb = 0; cb < p.CB; ++cb) {
                    if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag)) {
                        atomicExch(p.status, 141);
                        ok = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&full_bar[stage]);
                    mbar_arrive_expect_tx(bar, (uint32_t)stage_bytes);
                    tma_load_2d(smem_u32(smem_a + stage * stage_bytes), &tmap_x, bar, cb * HB_K,
                                tile * HB_M);
                    if (++stage == p.stages) {
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
            constexpr uint32_t idesc = make_idesc(false, false, HB_M, BLOCK_N);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = mbar_wait(smem_u32(w_full_bar), 0, abort_flag);
            if (!ok) atomicExch(p.status, 145);
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag)) {
                    atomicExch(p.status, 142);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BLOCK_N);
                for (int cb = 0; cb < p.CB; ++cb) {
                    if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag)) {
                        atomicExch(p.status, 143);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    // One thread issues every MMA of the CTA, so the issue loop is kept to a
                    // few integer adds per instruction: a descriptor's low bits are the
                    // shared-memory address >> 4, and moving an operand by a whole number of
                    // 16-byte units is an add to the 64-bit descriptor (addresses stay below
                    // 256 KiB, so nothing carries out of the 14-bit address field).
                    const uint64_t a_desc0 =
                        make_smem_desc(smem_u32(smem_a + stage * stage_bytes), 0, 1024);
                    const uint64_t b_desc0 =
                        make_smem_desc(smem_u32(smem_w + cb * W_TILE_BYTES), 0, 1024);
                    const uint64_t b_tap_step = (uint64_t)((p.CB * W_TILE_BYTES) >> 4);
                    uint64_t b_tap = b_desc0;
                    uint32_t accumulate = cb > 0 ? 1u : 0u;
                    for (int fi = 0; fi < p.FH; ++fi) {
                        uint64_t a_tap = a_desc0 + (uint64_t)(fi * p.Wp * 8);  // 128-byte rows
                        for (int fj = 0; fj < p.FW; ++fj, a_tap += 8, b_tap += b_tap_step) {
                            umma_bf16(d_tmem, a_tap, b_tap, idesc, accumulate);
                            accumulate = 1u;
#pragma unroll
                            for (int k = 1; k < HB_K / H_UMMA_K; ++k)
                                umma_bf16(d_tmem, a_tap + 2 * k, b_tap + 2 * k, idesc, 1u);
                        }
                    }
                    umma_commit(smem_u32(&empty_bar[stage]));
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(smem_u32(&tmem_full_bar[acc]));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------- epilogue
        const int quarter = warp % 4;
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag)) {
                if (lane == 0) atomicExch(p.status, 144);
                break;
            }
            tc_fence_after();
            const uint32_t q = (uint32_t)(tile * HB_M + quarter * 32 + lane);
            const uint32_t b = p.div_hw.div(q);
            const uint32_t rem = q - b * (uint32_t)(p.Hp * p.Wp);
            const uint32_t oy = p.div_w.div(rem);
            const uint32_t ox = rem - oy * (uint32_t)p.Wp;
            const bool valid = q < (uint32_t)p.R && oy < (uint32_t)p.OH && ox < (uint32_t)p.OW;
            const uint32_t taddr =
                tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BLOCK_N);
            __nv_bfloat16 *dst = p.y + (((int64_t)b * p.OH + oy) * p.OW + ox) * p.OCp;
#pragma unroll 1
            for (int chunk = 0; chunk < BLOCK_N / 32; ++chunk) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + chunk * 32, r);
                tmem_ld_wait();
                const int oc0 = chunk * 32;
                if (valid && oc0 < p.OCp) {
                    uint32_t packed[16];
                    const bool has_bias = p.bias != nullptr;
#pragma unroll
                    for (int j = 0; j < 32; j += 2)
                        packed[j / 2] = bf16_pair_epilogue(r[j], r[j + 1], s_bias[oc0 + j],
                                                           s_bias[oc0 + j + 1], has_bias, p.relu != 0);
                    uint4 *d4 = reinterpret_cast<uint4 *>(dst + oc0);
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4)
                        d4[k4] = make_uint4(packed[4 * k4], packed[4 * k4 + 1], packed[4 * k4 + 2],
                                            packed[4 * k4 + 3]);
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
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int BLOCK_N>
int launch_halo(ag_device *dev, const CUtensorMap &tx, const CUtensorMap &tw, const HaloParams &p,
                int smem) {
    auto kernel = conv2_bf16_tc_halo_kernel<BLOCK_N>;
    // the attribute belongs to the (kernel, GPU) pair: largest size set so far, per
    // instantiation and GPU
    static int configured_on[64] = {};
    int &configured = configured_on[dev->ordinal & 63];
    if (smem > configured) {
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = smem;
    }
    const int tiles = (p.R + HB_M - 1) / HB_M;
    const int grid = tiles < dev->sm_count ? tiles : dev->sm_count;
    kernel<<<grid, H_THREADS, smem, dev->stream>>>(tx, tw, p);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

}  // namespace

bool halo_plan(int64_t bs, int64_t cp, int64_t hp, int64_t wp, int64_t c_out, int fh, int fw,
               int *block_n, int *halo_rows, int *stages, int *smem_bytes) {
    if (c_out > 128) return false;
    const int bn = c_out <= 64 ? 64 : 128;
    const int64_t rows = ((HB_M + (int64_t)(fh - 1) * wp + (fw - 1)) + 7) / 8 * 8;
    if (rows > 256) return false;
    if (bs * hp * wp >= (int64_t(1) << 31) - 256) return false;
    const int64_t w_bytes = (int64_t)fh * fw * (cp / 64) * bn * 128;
    const int64_t budget = 226 * 1024 - 1024 - 256 - w_bytes;
    int st = (int)(budget / (rows * 128));
    if (st > H_MAX_STAGES) st = H_MAX_STAGES;
    if (st < 2) return false;
    *block_n = bn;
    *halo_rows = (int)rows;
    *stages = st;
    *smem_bytes = (int)(w_bytes + st * rows * 128 + 1024 + 256);
    return true;
}

int run_halo(ag_device *dev, const __nv_bfloat16 *act_rows, const __nv_bfloat16 *wk, int64_t bs,
             int64_t cp, int64_t hp, int64_t wp, int fh, int fw, int64_t c_out, int64_t out_h,
             int64_t out_w, const __nv_bfloat16 *bias, bool relu, __nv_bfloat16 *out_nhwc) {
    int block_n = 0, halo_rows = 0, stages = 0, smem = 0;
    AG_REQUIRE(halo_plan(bs, cp, hp, wp, c_out, fh, fw, &block_n, &halo_rows, &stages, &smem),
               AG_ERR_UNSUPPORTED, "shape not taken by the resident-filter convolution");
    HaloParams p;
    p.R = (int)(bs * hp * wp);
    p.Hp = (int)hp; p.Wp = (int)wp;
    p.OH = (int)out_h; p.OW = (int)out_w; p.OC = (int)c_out;
    p.OCp = (int)((c_out + 63) / 64 * 64);
    p.FH = fh; p.FW = fw;
    p.CB = (int)(cp / 64);
    p.halo_rows = halo_rows;
    p.stages = stages;
    p.div_w = FastDiv((uint32_t)wp);
    p.div_hw = FastDiv((uint32_t)(hp * wp));
    p.bias = bias;
    p.relu = relu ? 1 : 0;
    p.y = out_nhwc;
    p.status = dev->status_dev;
    CUtensorMap tx, tw;
    {
        const uint64_t dims[2] = {(uint64_t)cp, (uint64_t)p.R};
        const uint64_t strides[1] = {(uint64_t)cp};
        const uint32_t box[2] = {64, (uint32_t)halo_rows};
        AG_TRY(make_tmap_bf16(&tx, act_rows, 2, dims, strides, box));
    }
    {
        const uint64_t k = (uint64_t)fh * fw * (uint64_t)cp;
        const uint64_t dims[2] = {k, (uint64_t)c_out};
        const uint64_t strides[1] = {k};
        const uint32_t box[2] = {64, (uint32_t)block_n};
        AG_TRY(make_tmap_bf16(&tw, wk, 2, dims, strides, box));
    }
    if (block_n == 64) return launch_halo<64>(dev, tx, tw, p, smem);
    return launch_halo<128>(dev, tx, tw, p, smem);
}

}  // namespace convtc
}  // namespace ag
