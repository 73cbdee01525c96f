// bf16 weight gradient of a convolution on the Blackwell tensor cores.
//
//   dw[oc][ci][fi][fj] = sum over (b, oy, ox) of dy[b][oc][oy][ox] * x[b][ci][oy+fi-ph][ox+fj-pw]
//
// For one filter tap this is a product  dy^T . x_shifted  whose reduction index
// is the output pixel.  With both tensors rewritten channels-last, a chunk of 64
// pixels (a TH x TW rectangle of one image) of dy is a [64 pixels][64 channels]
// TMA box -- an MN-major operand tile for tcgen05.mma -- and the matching chunk
// of x for tap (fi, fj) is the same box shifted by the tap; pixels outside the
// image read as zero, which is both the padding and the ragged edge.
//
// A CTA owns one filter row (FW taps), one block of 128 output channels, one
// block of input channels and a contiguous range of pixel chunks: every stage of
// its ring holds one dy tile and FW shifted x tiles, the FW accumulators live in
// TMEM for the whole range, and the f32 partial result goes to a scratch plane
// [split][oc][tap][ci].  A second kernel adds the planes in split order (so the
// result is reproducible), applies beta and writes dw in its [oc][ci][fi][fj]
// layout.  Warp roles and the bounded waits are those of the GEMM kernel.
#include "conv_tc.cuh"
#include "tc_ptx.cuh"

namespace ag {
namespace convtc {

using namespace ::ag::tc;

namespace {

constexpr int WG_BLOCK_M = 128;
constexpr int WG_CHUNK = 64;                     // pixels per k step
constexpr int WG_ATOM_BYTES = 64 * WG_CHUNK * 2;  // one [64 pixels][64 channels] box
constexpr int WG_A_BYTES = 2 * WG_ATOM_BYTES;
constexpr int WG_UMMA_K = 16;
constexpr int WG_THREADS = 192;
constexpr int WG_MAX_STAGES = 8;

struct WgParams {
    int B, OH, OW;
    int TW, tw_shift;          // pixel chunk: TH x TW = 64, TW = 1 << tw_shift
    int chunks_y, chunks_x;    // chunks per image
    int total_chunks, chunks_per_split;
    int FW, groups;            // taps per CTA (one filter row); filter rows
    int m_blocks, n_blocks;
    int pad_h, pad_w;
    int Cp, taps;
    int stages, stage_bytes;
    float *partial;            // [splits][m_blocks * 128][taps][Cp]
    int *status;
};

template <int NT>
__global__ void __launch_bounds__(WG_THREADS, 1)
    conv2_wgrad_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmap_dy,
                               const __grid_constant__ CUtensorMap tmap_x, const WgParams p) {
    constexpr int ATOMS_N = NT / 64;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + p.stages * p.stage_bytes);
    uint64_t *full_bar = bars;
    uint64_t *empty_bar = bars + WG_MAX_STAGES;
    uint64_t *tmem_full_bar = bars + 2 * WG_MAX_STAGES;
    uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(bars + 2 * WG_MAX_STAGES + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_base_slot + 1);

    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;

    int r = blockIdx.x;
    const int n_blk = r % p.n_blocks;
    r /= p.n_blocks;
    const int m_blk = r % p.m_blocks;
    r /= p.m_blocks;
    const int group = r % p.groups;  // filter row
    const int split = r / p.groups;
    const int c_begin = split * p.chunks_per_split;
    const int c_end = min(p.total_chunks, c_begin + p.chunks_per_split);

    // TMEM columns: FW accumulators of NT columns, rounded up to a power of two >= 32.
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < p.FW * NT) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_dy);
        prefetch_tmap(&tmap_x);
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(tmem_full_bar), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_base_slot), tmem_cols);
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
            const int per_image = p.chunks_y * p.chunks_x;
            const int th = WG_CHUNK >> p.tw_shift;
            for (int c = c_begin; c < c_end; ++c) {
                const int b = c / per_image;
                const int rem = c - b * per_image;
                const int cy = rem / p.chunks_x, cx = rem - cy * p.chunks_x;
                const int oy0 = cy * th, ox0 = cx * p.TW;
                if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag)) {
                    atomicExch(p.status, 131);
                    break;
                }
                const uint32_t bar = smem_u32(&full_bar[stage]);
                mbar_arrive_expect_tx(bar, (uint32_t)p.stage_bytes);
                const uint32_t a_dst = smem_u32(smem + stage * p.stage_bytes);
                const uint32_t b_dst = a_dst + WG_A_BYTES;
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    tma_load_4d(a_dst + i * WG_ATOM_BYTES, &tmap_dy, bar, m_blk * WG_BLOCK_M + i * 64,
                                ox0, oy0, b);
                for (int g = 0; g < p.FW; ++g)
#pragma unroll
                    for (int j = 0; j < ATOMS_N; ++j)
                        tma_load_4d(b_dst + (g * ATOMS_N + j) * WG_ATOM_BYTES, &tmap_x, bar,
                                    n_blk * NT + j * 64, ox0 + g - p.pad_w, oy0 + group - p.pad_h, b);
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // The x tiles of the taps of a filter row lie one after the other in the stage and
            // their accumulators one after the other in TMEM, so several taps are ONE operand
            // of up to 256 columns: one tcgen05.mma per k step covers them all, which moves
            // far fewer operand bytes per flop than one 64-column instruction per tap.
            const int taps_per_mma = min(p.FW, 256 / NT);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int c = c_begin; c < c_end; ++c) {
                if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag)) {
                    atomicExch(p.status, 132);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_base = smem_u32(smem + stage * p.stage_bytes);
                const uint32_t b_base = a_base + WG_A_BYTES;
                for (int g0 = 0; g0 < p.FW; g0 += taps_per_mma) {
                    const int n_cols = min(taps_per_mma, p.FW - g0) * NT;
                    const uint32_t idesc = make_idesc(true, true, WG_BLOCK_M, n_cols);
#pragma unroll
                    for (int k = 0; k < WG_CHUNK / WG_UMMA_K; ++k) {
                        // 16 pixel rows of 128 bytes per k step
                        const uint64_t a_desc =
                            make_smem_desc(a_base + k * WG_UMMA_K * 128, WG_ATOM_BYTES, 1024);
                        const uint64_t b_desc =
                            make_smem_desc(b_base + g0 * ATOMS_N * WG_ATOM_BYTES + k * WG_UMMA_K * 128,
                                           WG_ATOM_BYTES, 1024);
                        umma_bf16(tmem_base + (uint32_t)(g0 * NT), a_desc, b_desc, idesc,
                                  (c > c_begin || k > 0) ? 1u : 0u);
                    }
                }
                umma_commit(smem_u32(&empty_bar[stage]));
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (ok) umma_commit(smem_u32(tmem_full_bar));
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------- epilogue
        const int quarter = warp % 4;
        if (mbar_wait(smem_u32(tmem_full_bar), 0, abort_flag)) {
            tc_fence_after();
            const int row = m_blk * WG_BLOCK_M + quarter * 32 + lane;  // output channel
            const int64_t m_total = (int64_t)p.m_blocks * WG_BLOCK_M;
            float *base = p.partial + (((int64_t)split * m_total + row) * p.taps) * p.Cp +
                          (int64_t)n_blk * NT;
            for (int g = 0; g < p.FW; ++g) {
                float *dst = base + (int64_t)(group * p.FW + g) * p.Cp;
#pragma unroll 1
                for (int chunk = 0; chunk < NT / 32; ++chunk) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) +
                                      (uint32_t)(g * NT + chunk * 32),
                                  v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        reinterpret_cast<uint4 *>(dst + chunk * 32)[j] =
                            make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
        } else if (lane == 0) {
            atomicExch(p.status, 133);
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
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

// dw[oc][ci][tap] = beta * dw + sum over splits (in order) of partial[s][oc][tap][ci]
// Block of 32 x 8 threads: 32 consecutive outputs, the split planes dealt round-robin to the 8
// rows (every load of a warp is 128 contiguous bytes of one plane); the 8 row sums are added in
// row order, so the result does not depend on scheduling.
__global__ void wgrad_reduce_kernel(const float *__restrict__ partial, int splits, int64_t m_total,
                                    int taps, int Cp, int OC, int IC, float beta,
                                    __nv_bfloat16 *__restrict__ dw) {
    __shared__ float part[8][33];
    const int64_t i = (int64_t)blockIdx.x * 32 + threadIdx.x;
    const bool live = i < (int64_t)OC * taps * IC;
    const int ci = live ? (int)(i % IC) : 0;
    const int tap = live ? (int)((i / IC) % taps) : 0;
    const int oc = live ? (int)(i / ((int64_t)IC * taps)) : 0;
    const int64_t plane = m_total * taps * Cp;
    const float *src = partial + ((int64_t)oc * taps + tap) * Cp + ci;
    float s = 0.f;
    if (live)
        for (int z = threadIdx.y; z < splits; z += 8) s += src[(int64_t)z * plane];
    part[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y != 0 || !live) return;
    s = part[0][threadIdx.x];
#pragma unroll
    for (int r = 1; r < 8; ++r) s += part[r][threadIdx.x];
    __nv_bfloat16 *d = dw + ((int64_t)oc * IC + ci) * taps + tap;
    if (beta != 0.f) s = fmaf(beta, __bfloat162float(*d), s);
    *d = __float2bfloat16_rn(s);
}

int64_t round_up64(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

template <int NT>
int launch_wgrad(ag_device *dev, const CUtensorMap &tdy, const CUtensorMap &tx, const WgParams &p,
                 int grid) {
    auto kernel = conv2_wgrad_bf16_tc_kernel<NT>;
    const int smem = p.stages * p.stage_bytes + 1024 + 256;
    // the attribute belongs to the (kernel, GPU) pair: largest size set so far, per
    // instantiation and GPU
    static int configured_on[64] = {};
    int &configured = configured_on[dev->ordinal & 63];
    if (smem > configured) {
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = smem;
    }
    kernel<<<grid, WG_THREADS, smem, dev->stream>>>(tdy, tx, p);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

}  // namespace

bool eligible_backward_weight(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
                              const ag_conv2_options *o) {
    if (!tc_conv_enabled() || encode_tiled_fn() == nullptr) return false;
    if (o->stride[0] != 1 || o->stride[1] != 1 || o->dilation[0] != 1 || o->dilation[1] != 1)
        return false;
    const int fh = o->filter[0], fw = o->filter[1];
    const int64_t oh = ih + 2 * o->padding[0] - fh + 1, ow = iw + 2 * o->padding[1] - fw + 1;
    if (bs <= 0 || ic <= 0 || oc < 32 || oh <= 0 || ow <= 0) return false;
    if (fw < 1 || fw > 8 || fh < 1 || fh > 8) return false;
    if (bs * oh * ow < 4096) return false;
    if (ih > 32768 || iw > 32768 || bs > 65535) return false;
    const int64_t cp = round_up64(ic, 64), ocp = round_up64(oc, 64);
    if (bs * ih * iw * cp >= (int64_t(1) << 40) || bs * oh * ow * ocp >= (int64_t(1) << 40))
        return false;
    return true;
}

int backward_weight(ag_device *dev, const __nv_bfloat16 *x, int64_t bs, int64_t ic, int64_t ih,
                    int64_t iw, const __nv_bfloat16 *dy, int64_t oc, const ag_conv2_options *o,
                    float beta, __nv_bfloat16 *dw) {
    const int fh = o->filter[0], fw = o->filter[1];
    const int64_t oh = ih + 2 * o->padding[0] - fh + 1, ow = iw + 2 * o->padding[1] - fw + 1;
    const int64_t cp = round_up64(ic, 64), ocp = round_up64(oc, 64);
    const int64_t x_bytes = round_up64(bs * ih * iw * cp * 2, 1024);
    const int64_t dy_bytes = round_up64(bs * oh * ow * ocp * 2, 1024);
    void *st = nullptr;
    AG_TRY(staging(dev, (size_t)(x_bytes + dy_bytes), &st));
    __nv_bfloat16 *xh = (__nv_bfloat16 *)st;
    __nv_bfloat16 *dyh = (__nv_bfloat16 *)((char *)st + x_bytes);
    AG_TRY(to_nhwc(dev, x, bs, ic, ih * iw, cp, xh));
    AG_TRY(to_nhwc(dev, dy, bs, oc, oh * ow, ocp, dyh));
    return backward_weight_nhwc(dev, xh, bs, ic, ih, iw, dyh, ow * ocp, oh * ow * ocp, oc, o, beta, dw);
}

int backward_weight_nhwc(ag_device *dev, const __nv_bfloat16 *xh, int64_t bs, int64_t ic, int64_t ih,
                         int64_t iw, const __nv_bfloat16 *dyh, int64_t dy_row_pitch,
                         int64_t dy_image_pitch, int64_t oc, const ag_conv2_options *o, float beta,
                         __nv_bfloat16 *dw) {
    const int fh = o->filter[0], fw = o->filter[1];
    const int64_t oh = ih + 2 * o->padding[0] - fh + 1, ow = iw + 2 * o->padding[1] - fw + 1;
    const int64_t cp = round_up64(ic, 64), ocp = round_up64(oc, 64);
    const int nt = (cp % 128 == 0 && fw * 128 <= 512) ? 128 : 64;
    AG_REQUIRE(dy_row_pitch % 8 == 0 && dy_image_pitch % 8 == 0 &&
                   (reinterpret_cast<uintptr_t>(dyh) & 15) == 0 && (reinterpret_cast<uintptr_t>(xh) & 15) == 0,
               AG_ERR_INVALID, "weight gradient: channels-last operands must keep 16-byte alignment");

    WgParams p;
    p.B = (int)bs; p.OH = (int)oh; p.OW = (int)ow;
    int best_shift = 3;
    int64_t best_cover = -1;
    for (int shift = 3; shift <= 6; ++shift) {
        const int64_t tw = 1 << shift, th = WG_CHUNK / tw;
        const int64_t cover = round_up64(ow, tw) * round_up64(oh, th);
        if (best_cover < 0 || cover <= best_cover) {  // ties: the wider chunk
            best_cover = cover;
            best_shift = shift;
        }
    }
    p.tw_shift = best_shift;
    p.TW = 1 << best_shift;
    const int th = WG_CHUNK / p.TW;
    p.chunks_y = (int)ceil_div(oh, th);
    p.chunks_x = (int)ceil_div(ow, p.TW);
    const int64_t total = bs * p.chunks_y * p.chunks_x;
    AG_REQUIRE(total < (int64_t(1) << 31), AG_ERR_LIMIT, "too many pixel chunks");
    p.total_chunks = (int)total;
    p.FW = fw;
    p.groups = fh;
    p.m_blocks = (int)ceil_div(ocp, WG_BLOCK_M);
    p.n_blocks = (int)(cp / nt);
    p.pad_h = o->padding[0];
    p.pad_w = o->padding[1];
    p.Cp = (int)cp;
    p.taps = fh * fw;
    p.stage_bytes = WG_A_BYTES + fw * nt * 128;
    p.stages = (200 * 1024) / p.stage_bytes;
    if (p.stages > WG_MAX_STAGES) p.stages = WG_MAX_STAGES;
    AG_REQUIRE(p.stages >= 2, AG_ERR_LIMIT, "filter too wide for the tensor-core weight gradient");
    const int base = p.groups * p.m_blocks * p.n_blocks;
    int splits = dev->sm_count / base;
    if (splits < 1) splits = 1;
    if (splits > p.total_chunks) splits = p.total_chunks;
    p.chunks_per_split = (int)ceil_div(p.total_chunks, splits);
    splits = (int)ceil_div(p.total_chunks, p.chunks_per_split);
    const int64_t m_total = (int64_t)p.m_blocks * WG_BLOCK_M;
    void *ws = nullptr;
    AG_TRY(workspace(dev, sizeof(float) * (size_t)splits * (size_t)m_total * p.taps * (size_t)cp,
                     &ws));
    p.partial = (float *)ws;
    p.status = dev->status_dev;

    CUtensorMap tdy, tx;
    {
        const uint64_t dims[4] = {(uint64_t)ocp, (uint64_t)ow, (uint64_t)oh, (uint64_t)bs};
        const uint64_t strides[3] = {(uint64_t)ocp, (uint64_t)dy_row_pitch, (uint64_t)dy_image_pitch};
        const uint32_t box[4] = {64, (uint32_t)p.TW, (uint32_t)th, 1};
        AG_TRY(make_tmap_bf16(&tdy, dyh, 4, dims, strides, box));
    }
    {
        const uint64_t dims[4] = {(uint64_t)cp, (uint64_t)iw, (uint64_t)ih, (uint64_t)bs};
        const uint64_t strides[3] = {(uint64_t)cp, (uint64_t)(iw * cp), (uint64_t)(ih * iw * cp)};
        const uint32_t box[4] = {64, (uint32_t)p.TW, (uint32_t)th, 1};
        AG_TRY(make_tmap_bf16(&tx, xh, 4, dims, strides, box));
    }
    const int grid = splits * base;
    if (nt == 128)
        AG_TRY(launch_wgrad<128>(dev, tdy, tx, p, grid));
    else
        AG_TRY(launch_wgrad<64>(dev, tdy, tx, p, grid));
    const int64_t outs = oc * p.taps * ic;
    wgrad_reduce_kernel<<<(unsigned)ceil_div(outs, 32), dim3(32, 8), 0, dev->stream>>>(
        p.partial, splits, m_total, p.taps, (int)cp, (int)oc, (int)ic, beta, dw);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

}  // namespace convtc
}  // namespace ag
