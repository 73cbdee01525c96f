// bf16 convolution as an implicit GEMM on the Blackwell tensor cores.
//
//   y[b][oc][oy][ox] = sum over (fi, fj, ci) of x[b][ci][oy+fi-ph][ox+fj-pw] * w[oc][ci][fi][fj]
//
// is the product of a [pixels x (fi,fj,ci)] matrix that is never materialised
// with the filter bank.  The activation is first rewritten channels-last
// (NHWC, channels padded to a multiple of 64), so that the 64 channels of one
// pixel are one 128-byte row.  An A tile of the GEMM -- 128 output pixels taken
// as a TH x TW rectangle of one image, 64 channels of one filter tap -- is then
// a single 4-D TMA box of the activation, shifted by the tap: the box lands in
// shared memory in exactly the 128-byte-swizzled K-major layout tcgen05.mma
// reads, padding comes for free from the zero fill of out-of-range
// coordinates, and the k loop walks (tap, channel block).  The filter bank is
// repacked once per call as [oc][fi][fj][ci] and loaded by a 2-D map.
//
// Warp roles are those of the GEMM kernel (gemm_tc.cu): warp 0 issues TMA, warp
// 1 issues tcgen05.mma into one of two TMEM accumulators, warps 2..5 drain the
// other accumulator: bias, ReLU, bf16 rounding and 16-byte stores of channels-last
// rows (a thread owns one pixel, 32 channels are 64 contiguous bytes).  A last
// kernel turns the channels-last result into the caller's NCHW tensor through
// shared memory, again with 16-byte accesses on both sides: scattering 2-byte
// NCHW stores straight from the epilogue cost more than the whole main loop.
//
// The gradient with respect to the input is the same kernel on the transposed
// problem: dy as the activation, zero border F-1-p, filter bank repacked with
// the channel axes swapped and the spatial axes reversed.
#include <cstdlib>

#include "conv_tc.cuh"
#include "tc_ptx.cuh"

namespace ag {
namespace convtc {

using namespace ::ag::tc;

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BLOCK_M * BLOCK_K * 2;
constexpr int NUM_THREADS = 192;

template <int BLOCK_N>
struct Cfg {
    static constexpr int B_TILE_BYTES = BLOCK_N * BLOCK_K * 2;
    static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    static constexpr int STAGES = BLOCK_N <= 128 ? 6 : 4;
    static constexpr int TMEM_COLS = 2 * BLOCK_N;  // 128, 256 or 512
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

struct Params {
    int B, OH, OW, OC, OCp;  // output geometry; OCp = OC rounded up to a multiple of 64
    int TW, tw_shift;        // pixel tile: TH x TW = 128, TW = 1 << tw_shift
    int tiles_y, tiles_x, n_blocks;
    int FH, FW, CB;          // filter taps; channel blocks of 64
    int pad_h, pad_w;
    const __nv_bfloat16 *bias;  // [OC] or null
    int relu;
    __nv_bfloat16 *y;        // channels-last [B][OH][OW][OCp]
    int *status;
};

struct TileCoord {
    int b, oy0, ox0, n_blk;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, const Params &p) {
    TileCoord t;
    t.n_blk = tile % p.n_blocks;
    int r = tile / p.n_blocks;
    const int tx = r % p.tiles_x;
    r /= p.tiles_x;
    const int ty = r % p.tiles_y;
    t.b = r / p.tiles_y;
    t.oy0 = ty * (BLOCK_M >> p.tw_shift);
    t.ox0 = tx * p.TW;
    return t;
}

template <int BLOCK_N>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    conv2_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmap_x,
                         const __grid_constant__ CUtensorMap tmap_w, const Params p) {
    using C = Cfg<BLOCK_N>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + STAGES * A_TILE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * C::STAGE_BYTES);
    uint64_t *full_bar = bars;
    uint64_t *empty_bar = bars + STAGES;
    uint64_t *tmem_full_bar = bars + 2 * STAGES;
    uint64_t *tmem_empty_bar = bars + 2 * STAGES + 2;
    uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_base_slot + 1);
    // bias of this CTA's output channels as f32 (zero where there is none): read from
    // shared memory in the epilogue instead of one global load per element
    __shared__ float s_bias[BLOCK_N];

    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int num_tiles = p.B * p.tiles_y * p.tiles_x * p.n_blocks;
    const int taps = p.FH * p.FW;
    const int num_kb = taps * p.CB;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_x);
        prefetch_tmap(&tmap_w);
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
        tmem_alloc(smem_u32(tmem_base_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    // one output-channel block per CTA keeps its bias resident; with several blocks the
    // epilogue reads the bias from global memory
    const bool bias_resident = p.n_blocks == 1;
    if (bias_resident)
        for (int i = threadIdx.x; i < BLOCK_N; i += NUM_THREADS)
            s_bias[i] = (p.bias != nullptr && i < p.OC) ? __bfloat162float(p.bias[i]) : 0.f;
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
                const TileCoord t = tile_coord(tile, p);
                int fi = 0, fj = 0, cb = 0;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag)) {
                        atomicExch(p.status, 121);
                        ok = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&full_bar[stage]);
                    mbar_arrive_expect_tx(bar, C::STAGE_BYTES);
                    // channels cb*64.., columns ox0+fj-pw.., rows oy0+fi-ph.., image b
                    tma_load_4d(smem_u32(smem_a + stage * A_TILE_BYTES), &tmap_x, bar, cb * BLOCK_K,
                                t.ox0 + fj - p.pad_w, t.oy0 + fi - p.pad_h, t.b);
                    tma_load_2d(smem_u32(smem_b + stage * C::B_TILE_BYTES), &tmap_w, bar,
                                kb * BLOCK_K, t.n_blk * BLOCK_N);
                    if (++cb == p.CB) {
                        cb = 0;
                        if (++fj == p.FW) {
                            fj = 0;
                            ++fi;
                        }
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
            constexpr uint32_t idesc = make_idesc(false, false, BLOCK_M, BLOCK_N);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag)) {
                    atomicExch(p.status, 122);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BLOCK_N);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag)) {
                        atomicExch(p.status, 123);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_base = smem_u32(smem_a + stage * A_TILE_BYTES);
                    const uint32_t b_base = smem_u32(smem_b + stage * C::B_TILE_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t a_desc = make_smem_desc(a_base + k * UMMA_K * 2, 0, 1024);
                        const uint64_t b_desc = make_smem_desc(b_base + k * UMMA_K * 2, 0, 1024);
                        umma_bf16(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&empty_bar[stage]));
                    if (++stage == STAGES) {
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
        const int quarter = warp % 4;  // TMEM lanes this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            const TileCoord t = tile_coord(tile, p);
            if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag)) {
                if (lane == 0) atomicExch(p.status, 124);
                break;
            }
            tc_fence_after();
            const int pix = quarter * 32 + lane;
            const int oy = t.oy0 + (pix >> p.tw_shift);
            const int ox = t.ox0 + (pix & (p.TW - 1));
            const bool valid = oy < p.OH && ox < p.OW;
            const uint32_t taddr =
                tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BLOCK_N);
            // channels-last row of this pixel: 32 channels = 64 contiguous, 16-byte aligned bytes
            __nv_bfloat16 *dst = p.y + (((int64_t)t.b * p.OH + oy) * p.OW + ox) * p.OCp;
#pragma unroll 1
            for (int chunk = 0; chunk < BLOCK_N / 32; ++chunk) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + chunk * 32, r);
                tmem_ld_wait();
                const int oc0 = t.n_blk * BLOCK_N + chunk * 32;
                if (valid && oc0 < p.OCp) {
                    uint32_t packed[16];
                    const bool has_bias = p.bias != nullptr;
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const int oc = oc0 + j;
                        float b0 = 0.f, b1 = 0.f;
                        if (has_bias) {
                            if (bias_resident) {
                                b0 = s_bias[oc];
                                b1 = s_bias[oc + 1];
                            } else {
                                b0 = oc < p.OC ? __bfloat162float(p.bias[oc]) : 0.f;
                                b1 = oc + 1 < p.OC ? __bfloat162float(p.bias[oc + 1]) : 0.f;
                            }
                        }
                        packed[j / 2] = bf16_pair_epilogue(r[j], r[j + 1], b0, b1, has_bias, p.relu != 0);
                    }
                    uint4 *d4 = reinterpret_cast<uint4 *>(dst + oc0);
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        d4[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2],
                                           packed[4 * q + 3]);
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
        // Loads issued before a wait expired may still be landing in shared memory.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------- layout conversions
// x [B][C][H*W] -> out [B][Hp][Wp][Cp] (Cp a multiple of 64, channels >= C are zero), the
// image placed at (pad_h, pad_w) of the Hp x Wp frame (the frame itself is cleared by
// the caller when it is larger than the image).
// A thread owns 16 channels of one pixel: 16 independent 2-byte loads, each
// coalesced across the warp (lanes are consecutive pixels of one channel plane),
// then one full 32-byte sector of the channels-last copy.  No shared memory.
// grid (ceil(HW / 256), Cp / 16, B), 256 threads.
__global__ void __launch_bounds__(256)
    nchw_to_nhwc_kernel(const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ out, int C,
                        int HW, int Cp, int W, int Hp, int Wp, int pad_h, int pad_w) {
    const int px = blockIdx.x * 256 + threadIdx.x;
    if (px >= HW) return;
    const int c0 = blockIdx.y * 16;
    const int b = blockIdx.z;
    const unsigned short *src =
        reinterpret_cast<const unsigned short *>(x) + ((int64_t)b * C + c0) * HW + px;
    unsigned short v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = (c0 + j < C) ? src[(int64_t)j * HW] : (unsigned short)0;
    uint4 lo, hi;
    lo.x = v[0] | ((uint32_t)v[1] << 16);   lo.y = v[2] | ((uint32_t)v[3] << 16);
    lo.z = v[4] | ((uint32_t)v[5] << 16);   lo.w = v[6] | ((uint32_t)v[7] << 16);
    hi.x = v[8] | ((uint32_t)v[9] << 16);   hi.y = v[10] | ((uint32_t)v[11] << 16);
    hi.z = v[12] | ((uint32_t)v[13] << 16); hi.w = v[14] | ((uint32_t)v[15] << 16);
    const int yy = px / W, xx = px - yy * W;
    const int64_t row = ((int64_t)b * Hp + yy + pad_h) * Wp + xx + pad_w;
    uint4 *dst = reinterpret_cast<uint4 *>(out + row * Cp + c0);
    dst[0] = lo;
    dst[1] = hi;
}

// in [B][HW][Cp] -> out [B][C][HW].  A CTA takes 16 channels of up to 1024 pixels
// of one image: 32-byte loads (lanes are consecutive pixels), a transposed copy
// in shared memory whose rows start at the same offset modulo 8 elements as the
// runs they are written to, then 16-byte stores of whole runs (2-byte stores only
// at ragged ends).  grid (ceil(HW / 1024), ceil(C / 16), B), 256 threads.
constexpr int NCHW_PIX = 1024;
constexpr int NCHW_PITCH = NCHW_PIX + 16;
__global__ void __launch_bounds__(256)
    nhwc_to_nchw_kernel(const __nv_bfloat16 *__restrict__ in, __nv_bfloat16 *__restrict__ out, int C,
                        int HW, int Cp) {
    __shared__ __align__(16) unsigned short tile[16 * NCHW_PITCH];
    const int p0 = blockIdx.x * NCHW_PIX;
    const int c0 = blockIdx.y * 16;
    const int b = blockIdx.z;
    const int np = min(NCHW_PIX, HW - p0);
    const int nc = min(16, C - c0);
    // a staged row starts at the same offset modulo 8 elements (16 bytes) as its run in out
    const int64_t run0 = ((int64_t)b * C + c0) * HW + p0;
    for (int px = threadIdx.x; px < np; px += 256) {
        const uint4 *src =
            reinterpret_cast<const uint4 *>(in + ((int64_t)b * HW + p0 + px) * Cp + c0);
        const uint4 lo = src[0], hi = src[1];
        const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int off = (int)((reinterpret_cast<uintptr_t>(out + run0 + (int64_t)j * HW) >> 1) & 7);
            tile[j * NCHW_PITCH + off + px] =
                (unsigned short)((j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xffffu));
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int j = warp; j < nc; j += 8) {
        const int64_t start = run0 + (int64_t)j * HW;  // element index of the run in out
        const int off = (int)((reinterpret_cast<uintptr_t>(out + start) >> 1) & 7);
        const unsigned short *row = tile + j * NCHW_PITCH;   // row[off + i] = element i of the run
        unsigned short *dst = reinterpret_cast<unsigned short *>(out) + start;
        const int head = min(np, (8 - off) & 7);
        const int nvec = (np - head) / 8;
        if (lane < head) dst[lane] = row[off + lane];
        for (int v = lane; v < nvec; v += 32)
            *reinterpret_cast<uint4 *>(dst + head + v * 8) =
                *reinterpret_cast<const uint4 *>(row + off + head + v * 8);
        const int tail0 = head + nvec * 8;
        if (tail0 + lane < np) dst[tail0 + lane] = row[off + tail0 + lane];
    }
}

// Filter bank for the forward pass: w [OC][IC][FH][FW] -> wk [OC][FH][FW][Cp].
__global__ void repack_filters_kernel(const __nv_bfloat16 *__restrict__ w,
                                      __nv_bfloat16 *__restrict__ wk, int OC, int IC, int taps,
                                      int Cp) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)OC * taps * Cp) return;
    const int c = (int)(i % Cp);
    const int tap = (int)((i / Cp) % taps);
    const int oc = (int)(i / ((int64_t)Cp * taps));
    wk[i] = c < IC ? w[((int64_t)oc * IC + c) * taps + tap] : __float2bfloat16_rn(0.f);
}

// Filter bank for the input gradient: w [OC][IC][FH][FW] -> wk [IC][FH][FW][OCp] with
// both spatial axes reversed.
__global__ void repack_filters_transposed_kernel(const __nv_bfloat16 *__restrict__ w,
                                                 __nv_bfloat16 *__restrict__ wk, int OC, int IC,
                                                 int taps, int OCp) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)IC * taps * OCp) return;
    const int oc = (int)(i % OCp);
    const int tap = (int)((i / OCp) % taps);
    const int ic = (int)(i / ((int64_t)OCp * taps));
    wk[i] = oc < OC ? w[((int64_t)oc * IC + ic) * taps + (taps - 1 - tap)]
                    : __float2bfloat16_rn(0.f);
}

// ------------------------------------------------------------------ host side
bool tc_conv_enabled() {
    static int v = []() {
        const char *a = getenv("AG_TC");
        const char *c = getenv("AG_CONV_TC");
        return ((a && a[0] == '0') || (c && c[0] == '0')) ? 0 : 1;
    }();
    return v != 0;
}

static int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

static bool halo_enabled() {
    static int v = []() {
        const char *e = getenv("AG_CONV_HALO");
        return (e && e[0] == '0') ? 0 : 1;
    }();
    return v != 0;
}

int to_nhwc(ag_device *dev, const __nv_bfloat16 *x, int64_t bs, int64_t c, int64_t hw, int64_t cp,
            __nv_bfloat16 *out) {
    // no border: the frame is the image, any width gives the same row index
    nchw_to_nhwc_kernel<<<dim3((unsigned)ceil_div(hw, 256), (unsigned)(cp / 16), (unsigned)bs), 256,
                          0, dev->stream>>>(x, out, (int)c, (int)hw, (int)cp, (int)hw, 1, (int)hw, 0,
                                            0);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

int to_nhwc_framed(ag_device *dev, const __nv_bfloat16 *x, int64_t bs, int64_t c, int64_t h,
                   int64_t w, int64_t cp, int pad_h, int pad_w, __nv_bfloat16 *out) {
    const int64_t hp = h + 2 * pad_h, wp = w + 2 * pad_w;
    if (pad_h || pad_w)
        AG_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)(bs * hp * wp * cp * 2), dev->stream));
    nchw_to_nhwc_kernel<<<dim3((unsigned)ceil_div(h * w, 256), (unsigned)(cp / 16), (unsigned)bs),
                          256, 0, dev->stream>>>(x, out, (int)c, (int)(h * w), (int)cp, (int)w,
                                                 (int)hp, (int)wp, pad_h, pad_w);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

// Shared test for both directions, in the kernel's view: `c_in` channels of
// in_h x in_w are correlated into `c_out` channels of out_h x out_w.
static bool shape_ok(int64_t bs, int64_t c_in, int64_t in_h, int64_t in_w, int64_t c_out,
                     int64_t out_h, int64_t out_w, int fh, int fw) {
    if (!tc_conv_enabled() || encode_tiled_fn() == nullptr) return false;
    if (bs <= 0 || c_in < 16 || c_out < 32 || out_h <= 0 || out_w <= 0) return false;
    if (fh < 1 || fw < 1 || fh * fw > 49) return false;
    if (bs * out_h * out_w < 4096) return false;  // too little work for 128-pixel tiles
    if (in_h > 32768 || in_w > 32768 || bs > 65535) return false;
    const int64_t cp = round_up(c_in, 64);
    if (bs * in_h * in_w * cp >= (int64_t(1) << 40)) return false;
    if (c_out * (int64_t)fh * fw * cp >= (int64_t(1) << 31)) return false;
    return true;
}

bool eligible_forward(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
                      const ag_conv2_options *o) {
    if (o->stride[0] != 1 || o->stride[1] != 1 || o->dilation[0] != 1 || o->dilation[1] != 1)
        return false;
    const int64_t oh = ih + 2 * o->padding[0] - o->filter[0] + 1;
    const int64_t ow = iw + 2 * o->padding[1] - o->filter[1] + 1;
    return shape_ok(bs, ic, ih, iw, oc, oh, ow, o->filter[0], o->filter[1]);
}

bool eligible_backward_input(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
                             const ag_conv2_options *o) {
    if (o->stride[0] != 1 || o->stride[1] != 1 || o->dilation[0] != 1 || o->dilation[1] != 1)
        return false;
    if (o->padding[0] > o->filter[0] - 1 || o->padding[1] > o->filter[1] - 1) return false;
    const int64_t oh = ih + 2 * o->padding[0] - o->filter[0] + 1;
    const int64_t ow = iw + 2 * o->padding[1] - o->filter[1] + 1;
    return shape_ok(bs, oc, oh, ow, ic, ih, iw, o->filter[0], o->filter[1]);
}

template <int BLOCK_N>
static int launch(ag_device *dev, const CUtensorMap &tx, const CUtensorMap &tw, const Params &p) {
    using C = Cfg<BLOCK_N>;
    auto kernel = conv2_bf16_tc_kernel<BLOCK_N>;
    // the attribute belongs to the (kernel, GPU) pair: remembered per instantiation and GPU
    static bool configured_on[64] = {};
    bool &configured = configured_on[dev->ordinal & 63];
    if (!configured) {
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES));
        configured = true;
    }
    const int64_t tiles = (int64_t)p.B * p.tiles_y * p.tiles_x * p.n_blocks;
    const int grid = (int)(tiles < dev->sm_count ? tiles : dev->sm_count);
    kernel<<<grid, NUM_THREADS, C::SMEM_BYTES, dev->stream>>>(tx, tw, p);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

bool nhwc_wants_frame(const NhwcConv &c) {
    const int64_t cp = round_up(c.c_in, 64);
    int n = 0, rows = 0, stages = 0, smem = 0;
    return halo_enabled() && halo_plan(c.bs, cp, c.in_h + 2 * c.pad_h, c.in_w + 2 * c.pad_w, c.c_out,
                                       c.fh, c.fw, &n, &rows, &stages, &smem);
}

int64_t nhwc_filter_scratch_bytes(const NhwcConv &c) {
    return round_up(c.c_out * (int64_t)c.fh * c.fw * round_up(c.c_in, 64) * 2, 1024);
}

int from_nhwc(ag_device *dev, const __nv_bfloat16 *in, int64_t bs, int64_t c, int64_t hw, int64_t cp,
              __nv_bfloat16 *out) {
    nhwc_to_nchw_kernel<<<dim3((unsigned)ceil_div(hw, NCHW_PIX), (unsigned)ceil_div(c, 16), (unsigned)bs),
                          256, 0, dev->stream>>>(in, out, (int)c, (int)hw, (int)cp);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

// The tensor-core correlation on channels-last data.  `act` is [bs][in_h][in_w][cp], or, when
// `framed` (required when nhwc_wants_frame says so, not allowed otherwise), the same inside a
// zero frame of pad_h rows / pad_w columns; `out` is [bs][out_h * out_w][ocp]; `wk` is scratch of
// nhwc_filter_scratch_bytes for the repacked filter bank.
int correlate_nhwc(ag_device *dev, const NhwcConv &c, const __nv_bfloat16 *act_nhwc, bool framed,
                   const __nv_bfloat16 *w, int64_t w_oc, int64_t w_ic, const __nv_bfloat16 *bias,
                   bool relu, __nv_bfloat16 *wk, __nv_bfloat16 *out_nhwc) {
    const int64_t bs = c.bs, in_h = c.in_h, in_w = c.in_w, c_out = c.c_out, out_h = c.out_h,
                  out_w = c.out_w;
    const int fh = c.fh, fw = c.fw, pad_h = c.pad_h, pad_w = c.pad_w;
    const int64_t cp = round_up(c.c_in, 64);
    const int taps = fh * fw;
    const int64_t hp = in_h + 2 * pad_h, wp = in_w + 2 * pad_w;
    const bool halo = nhwc_wants_frame(c);
    AG_REQUIRE(halo == framed, AG_ERR_INVALID, "conv: activation frame does not match the kernel's plan");
    const int64_t wk_elems = c_out * taps * cp;
    const int64_t ocp = round_up(c_out, 64);
    const unsigned rgrid = (unsigned)ceil_div(wk_elems, 256);
    if (c.transposed)
        repack_filters_transposed_kernel<<<rgrid, 256, 0, dev->stream>>>(w, wk, (int)w_oc, (int)w_ic,
                                                                         taps, (int)cp);
    else
        repack_filters_kernel<<<rgrid, 256, 0, dev->stream>>>(w, wk, (int)w_oc, (int)w_ic, taps,
                                                              (int)cp);
    AG_CHECK_LAUNCH();
    if (halo)
        return run_halo(dev, act_nhwc, wk, bs, cp, hp, wp, fh, fw, c_out, out_h, out_w, bias, relu,
                        out_nhwc);

    // Pixel tile: the TH x TW rectangle (TH * TW = 128) that wastes the fewest pixels.
    int best_shift = 3;
    int64_t best_cover = -1;
    for (int shift = 3; shift <= 7; ++shift) {
        const int64_t tw = 1 << shift, th = BLOCK_M / tw;
        const int64_t cover = round_up(out_w, tw) * round_up(out_h, th);
        if (best_cover < 0 || cover <= best_cover) {  // ties: the wider tile (longer store runs)
            best_cover = cover;
            best_shift = shift;
        }
    }
    Params p;
    p.B = (int)bs; p.OH = (int)out_h; p.OW = (int)out_w; p.OC = (int)c_out;
    p.OCp = (int)ocp;
    p.tw_shift = best_shift;
    p.TW = 1 << best_shift;
    const int th = BLOCK_M / p.TW;
    p.tiles_y = (int)ceil_div(out_h, th);
    p.tiles_x = (int)ceil_div(out_w, p.TW);
    p.FH = fh; p.FW = fw;
    p.CB = (int)(cp / 64);
    p.pad_h = pad_h; p.pad_w = pad_w;
    p.bias = bias;
    p.relu = relu ? 1 : 0;
    p.y = out_nhwc;
    p.status = dev->status_dev;
    const int block_n = c_out <= 64 ? 64 : (c_out <= 128 ? 128 : 256);
    p.n_blocks = (int)ceil_div(c_out, block_n);

    CUtensorMap tx, tw;
    {
        const uint64_t dims[4] = {(uint64_t)cp, (uint64_t)in_w, (uint64_t)in_h, (uint64_t)bs};
        const uint64_t strides[3] = {(uint64_t)cp, (uint64_t)(in_w * cp), (uint64_t)(in_h * in_w * cp)};
        const uint32_t box[4] = {64, (uint32_t)p.TW, (uint32_t)th, 1};
        AG_TRY(make_tmap_bf16(&tx, act_nhwc, 4, dims, strides, box));
    }
    {
        const uint64_t k = (uint64_t)taps * (uint64_t)cp;
        const uint64_t dims[2] = {k, (uint64_t)c_out};
        const uint64_t strides[1] = {k};
        const uint32_t box[2] = {64, (uint32_t)block_n};
        AG_TRY(make_tmap_bf16(&tw, wk, 2, dims, strides, box));
    }
    if (block_n == 64)
        AG_TRY(launch<64>(dev, tx, tw, p));
    else if (block_n == 128)
        AG_TRY(launch<128>(dev, tx, tw, p));
    else
        AG_TRY(launch<256>(dev, tx, tw, p));
    return AG_OK;
}

// The common path of the NCHW entry points.  `act` is the NCHW activation [bs][c_in][in_h][in_w];
// the output is NCHW [bs][c_out][out_h][out_w]; `transposed` selects the filter repacking of the
// input gradient.
static int run(ag_device *dev, const __nv_bfloat16 *act, int64_t bs, int64_t c_in, int64_t in_h,
               int64_t in_w, const __nv_bfloat16 *w, int64_t w_oc, int64_t w_ic, int fh, int fw,
               int pad_h, int pad_w, bool transposed, int64_t c_out, int64_t out_h, int64_t out_w,
               const __nv_bfloat16 *bias, bool relu, __nv_bfloat16 *y) {
    NhwcConv c;
    c.bs = bs; c.c_in = c_in; c.in_h = in_h; c.in_w = in_w;
    c.c_out = c_out; c.out_h = out_h; c.out_w = out_w;
    c.fh = fh; c.fw = fw; c.pad_h = pad_h; c.pad_w = pad_w;
    c.transposed = transposed;
    const int64_t cp = round_up(c_in, 64);
    const int64_t hp = in_h + 2 * pad_h, wp = in_w + 2 * pad_w;
    const bool halo = nhwc_wants_frame(c);
    const int64_t act_bytes =
        round_up((halo ? bs * hp * wp : bs * in_h * in_w) * cp * 2, 1024);
    const int64_t wk_bytes = nhwc_filter_scratch_bytes(c);
    const int64_t ocp = round_up(c_out, 64);
    const int64_t out_bytes = bs * out_h * out_w * ocp * 2;
    void *ws = nullptr;
    AG_TRY(staging(dev, (size_t)(act_bytes + wk_bytes + out_bytes), &ws));
    __nv_bfloat16 *act_nhwc = (__nv_bfloat16 *)ws;
    __nv_bfloat16 *wk = (__nv_bfloat16 *)((char *)ws + act_bytes);
    __nv_bfloat16 *out_nhwc = (__nv_bfloat16 *)((char *)ws + act_bytes + wk_bytes);
    if (halo)
        AG_TRY(to_nhwc_framed(dev, act, bs, c_in, in_h, in_w, cp, pad_h, pad_w, act_nhwc));
    else
        AG_TRY(to_nhwc(dev, act, bs, c_in, in_h * in_w, cp, act_nhwc));
    AG_TRY(correlate_nhwc(dev, c, act_nhwc, halo, w, w_oc, w_ic, bias, relu, wk, out_nhwc));
    return from_nhwc(dev, out_nhwc, bs, c_out, out_h * out_w, ocp, y);
}

int forward(ag_device *dev, const __nv_bfloat16 *x, int64_t bs, int64_t ic, int64_t ih, int64_t iw,
            const __nv_bfloat16 *w, int64_t oc, const __nv_bfloat16 *bias,
            const ag_conv2_options *o, bool relu, __nv_bfloat16 *y) {
    const int fh = o->filter[0], fw = o->filter[1];
    const int64_t oh = ih + 2 * o->padding[0] - fh + 1, ow = iw + 2 * o->padding[1] - fw + 1;
    return run(dev, x, bs, ic, ih, iw, w, oc, ic, fh, fw, o->padding[0], o->padding[1], false, oc,
               oh, ow, bias, relu, y);
}

int backward_input(ag_device *dev, const __nv_bfloat16 *w, int64_t oc, int64_t ic,
                   const __nv_bfloat16 *dy, int64_t bs, int64_t ih, int64_t iw,
                   const ag_conv2_options *o, __nv_bfloat16 *dx) {
    const int fh = o->filter[0], fw = o->filter[1];
    const int64_t oh = ih + 2 * o->padding[0] - fh + 1, ow = iw + 2 * o->padding[1] - fw + 1;
    return run(dev, dy, bs, oc, oh, ow, w, oc, ic, fh, fw, fh - 1 - o->padding[0],
               fw - 1 - o->padding[1], true, ic, ih, iw, nullptr, false, dx);
}

}  // namespace convtc
}  // namespace ag
