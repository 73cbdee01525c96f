// bf16 variant of the LeNet5-geometry whole-network kernel (conv_chain_lenet.cuh) whose second
// convolution, 54 % of the network's multiply-adds, runs on the tensor cores (tcgen05.mma, f32
// accumulators in tensor memory).
//
// No im2col matrix is built.  The pooled output of conv1 is kept channels-last in shared
// memory, one 32-byte row per pixel (6 channels + 10 zeros = one K step of 16 bf16), image
// after image: row = image * 144 + y * 12 + x.  For filter tap (fi, fj) the A operand of the
// product "pixels x channels" is that same matrix moved down fi * 12 + fj rows, so each of the
// 25 taps is ONE tcgen05.mma (M = 128 pixel rows, N = 16 output channels, K = 16) whose
// shared-memory descriptor starts fi * 12 + fj rows further on; the 25 MMAs of a tile
// accumulate in tensor memory.  Rows whose window would leave the 12 x 12 plane (x > 7 or
// y > 7) compute values nobody reads: 36 % of the MMA work, which costs nothing next to the
// im2col traffic it replaces.  Operands use the 32-byte swizzle (address bit 4 ^= bit 7), which
// the SM applies when it writes the rows and the tensor core undoes when it reads them; it is
// a function of the absolute shared-memory address, so a descriptor may start at any row.
//
// K = 16 per tap with 6 channels in use wastes 62 % of each MMA as well; the tensor core is
// still ~7 times faster here than the FFMA pipe (measured), and operands that are written by
// the SM need no TMA (whose 16-byte rules the 150-wide rows of an im2col matrix break).
//
// conv1 (one input channel: nothing for a tensor core to contract over) and the dense chain
// run as in the f32 kernel.  The f32 sums of conv2 are added in the tensor core's order, so
// the logits equal the layer-by-layer kernels within bf16 rounding, not bit for bit.
// Waits on the MMA-completion barriers and on the weight copy are bounded (status 172 / 170).
#pragma once

#include "conv_chain_lenet.cuh"

namespace ag {
namespace conv_chain {
namespace lenet_tc {

using dense_small::ROWS;
using namespace lenet;   // geometry constants, bulk_g2s, round_t
// this kernel's first convolution keeps the [channel triple 2][tap 25][4] filter layout
constexpr int W1_TRIPLE = F * F * 4;         // 100
constexpr int W1_TC_FLOATS = 2 * W1_TRIPLE;  // 200

constexpr int TILES = (kGroup * P1 * P1 + 127) / 128;   // 8 tiles of 128 pixel rows
constexpr int ACT_ROWS = TILES * 128 + 64;          // rows a tile plus the largest tap shift (52) can reach
constexpr int ACT_BYTES = ACT_ROWS * 32;
constexpr int W2B_BYTES = F * F * 16 * 32;          // per tap: 16 output channels x 32 bytes
constexpr int C2_BYTES = TILES * 128 * 32;          // conv2 + relu, bf16, [pixel row][16 channels]
constexpr int TMEM_COLS = 128;                      // 8 tiles x 16 columns

struct Plan {
    int bs, group;
    const void *w1, *w2;
    dense_small::ChainParams chain;
    int w_smem[dense_small::kMaxChain];   // byte offset of the layer's weights in shared memory, or -1
    int w_bytes[dense_small::kMaxChain];
    int in_off, act_off, w2b_off, c2_off, w1_off, xa_off, xb_off, red_off, bar_off;   // bytes
    int *status;
};

// 32-byte swizzle on an absolute shared-memory address.
__device__ __forceinline__ uint32_t swz32(uint32_t addr) { return addr ^ (((addr >> 7) & 1u) << 4); }

__device__ __forceinline__ uint64_t make_desc_sw32(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(256u >> 4) << 32;   // stride between groups of 8 rows
    d |= 1ull << 46;                    // descriptor version
    d |= 6ull << 61;                    // SWIZZLE_32B
    return d;
}

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
    lenet_chain_tc_kernel(const __nv_bfloat16 *__restrict__ x, const uint8_t *__restrict__ x8, float alpha,
                          __nv_bfloat16 *__restrict__ y, const Plan pl) {
    using T = __nv_bfloat16;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ int s_abort;
    __shared__ uint32_t s_tmem;
    // the operand buffers want 1 KiB alignment of their absolute addresses
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b0 = blockIdx.x * pl.group;
    const int nimg = min(pl.group, pl.bs - b0);
    float *s_in = reinterpret_cast<float *>(smem + pl.in_off);
    uint8_t *s_act = smem + pl.act_off, *s_w2b = smem + pl.w2b_off, *s_c2 = smem + pl.c2_off;
    float *s_w1 = reinterpret_cast<float *>(smem + pl.w1_off);
    float *xa = reinterpret_cast<float *>(smem + pl.xa_off), *xb = reinterpret_cast<float *>(smem + pl.xb_off);
    const uint32_t bar_w = tc::smem_u32(smem + pl.bar_off);   // weight copy
    const uint32_t bar_tile0 = bar_w + 8;                      // [TILES] MMA completion
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    AG_STAMP(0);

    if (tid == kThreads - 1) {
        s_abort = 0;
        tc::mbar_init(bar_w, 1);
        for (int t = 0; t < TILES; ++t) tc::mbar_init(bar_tile0 + 8 * t, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        uint32_t bytes = 0;
        for (int l = 0; l < pl.chain.n_layers; ++l)
            if (pl.w_smem[l] >= 0) bytes += (uint32_t)pl.w_bytes[l];
        if (bytes) {
            tc::mbar_arrive_expect_tx(bar_w, bytes);
            for (int l = 0; l < pl.chain.n_layers; ++l)
                if (pl.w_smem[l] >= 0)
                    bulk_g2s(tc::smem_u32(smem + pl.w_smem[l]), pl.chain.s[l].w, (uint32_t)pl.w_bytes[l], bar_w);
        }
    }
    if (warp == 0) {   // tensor memory for the eight accumulators
        tc::tmem_alloc(tc::smem_u32(&s_tmem), TMEM_COLS);
        tc::tmem_relinquish();
    }

    // ---- images, conv1 filter bank; zeroed operand buffers; conv2 filter bank as B operands
    if (x8 != nullptr) {
        const float a = round_t<T>(alpha);
        const uint8_t *src = x8 + (int64_t)b0 * (IH * IW);
        const int total = nimg * IH * IW;
        const int nvec = (reinterpret_cast<uintptr_t>(src) & 3) == 0 ? total / 4 : 0;
        for (int i = tid; i < nvec; i += kThreads) {
            const uint32_t q = reinterpret_cast<const uint32_t *>(src)[i];
            float4 v;
            v.x = round_t<T>(a * (float)(q & 0xffu));
            v.y = round_t<T>(a * (float)((q >> 8) & 0xffu));
            v.z = round_t<T>(a * (float)((q >> 16) & 0xffu));
            v.w = round_t<T>(a * (float)(q >> 24));
            reinterpret_cast<float4 *>(s_in)[i] = v;
        }
        for (int i = nvec * 4 + tid; i < total; i += kThreads) s_in[i] = round_t<T>(a * (float)src[i]);
    } else {
        direct::stage_contiguous<T>(x + (int64_t)b0 * (IH * IW), s_in, nimg * IH * IW);
    }
    {
        const T *w1 = reinterpret_cast<const T *>(pl.w1);
        for (int i = tid; i < W1_TC_FLOATS; i += kThreads) {
            const int triple = i / W1_TRIPLE, r = i - triple * W1_TRIPLE;
            const int tap = r >> 2, o = r & 3;
            s_w1[i] = o < 3 ? to_f32(w1[(triple * 3 + o) * (F * F) + tap]) : 0.f;
        }
        for (int i = tid; i < (ACT_BYTES + W2B_BYTES) / 16; i += kThreads)   // act and w2b are adjacent
            reinterpret_cast<uint4 *>(s_act)[i] = make_uint4(0, 0, 0, 0);
    }
    if (nimg < ROWS)
        for (int i = tid; i < kFlat * ROWS; i += kThreads) xa[i] = 0.f;
    __syncthreads();
    {
        // B operand of tap (fi, fj): row = output channel, 16 bf16 = input channels (6 in use)
        const unsigned short *w2 = reinterpret_cast<const unsigned short *>(pl.w2);
        const uint32_t w2b_addr = tc::smem_u32(s_w2b);
        for (int i = tid; i < C2 * C1 * F * F; i += kThreads) {
            const int oc = i / (C1 * F * F), r = i - oc * (C1 * F * F);
            const int ci = r / (F * F), tap = r - ci * (F * F);
            const uint32_t a = swz32(w2b_addr + tap * 512 + oc * 32 + ci * 2);
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "h"(w2[i]) : "memory");
        }
    }
    AG_STAMP(1);

    // ---- conv1 + relu + pool on the FFMA pipe; the pooled values go to the channels-last
    //      operand buffer as bf16
    if (tid < nimg * 72) {
        const int g = tid / 72, r = tid - g * 72;
        const int triple = r & 1, blk = r >> 1;
        const int by = blk / 3, bx = blk - by * 3;
        const float *img = s_in + g * (IH * IW) + (2 * by) * IW + 8 * bx;
        const float *wt = s_w1 + triple * W1_TRIPLE;
        float acc[2][8][3];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < 8; ++b) acc[a][b][0] = acc[a][b][1] = acc[a][b][2] = 0.f;
        float wprev[F][3];
#pragma unroll
        for (int pr = 0; pr < F + 1; ++pr) {
            float p[12];
#pragma unroll
            for (int q = 0; q < 3; ++q)
                *reinterpret_cast<float4 *>(p + 4 * q) =
                    *reinterpret_cast<const float4 *>(img + pr * IW + 4 * q);
            float wcur[F][3];
#pragma unroll
            for (int fj = 0; fj < F; ++fj) {
                if (pr < F) {
                    const float4 w4 = *reinterpret_cast<const float4 *>(wt + (pr * F + fj) * 4);
                    wcur[fj][0] = w4.x; wcur[fj][1] = w4.y; wcur[fj][2] = w4.z;
#pragma unroll
                    for (int b = 0; b < 8; ++b)
#pragma unroll
                        for (int o = 0; o < 3; ++o)
                            acc[0][b][o] = fmaf(p[fj + b], wcur[fj][o], acc[0][b][o]);
                }
                if (pr >= 1) {
#pragma unroll
                    for (int b = 0; b < 8; ++b)
#pragma unroll
                        for (int o = 0; o < 3; ++o)
                            acc[1][b][o] = fmaf(p[fj + b], wprev[fj][o], acc[1][b][o]);
                }
            }
            if (pr < F) {
#pragma unroll
                for (int fj = 0; fj < F; ++fj)
#pragma unroll
                    for (int o = 0; o < 3; ++o) wprev[fj][o] = wcur[fj][o];
            }
        }
        const uint32_t act_addr = tc::smem_u32(s_act);
#pragma unroll
        for (int wx = 0; wx < 4; ++wx) {
            const uint32_t row = (uint32_t)(g * (P1 * P1) + by * P1 + 4 * bx + wx);
#pragma unroll
            for (int o = 0; o < 3; ++o) {
                float v00 = round_t<T>(acc[0][2 * wx][o]), v01 = round_t<T>(acc[0][2 * wx + 1][o]);
                float v10 = round_t<T>(acc[1][2 * wx][o]), v11 = round_t<T>(acc[1][2 * wx + 1][o]);
                v00 = v00 >= 0.f ? v00 : 0.f; v01 = v01 >= 0.f ? v01 : 0.f;
                v10 = v10 >= 0.f ? v10 : 0.f; v11 = v11 >= 0.f ? v11 : 0.f;
                float mm = v00;
                if (v01 > mm) mm = v01;
                if (v10 > mm) mm = v10;
                if (v11 > mm) mm = v11;
                const __nv_bfloat16 h = __float2bfloat16_rn(mm);   // exact: mm is a bf16 value
                const uint32_t a = swz32(act_addr + row * 32 + (triple * 3 + o) * 2);
                asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "h"(*reinterpret_cast<const unsigned short *>(&h))
                             : "memory");
            }
        }
    }
    // the operands were written through the generic proxy; the tensor core reads them through
    // the async proxy
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    AG_STAMP(2);

    // ---- conv2 on the tensor cores: per tile of 128 pixel rows, 25 MMAs (one per tap)
    const uint32_t tmem = s_tmem;
    const int tiles = (nimg * (P1 * P1) + 127) / 128;
    if (tid == 0) {
        const uint32_t act_addr = tc::smem_u32(s_act), w2b_addr = tc::smem_u32(s_w2b);
        const uint32_t idesc = tc::make_idesc(false, false, 128, 16);
        // Tap by tap across the tiles: consecutive MMAs go to different accumulators, so they
        // pipeline; 25 MMAs into ONE accumulator run one after the other (measured: 13 us
        // against 2 us for the phase).
#pragma unroll 1
        for (int tap = 0; tap < F * F; ++tap) {
            const int fi = tap / F, fj = tap - fi * F;
            const uint64_t b_desc = make_desc_sw32(w2b_addr + (uint32_t)tap * 512);
            for (int t = 0; t < tiles; ++t) {
                const uint64_t a_desc = make_desc_sw32(act_addr + (uint32_t)(t * 128 + fi * P1 + fj) * 32);
                tc::umma_bf16(tmem + (uint32_t)(t * 16), a_desc, b_desc, idesc, tap > 0 ? 1u : 0u);
            }
        }
        for (int t = 0; t < tiles; ++t) tc::umma_commit(bar_tile0 + 8 * t);
    }
    // epilogue: warp group (t % 4) takes tile t; a thread owns one pixel row of the tile
    {
        const int group4 = warp >> 2, quarter = warp & 3;
        for (int t = group4; t < tiles; t += 4) {
            if (!tc::mbar_wait(bar_tile0 + 8 * t, 0, &s_abort)) {
                if (lane == 0) atomicCAS(pl.status, 0, 172);
                break;
            }
            tc::tc_fence_after();
            uint32_t r[16];
            tmem_ld_32x16(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(t * 16), r);
            tc::tmem_ld_wait();
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                o[j] = tc::bf16_pair_epilogue(r[2 * j], r[2 * j + 1], 0.f, 0.f, false, true);
            uint4 *dst = reinterpret_cast<uint4 *>(s_c2 + (size_t)(t * 128 + quarter * 32 + lane) * 32);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (s_abort) {
        if (warp == 0) tc::tmem_dealloc(tmem, TMEM_COLS);
        return;
    }
    // 2x2 pool of relu(conv2) into the dense chain's input [k][ROWS], k = (c, py, px)
    for (int i = tid; i < nimg * kFlat; i += kThreads) {
        const int g = i >> 8, k = i & 255;
        const int oc = k >> 4, py = (k >> 2) & 3, px = k & 3;
        const unsigned short *base = reinterpret_cast<const unsigned short *>(s_c2) +
                                     (size_t)(g * (P1 * P1) + (2 * py) * P1 + 2 * px) * 16 + oc;
        const float v00 = __uint_as_float((uint32_t)base[0] << 16), v01 = __uint_as_float((uint32_t)base[16] << 16);
        const float v10 = __uint_as_float((uint32_t)base[P1 * 16] << 16);
        const float v11 = __uint_as_float((uint32_t)base[P1 * 16 + 16] << 16);
        float mm = v00;
        if (v01 > mm) mm = v01;
        if (v10 > mm) mm = v10;
        if (v11 > mm) mm = v11;
        xa[k * ROWS + g] = mm;
    }
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem, TMEM_COLS);
    AG_STAMP(3);

    // ---- dense chain (FFMA pipe), weights from shared memory
    float *red = reinterpret_cast<float *>(smem + pl.red_off);
    bool waited = false;
    for (int l = 0; l < pl.chain.n_layers; ++l) {
        const T *w = reinterpret_cast<const T *>(pl.chain.s[l].w);
        const bool last = l + 1 == pl.chain.n_layers;
        if (l == 0) AG_STAMP(4);
        if (pl.w_smem[l] >= 0) {
            if (!waited) {
                if (!tc::mbar_wait(bar_w, 0, &s_abort)) {
                    if (tid == 0) atomicCAS(pl.status, 0, 170);
                    return;
                }
                waited = true;
            }
            dense_small::chain_layer<T, true, true>(pl.chain.s[l], reinterpret_cast<const T *>(smem + pl.w_smem[l]),
                                                    xa, xb, red, b0, nimg, last, y);
        } else {
            dense_small::chain_layer<T, true, false>(pl.chain.s[l], w, xa, xb, red, b0, nimg, last, y);
        }
        if (l < 2) AG_STAMP(5 + l);
        float *t = xa;
        xa = xb;
        xb = t;
    }
    AG_STAMP(7);
}

// Plan for a bf16 network of LeNet5's geometry; returns the dynamic shared memory in bytes or 0.
inline size_t make_plan(Plan *pl, int64_t bs, int64_t ic, int64_t ih, int64_t iw, int n_conv,
                        const ag_conv_stage *stages, int n_dense, const dense_small::ChainLayer *layers) {
    lenet::Plan base;   // reuse the geometry checks
    if (lenet::make_plan(&base, AG_BF16, bs, ic, ih, iw, n_conv, stages, n_dense, layers) == 0) return 0;
    pl->bs = (int)bs;
    pl->w1 = stages[0].w;
    pl->w2 = stages[1].w;
    if ((reinterpret_cast<uintptr_t>(pl->w2) & 1) != 0) return 0;
    pl->chain = base.chain;
    int off = 0;
    auto take = [&](int bytes, int align) {
        off = (off + align - 1) / align * align;
        const int at = off;
        off += bytes;
        return at;
    };
    pl->act_off = take(ACT_BYTES, 1024);
    pl->w2b_off = take(W2B_BYTES, 256);    // directly behind act (ACT_BYTES is a multiple of 256)
    if (pl->w2b_off != pl->act_off + ACT_BYTES) return 0;
    pl->c2_off = take(C2_BYTES, 128);
    pl->red_off = pl->c2_off;               // red overlays the conv2 output (dead after the pool)
    if (pl->chain.red_floats * 4 > C2_BYTES) return 0;
    pl->in_off = take(kGroup * IH * IW * 4, 16);
    pl->w1_off = take(W1_TC_FLOATS * 4, 16);
    pl->xa_off = take(kFlat * ROWS * 4, 16);
    pl->xb_off = take(kFlat * ROWS * 4, 16);
    pl->bar_off = take(8 * (1 + TILES), 16);
    constexpr int kBudget = 227 * 1024 - 64 - 1024;   // static words and the alignment slack
    for (int l = 0; l < n_dense; ++l) {
        pl->w_smem[l] = -1;
        const int64_t bytes = (int64_t)layers[l].inputs * layers[l].outputs * 2;
        pl->w_bytes[l] = (int)bytes;
        const bool copyable = (reinterpret_cast<uintptr_t>(layers[l].w) & 15) == 0 && bytes % 16 == 0 &&
                              bytes < (1 << 20);
        if (copyable && off + bytes + 16 <= kBudget) pl->w_smem[l] = take((int)bytes, 16);
    }
    return (size_t)off + 1024;
}

}  // namespace lenet_tc
}  // namespace conv_chain
}  // namespace ag
