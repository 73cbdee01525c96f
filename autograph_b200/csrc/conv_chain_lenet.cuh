// The whole-network kernel specialised for the geometry of LeNet5
// (benches/neural-network-benches/src/autograph_backend.rs:129-146):
//   [B,1,28,28] -> Conv2 1->6 5x5 -> Relu -> MaxPool2 2x2 -> Conv2 6->16 5x5 -> Relu ->
//   MaxPool2 2x2 -> Flatten (256) -> a chain of Dense (+ Relu) layers.
// The generic kernel (conv_chain.cu) takes any small network; this one fixes every extent of
// the two convolution stages at compile time, which buys:
//  * register tiles sized for the shared-memory return path.  Shared memory delivers 128 bytes
//    per clock to the register file, broadcasts included, while the four schedulers retire 128
//    FFMAs per clock: a thread has to get at least four FFMAs out of every float it loads.
//    conv1: one item is 2 x 12 pixels x 2 channels (48 accumulators; 7 images are 504 items, one
//    round of the 512 threads); conv2: 2 x 4 pixels x 2 channels (448 items: wider tiles leave
//    too few warps to cover the load latency, measured).  The two channels of an item are the
//    halves of one fma.rn.f32x2: half the instructions for the same FMAs.
//    Patch rows stream through registers one at a time (row r feeds filter row r of the
//    block's first pixel row and filter row r-1 of its second, whose weights are kept from the
//    previous step), so a thread holds one patch row and two filter rows, not a whole patch.
//  * every shared-memory offset is an immediate.
//  * the dense weights do not stream from L2 inside the dense phase: the first layer's matrix
//    is brought into shared memory by one bulk asynchronous copy issued when the kernel
//    starts (it lands while the convolutions run), the later layers' by copies issued when the
//    second convolution has released its buffers.  The waits on the copies' mbarriers are
//    bounded (status 170 / 171).
// Every output is the same chain of FFMAs in the same order, with the same roundings, as in
// the generic kernel and the stand-alone layer kernels, so the logits are identical bit for
// bit (tests/test_fused_gpu.py).
#pragma once

#include "conv2_direct_device.cuh"
#include "dense_small_device.cuh"
#include "tc_ptx.cuh"

namespace ag {
namespace conv_chain {
namespace lenet {

using dense_small::ROWS;

constexpr int kThreads = 512;
constexpr int kGroup = 7;             // images per CTA (504 conv1 items, 448 conv2 items)
constexpr int IH = 28, IW = 28, F = 5;
constexpr int C1 = 6, H1 = 24, P1 = 12;   // conv1 output channels / size, pooled size
constexpr int C2 = 16, H2 = 8, P2 = 4;    // conv2
constexpr int kFlat = C2 * P2 * P2;       // 256
// Filter banks in shared memory.  conv1: [channel pair 3][filter row 5][tap 5][2], rows padded to 12.
// conv2: [channel pair 8][input channel 6][filter row 5][tap 5][2] with filter rows padded to
// 12 floats: a filter row of a pair is three 16-byte loads; the pair pitch keeps the eight
// pairs of a warp on different banks.
constexpr int W1_ROW = 12;                // a filter row of a channel pair: 5 taps x 2 channels + 2 zeros
constexpr int W1_PAIR = F * W1_ROW + 4;   // 64: the three pairs of a block on different banks
constexpr int W1_FLOATS = (C1 / 2) * W1_PAIR;  // 192
constexpr int W2_ROW = 12;
constexpr int W2_CI = F * W2_ROW;         // 60
constexpr int W2_PAIR = C1 * W2_CI + 4;   // 364
constexpr int W2_FLOATS = (C2 / 2) * W2_PAIR;

// Shared-memory plan in floats (every offset a multiple of 4).
constexpr int IN_OFF = 0;                              // [kGroup][784]
constexpr int MID_OFF = IN_OFF + kGroup * IH * IW;     // [kGroup][6][144]
constexpr int CONV_END = MID_OFF + kGroup * C1 * P1 * P1;

struct Plan {
    int bs;
    int group;                        // images per CTA (<= kGroup)
    const void *w1, *w2;              // conv filter banks [6][1][5][5], [16][6][5][5]
    dense_small::ChainParams chain;   // the dense layers (weights read from w_off when >= 0)
    int w_smem[dense_small::kMaxChain];  // float offset of the layer's weights in shared memory, or -1
    int w_bytes[dense_small::kMaxChain];
    int early;                        // layers [0, early) are copied at kernel start, the rest after conv2
    int w1_off, w2_off, xa_off, xb_off, red_off, bar_off;
    int *status;
    int persist, in2_off;   // split form: CTAs walk over several groups (second image buffer at in2_off)
    // When set, the kernel stops after the flatten and writes the activations [bs, 256] here
    // (the dense layers then run as separate products over the whole batch).
    void *flat_out;
};

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

template <class T>
__device__ __forceinline__ float round_t(float v) {
    return to_f32(from_f32<T>(v));
}

template <class T>
__global__ void __launch_bounds__(kThreads, 1)
    lenet_chain_kernel(const T *__restrict__ x, const uint8_t *__restrict__ x8, float alpha,
                       T *__restrict__ y, const Plan pl) {
    extern __shared__ __align__(16) float smem[];
    __shared__ int s_abort;
    const int tid = threadIdx.x;
    int b0 = blockIdx.x * pl.group;
    int nimg = min(pl.group, pl.bs - b0);
    float *s_in = smem + IN_OFF, *s_mid = smem + MID_OFF;
    // Large batches that stop after the flatten: fewer CTAs than groups, each CTA walks over
    // its groups and fetches the next group's images (asynchronous copies into a second buffer)
    // while it convolves the current one; the filter banks are staged once.
    const bool persist = pl.persist != 0 && pl.flat_out != nullptr && x8 == nullptr;
    float *s_in_next = smem + pl.in2_off;
    int grp = blockIdx.x;
    const int ngroups = (pl.bs + pl.group - 1) / pl.group;
    float *s_w1 = smem + pl.w1_off, *s_w2 = smem + pl.w2_off;
    float *xa = smem + pl.xa_off, *xb = smem + pl.xb_off;
    const uint32_t bar0 = tc::smem_u32(smem + pl.bar_off), bar1 = bar0 + 8;
    // Programmatic dependent launch: let the next kernel of the stream (if it was launched with
    // the matching attribute) place its CTAs as soon as SMs become free, and, being such a
    // kernel itself, wait here until everything the previous kernel wrote is visible.  Nothing
    // before this point touches global memory.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    AG_STAMP(0);

    // ---- the dense weights of the early layers start their way into shared memory (issued by
    // a thread of the last warp, which has the least other work)
    if (tid == kThreads - 1) {
        s_abort = 0;
        tc::mbar_init(bar0, 1);
        tc::mbar_init(bar1, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        uint32_t bytes = 0;
        for (int l = 0; l < pl.early; ++l) bytes += (uint32_t)pl.w_bytes[l];
        if (bytes) {
            tc::mbar_arrive_expect_tx(bar0, bytes);
            for (int l = 0; l < pl.early; ++l)
                bulk_g2s(tc::smem_u32(smem + pl.w_smem[l]), pl.chain.s[l].w, (uint32_t)pl.w_bytes[l], bar0);
        }
    }

    // ---- images and filter banks
    if (x8 != nullptr) {
        const float a = round_t<T>(alpha);  // scaled_cast: alpha rounded to T, product rounded once
        const uint8_t *src = x8 + (int64_t)b0 * (IH * IW);
        const int total = nimg * IH * IW;   // a multiple of 4; b0 * 784 keeps 4-byte alignment
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
        for (int i = tid; i < W1_FLOATS; i += kThreads) {
            const int pair = i / W1_PAIR, r = i - pair * W1_PAIR;
            const int fi = r / W1_ROW, r2 = r - fi * W1_ROW;
            const int fj = r2 >> 1, o = r2 & 1;
            s_w1[i] = (fi < F && fj < F) ? to_f32(w1[((pair * 2 + o) * F + fi) * F + fj]) : 0.f;
        }
        const T *w2 = reinterpret_cast<const T *>(pl.w2);
        float v[(W2_FLOATS + kThreads - 1) / kThreads];
#pragma unroll
        for (int j = 0; j < (W2_FLOATS + kThreads - 1) / kThreads; ++j) {   // loads first, stores after
            const int i = tid + j * kThreads;
            const int pair = i / W2_PAIR, r = i - pair * W2_PAIR;
            const int ci = r / W2_CI, r2 = r - ci * W2_CI;
            const int fi = r2 / W2_ROW, r3 = r2 - fi * W2_ROW;
            const int fj = r3 >> 1, o = r3 & 1;
            v[j] = (i < W2_FLOATS && ci < C1 && fj < F)
                       ? to_f32(w2[(((pair * 2 + o) * C1 + ci) * F + fi) * F + fj]) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < (W2_FLOATS + kThreads - 1) / kThreads; ++j)
            if (tid + j * kThreads < W2_FLOATS) s_w2[tid + j * kThreads] = v[j];
    }
    if (nimg < ROWS)  // rows without an image still flow through the dense layers: zeros
        for (int i = tid; i < kFlat * ROWS; i += kThreads) xa[i] = 0.f;
    __syncthreads();
    AG_STAMP(1);

    for (;;) {
    if (persist && grp + (int)gridDim.x < ngroups) {
        // 16-byte pieces of the next group's images as they lie in memory (f32: the buffer the
        // convolution will read; bf16: raw, converted when the current group is done)
        const int nb0 = (grp + (int)gridDim.x) * pl.group;
        const int total = min(pl.group, pl.bs - nb0) * (IH * IW * (int)sizeof(T) / 16);
        const char *src = reinterpret_cast<const char *>(x + (int64_t)nb0 * (IH * IW));
        for (int q = tid; q < total; q += kThreads)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(tc::smem_u32(s_in_next) + 16 * q),
                         "l"(src + 16 * q)
                         : "memory");
    }
    // ---- conv1 + relu + pool: item = (image, 2 rows x 12 columns, channel pair).  The two
    // channels of a pair are the halves of one fma.rn.f32x2 (the pixel's value in both halves of
    // the multiplier): per patch row 120 packed FMAs and 20 moves instead of 240 FFMAs, the same
    // sums in the same order.
    if (tid < nimg * 72) {
        const int g = tid / 72, r = tid - g * 72;
        const int pair = r % 3, blk = r / 3;           // the three pairs of a block sit in adjacent lanes
        const int by = blk >> 1, hx = blk & 1;
        const float *img = s_in + g * (IH * IW) + (2 * by) * IW + 12 * hx;
        const float *wt = s_w1 + pair * W1_PAIR;
        unsigned long long acc2[2][12];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < 12; ++b) acc2[a][b] = 0ull;
        unsigned long long wprev[W1_ROW / 2];
#pragma unroll
        for (int pr = 0; pr < F + 1; ++pr) {       // patch row pr = filter row pr of pixel row 0
            float p[16];                           // and filter row pr - 1 of pixel row 1
#pragma unroll
            for (int q = 0; q < 4; ++q)
                *reinterpret_cast<float4 *>(p + 4 * q) =
                    *reinterpret_cast<const float4 *>(img + pr * IW + 4 * q);
            unsigned long long wcur[W1_ROW / 2];
            if (pr < F) {
#pragma unroll
                for (int q = 0; q < W1_ROW / 4; ++q) {
                    const ulonglong2 w2 = *reinterpret_cast<const ulonglong2 *>(wt + pr * W1_ROW + 4 * q);
                    wcur[2 * q] = w2.x;
                    wcur[2 * q + 1] = w2.y;
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {          // six pixels at a time: ten doubled patch values live
                unsigned long long pp[10];
#pragma unroll
                for (int q = 0; q < 10; ++q) asm("mov.b64 %0, {%1, %1};" : "=l"(pp[q]) : "f"(p[6 * h + q]));
#pragma unroll
                for (int fj = 0; fj < F; ++fj) {
                    if (pr < F) {
#pragma unroll
                        for (int b = 0; b < 6; ++b)
                            asm("fma.rn.f32x2 %0, %1, %2, %0;"
                                : "+l"(acc2[0][6 * h + b]) : "l"(pp[fj + b]), "l"(wcur[fj]));
                    }
                    if (pr >= 1) {
#pragma unroll
                        for (int b = 0; b < 6; ++b)
                            asm("fma.rn.f32x2 %0, %1, %2, %0;"
                                : "+l"(acc2[1][6 * h + b]) : "l"(pp[fj + b]), "l"(wprev[fj]));
                    }
                }
            }
            if (pr < F) {
#pragma unroll
                for (int q = 0; q < W1_ROW / 2; ++q) wprev[q] = wcur[q];
            }
        }
        // round to T, relu, 2x2 pool (window order (0,0),(0,1),(1,0),(1,1); first maximum wins)
        float acc[2][12][2];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < 12; ++b)
                asm("mov.b64 {%0, %1}, %2;" : "=f"(acc[a][b][0]), "=f"(acc[a][b][1]) : "l"(acc2[a][b]));
        float *dst = s_mid + (g * C1 + pair * 2) * (P1 * P1) + by * P1 + 6 * hx;
#pragma unroll
        for (int o = 0; o < 2; ++o) {
            float m[6];
#pragma unroll
            for (int wx = 0; wx < 6; ++wx) {
                float v00 = round_t<T>(acc[0][2 * wx][o]), v01 = round_t<T>(acc[0][2 * wx + 1][o]);
                float v10 = round_t<T>(acc[1][2 * wx][o]), v11 = round_t<T>(acc[1][2 * wx + 1][o]);
                v00 = v00 >= 0.f ? v00 : 0.f; v01 = v01 >= 0.f ? v01 : 0.f;
                v10 = v10 >= 0.f ? v10 : 0.f; v11 = v11 >= 0.f ? v11 : 0.f;
                float mm = v00;
                if (v01 > mm) mm = v01;
                if (v10 > mm) mm = v10;
                if (v11 > mm) mm = v11;
                m[wx] = mm;
            }
#pragma unroll
            for (int q = 0; q < 3; ++q)
                *reinterpret_cast<float2 *>(dst + o * (P1 * P1) + 2 * q) = make_float2(m[2 * q], m[2 * q + 1]);
        }
    }
    __syncthreads();
    AG_STAMP(2);

    // ---- conv2 + relu + pool: item = (image, 2 rows x 4 columns, channel pair)
    if (tid < nimg * 64) {
        const int g = tid >> 6, r = tid & 63;
        const int pair = r & 7, blk = r >> 3;          // the eight pairs of a block sit in adjacent lanes
        const int by = blk >> 1, bx = blk & 1;
        const float *img = s_mid + g * (C1 * P1 * P1) + (2 * by) * P1 + 4 * bx;
        const float *wp = s_w2 + pair * W2_PAIR;
        // Two channels per instruction: fma.rn.f32x2 on the (channel 2 * pair, channel 2 * pair + 1)
        // register pair, the pixel's value in both halves of the multiplier.  Same FMAs in the same
        // order per accumulator, half the instructions to issue.
        unsigned long long acc2[2][4];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc2[a][b] = 0ull;
        // The loop over input channels stays rolled: the phase runs once per launch, and 2400
        // FFMAs of straight-line code fetched for a single use cost more in instruction fetch
        // than the loop costs in branches (measured both ways; the patch-row loop inside, and
        // conv1's, are faster unrolled).
#pragma unroll 1
        for (int ci = 0; ci < C1; ++ci) {
            unsigned long long wprev[W2_ROW / 2];
#pragma unroll
            for (int pr = 0; pr < F + 1; ++pr) {
                float p[8];
                *reinterpret_cast<float4 *>(p) =
                    *reinterpret_cast<const float4 *>(img + ci * (P1 * P1) + pr * P1);
                *reinterpret_cast<float4 *>(p + 4) =
                    *reinterpret_cast<const float4 *>(img + ci * (P1 * P1) + pr * P1 + 4);
                unsigned long long pp[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) asm("mov.b64 %0, {%1, %1};" : "=l"(pp[q]) : "f"(p[q]));
                unsigned long long wcur[W2_ROW / 2];
                if (pr < F) {
#pragma unroll
                    for (int q = 0; q < W2_ROW / 4; ++q) {
                        const ulonglong2 w2 =
                            *reinterpret_cast<const ulonglong2 *>(wp + ci * W2_CI + pr * W2_ROW + 4 * q);
                        wcur[2 * q] = w2.x;
                        wcur[2 * q + 1] = w2.y;
                    }
                }
#pragma unroll
                for (int fj = 0; fj < F; ++fj) {
                    if (pr < F) {
#pragma unroll
                        for (int b = 0; b < 4; ++b)
                            asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc2[0][b]) : "l"(pp[fj + b]), "l"(wcur[fj]));
                    }
                    if (pr >= 1) {
#pragma unroll
                        for (int b = 0; b < 4; ++b)
                            asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc2[1][b]) : "l"(pp[fj + b]), "l"(wprev[fj]));
                    }
                }
                if (pr < F) {
#pragma unroll
                    for (int q = 0; q < W2_ROW / 2; ++q) wprev[q] = wcur[q];
                }
            }
        }
        float acc[2][4][2];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b)
                asm("mov.b64 {%0, %1}, %2;" : "=f"(acc[a][b][0]), "=f"(acc[a][b][1]) : "l"(acc2[a][b]));
        // flattened (c, h, w) index of the dense chain's input, [k][ROWS]
#pragma unroll
        for (int o = 0; o < 2; ++o) {
            const int oc = pair * 2 + o;
#pragma unroll
            for (int wx = 0; wx < 2; ++wx) {
                float v00 = round_t<T>(acc[0][2 * wx][o]), v01 = round_t<T>(acc[0][2 * wx + 1][o]);
                float v10 = round_t<T>(acc[1][2 * wx][o]), v11 = round_t<T>(acc[1][2 * wx + 1][o]);
                v00 = v00 >= 0.f ? v00 : 0.f; v01 = v01 >= 0.f ? v01 : 0.f;
                v10 = v10 >= 0.f ? v10 : 0.f; v11 = v11 >= 0.f ? v11 : 0.f;
                float mm = v00;
                if (v01 > mm) mm = v01;
                if (v10 > mm) mm = v10;
                if (v11 > mm) mm = v11;
                xa[((oc * P2 + by) * P2 + 2 * bx + wx) * ROWS + g] = mm;
            }
        }
    }
    __syncthreads();
    AG_STAMP(3);
    if (pl.flat_out != nullptr) {
        T *flat = reinterpret_cast<T *>(pl.flat_out) + (int64_t)b0 * kFlat;
        for (int i = tid; i < nimg * kFlat; i += kThreads) {
            const int g = i >> 8, k = i & (kFlat - 1);
            flat[i] = from_f32<T>(xa[k * ROWS + g]);   // exact: the values are already T's
        }
        if (!persist || grp + (int)gridDim.x >= ngroups) return;
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();   // the next group's images have landed; xa and s_mid may be rewritten
        grp += (int)gridDim.x;
        b0 = grp * pl.group;
        nimg = min(pl.group, pl.bs - b0);
        if constexpr (sizeof(T) == 4) {
            float *t = s_in;
            s_in = s_in_next;
            s_in_next = t;
        } else {
            const T *raw = reinterpret_cast<const T *>(s_in_next);
            for (int i = tid; i < nimg * (IH * IW) / 4; i += kThreads)
                direct::load4_to_f32<T>(raw + 4 * i, s_in + 4 * i);
            __syncthreads();
        }
        continue;
    }
    break;
    }

    // ---- the later dense layers' weights go where the convolutions' buffers were
    if (tid == kThreads - 1 && pl.early < pl.chain.n_layers) {
        uint32_t bytes = 0;
        for (int l = pl.early; l < pl.chain.n_layers; ++l)
            if (pl.w_smem[l] >= 0) bytes += (uint32_t)pl.w_bytes[l];
        if (bytes) {
            // the buffers were read through the generic proxy until the barrier above
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc::mbar_arrive_expect_tx(bar1, bytes);
            for (int l = pl.early; l < pl.chain.n_layers; ++l)
                if (pl.w_smem[l] >= 0)
                    bulk_g2s(tc::smem_u32(smem + pl.w_smem[l]), pl.chain.s[l].w, (uint32_t)pl.w_bytes[l],
                             bar1);
        }
    }

    // ---- dense chain
    float *red = smem + pl.red_off;
    bool waited0 = false, waited1 = false;
    for (int l = 0; l < pl.chain.n_layers; ++l) {
        const T *w = reinterpret_cast<const T *>(pl.chain.s[l].w);
        if (pl.w_smem[l] >= 0) {
            const bool early = l < pl.early;
            if (early ? !waited0 : !waited1) {
                // the copy either completes for every thread or for none, so all threads take
                // the same way out
                if (!tc::mbar_wait(early ? bar0 : bar1, 0, &s_abort)) {
                    if (tid == 0) atomicCAS(pl.status, 0, early ? 170 : 171);
                    return;
                }
                (early ? waited0 : waited1) = true;
            }
            w = reinterpret_cast<const T *>(smem + pl.w_smem[l]);
        }
        if (l == 0) AG_STAMP(4);
        const bool last = l + 1 == pl.chain.n_layers;
        if (pl.w_smem[l] >= 0)
            dense_small::chain_layer<T, true, true>(pl.chain.s[l], w, xa, xb, red, b0, nimg, last, y);
        else
            dense_small::chain_layer<T, true, false>(pl.chain.s[l], w, xa, xb, red, b0, nimg, last, y);
        if (l < 2) AG_STAMP(5 + l);
        float *t = xa;
        xa = xb;
        xb = t;
    }
    AG_STAMP(7);
}

// Fills the plan for a network of this geometry; returns the dynamic shared memory in bytes,
// or 0 when the kernel does not take it (the caller then uses the generic kernel).
inline size_t make_plan(Plan *pl, ag_dtype dtype, int64_t bs, int64_t ic, int64_t ih, int64_t iw,
                        int n_conv, const ag_conv_stage *stages, int n_dense,
                        const dense_small::ChainLayer *layers, void *flat_out = nullptr) {
    pl->flat_out = flat_out;
    pl->persist = 0;
    pl->in2_off = 0;
    if (n_conv != 2 || ic != 1 || ih != IH || iw != IW) return 0;
    if (bs <= 0 || bs > (int64_t)kGroup * 0x7fffffff / 8) return 0;
    const int ocs[2] = {C1, C2};
    for (int s = 0; s < 2; ++s) {
        const ag_conv_stage &cs = stages[s];
        const ag_conv2_options &o = cs.options;
        if (cs.oc != ocs[s] || cs.bias != nullptr || !cs.relu || cs.pool[0] != 2 || cs.pool[1] != 2)
            return 0;
        if (o.filter[0] != F || o.filter[1] != F || o.padding[0] || o.padding[1] || o.stride[0] != 1 ||
            o.stride[1] != 1 || o.dilation[0] != 1 || o.dilation[1] != 1)
            return 0;
    }
    if (n_dense < 1 || n_dense > dense_small::kMaxChain || layers[0].inputs != kFlat) return 0;
    for (int i = 0; i < n_dense; ++i) {
        if (!dense_small::eligible(ROWS, layers[i].inputs, layers[i].outputs)) return 0;
        if (i > 0 && layers[i].inputs != layers[i - 1].outputs) return 0;
    }
    const size_t es = dtype_size(dtype);
    pl->bs = (int)bs;
    pl->w1 = stages[0].w;
    pl->w2 = stages[1].w;
    dense_small::plan_chain(&pl->chain, (int)bs, n_dense, layers);
    if (pl->chain.max_k > kFlat) return 0;
    // Budget: 227 KiB per CTA minus the kernel's few static words.
    constexpr int kMaxFloats = (227 * 1024 - 64) / 4;
    // Layout: [in | mid] [spare] [w1] [w2] [xa] [xb] [mbarriers] [layer 0 weights].  red overlays
    // the start of [in | mid]; what follows red up to the end of the spare region, and later the
    // filter banks, take the later layers' weights once the convolutions are done.
    const int xb_floats = [&] {
        int n = 0;
        for (int i = 0; i < n_dense; ++i) n = layers[i].outputs > n ? layers[i].outputs : n;
        return n * ROWS;
    }();
    auto r4 = [](int64_t v) { return (int)((v + 3) & ~3ll); };
    const int64_t l0_bytes = (int64_t)layers[0].inputs * layers[0].outputs * (int64_t)es;
    const bool l0_copyable = (reinterpret_cast<uintptr_t>(layers[0].w) & 15) == 0 &&
                             l0_bytes % 16 == 0 && l0_bytes < (1 << 20);
    const int fixed = r4(W1_FLOATS) + r4(W2_FLOATS) + r4(kFlat * ROWS) + r4(xb_floats) + 4;
    int l0_floats = l0_copyable ? r4((l0_bytes + 3) / 4) : 0;
    if (CONV_END + fixed + l0_floats > kMaxFloats) l0_floats = 0;   // layer 0 stays in global memory
    const int spare = kMaxFloats - (CONV_END + fixed + l0_floats);
    if (spare < 0 || pl->chain.red_floats > CONV_END + spare) return 0;
    // the second image buffer of the group-walking form sits in the spare region (nothing else
    // uses it when the dense layers do not run in this kernel)
    if (flat_out != nullptr && spare >= kGroup * IH * IW) {
        pl->persist = 1;
        pl->in2_off = CONV_END;
    }
    int off = CONV_END + spare;
    auto take = [&](int floats) {
        const int at = off;
        off += r4(floats);
        return at;
    };
    pl->w1_off = take(W1_FLOATS);
    pl->w2_off = take(W2_FLOATS);
    pl->xa_off = take(kFlat * ROWS);
    pl->xb_off = take(xb_floats);
    pl->bar_off = take(4);
    pl->red_off = IN_OFF;
    struct Hole { int at, floats; };
    Hole holes[2] = {{r4(pl->chain.red_floats), 0}, {pl->w1_off, pl->xa_off - pl->w1_off}};
    holes[0].floats = CONV_END + spare - holes[0].at;
    pl->early = 0;
    for (int l = 0; l < n_dense; ++l) {
        pl->w_smem[l] = -1;
        const int64_t bytes = (int64_t)layers[l].inputs * layers[l].outputs * (int64_t)es;
        pl->w_bytes[l] = (int)bytes;
        if (flat_out != nullptr) continue;   // the dense layers do not run in this kernel
        if (l == 0) {
            if (l0_floats) {
                pl->w_smem[0] = take(l0_floats);
                pl->early = 1;
            }
            continue;
        }
        const bool copyable = (reinterpret_cast<uintptr_t>(layers[l].w) & 15) == 0 && bytes % 16 == 0 &&
                              bytes < (1 << 20);
        if (!copyable) continue;
        const int floats = r4((bytes + 3) / 4);
        for (Hole &h : holes) {
            if (floats <= h.floats) {
                pl->w_smem[l] = h.at;
                h.at += floats;
                h.floats -= floats;
                break;
            }
        }
    }
    return (size_t)kMaxFloats * sizeof(float);
}

}  // namespace lenet
}  // namespace conv_chain
}  // namespace ag
