// PTX wrappers shared by the tcgen05 kernels: mbarriers with bounded waits, TMA
// tile loads, tensor-memory allocation, tcgen05.mma / commit / ld, and the
// shared-memory and instruction descriptors for bf16 operands with f32
// accumulation.  Host side: the cuTensorMapEncodeTiled entry point.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace ag {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait: gives up after limit_ns, or as soon as another thread of the CTA has given
// up, and reports through *abort_flag.
__device__ __forceinline__ bool mbar_wait_for(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                              uint64_t limit_ns) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 1023u) == 1023u) {
            if (*abort_flag) return false;
            uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > limit_ns) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// The limit every kernel of the library uses: about two seconds.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    return mbar_wait_for(bar, parity, abort_flag, 2000000000ull);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(cols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] . B[smem]; one thread issues for the whole CTA.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The mbarrier receives one arrival once every tcgen05 operation issued so far
// by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives row
// (lane base + t), columns [col, col + 32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (tcgen05): start address, leading / stride
// byte offsets (all >> 4), descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;  // descriptor version for sm_100
    d |= 2ull << 61;  // SWIZZLE_128B
    return d;
}

// Two accumulator values -> one packed bf16 pair with the layer's epilogue:
// round the sums to bf16, add the bias in f32 and round again, ReLU (x >= 0 ? x : 0).
// Conversions are the slow instructions of an epilogue, so the pair is rounded with
// one packed conversion, unpacked with shifts, and packed again only when a bias
// changed the values.
__device__ __forceinline__ uint32_t bf16_pair_epilogue(uint32_t acc0, uint32_t acc1, float b0,
                                                       float b1, bool has_bias, bool relu) {
    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(acc0), __uint_as_float(acc1));
    uint32_t u = *reinterpret_cast<uint32_t *>(&h);
    if (!has_bias && !relu) return u;
    float x0 = __uint_as_float(u << 16), x1 = __uint_as_float(u & 0xffff0000u);
    if (has_bias) {
        h = __floats2bfloat162_rn(x0 + b0, x1 + b1);
        u = *reinterpret_cast<uint32_t *>(&h);
        if (!relu) return u;
        x0 = __uint_as_float(u << 16);
        x1 = __uint_as_float(u & 0xffff0000u);
    }
    // ReLU on exact bf16 values: clear a half whose value is negative (or NaN)
    const uint32_t lo = (x0 >= 0.f) ? (u & 0x0000ffffu) : 0u;
    const uint32_t hi = (x1 >= 0.f) ? (u & 0xffff0000u) : 0u;
    return lo | hi;
}

// Instruction descriptor for kind::f16: f32 accumulate, bf16 A and B.
__host__ __device__ constexpr uint32_t make_idesc(bool a_mn_major, bool b_mn_major, int m, int n) {
    return (1u << 4)                         // D format: f32
           | (1u << 7)                       // A format: bf16
           | (1u << 10)                      // B format: bf16
           | ((a_mn_major ? 1u : 0u) << 15)  // A major: 0 = K, 1 = MN
           | ((b_mn_major ? 1u : 0u) << 16)  // B major
           | ((uint32_t)(n >> 3) << 17)      // N / 8
           | ((uint32_t)(m >> 4) << 24);     // M / 16
}


__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point query (the
// library does not link libcuda), or null.
EncodeTiledFn encode_tiled_fn();

// bf16 tensor map of `rank` dimensions (innermost first): dims in elements,
// strides in elements for dimensions 1..rank-1, box in elements; 128-byte
// swizzle, out-of-range elements read as zero.
int make_tmap_bf16(CUtensorMap *map, const void *base, int rank, const uint64_t *dims,
                   const uint64_t *strides, const uint32_t *box);

}  // namespace tc
}  // namespace ag
