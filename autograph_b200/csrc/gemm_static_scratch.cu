// ag_gemm_static_scratch: the split-k GEMM for callers that must not allocate.
//
// Some hosts give the library no way to obtain device memory after start-up: a
// serving process that handed all of a GPU's memory to its own arena, a plugin
// whose host forbids driver allocations on its worker threads, or code that
// runs where a cudaMalloc would stall the whole device.  ag_gemm cannot serve
// them when it splits a product along k, because the partial sums go to a
// workspace that is grown with cudaMalloc.  This entry point keeps the partial
// sums in a fixed array that is part of the library image instead, and takes a
// device ordinal and a stream rather than an ag_device (creating an ag_device
// allocates).  It calls no cudaMalloc, cudaFree or other allocating routine.
//
// The array costs kStaticScratchBytes of device memory on every GPU that loads
// the library, for the life of the process.  All calls on a GPU share it: two
// calls that overlap on the GPU (different streams) race on it, so keep them
// on one stream or order them with events.  Nothing in it has to start at
// zero: every partial sum that is read was written by the same call.
#include <mutex>

#include "gemm_simt_launch.cuh"

namespace ag {

constexpr size_t kStaticScratchBytes = size_t(4) << 20;  // 4 MiB
constexpr int kMaxDevices = 64;

// Device-side storage.  In host code this name is only a handle for
// cudaGetSymbolAddress; the address kernels may use is looked up per device.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticSetup {
    bool ready = false;
    void *scratch = nullptr;  // device address of g_static_scratch on this GPU
    int sm_count = 0;
};
static StaticSetup g_setup[kMaxDevices];
static std::mutex g_setup_mutex;

// Once per GPU, with that GPU current: resolve the device address of the array.
static int static_setup(int ordinal, StaticSetup *out) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    StaticSetup &s = g_setup[ordinal];
    if (!s.ready) {
        void *ptr = nullptr;
        AG_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
        AG_REQUIRE(ptr != nullptr, AG_ERR_CUDA, "static scratch has no device address");
        int sms = 0;
        AG_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ordinal));
        int major = 0;
        AG_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, ordinal));
        AG_REQUIRE(major == 10, AG_ERR_UNSUPPORTED,
                   "device %d is not sm_100; this library only carries sm_100a code", ordinal);
        s.scratch = ptr;
        s.sm_count = sms;
        s.ready = true;
    }
    *out = s;
    return AG_OK;
}

template <class T>
static bool vec_aligned(const T *p) {
    return (reinterpret_cast<uintptr_t>(p) % (4 * sizeof(T))) == 0;
}

template <class T, bool AK, bool BK_>
static int run_typed(ag_device *dev, void *scratch, int m, int k, int n, float alpha, const T *a,
                     int64_t rsa, int64_t csa, const T *b, int64_t rsb, int64_t csb, float beta,
                     T *c, int64_t rsc, int64_t csc) {
    simt::StridedOperand<T, AK> A{a, rsa, csa, m, k, false};
    simt::StridedOperand<T, BK_> B{b, csb, rsb, n, k, false};
    A.vec = AK ? ((csa == 1) && (rsa % 4 == 0 || m == 1) && vec_aligned(a))
               : ((rsa == 1) && (csa % 4 == 0 || k == 1) && vec_aligned(a));
    B.vec = BK_ ? ((rsb == 1) && (csb % 4 == 0 || n == 1) && vec_aligned(b))
                : ((csb == 1) && (rsb % 4 == 0 || k == 1) && vec_aligned(b));
    simt::StridedEpilogue<T> E{c, rsc, csc, alpha, beta, false, n};
    E.vec = (csc == 1) && (rsc % 4 == 0 || m == 1) && vec_aligned(c);
    return simt::gemm(dev, m, n, k, A, B, E, /*allow_split=*/true, scratch, kStaticScratchBytes);
}

template <class T>
static int run(ag_device *dev, void *scratch, int m, int k, int n, float alpha, const T *a,
               int64_t rsa, int64_t csa, const T *b, int64_t rsb, int64_t csb, float beta, T *c,
               int64_t rsc, int64_t csc) {
    const bool ak = (csa == 1 && rsa != 1) || (csa == 1 && m == 1);
    const bool bk = (rsb == 1 && csb != 1) || (rsb == 1 && n == 1);
    if (ak && bk)
        return run_typed<T, true, true>(dev, scratch, m, k, n, alpha, a, rsa, csa, b, rsb, csb,
                                        beta, c, rsc, csc);
    if (ak)
        return run_typed<T, true, false>(dev, scratch, m, k, n, alpha, a, rsa, csa, b, rsb, csb,
                                         beta, c, rsc, csc);
    if (bk)
        return run_typed<T, false, true>(dev, scratch, m, k, n, alpha, a, rsa, csa, b, rsb, csb,
                                         beta, c, rsc, csc);
    return run_typed<T, false, false>(dev, scratch, m, k, n, alpha, a, rsa, csa, b, rsb, csb, beta,
                                      c, rsc, csc);
}

}  // namespace ag

using namespace ag;

extern "C" int ag_gemm_static_scratch(int ordinal, void *cuda_stream, ag_dtype dtype, int64_t m,
                                      int64_t k, int64_t n, float alpha, const void *a,
                                      int64_t off_a, int64_t rsa, int64_t csa, const void *b,
                                      int64_t off_b, int64_t rsb, int64_t csb, float beta, void *c,
                                      int64_t off_c, int64_t rsc, int64_t csc) {
    AG_REQUIRE(ordinal >= 0 && ordinal < kMaxDevices, AG_ERR_INVALID,
               "device ordinal %d out of range", ordinal);
    AG_REQUIRE(dtype == AG_F32 || dtype == AG_BF16, AG_ERR_DTYPE,
               "Dot unimplemented for dtype %d", (int)dtype);
    AG_REQUIRE(m >= 0 && k >= 0 && n >= 0, AG_ERR_SHAPE, "negative dimension");
    AG_REQUIRE(m < (1ll << 31) && k < (1ll << 31) && n < (1ll << 31), AG_ERR_LIMIT,
               "dimension beyond 2^31");
    // Room for at least two planes of f32 partial sums.
    const int64_t max_outputs = (int64_t)(kStaticScratchBytes / (2 * sizeof(float)));
    AG_REQUIRE(m * n <= max_outputs, AG_ERR_LIMIT,
               "m*n = %lld exceeds the static scratch limit of %lld output elements "
               "(%zu bytes of fixed scratch); use ag_gemm for larger outputs",
               (long long)(m * n), (long long)max_outputs, kStaticScratchBytes);
    if (m == 0 || n == 0) return AG_OK;
    AG_REQUIRE(c != nullptr && (k == 0 || (a != nullptr && b != nullptr)), AG_ERR_INVALID,
               "null operand pointer");
    AG_REQUIRE(off_a >= 0 && off_b >= 0 && off_c >= 0, AG_ERR_INVALID, "negative offset");

    int previous = 0;
    AG_CUDA_TRY(cudaGetDevice(&previous));
    AG_CUDA_TRY(cudaSetDevice(ordinal));
    StaticSetup setup;
    int status = static_setup(ordinal, &setup);
    if (status == AG_OK) {
        // A stack-only stand-in for an ag_device: stream and SM count, no resources.
        ag_device dev;
        dev.ordinal = ordinal;
        dev.stream = (cudaStream_t)cuda_stream;
        dev.sm_count = setup.sm_count;
        if (dtype == AG_F32)
            status = run<float>(&dev, setup.scratch, (int)m, (int)k, (int)n, alpha,
                                (const float *)a + off_a, rsa, csa, (const float *)b + off_b, rsb,
                                csb, beta, (float *)c + off_c, rsc, csc);
        else
            status = run<__nv_bfloat16>(&dev, setup.scratch, (int)m, (int)k, (int)n, alpha,
                                        (const __nv_bfloat16 *)a + off_a, rsa, csa,
                                        (const __nv_bfloat16 *)b + off_b, rsb, csb, beta,
                                        (__nv_bfloat16 *)c + off_c, rsc, csc);
    }
    if (previous != ordinal) cudaSetDevice(previous);
    return status;
}
