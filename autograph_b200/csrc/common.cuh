// Shared declarations of the library: device object, error reporting, dtype helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <vector>

#include "../../include/autograph_b200.h"

namespace ag {

// ---- error reporting -----------------------------------------------------
// Thread-local message behind ag_last_error().
char *error_buffer();
int fail(int status, const char *fmt, ...) __attribute__((format(printf, 2, 3)));

#define AG_CUDA_TRY(expr)                                                                      \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess) {                                                               \
            /* reported here: it must not also fail the next call's launch check */           \
            cudaGetLastError();                                                                \
            return ::ag::fail(_e == cudaErrorMemoryAllocation ? AG_ERR_OOM : AG_ERR_CUDA,      \
                              "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, \
                              __LINE__);                                                       \
        }                                                                                      \
    } while (0)

#define AG_TRY(expr)              \
    do {                          \
        int _s = (expr);          \
        if (_s != AG_OK) return _s; \
    } while (0)

#define AG_REQUIRE(cond, status, ...)                   \
    do {                                                \
        if (!(cond)) return ::ag::fail(status, __VA_ARGS__); \
    } while (0)

// Counts kernel launches enqueued by the library (ag_kernel_launch_count).
void count_launch();
void count_launches(uint64_t n);
uint64_t launch_count();

// Checks the launch that was just enqueued.
#define AG_CHECK_LAUNCH()                  \
    do {                                   \
        ::ag::count_launch();              \
        AG_CUDA_TRY(cudaGetLastError());   \
    } while (0)

}  // namespace ag

// ---- device object ---------------------------------------------------------
// One per (GPU, stream).  Owns a scratch workspace that kernels such as the
// split-k GEMM use for partial sums, a device status word that bounded device
// waits report into, and a pinned host word for scalar read-backs.
struct ag_device {
    int ordinal = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 0;
    std::recursive_mutex mu;
    void *workspace = nullptr;
    size_t workspace_bytes = 0;
    void *staging = nullptr;        // second scratch block: operand re-layouts of the
    size_t staging_bytes = 0;       // tensor-core convolution (may be live next to workspace)
    std::vector<void *> retired;    // outgrown scratch blocks that captured graphs may still use
    int *status_dev = nullptr;      // device word: 0 = ok, else a timeout code
    int *status_host = nullptr;     // pinned mirror
    float *scalar_dev = nullptr;    // small device buffer for loss / accuracy sums (64 B)
    float *scalar_host = nullptr;   // pinned mirror
};

namespace ag {

// Makes `dev` current on the calling thread and locks it for the call.
class DeviceGuard {
   public:
    explicit DeviceGuard(ag_device *dev) : lock_(dev->mu) { err_ = cudaSetDevice(dev->ordinal); }
    cudaError_t error() const { return err_; }

   private:
    std::lock_guard<std::recursive_mutex> lock_;
    cudaError_t err_;
};

#define AG_ENTER(dev)                                                                     \
    AG_REQUIRE((dev) != nullptr, AG_ERR_INVALID, "device is null");                       \
    ::ag::DeviceGuard _guard(dev);                                                        \
    if (_guard.error() != cudaSuccess)                                                    \
    return ::ag::fail(AG_ERR_CUDA, "cudaSetDevice(%d) failed: %s", (dev)->ordinal,        \
                      cudaGetErrorString(_guard.error()))

// Returns a workspace of at least `bytes` (grown on demand; outgrown blocks stay allocated
// until the device is destroyed because captured graphs may still point into them).
int workspace(ag_device *dev, size_t bytes, void **out);
// The same for the second scratch block.
int staging(ag_device *dev, size_t bytes, void **out);

inline size_t dtype_size(ag_dtype t) {
    switch (t) {
        case AG_F32: return 4;
        case AG_BF16: return 2;
        case AG_U8: return 1;
        case AG_U16: return 2;
        case AG_U32: return 4;
    }
    return 0;
}

inline bool is_float_dtype(ag_dtype t) { return t == AG_F32 || t == AG_BF16; }
inline bool is_label_dtype(ag_dtype t) { return t == AG_U8 || t == AG_U16 || t == AG_U32; }

// ---- element conversion (device) ------------------------------------------
__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
template <class T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) {
    return x;
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

// Unsigned division by a runtime constant without a divide instruction.
// Valid for dividends below 2^31.
struct FastDiv {
    uint32_t d = 1, mul = 0, shr = 0;
    FastDiv() = default;
    explicit FastDiv(uint32_t divisor) : d(divisor) {
        if (divisor <= 1) {
            d = 1;
            return;
        }
        uint32_t l = 0;
        while ((1ull << l) < divisor) ++l;  // ceil(log2 d)
        uint64_t p = 31 + l;
        mul = (uint32_t)(((1ull << p) + divisor - 1) / divisor);
        shr = l - 1;
    }
    __device__ __forceinline__ uint32_t div(uint32_t n) const {
        return d == 1 ? n : (__umulhi(n, mul) >> shr);
    }
    __device__ __forceinline__ void divmod(uint32_t n, uint32_t &q, uint32_t &r) const {
        q = div(n);
        r = n - q * d;
    }
};

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace ag
