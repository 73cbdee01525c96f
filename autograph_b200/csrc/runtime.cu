// Device objects, memory, transfers and error reporting of the C ABI.
#include <atomic>
#include <cstring>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace ag {

char *error_buffer() {
    static thread_local char buf[1024] = {0};
    return buf;
}

int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 1024, fmt, ap);
    va_end(ap);
    return status;
}

static std::atomic<uint64_t> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
void count_launches(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
uint64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

// Growing a scratch block never frees the old one: captured CUDA graphs (the model's
// inference and training passes) carry the old address in their kernel parameters and
// tensor maps, and may be replayed after the growth.  The old block is retired instead and
// lives until the device object is destroyed; sizes at least double, so all retired blocks
// together are smaller than the live one.
static int grow_block(ag_device *dev, void **block, size_t *have, size_t bytes, size_t floor) {
    size_t want = *have ? *have * 2 : floor;
    if (want < bytes) want = bytes + bytes / 4;
    void *fresh = nullptr;
    AG_CUDA_TRY(cudaMalloc(&fresh, want));
    if (*block) dev->retired.push_back(*block);
    *block = fresh;
    *have = want;
    return AG_OK;
}

int workspace(ag_device *dev, size_t bytes, void **out) {
    if (bytes > dev->workspace_bytes)
        AG_TRY(grow_block(dev, &dev->workspace, &dev->workspace_bytes, bytes, size_t(8) << 20));
    *out = dev->workspace;
    return AG_OK;
}

int staging(ag_device *dev, size_t bytes, void **out) {
    if (bytes > dev->staging_bytes)
        AG_TRY(grow_block(dev, &dev->staging, &dev->staging_bytes, bytes, size_t(1) << 20));
    *out = dev->staging;
    return AG_OK;
}

static int device_init(int ordinal, cudaStream_t stream, bool owns, ag_device **out) {
    AG_REQUIRE(out != nullptr, AG_ERR_INVALID, "out is null");
    int count = 0;
    AG_CUDA_TRY(cudaGetDeviceCount(&count));
    AG_REQUIRE(ordinal >= 0 && ordinal < count, AG_ERR_INVALID,
               "device ordinal %d out of range (%d devices)", ordinal, count);
    AG_CUDA_TRY(cudaSetDevice(ordinal));
    cudaDeviceProp prop;
    AG_CUDA_TRY(cudaGetDeviceProperties(&prop, ordinal));
    AG_REQUIRE(prop.major == 10, AG_ERR_UNSUPPORTED,
               "device %d is sm_%d%d; this library only carries sm_100a code", ordinal, prop.major,
               prop.minor);
    ag_device *dev = new ag_device();
    dev->ordinal = ordinal;
    dev->sm_count = prop.multiProcessorCount;
    dev->owns_stream = owns;
    if (owns) {
        cudaError_t e = cudaStreamCreateWithFlags(&dev->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            delete dev;
            return fail(AG_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(e));
        }
    } else {
        dev->stream = stream;
    }
    cudaError_t e = cudaMalloc(&dev->status_dev, 64);
    if (e == cudaSuccess) e = cudaMalloc(&dev->scalar_dev, 64);
    if (e == cudaSuccess) e = cudaMallocHost(&dev->status_host, 64);
    if (e == cudaSuccess) e = cudaMallocHost(&dev->scalar_host, 64);
    if (e == cudaSuccess) e = cudaMemsetAsync(dev->status_dev, 0, 64, dev->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(dev->scalar_dev, 0, 64, dev->stream);
    if (e != cudaSuccess) {
        ag_device_destroy(dev);
        return fail(AG_ERR_CUDA, "device set-up failed: %s", cudaGetErrorString(e));
    }
    *out = dev;
    return AG_OK;
}

// One CTA waits on an mbarrier that nothing will ever complete, with the library's bounded wait
// and the caller's limit: the wait runs out, the kernel records status 199 and returns.
__global__ void expiring_wait_kernel(uint64_t limit_ns, int *status) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        tc::mbar_init(tc::smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (!tc::mbar_wait_for(tc::smem_u32(&bar), 0, &abort_flag, limit_ns) && threadIdx.x == 0)
        atomicCAS(status, 0, 199);
}

}  // namespace ag

using namespace ag;

extern "C" {

int ag_debug_expiring_wait(ag_device *dev, uint64_t limit_ns) {
    AG_ENTER(dev);
    AG_REQUIRE(limit_ns > 0 && limit_ns <= 1000000000ull, AG_ERR_INVALID,
               "limit must be between 1 ns and 1 s");
    expiring_wait_kernel<<<1, 64, 0, dev->stream>>>(limit_ns, dev->status_dev);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

const char *ag_last_error(void) { return error_buffer(); }

const char *ag_version(void) { return "autograph_b200 0.1 (sm_100a)"; }

int ag_kernel_launch_count(uint64_t *count) {
    AG_REQUIRE(count != nullptr, AG_ERR_INVALID, "count is null");
    *count = g_launches.load(std::memory_order_relaxed);
    return AG_OK;
}

int ag_device_count(int *count) {
    AG_REQUIRE(count != nullptr, AG_ERR_INVALID, "count is null");
    AG_CUDA_TRY(cudaGetDeviceCount(count));
    return AG_OK;
}

int ag_device_create(int ordinal, ag_device **out) { return device_init(ordinal, nullptr, true, out); }

int ag_device_create_on_stream(int ordinal, void *cuda_stream, ag_device **out) {
    return device_init(ordinal, (cudaStream_t)cuda_stream, false, out);
}

int ag_device_destroy(ag_device *dev) {
    if (!dev) return AG_OK;
    cudaSetDevice(dev->ordinal);
    if (dev->stream) cudaStreamSynchronize(dev->stream);
    if (dev->workspace) cudaFree(dev->workspace);
    if (dev->staging) cudaFree(dev->staging);
    for (void *p : dev->retired) cudaFree(p);
    if (dev->status_dev) cudaFree(dev->status_dev);
    if (dev->scalar_dev) cudaFree(dev->scalar_dev);
    if (dev->status_host) cudaFreeHost(dev->status_host);
    if (dev->scalar_host) cudaFreeHost(dev->scalar_host);
    if (dev->owns_stream && dev->stream) cudaStreamDestroy(dev->stream);
    delete dev;
    return AG_OK;
}

int ag_device_wait(ag_device *dev) {
    AG_ENTER(dev);
    AG_CUDA_TRY(cudaMemcpyAsync(dev->status_host, dev->status_dev, sizeof(int),
                                cudaMemcpyDeviceToHost, dev->stream));
    AG_CUDA_TRY(cudaStreamSynchronize(dev->stream));
    if (*dev->status_host != 0) {
        int code = *dev->status_host;
        cudaMemsetAsync(dev->status_dev, 0, sizeof(int), dev->stream);
        return fail(AG_ERR_DEVICE_TIMEOUT, "a bounded device-side wait gave up (code %d)", code);
    }
    return AG_OK;
}

void *ag_device_stream(ag_device *dev) { return dev ? (void *)dev->stream : nullptr; }

int ag_device_ordinal(ag_device *dev) { return dev ? dev->ordinal : -1; }

int ag_alloc(ag_device *dev, size_t bytes, void **dptr) {
    AG_ENTER(dev);
    AG_REQUIRE(dptr != nullptr, AG_ERR_INVALID, "dptr is null");
    *dptr = nullptr;
    if (bytes == 0) return AG_OK;
    AG_CUDA_TRY(cudaMalloc(dptr, bytes));
    return AG_OK;
}

int ag_free(ag_device *dev, void *dptr) {
    AG_ENTER(dev);
    if (!dptr) return AG_OK;
    AG_CUDA_TRY(cudaStreamSynchronize(dev->stream));
    AG_CUDA_TRY(cudaFree(dptr));
    return AG_OK;
}

int ag_host_alloc(size_t bytes, void **hptr) {
    AG_REQUIRE(hptr != nullptr, AG_ERR_INVALID, "hptr is null");
    *hptr = nullptr;
    if (bytes == 0) return AG_OK;
    AG_CUDA_TRY(cudaMallocHost(hptr, bytes));
    return AG_OK;
}

int ag_host_free(void *hptr) {
    if (hptr) AG_CUDA_TRY(cudaFreeHost(hptr));
    return AG_OK;
}

int ag_upload(ag_device *dev, void *dptr, const void *host, size_t bytes) {
    AG_ENTER(dev);
    if (bytes == 0) return AG_OK;
    AG_REQUIRE(dptr && host, AG_ERR_INVALID, "null pointer in upload");
    AG_CUDA_TRY(cudaMemcpyAsync(dptr, host, bytes, cudaMemcpyHostToDevice, dev->stream));
    return AG_OK;
}

int ag_download(ag_device *dev, void *host, const void *dptr, size_t bytes) {
    AG_ENTER(dev);
    if (bytes == 0) return AG_OK;
    AG_REQUIRE(dptr && host, AG_ERR_INVALID, "null pointer in download");
    AG_CUDA_TRY(cudaMemcpyAsync(host, dptr, bytes, cudaMemcpyDeviceToHost, dev->stream));
    AG_CUDA_TRY(cudaStreamSynchronize(dev->stream));
    return AG_OK;
}

int ag_copy(ag_device *dev, void *dst, const void *src, size_t bytes) {
    AG_ENTER(dev);
    if (bytes == 0) return AG_OK;
    AG_REQUIRE(dst && src, AG_ERR_INVALID, "null pointer in copy");
    AG_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, dev->stream));
    return AG_OK;
}

int ag_fill_zero(ag_device *dev, void *dptr, size_t bytes) {
    AG_ENTER(dev);
    if (bytes == 0) return AG_OK;
    AG_REQUIRE(dptr != nullptr, AG_ERR_INVALID, "null pointer in fill");
    AG_CUDA_TRY(cudaMemsetAsync(dptr, 0, bytes, dev->stream));
    return AG_OK;
}

}  // extern "C"
