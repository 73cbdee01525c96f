// Cross-entropy loss (value and gradient) and accuracy.  One warp per row; the
// row maximum and the sum of exponentials are warp-shuffle reductions in f32,
// as the reference computes them in f32 for both element types.
#include "common.cuh"

namespace ag {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <class L>
__device__ __forceinline__ uint32_t label_at(const L *t, int64_t i) {
    return (uint32_t)t[i];
}

// row_loss[r] = ln(sum exp(x - m)) - (x_t - m); a label outside [0, classes)
// contributes x_t = 0 like the reference's device kernel.
template <class T, class L>
__global__ void ce_loss_rows_kernel(const T *__restrict__ x, const L *__restrict__ t, int64_t bs,
                                    int classes, float *__restrict__ row_loss) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < bs; r += warps) {
        const T *row = x + r * classes;
        float m = -INFINITY;
        for (int i = lane; i < classes; i += 32) m = fmaxf(m, to_f32(row[i]));
        m = warp_max(m);
        float s = 0.f;
        for (int i = lane; i < classes; i += 32) s += expf(to_f32(row[i]) - m);
        s = warp_sum(s);
        if (lane == 0) {
            uint32_t tt = label_at(t, r);
            float xt = tt < (uint32_t)classes ? to_f32(row[tt]) : 0.f;
            row_loss[r] = logf(s) - (xt - m);
        }
    }
}

// Sums n floats into out[0] with one CTA (fixed order: deterministic).
__global__ void sum_rows_kernel(const float *__restrict__ v, int64_t n, float *__restrict__ out) {
    __shared__ float part[1024];
    float s = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) s += v[i];
    part[threadIdx.x] = s;
    __syncthreads();
    for (int off = blockDim.x / 2; off > 0; off >>= 1) {
        if ((int)threadIdx.x < off) part[threadIdx.x] += part[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[0] = part[0];
}

// Both steps in one CTA for bs <= 1024: the row losses stay in shared memory and are added
// by the same tree as sum_rows_kernel.
template <class T, class L>
__global__ void __launch_bounds__(1024)
    ce_loss_small_kernel(const T *__restrict__ x, const L *__restrict__ t, int bs, int classes,
                         float *__restrict__ out, float dy, T *__restrict__ dx) {
    __shared__ float part[1024];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    part[threadIdx.x] = 0.f;
    __syncthreads();
    if (classes <= 32) {
        // a thread per row: the rows' loads are all in flight together
        const int r = threadIdx.x;
        if (r < bs) {
            const T *row = x + (int64_t)r * classes;
            const uint32_t tt = label_at(t, r);
            float m = -INFINITY;
            for (int i = 0; i < classes; ++i) m = fmaxf(m, to_f32(row[i]));
            float s = 0.f, xt = 0.f;
            for (int i = 0; i < classes; ++i) {
                const float v = to_f32(row[i]);
                s += expf(v - m);
                if ((uint32_t)i == tt) xt = v;
            }
            part[r] = logf(s) - (xt - m);
            if (dx != nullptr)  // the gradient the backward edge would compute: dy (softmax - onehot)
                for (int i = 0; i < classes; ++i) {
                    const float onehot = ((uint32_t)i == tt) ? 1.f : 0.f;
                    const float g = __fmul_rn(
                        dy, __fsub_rn(__fdiv_rn(expf(to_f32(row[i]) - m), s), onehot));
                    dx[(int64_t)r * classes + i] = from_f32<T>(g);
                }
        }
    } else {
        for (int r = warp; r < bs; r += 32) {
            const T *row = x + (int64_t)r * classes;
            float m = -INFINITY;
            for (int i = lane; i < classes; i += 32) m = fmaxf(m, to_f32(row[i]));
            m = warp_max(m);
            float s = 0.f;
            for (int i = lane; i < classes; i += 32) s += expf(to_f32(row[i]) - m);
            s = warp_sum(s);
            const uint32_t tt = label_at(t, r);
            if (lane == 0) {
                float xt = tt < (uint32_t)classes ? to_f32(row[tt]) : 0.f;
                part[r] = logf(s) - (xt - m);
            }
            if (dx != nullptr)
                for (int i = lane; i < classes; i += 32) {
                    const float onehot = ((uint32_t)i == tt) ? 1.f : 0.f;
                    const float g = __fmul_rn(
                        dy, __fsub_rn(__fdiv_rn(expf(to_f32(row[i]) - m), s), onehot));
                    dx[(int64_t)r * classes + i] = from_f32<T>(g);
                }
        }
    }
    __syncthreads();
    for (int off = 512; off > 0; off >>= 1) {
        if ((int)threadIdx.x < off) part[threadIdx.x] += part[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[0] = part[0];
}

template <class T, class L>
__global__ void ce_backward_kernel(const T *__restrict__ x, const L *__restrict__ t, int64_t bs,
                                   int classes, float dy, T *__restrict__ dx) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < bs; r += warps) {
        const T *row = x + r * classes;
        float m = -INFINITY;
        for (int i = lane; i < classes; i += 32) m = fmaxf(m, to_f32(row[i]));
        m = warp_max(m);
        float s = 0.f;
        for (int i = lane; i < classes; i += 32) s += expf(to_f32(row[i]) - m);
        s = warp_sum(s);
        const uint32_t tt = label_at(t, r);
        for (int i = lane; i < classes; i += 32) {
            float onehot = ((uint32_t)i == tt) ? 1.f : 0.f;
            float g = __fmul_rn(dy, __fsub_rn(__fdiv_rn(expf(to_f32(row[i]) - m), s), onehot));
            dx[r * classes + i] = from_f32<T>(g);
        }
    }
}

template <class T, class L>
__global__ void accuracy_kernel(const T *__restrict__ x, const L *__restrict__ t, int64_t bs,
                                int classes, unsigned long long *__restrict__ correct) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < bs; r += warps) {
        const T *row = x + r * classes;
        const uint32_t tt = label_at(t, r);
        bool ok = tt < (uint32_t)classes;
        if (ok) {
            const float xt = to_f32(row[tt]);
            for (int i = lane; i < classes; i += 32)
                if ((uint32_t)i != tt && !(xt > to_f32(row[i]))) ok = false;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok && lane == 0) atomicAdd(correct, 1ull);
    }
}

static unsigned warp_grid(int64_t rows, int threads, int sms) {
    int64_t blocks = ceil_div(rows * 32, threads);
    int64_t cap = (int64_t)sms * 8;
    return (unsigned)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

// Sum of the row losses into *loss_dev (device memory); no synchronisation.
template <class T, class L>
static int ce_loss_device(ag_device *dev, const T *x, const L *t, int64_t bs, int classes,
                          float *loss_dev, float dy = 0.f, T *dx = nullptr) {
    if (bs <= 1024) {
        ce_loss_small_kernel<T, L><<<1, 1024, 0, dev->stream>>>(x, t, (int)bs, classes, loss_dev,
                                                                dy / (float)bs, dx);
        AG_CHECK_LAUNCH();
        return AG_OK;
    }
    if (dx != nullptr) {
        const int threads = 256;
        ce_backward_kernel<T, L><<<warp_grid(bs, threads, dev->sm_count), threads, 0, dev->stream>>>(
            x, t, bs, classes, dy / (float)bs, dx);
        AG_CHECK_LAUNCH();
    }
    void *ws;
    AG_TRY(workspace(dev, sizeof(float) * (size_t)bs, &ws));
    const int threads = 256;
    ce_loss_rows_kernel<T, L><<<warp_grid(bs, threads, dev->sm_count), threads, 0, dev->stream>>>(
        x, t, bs, classes, (float *)ws);
    AG_CHECK_LAUNCH();
    sum_rows_kernel<<<1, 1024, 0, dev->stream>>>((const float *)ws, bs, loss_dev);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

template <class T, class L>
static int ce_loss(ag_device *dev, const T *x, const L *t, int64_t bs, int classes,
                   float *loss_host) {
    AG_TRY((ce_loss_device<T, L>(dev, x, t, bs, classes, dev->scalar_dev)));
    AG_CUDA_TRY(cudaMemcpyAsync(dev->scalar_host, dev->scalar_dev, sizeof(float),
                                cudaMemcpyDeviceToHost, dev->stream));
    AG_CUDA_TRY(cudaStreamSynchronize(dev->stream));
    *loss_host = dev->scalar_host[0];
    return AG_OK;
}

}  // namespace ag

using namespace ag;

#define AG_DISPATCH_XT(dtype, label, T, L, ...)                         \
    do {                                                                \
        if ((dtype) == AG_F32) {                                        \
            using T = float;                                            \
            if ((label) == AG_U8) { using L = uint8_t; __VA_ARGS__ }    \
            else if ((label) == AG_U16) { using L = uint16_t; __VA_ARGS__ } \
            else { using L = uint32_t; __VA_ARGS__ }                    \
        } else {                                                        \
            using T = __nv_bfloat16;                                    \
            if ((label) == AG_U8) { using L = uint8_t; __VA_ARGS__ }    \
            else if ((label) == AG_U16) { using L = uint16_t; __VA_ARGS__ } \
            else { using L = uint32_t; __VA_ARGS__ }                    \
        }                                                               \
    } while (0)

static int check_ce_args(ag_dtype dtype, ag_dtype label_dtype, int64_t bs, int64_t classes) {
    AG_REQUIRE(is_float_dtype(dtype) && is_label_dtype(label_dtype), AG_ERR_DTYPE,
               "CrossEntropyLoss %d %d unimplemented", (int)dtype, (int)label_dtype);
    AG_REQUIRE(bs >= 0 && classes > 0 && classes < (1ll << 31), AG_ERR_SHAPE,
               "bad shape [%lld,%lld]", (long long)bs, (long long)classes);
    return AG_OK;
}

extern "C" {

int ag_cross_entropy_loss(ag_device *dev, ag_dtype dtype, ag_dtype label_dtype, const void *x,
                          const void *t, int64_t bs, int64_t classes, float *loss_host) {
    AG_ENTER(dev);
    AG_TRY(check_ce_args(dtype, label_dtype, bs, classes));
    AG_REQUIRE(loss_host != nullptr, AG_ERR_INVALID, "loss_host is null");
    *loss_host = 0.f;
    if (bs == 0) return AG_OK;
    AG_REQUIRE(x && t, AG_ERR_INVALID, "null tensor pointer");
    AG_DISPATCH_XT(dtype, label_dtype, T, L,
                   return ce_loss<T, L>(dev, (const T *)x, (const L *)t, bs, (int)classes, loss_host););
}

int ag_cross_entropy_loss_device(ag_device *dev, ag_dtype dtype, ag_dtype label_dtype,
                                 const void *x, const void *t, int64_t bs, int64_t classes,
                                 float *loss_dev) {
    AG_ENTER(dev);
    AG_TRY(check_ce_args(dtype, label_dtype, bs, classes));
    AG_REQUIRE(loss_dev != nullptr, AG_ERR_INVALID, "loss_dev is null");
    if (bs == 0) return ag_fill_zero(dev, loss_dev, sizeof(float));
    AG_REQUIRE(x && t, AG_ERR_INVALID, "null tensor pointer");
    AG_DISPATCH_XT(dtype, label_dtype, T, L,
                   return ce_loss_device<T, L>(dev, (const T *)x, (const L *)t, bs, (int)classes, loss_dev););
}

int ag_cross_entropy_loss_device_grad(ag_device *dev, ag_dtype dtype, ag_dtype label_dtype,
                                      const void *x, const void *t, int64_t bs, int64_t classes,
                                      float *loss_dev, float dy, void *dx) {
    AG_ENTER(dev);
    AG_TRY(check_ce_args(dtype, label_dtype, bs, classes));
    AG_REQUIRE(loss_dev != nullptr, AG_ERR_INVALID, "loss_dev is null");
    if (bs == 0) return ag_fill_zero(dev, loss_dev, sizeof(float));
    AG_REQUIRE(x && t && dx, AG_ERR_INVALID, "null tensor pointer");
    AG_DISPATCH_XT(dtype, label_dtype, T, L,
                   return ce_loss_device<T, L>(dev, (const T *)x, (const L *)t, bs, (int)classes,
                                               loss_dev, dy, (T *)dx););
}

int ag_cross_entropy_loss_backward(ag_device *dev, ag_dtype dtype, ag_dtype label_dtype,
                                   const void *x, const void *t, int64_t bs, int64_t classes,
                                   float dy, void *dx) {
    AG_ENTER(dev);
    AG_TRY(check_ce_args(dtype, label_dtype, bs, classes));
    if (bs == 0) return AG_OK;
    AG_REQUIRE(x && t && dx, AG_ERR_INVALID, "null tensor pointer");
    const float scaled = dy / (float)bs;
    const int threads = 256;
    const unsigned grid = warp_grid(bs, threads, dev->sm_count);
    AG_DISPATCH_XT(dtype, label_dtype, T, L,
                   ce_backward_kernel<T, L><<<grid, threads, 0, dev->stream>>>(
                       (const T *)x, (const L *)t, bs, (int)classes, scaled, (T *)dx););
    AG_CHECK_LAUNCH();
    return AG_OK;
}

int ag_accuracy(ag_device *dev, ag_dtype dtype, ag_dtype label_dtype, const void *x, const void *t,
                int64_t bs, int64_t classes, uint64_t *correct_host) {
    AG_ENTER(dev);
    AG_TRY(check_ce_args(dtype, label_dtype, bs, classes));
    AG_REQUIRE(correct_host != nullptr, AG_ERR_INVALID, "correct_host is null");
    *correct_host = 0;
    if (bs == 0) return AG_OK;
    AG_REQUIRE(x && t, AG_ERR_INVALID, "null tensor pointer");
    unsigned long long *counter = reinterpret_cast<unsigned long long *>(dev->scalar_dev + 2);
    AG_CUDA_TRY(cudaMemsetAsync(counter, 0, sizeof(unsigned long long), dev->stream));
    const int threads = 256;
    const unsigned grid = warp_grid(bs, threads, dev->sm_count);
    AG_DISPATCH_XT(dtype, label_dtype, T, L,
                   accuracy_kernel<T, L><<<grid, threads, 0, dev->stream>>>(
                       (const T *)x, (const L *)t, bs, (int)classes, counter););
    AG_CHECK_LAUNCH();
    AG_CUDA_TRY(cudaMemcpyAsync(dev->scalar_host + 2, counter, sizeof(unsigned long long),
                                cudaMemcpyDeviceToHost, dev->stream));
    AG_CUDA_TRY(cudaStreamSynchronize(dev->stream));
    *correct_host = *reinterpret_cast<unsigned long long *>(dev->scalar_host + 2);
    return AG_OK;
}

}  // extern "C"
