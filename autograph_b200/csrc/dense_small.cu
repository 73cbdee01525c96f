// Latency-oriented kernel for small dense products (m up to a few thousand
// rows, n <= 256 outputs): y[m,n] = x[m,k] . w[k,n] (+ bias) (relu), row-major.
//
// At these sizes a shared-memory-tiled GEMM runs two warps per SM through a
// chain of load -> barrier -> multiply steps and is bound by memory and
// instruction-fetch latency.  Here a CTA owns 8 rows of x (staged once in
// shared memory, transposed so that the 8 row values of one k are two 16-byte
// loads) and up to 1024 threads split the work as (output column, k slice):
// each thread streams its weights straight from L2 with coalesced loads and
// keeps 8 accumulators.  The k slices are then summed in a fixed order, so the
// result is deterministic.  The code is small on purpose.
#include "dense_small.cuh"
#include "dense_small_device.cuh"

namespace ag {
namespace dense_small {

template <class T>
__global__ void __launch_bounds__(1024)
    dense_small_kernel(const T *__restrict__ x, const T *__restrict__ w,
                       const T *__restrict__ bias, T *__restrict__ y, int M, int K, int N, int np,
                       int slices, int kchunk, int relu) {
    extern __shared__ __align__(16) float smem[];
    float *xs = smem;                          // [K][ROWS]
    float *red = smem + (size_t)K * ROWS;      // [slices][ROWS][np]
    const int m0 = blockIdx.x * ROWS;
    const int rows = min(ROWS, M - m0);

    for (int i = threadIdx.x; i < ROWS * K; i += blockDim.x) {
        const int r = i / K, k = i - r * K;    // coalesced along k
        xs[k * ROWS + r] = (r < rows) ? to_f32(x[(int64_t)(m0 + r) * K + k]) : 0.f;
    }
    __syncthreads();

    const int n = threadIdx.x % np, slice = threadIdx.x / np;
    float acc[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
    if (n < N && slice < slices) {
        const int k0 = slice * kchunk, k1 = min(K, k0 + kchunk);
        const T *wp = w + (int64_t)k0 * N + n;
#pragma unroll 8
        for (int k = k0; k < k1; ++k, wp += N) {
            const float wv = to_f32(*wp);
            const float4 a = *reinterpret_cast<const float4 *>(xs + k * ROWS);
            const float4 b = *reinterpret_cast<const float4 *>(xs + k * ROWS + 4);
            acc[0] = fmaf(a.x, wv, acc[0]); acc[1] = fmaf(a.y, wv, acc[1]);
            acc[2] = fmaf(a.z, wv, acc[2]); acc[3] = fmaf(a.w, wv, acc[3]);
            acc[4] = fmaf(b.x, wv, acc[4]); acc[5] = fmaf(b.y, wv, acc[5]);
            acc[6] = fmaf(b.z, wv, acc[6]); acc[7] = fmaf(b.w, wv, acc[7]);
        }
    }
    if (slice < slices) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) red[(slice * ROWS + r) * np + n] = acc[r];
    }
    __syncthreads();

    for (int i = threadIdx.x; i < ROWS * np; i += blockDim.x) {
        const int r = i / np, c = i - r * np;
        if (r >= rows || c >= N) continue;
        float s = 0.f;
        for (int sl = 0; sl < slices; ++sl) s += red[(sl * ROWS + r) * np + c];
        float v = to_f32(from_f32<T>(s));
        if (bias != nullptr) v = to_f32(from_f32<T>(__fadd_rn(v, to_f32(bias[c]))));
        if (relu) v = (v >= 0.f) ? v : 0.f;
        y[(int64_t)(m0 + r) * N + c] = from_f32<T>(v);
    }
}

bool eligible(int64_t m, int64_t k, int64_t n) {
    return m > 0 && m <= 4096 && n > 0 && n <= 256 && k > 0 && k <= 2048;
}

template <class T>
int forward(ag_device *dev, const T *x, int m, int k, const T *w, int n, const T *bias, bool relu,
            T *y) {
    const int np = ((n + 31) / 32) * 32;
    int slices = 1024 / np;
    if (slices > 16) slices = 16;
    if (slices > k / 8) slices = k / 8;
    if (slices < 1) slices = 1;
    const int kchunk = (k + slices - 1) / slices;
    slices = (k + kchunk - 1) / kchunk;
    const int threads = np * slices;
    const size_t smem = ((size_t)k * ROWS + (size_t)slices * ROWS * np) * sizeof(float);
    auto kernel = dense_small_kernel<T>;
    if (smem > 48 * 1024)
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    kernel<<<(unsigned)ceil_div(m, ROWS), threads, smem, dev->stream>>>(x, w, bias, y, m, k, n, np,
                                                                         slices, kchunk, relu ? 1 : 0);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

// ---------------------------------------------------------------- layer chain
template <class T>
__global__ void __launch_bounds__(1024)
    dense_chain_kernel(const T *__restrict__ x, T *__restrict__ y, const ChainParams p) {
    extern __shared__ __align__(16) float smem[];
    float *xa = smem;                              // [max_k][ROWS] current layer input
    float *xb = smem + (size_t)p.max_k * ROWS;     // next layer input
    float *red = xb + (size_t)p.max_k * ROWS;      // [slices][ROWS][np]
    const int m0 = blockIdx.x * ROWS;
    const int rows = min(ROWS, p.M - m0);
    {
        const int K = p.s[0].K;
        for (int i = threadIdx.x; i < ROWS * K; i += blockDim.x) {
            const int r = i / K, k = i - r * K;
            xa[k * ROWS + r] = (r < rows) ? to_f32(x[(int64_t)(m0 + r) * K + k]) : 0.f;
        }
    }
    __syncthreads();
    chain_layers<T>(xa, xb, red, p, m0, rows, y);
}

bool chain_eligible(int64_t m, int n_layers, const ChainLayer *layers) {
    if (n_layers < 2 || n_layers > kMaxChain) return false;
    for (int i = 0; i < n_layers; ++i) {
        if (!eligible(m, layers[i].inputs, layers[i].outputs)) return false;
        if (i > 0 && layers[i].inputs != layers[i - 1].outputs) return false;
    }
    return true;
}

template <class T>
int chain_forward(ag_device *dev, const T *x, int m, int n_layers, const ChainLayer *layers, T *y) {
    ChainParams p;
    const size_t smem = plan_chain(&p, m, n_layers, layers) * sizeof(float);
    const int threads = p.threads;
    auto kernel = dense_chain_kernel<T>;
    if (smem > 48 * 1024)
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    kernel<<<(unsigned)ceil_div(m, ROWS), threads, smem, dev->stream>>>(x, y, p);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

template int chain_forward<float>(ag_device *, const float *, int, int, const ChainLayer *, float *);
template int chain_forward<__nv_bfloat16>(ag_device *, const __nv_bfloat16 *, int, int,
                                          const ChainLayer *, __nv_bfloat16 *);

template int forward<float>(ag_device *, const float *, int, int, const float *, int, const float *,
                            bool, float *);
template int forward<__nv_bfloat16>(ag_device *, const __nv_bfloat16 *, int, int,
                                    const __nv_bfloat16 *, int, const __nv_bfloat16 *, bool,
                                    __nv_bfloat16 *);

}  // namespace dense_small
}  // namespace ag
