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

    // one layer of the chain code: the same sums in the same order as inside every fused kernel
    ChainStep st;
    st.w = w; st.bias = bias;
    st.K = K; st.N = N; st.np = np; st.slices = slices; st.kchunk = kchunk; st.relu = relu;
    st.pre = nullptr; st.act = nullptr;
    st.transposed = 0; st.gate = nullptr;
    chain_layer<T>(st, w, xs, nullptr, red, m0, rows, true, y);
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

// ---------------------------------------------------------------- backward
template <class T>
__global__ void __launch_bounds__(1024)
    dense_chain_backward_kernel(const T *__restrict__ dy, const T *__restrict__ gate_last,
                                T *__restrict__ g_last, T *__restrict__ y, const ChainParams p) {
    extern __shared__ __align__(16) float smem[];
    float *xa = smem;
    float *xb = smem + (size_t)p.max_k * ROWS;
    float *red = xb + (size_t)p.max_k * ROWS;
    const int m0 = blockIdx.x * ROWS;
    const int rows = min(ROWS, p.M - m0);
    {
        const int K = p.s[0].K;
        for (int i = threadIdx.x; i < ROWS * K; i += blockDim.x) {
            const int r = i / K, k = i - r * K;
            float v = 0.f;
            if (r < rows) {
                const int64_t at = (int64_t)(m0 + r) * K + k;
                v = to_f32(dy[at]);
                if (gate_last != nullptr) {
                    if (!(to_f32(gate_last[at]) >= 0.f)) v = 0.f;
                    g_last[at] = from_f32<T>(v);
                }
            }
            xa[k * ROWS + r] = v;
        }
    }
    __syncthreads();
    chain_layers<T>(xa, xb, red, p, m0, rows, y);
}

bool chain_backward_eligible(int64_t m, int n_steps, const ChainLayer *steps) {
    if (n_steps < 1 || n_steps > kMaxChain) return false;
    for (int i = 0; i < n_steps; ++i) {
        if (!eligible(m, steps[i].inputs, steps[i].outputs)) return false;
        if (i > 0 && steps[i].inputs != steps[i - 1].outputs) return false;
    }
    return true;
}

template <class T>
int chain_backward_input(ag_device *dev, const T *dy, int m, int n_steps, const ChainLayer *steps,
                         const T *gate_last, T *g_last, T *y) {
    ChainParams p;
    const size_t smem = plan_chain(&p, m, n_steps, steps) * sizeof(float);
    auto kernel = dense_chain_backward_kernel<T>;
    if (smem > 48 * 1024)
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    kernel<<<(unsigned)ceil_div(m, ROWS), p.threads, smem, dev->stream>>>(dy, gate_last, g_last, y, p);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

// A 32 x 32 tile of one problem's dw per CTA of 256 threads.  The reduction runs over the
// batch in chunks of 128 rows staged whole in shared memory; the four groups of 64 threads
// each take a quarter of every chunk for the full tile (4 x 4 outputs per thread) and their
// sums are added in group order.  The CTAs of a problem's first tile row also add up the
// columns of g (the bias gradient), row after row.
constexpr int kWgChunk = 128, kWgPitch = 36;
struct WgradParams {
    WgradProblem p[kMaxChain];
    int n, M;
};

template <class T>
__global__ void __launch_bounds__(256) dense_wgrad_group_kernel(const WgradParams P) {
    __shared__ __align__(16) float As[kWgChunk][kWgPitch];
    __shared__ __align__(16) float Bs[kWgChunk][kWgPitch];
    int q = 0;
    while (q + 1 < P.n && (int)blockIdx.x >= P.p[q + 1].tile0) ++q;
    const WgradProblem pr = P.p[q];
    const int tile = blockIdx.x - pr.tile0;
    const int tm = tile / pr.tiles_n, tn = tile - tm * pr.tiles_n;
    const int m0 = tm * 32, n0 = tn * 32;
    const T *in = reinterpret_cast<const T *>(pr.in), *g = reinterpret_cast<const T *>(pr.g);
    const int tid = threadIdx.x;
    const int mn = tid & 31, kb = tid >> 5;  // staging: 32 consecutive columns of one batch row
    const int kg = tid >> 6, t = tid & 63, tx = t & 7, ty = t >> 3;
    const bool sums = pr.db != nullptr && tm == 0 && tid < 32;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    float bsum = 0.f;

    for (int kc = 0; kc < P.M; kc += kWgChunk) {
        const int chunk = min(kWgChunk, P.M - kc);
        float ra[kWgChunk / 8], rb[kWgChunk / 8];
#pragma unroll
        for (int i = 0; i < kWgChunk / 8; ++i)
            if (i * 8 < chunk) {
                const int k = i * 8 + kb;
                const bool ok = k < chunk;
                ra[i] = (ok && m0 + mn < pr.rows)
                            ? to_f32(in[(int64_t)(kc + k) * pr.rows + m0 + mn]) : 0.f;
                rb[i] = (ok && n0 + mn < pr.cols)
                            ? to_f32(g[(int64_t)(kc + k) * pr.cols + n0 + mn]) : 0.f;
            }
        if (kc > 0) __syncthreads();  // the previous chunk is no longer read
#pragma unroll
        for (int i = 0; i < kWgChunk / 8; ++i)
            if (i * 8 < chunk) {
                As[i * 8 + kb][mn] = ra[i];
                Bs[i * 8 + kb][mn] = rb[i];
            }
        __syncthreads();
        const int kp = (chunk + 7) & ~7;
        const int kq = (kp / 8 + 3) / 4 * 8;
        const int k0 = min(kp, kg * kq), k1 = min(kp, k0 + kq);
#pragma unroll 4
        for (int k = k0; k < k1; ++k) {
            const float4 a4 = *reinterpret_cast<const float4 *>(&As[k][ty * 4]);
            const float4 b4 = *reinterpret_cast<const float4 *>(&Bs[k][tx * 4]);
            const float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (sums)
            for (int k = 0; k < chunk; ++k) bsum += Bs[k][tid];
    }
    __syncthreads();
    float *red = &As[0][0];  // [3 groups][16 values][64 threads]
    if (kg > 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) red[((kg - 1) * 16 + i) * 64 + t] = acc[i / 4][i % 4];
    }
    __syncthreads();
    if (sums && n0 + tid < pr.cols) reinterpret_cast<T *>(pr.db)[n0 + tid] = from_f32<T>(bsum);
    if (kg > 0) return;
#pragma unroll
    for (int gi = 0; gi < 3; ++gi)
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i / 4][i % 4] += red[(gi * 16 + i) * 64 + t];
    T *dw = reinterpret_cast<T *>(pr.dw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= pr.rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < pr.cols) dw[(int64_t)m * pr.cols + n] = from_f32<T>(acc[i][j]);
        }
    }
}

template <class T>
int chain_weight_grads(ag_device *dev, int m, int n, WgradProblem *problems) {
    WgradParams P;
    P.n = n;
    P.M = m;
    int tiles = 0;
    for (int i = 0; i < n; ++i) {
        problems[i].tile0 = tiles;
        problems[i].tiles_n = (problems[i].cols + 31) / 32;
        tiles += ((problems[i].rows + 31) / 32) * problems[i].tiles_n;
        P.p[i] = problems[i];
    }
    if (tiles == 0) return AG_OK;
    dense_wgrad_group_kernel<T><<<(unsigned)tiles, 256, 0, dev->stream>>>(P);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

template int chain_backward_input<float>(ag_device *, const float *, int, int, const ChainLayer *,
                                         const float *, float *, float *);
template int chain_backward_input<__nv_bfloat16>(ag_device *, const __nv_bfloat16 *, int, int,
                                                 const ChainLayer *, const __nv_bfloat16 *,
                                                 __nv_bfloat16 *, __nv_bfloat16 *);
template int chain_weight_grads<float>(ag_device *, int, int, WgradProblem *);
template int chain_weight_grads<__nv_bfloat16>(ag_device *, int, int, WgradProblem *);

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
