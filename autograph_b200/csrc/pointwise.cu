// Memory-bound operators: relu, max-pool, scaled add, bias add / bias gradient
// and the SGD updates.  Each kernel moves 16 bytes per thread per access where
// the layout allows it and is sized as a grid-stride loop over a multiple of
// the SM count.  Arithmetic is written with explicit round-to-nearest multiply
// and add (no fused multiply-add) so that results are bit-identical to the
// reference's host code, which does not contract.
#include <algorithm>

#include "common.cuh"

namespace ag {

static unsigned grid_for(int64_t items, int threads, int sms) {
    int64_t blocks = ceil_div(items, threads);
    int64_t cap = (int64_t)sms * 8;
    return (unsigned)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

// 16-byte vector of T.
template <class T>
struct Vec16 {
    static constexpr int N = 16 / sizeof(T);
    uint4 raw;
    __device__ __forceinline__ float get(int i) const;
    __device__ __forceinline__ void set(int i, float v);
};
template <>
__device__ __forceinline__ float Vec16<float>::get(int i) const {
    return __uint_as_float((&raw.x)[i]);
}
template <>
__device__ __forceinline__ void Vec16<float>::set(int i, float v) {
    (&raw.x)[i] = __float_as_uint(v);
}
template <>
__device__ __forceinline__ float Vec16<__nv_bfloat16>::get(int i) const {
    uint32_t w = (&raw.x)[i >> 1];
    return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
}
template <>
__device__ __forceinline__ void Vec16<__nv_bfloat16>::set(int i, float v) {
    __nv_bfloat16 h = __float2bfloat16_rn(v);
    uint32_t bits = *reinterpret_cast<unsigned short *>(&h);
    uint32_t &w = (&raw.x)[i >> 1];
    w = (i & 1) ? ((w & 0x0000ffffu) | (bits << 16)) : ((w & 0xffff0000u) | bits);
}

template <class T>
static bool aligned16(const T *p) {
    return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

// ---- generic unary / binary / ternary element-wise driver --------------------
// f(i, in0[i], in1[i]) -> out[i]; vector body when every pointer is 16-byte aligned.
template <class T, class F>
__global__ void map2_kernel(const T *a, const T *b, T *out,
                            int64_t n, bool vec, F f) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    constexpr int V = Vec16<T>::N;
    int64_t done = 0;
    if (vec) {
        const int64_t nv = n / V;
        for (int64_t i = tid; i < nv; i += stride) {
            Vec16<T> va, vb, vo;
            va.raw = reinterpret_cast<const uint4 *>(a)[i];
            vb.raw = b ? reinterpret_cast<const uint4 *>(b)[i] : va.raw;
            vo.raw = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int j = 0; j < V; ++j) vo.set(j, f(va.get(j), vb.get(j)));
            reinterpret_cast<uint4 *>(out)[i] = vo.raw;
        }
        done = nv * V;
    }
    for (int64_t i = done + tid; i < n; i += stride) {
        float x = to_f32(a[i]);
        float y = b ? to_f32(b[i]) : x;
        out[i] = from_f32<T>(f(x, y));
    }
}

template <class T, class F>
static int map2(ag_device *dev, const T *a, const T *b, T *out, int64_t n, F f) {
    if (n == 0) return AG_OK;
    const bool vec = aligned16(a) && aligned16(out) && (b == nullptr || aligned16(b));
    const int threads = 256;
    const int64_t items = vec ? ceil_div(n, Vec16<T>::N) : n;
    map2_kernel<T, F><<<grid_for(items, threads, dev->sm_count), threads, 0, dev->stream>>>(
        a, b, out, n, vec, f);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

struct ReluF {
    __device__ __forceinline__ float operator()(float x, float) const {
        return (x >= 0.f) ? x : 0.f;
    }
};
struct ReluBackwardF {  // (x, dy)
    __device__ __forceinline__ float operator()(float x, float dy) const {
        return (x >= 0.f) ? dy : 0.f;
    }
};
template <class T>
struct ScaledAddF {  // (x, y) -> alpha*x + y in T arithmetic
    float alpha;
    __device__ __forceinline__ float operator()(float x, float y) const {
        float p = to_f32(from_f32<T>(__fmul_rn(alpha, x)));
        return __fadd_rn(p, y);
    }
};

// ---- max pool ---------------------------------------------------------------
template <class T>
__global__ void max_pool2_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t planes,
                                 int ih, int iw, int oh, int ow, int h, int w, int sh, int sw) {
    const int64_t total = planes * oh * ow;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int wid = (int)(i % ow);
        int64_t t = i / ow;
        int hid = (int)(t % oh);
        int64_t plane = t / oh;
        const T *src = x + (plane * ih + (int64_t)hid * sh) * iw + (int64_t)wid * sw;
        float m = 0.f;
        for (int fi = 0; fi < h; ++fi)
            for (int fj = 0; fj < w; ++fj) {
                float v = to_f32(src[fi * iw + fj]);
                if ((fi == 0 && fj == 0) || v > m) m = v;
            }
        y[i] = from_f32<T>(m);
    }
}

// 2x2 window, stride 2, even width, 16-byte aligned rows: each thread reads two
// 16-byte row segments and writes V/2 outputs.
template <class T>
__global__ void max_pool2_2x2_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t planes,
                                     int ih, int iw, int oh, int ow) {
    constexpr int V = Vec16<T>::N;  // inputs per vector
    const int vec_per_row = iw / V;
    const int64_t total = planes * oh * vec_per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int vx = (int)(i % vec_per_row);
        int64_t t = i / vec_per_row;
        int hid = (int)(t % oh);
        int64_t plane = t / oh;
        const T *r0 = x + (plane * ih + 2 * (int64_t)hid) * iw + vx * V;
        Vec16<T> a, b;
        a.raw = *reinterpret_cast<const uint4 *>(r0);
        b.raw = *reinterpret_cast<const uint4 *>(r0 + iw);
        T *dst = y + (plane * oh + hid) * (int64_t)ow + vx * (V / 2);
#pragma unroll
        for (int j = 0; j < V / 2; ++j) {
            float m = a.get(2 * j);
            float v = a.get(2 * j + 1);
            if (v > m) m = v;
            v = b.get(2 * j);
            if (v > m) m = v;
            v = b.get(2 * j + 1);
            if (v > m) m = v;
            dst[j] = from_f32<T>(m);
        }
    }
}

// One thread per window; windows do not overlap, so no two threads touch the
// same cell.  dx holds the forward input on entry.
template <class T>
__global__ void max_pool2_backward_kernel(T *__restrict__ dx, const T *__restrict__ dy,
                                          int64_t planes, int ih, int iw, int oh, int ow, int h,
                                          int w, int sh, int sw) {  // in place only
    const int64_t total = planes * oh * ow;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int wid = (int)(i % ow);
        int64_t t = i / ow;
        int hid = (int)(t % oh);
        int64_t plane = t / oh;
        T *win = dx + (plane * ih + (int64_t)hid * sh) * iw + (int64_t)wid * sw;
        float m = 0.f;
        int am = 0;
        for (int fi = 0; fi < h; ++fi)
            for (int fj = 0; fj < w; ++fj) {
                float v = to_f32(win[fi * iw + fj]);
                if ((fi == 0 && fj == 0) || v > m) {
                    m = v;
                    am = fi * iw + fj;
                }
                win[fi * iw + fj] = from_f32<T>(0.f);
            }
        win[am] = from_f32<T>(__fadd_rn(0.f, to_f32(dy[i])));
    }
}

// 2x2 window, stride 2, width a multiple of the vector length, 16-byte aligned rows:
// each thread owns V/2 adjacent windows, reads and rewrites two 16-byte row segments.
template <class T>
__global__ void max_pool2_backward_2x2_kernel(const T *src, T *dx, const T *__restrict__ dy,
                                              int64_t planes, int ih, int iw, int oh, int ow) {
    constexpr int V = Vec16<T>::N;
    const int vec_per_row = iw / V;
    const int64_t total = planes * oh * vec_per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int vx = (int)(i % vec_per_row);
        int64_t t = i / vec_per_row;
        int hid = (int)(t % oh);
        int64_t plane = t / oh;
        const int64_t off = (plane * ih + 2 * (int64_t)hid) * iw + vx * V;
        T *r0 = dx + off;
        const T *g = dy + (plane * oh + hid) * (int64_t)ow + vx * (V / 2);
        Vec16<T> a, b, oa, ob;
        a.raw = *reinterpret_cast<const uint4 *>(src + off);
        b.raw = *reinterpret_cast<const uint4 *>(src + off + iw);
        oa.raw = make_uint4(0, 0, 0, 0);
        ob.raw = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < V / 2; ++j) {
            // window order (0,0),(0,1),(1,0),(1,1); the first maximum wins
            float m = a.get(2 * j);
            int am = 0;
            float v = a.get(2 * j + 1);
            if (v > m) { m = v; am = 1; }
            v = b.get(2 * j);
            if (v > m) { m = v; am = 2; }
            v = b.get(2 * j + 1);
            if (v > m) { m = v; am = 3; }
            const float gv = __fadd_rn(0.f, to_f32(g[j]));
            oa.set(2 * j, am == 0 ? gv : 0.f);
            oa.set(2 * j + 1, am == 1 ? gv : 0.f);
            ob.set(2 * j, am == 2 ? gv : 0.f);
            ob.set(2 * j + 1, am == 3 ? gv : 0.f);
        }
        *reinterpret_cast<uint4 *>(r0) = oa.raw;
        *reinterpret_cast<uint4 *>(r0 + iw) = ob.raw;
    }
}

// 2x2 window, stride 2, even width and height, rows that keep pairs aligned (4 bytes for
// bf16, 8 for f32): a thread owns one window and reads each of its two rows as one pair;
// consecutive threads read consecutive pairs, so every load instruction covers a contiguous
// 128 / 256 bytes.
template <class T>
__device__ __forceinline__ void load_pair(const T *p, float &a, float &b);
template <>
__device__ __forceinline__ void load_pair<float>(const float *p, float &a, float &b) {
    const float2 v = *reinterpret_cast<const float2 *>(p);
    a = v.x;
    b = v.y;
}
template <>
__device__ __forceinline__ void load_pair<__nv_bfloat16>(const __nv_bfloat16 *p, float &a, float &b) {
    const uint32_t v = *reinterpret_cast<const uint32_t *>(p);
    a = __uint_as_float(v << 16);
    b = __uint_as_float(v & 0xffff0000u);
}
template <class T>
__device__ __forceinline__ void store_pair(T *p, float a, float b);
template <>
__device__ __forceinline__ void store_pair<float>(float *p, float a, float b) {
    *reinterpret_cast<float2 *>(p) = make_float2(a, b);
}
template <>
__device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16 *p, float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    *reinterpret_cast<uint32_t *>(p) = *reinterpret_cast<uint32_t *>(&h);
}

// RELU: the window is taken over relu(x) (x >= 0 ? x : 0), i.e. Relu followed by the pool.
template <class T, bool RELU = false>
__global__ void max_pool2_2x2_pair_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t planes,
                                          int ih, int iw, int oh, int ow) {
    const int64_t total = planes * oh * ow;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int wid = (int)(i % ow);
        const int64_t t = i / ow;
        const int hid = (int)(t % oh);
        const int64_t plane = t / oh;
        const T *r0 = x + (plane * ih + 2 * (int64_t)hid) * iw + 2 * wid;
        float a0, a1, b0, b1;
        load_pair<T>(r0, a0, a1);
        load_pair<T>(r0 + iw, b0, b1);
        if (RELU) {
            a0 = a0 >= 0.f ? a0 : 0.f;
            a1 = a1 >= 0.f ? a1 : 0.f;
            b0 = b0 >= 0.f ? b0 : 0.f;
            b1 = b1 >= 0.f ? b1 : 0.f;
        }
        float m = a0;  // window order (0,0),(0,1),(1,0),(1,1); the first maximum wins
        if (a1 > m) m = a1;
        if (b0 > m) m = b0;
        if (b1 > m) m = b1;
        y[i] = from_f32<T>(m);
    }
}

// Gradient of the same: src holds the forward input, dx receives dy at the first maximum
// of every window and zero elsewhere (every cell belongs to a window).  src may be dx.
// RELU: src is the input of a Relu whose output was pooled; the result is the gradient at
// that input (the pool's gradient gated by src >= 0, as Relu's backward gates it).
template <class T, bool RELU = false>
__global__ void max_pool2_backward_2x2_pair_kernel(const T *src, T *dx, const T *__restrict__ dy,
                                                   int64_t planes, int ih, int iw, int oh, int ow) {
    const int64_t total = planes * oh * ow;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int wid = (int)(i % ow);
        const int64_t t = i / ow;
        const int hid = (int)(t % oh);
        const int64_t plane = t / oh;
        const int64_t off = (plane * ih + 2 * (int64_t)hid) * iw + 2 * wid;
        float a0, a1, b0, b1;
        load_pair<T>(src + off, a0, a1);
        load_pair<T>(src + off + iw, b0, b1);
        bool p0 = true, p1 = true, p2 = true, p3 = true;  // Relu lets the gradient pass
        if (RELU) {
            p0 = a0 >= 0.f; p1 = a1 >= 0.f; p2 = b0 >= 0.f; p3 = b1 >= 0.f;
            a0 = p0 ? a0 : 0.f; a1 = p1 ? a1 : 0.f; b0 = p2 ? b0 : 0.f; b1 = p3 ? b1 : 0.f;
        }
        float m = a0;
        int am = 0;
        if (a1 > m) { m = a1; am = 1; }
        if (b0 > m) { m = b0; am = 2; }
        if (b1 > m) { m = b1; am = 3; }
        const float g = __fadd_rn(0.f, to_f32(dy[i]));
        store_pair<T>(dx + off, (am == 0 && p0) ? g : 0.f, (am == 1 && p1) ? g : 0.f);
        store_pair<T>(dx + off + iw, (am == 2 && p2) ? g : 0.f, (am == 3 && p3) ? g : 0.f);
    }
}

// Any non-overlapping window, any width: a CTA stages a run of whole planes in
// shared memory with 16-byte loads (the staged copy keeps the alignment of the
// global run), works on the windows there, and writes the run back with 16-byte
// stores, so the 2- and 4-byte window accesses never reach global memory.
template <class T>
__global__ void max_pool2_backward_staged_kernel(const T *src, T *dx, const T *__restrict__ dy,
                                                 int64_t planes, int ih, int iw, int oh, int ow,
                                                 int h, int w, int sh, int sw, int per_cta) {
    extern __shared__ __align__(16) unsigned char staged_raw[];
    T *s = reinterpret_cast<T *>(staged_raw);
    constexpr int V = 16 / (int)sizeof(T);
    const int plane_len = ih * iw;
    for (int64_t p0 = (int64_t)blockIdx.x * per_cta; p0 < planes;
         p0 += (int64_t)gridDim.x * per_cta) {
        const int np = (int)min((int64_t)per_cta, planes - p0);
        const int n = np * plane_len;
        const T *in = src + p0 * plane_len;
        T *base = dx + p0 * plane_len;
        // the staged copy keeps the 16-byte phase of the source run; the run is written back
        // with 16-byte stores when the destination run has the same phase (always, in place)
        const int shift = (int)((reinterpret_cast<uintptr_t>(in) & 15) / sizeof(T));
        const bool same_phase =
            shift == (int)((reinterpret_cast<uintptr_t>(base) & 15) / sizeof(T));
        const int head = min(n, (V - shift) % V);
        const int nv = (n - head) / V;
        const int tail0 = head + nv * V;
        for (int i = threadIdx.x; i < head; i += blockDim.x) s[shift + i] = in[i];
        for (int v = threadIdx.x; v < nv; v += blockDim.x)
            *reinterpret_cast<uint4 *>(s + shift + head + v * V) =
                *reinterpret_cast<const uint4 *>(in + head + v * V);
        for (int i = tail0 + threadIdx.x; i < n; i += blockDim.x) s[shift + i] = in[i];
        __syncthreads();
        const int windows = np * oh * ow;
        const T *g = dy + p0 * oh * ow;
        for (int i = threadIdx.x; i < windows; i += blockDim.x) {
            const int wid = i % ow;
            const int t = i / ow;
            const int hid = t % oh, plane = t / oh;
            T *win = s + shift + plane * plane_len + hid * sh * iw + wid * sw;
            float m = 0.f;
            int am = 0;
            for (int fi = 0; fi < h; ++fi)
                for (int fj = 0; fj < w; ++fj) {
                    const float v = to_f32(win[fi * iw + fj]);
                    if ((fi == 0 && fj == 0) || v > m) {
                        m = v;
                        am = fi * iw + fj;
                    }
                    win[fi * iw + fj] = from_f32<T>(0.f);
                }
            win[am] = from_f32<T>(__fadd_rn(0.f, to_f32(g[i])));
        }
        __syncthreads();
        if (same_phase) {
            for (int i = threadIdx.x; i < head; i += blockDim.x) base[i] = s[shift + i];
            for (int v = threadIdx.x; v < nv; v += blockDim.x)
                *reinterpret_cast<uint4 *>(base + head + v * V) =
                    *reinterpret_cast<const uint4 *>(s + shift + head + v * V);
            for (int i = tail0 + threadIdx.x; i < n; i += blockDim.x) base[i] = s[shift + i];
        } else {
            for (int i = threadIdx.x; i < n; i += blockDim.x) base[i] = s[shift + i];
        }
        __syncthreads();
    }
}

// ---- u8 images -> float ----------------------------------------------------------
// y = alpha * x in the output type (alpha rounded to T first, one rounding of the product).
// A thread converts 16 bytes when both pointers allow 16-byte accesses.
template <class T>
__global__ void scaled_cast_u8_kernel(const uint8_t *__restrict__ x, T *__restrict__ y, int64_t n,
                                      float alpha) {
    const float a = to_f32(from_f32<T>(alpha));
    const bool vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(y) & 15) == 0;
    const int64_t nvec = vec ? n / 16 : 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const uint4 q = reinterpret_cast<const uint4 *>(x)[i];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        __align__(16) T out[16];
#pragma unroll
        for (int j = 0; j < 16; ++j)
            out[j] = from_f32<T>(a * (float)((w[j >> 2] >> (8 * (j & 3))) & 0xffu));
        uint4 *dst = reinterpret_cast<uint4 *>(y + i * 16);
        const uint4 *src = reinterpret_cast<const uint4 *>(out);
#pragma unroll
        for (int j = 0; j < (int)(16 * sizeof(T) / 16); ++j) dst[j] = src[j];
    }
    for (int64_t i = nvec * 16 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        y[i] = from_f32<T>(a * (float)x[i]);
}

// ---- bias ---------------------------------------------------------------------
template <class T>
__global__ void bias_add_kernel(T *__restrict__ y, const T *__restrict__ bias, int64_t total,
                                int64_t cols, int64_t inner) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t c = (i / inner) % cols;
        y[i] = from_f32<T>(__fadd_rn(to_f32(y[i]), to_f32(bias[c])));
    }
}

// Bias gradient y[c] = beta*y[c] + sum over (r, i) of x[r, c, i], in two passes with a
// fixed summation order (deterministic):
//   pass 1  partial[chunk][c] over a chunk of rows, reading x coalesced
//   pass 2  y[c] = beta*y[c] + sum over chunks
// inner == 1 (Dense): threads walk the columns.  inner > 1 (Conv2, NCHW): threads walk
// the contiguous inner positions of one channel.
template <class T>
__global__ void bias_grad_cols_kernel(const T *__restrict__ x, float *__restrict__ partial,
                                      int64_t rows, int64_t cols, int64_t rows_per_chunk,
                                      T *__restrict__ y, float beta) {
    __shared__ float part[8][33];
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;  // 32 columns x 8 row lanes
    const int64_t c = (int64_t)blockIdx.x * 32 + cx;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_chunk;
    const int64_t r1 = min(rows, r0 + rows_per_chunk);
    float s = 0.f;
    if (c < cols)
        for (int64_t r = r0 + ry; r < r1; r += 8) s += to_f32(x[r * cols + c]);
    part[ry][cx] = s;
    __syncthreads();
    if (ry == 0 && c < cols) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += part[k][cx];
        if (y != nullptr) {  // a single chunk: this is the whole sum
            if (beta != 0.f) t = __fadd_rn(t, __fmul_rn(beta, to_f32(y[c])));
            y[c] = from_f32<T>(t);
        } else {
            partial[(int64_t)blockIdx.y * cols + c] = t;
        }
    }
}

// The same for wide matrices whose rows keep 16-byte alignment: a thread owns the columns of one
// 16-byte vector (4 f32 / 8 bf16) and has four rows' loads in flight before it adds them, in row
// order, to its running sums.
template <class T>
__global__ void bias_grad_cols_vec_kernel(const T *__restrict__ x, float *__restrict__ partial,
                                          int64_t rows, int64_t cols, int64_t rows_per_chunk,
                                          T *__restrict__ y, float beta) {
    constexpr int V = Vec16<T>::N;
    __shared__ float part[8][32 * V + 1];
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int64_t c = ((int64_t)blockIdx.x * 32 + cx) * V;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_chunk;
    const int64_t r1 = min(rows, r0 + rows_per_chunk);
    float s[V];
#pragma unroll
    for (int j = 0; j < V; ++j) s[j] = 0.f;
    if (c < cols) {
        int64_t r = r0 + ry;
        for (; r + 24 < r1; r += 32) {
            Vec16<T> v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                v[u].raw = *reinterpret_cast<const uint4 *>(x + (r + 8 * u) * cols + c);
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int j = 0; j < V; ++j) s[j] += v[u].get(j);
        }
        for (; r < r1; r += 8) {
            Vec16<T> v;
            v.raw = *reinterpret_cast<const uint4 *>(x + r * cols + c);
#pragma unroll
            for (int j = 0; j < V; ++j) s[j] += v.get(j);
        }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) part[ry][cx * V + j] = s[j];
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * V; i += blockDim.x) {
        const int64_t col = (int64_t)blockIdx.x * 32 * V + i;
        if (col >= cols) continue;
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += part[k][i];
        if (y != nullptr) {  // a single chunk: this is the whole sum
            if (beta != 0.f) t = __fadd_rn(t, __fmul_rn(beta, to_f32(y[col])));
            y[col] = from_f32<T>(t);
        } else {
            partial[(int64_t)blockIdx.y * cols + col] = t;
        }
    }
}

template <class T>
__global__ void bias_grad_inner_kernel(const T *__restrict__ x, float *__restrict__ partial,
                                       int64_t rows, int64_t cols, int64_t inner,
                                       int64_t rows_per_chunk) {
    __shared__ float part[256];
    const int64_t c = blockIdx.x;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_chunk;
    const int64_t r1 = min(rows, r0 + rows_per_chunk);
    float s = 0.f;
    for (int64_t r = r0; r < r1; ++r) {
        const T *seg = x + (r * cols + c) * inner;
        for (int64_t i = threadIdx.x; i < inner; i += blockDim.x) s += to_f32(seg[i]);
    }
    part[threadIdx.x] = s;
    __syncthreads();
    for (int off = blockDim.x / 2; off > 0; off >>= 1) {
        if ((int)threadIdx.x < off) part[threadIdx.x] += part[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[(int64_t)blockIdx.y * cols + c] = part[0];
}

// Block of 32 x 8 threads: 32 consecutive columns, the chunk rows dealt round-robin to the eight
// thread rows; the eight sums are added in row order (reproducible).
template <class T>
__global__ void bias_grad_final_kernel(const float *__restrict__ partial, T *__restrict__ y,
                                       int64_t cols, int chunks, float beta) {
    __shared__ float part[8][33];
    const int64_t c = (int64_t)blockIdx.x * 32 + threadIdx.x;
    float v = 0.f;
    if (c < cols)
        for (int k = threadIdx.y; k < chunks; k += 8) v += partial[(int64_t)k * cols + c];
    part[threadIdx.y][threadIdx.x] = v;
    __syncthreads();
    if (threadIdx.y != 0 || c >= cols) return;
    v = part[0][threadIdx.x];
#pragma unroll
    for (int r = 1; r < 8; ++r) v += part[r][threadIdx.x];
    if (beta != 0.f) v = __fadd_rn(v, __fmul_rn(beta, to_f32(y[c])));
    y[c] = from_f32<T>(v);
}

template <class T>
static int bias_grad_run(ag_device *dev, const T *x, int64_t rows, int64_t cols, int64_t inner,
                         float beta, T *y) {
    // Wide, aligned matrices: 16-byte loads (a CTA covers 32 vectors of columns).
    constexpr int V = Vec16<T>::N;
    const bool vec = inner == 1 && cols % V == 0 && cols >= 32 * V && rows > 1024 &&
                     (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    // Enough row chunks to fill the GPU (eight CTAs per SM for the vector form), at most 1024.
    int64_t col_blocks = inner == 1 ? ceil_div(cols, vec ? 32 * V : 32) : cols;
    int64_t chunks = ceil_div((int64_t)dev->sm_count * (vec ? 8 : 4), col_blocks);
    if (chunks > rows) chunks = rows;
    if (chunks > 1024) chunks = 1024;
    if (chunks < 1) chunks = 1;
    // Few rows (a Dense layer's small batch): one launch, no second pass.
    if (inner == 1 && rows <= 1024) chunks = 1;
    const int64_t rows_per_chunk = ceil_div(rows > 0 ? rows : 1, chunks);
    chunks = rows > 0 ? ceil_div(rows, rows_per_chunk) : 1;
    if (inner == 1 && chunks == 1) {
        bias_grad_cols_kernel<T><<<(unsigned)col_blocks, 256, 0, dev->stream>>>(
            x, nullptr, rows, cols, rows_per_chunk, y, beta);
        AG_CHECK_LAUNCH();
        return AG_OK;
    }
    void *ws = nullptr;
    AG_TRY(workspace(dev, sizeof(float) * (size_t)chunks * (size_t)cols, &ws));
    dim3 grid((unsigned)col_blocks, (unsigned)chunks);
    AG_REQUIRE(col_blocks < (1ll << 31), AG_ERR_LIMIT, "too many columns");
    if (vec)
        bias_grad_cols_vec_kernel<T><<<grid, 256, 0, dev->stream>>>(x, (float *)ws, rows, cols,
                                                                    rows_per_chunk, nullptr, 0.f);
    else if (inner == 1)
        bias_grad_cols_kernel<T><<<grid, 256, 0, dev->stream>>>(x, (float *)ws, rows, cols,
                                                                rows_per_chunk, nullptr, 0.f);
    else
        bias_grad_inner_kernel<T><<<grid, 256, 0, dev->stream>>>(x, (float *)ws, rows, cols, inner,
                                                                 rows_per_chunk);
    AG_CHECK_LAUNCH();
    bias_grad_final_kernel<T><<<(unsigned)ceil_div(cols, 32), dim3(32, 8), 0, dev->stream>>>(
        (const float *)ws, y, cols, (int)chunks, beta);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

// ---- SGD ------------------------------------------------------------------------
template <class T>
__global__ void sgd_momentum_kernel(T *__restrict__ w, const T *__restrict__ g, T *__restrict__ v,
                                    int64_t n, float lr, float mom) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        float vv = __fadd_rn(__fmul_rn(mom, to_f32(v[i])), to_f32(g[i]));
        float ww = __fsub_rn(to_f32(w[i]), __fmul_rn(lr, vv));
        v[i] = from_f32<T>(vv);
        w[i] = from_f32<T>(ww);
    }
}

// Any window, any width: a CTA stages a run of whole planes in shared memory with
// 16-byte loads (the staged copy keeps the alignment of the global run) and takes the
// window maxima from there; consecutive threads write consecutive outputs.
template <class T>
__global__ void max_pool2_staged_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t planes,
                                        int ih, int iw, int oh, int ow, int h, int w, int sh,
                                        int sw, int per_cta) {
    extern __shared__ __align__(16) unsigned char staged_raw[];
    T *s = reinterpret_cast<T *>(staged_raw);
    constexpr int V = 16 / (int)sizeof(T);
    const int plane_len = ih * iw;
    for (int64_t p0 = (int64_t)blockIdx.x * per_cta; p0 < planes;
         p0 += (int64_t)gridDim.x * per_cta) {
        const int np = (int)min((int64_t)per_cta, planes - p0);
        const int n = np * plane_len;
        const T *base = x + p0 * plane_len;
        const int shift = (int)((reinterpret_cast<uintptr_t>(base) & 15) / sizeof(T));
        const int head = min(n, (V - shift) % V);
        const int nv = (n - head) / V;
        const int tail0 = head + nv * V;
        for (int i = threadIdx.x; i < head; i += blockDim.x) s[shift + i] = base[i];
        for (int v = threadIdx.x; v < nv; v += blockDim.x)
            *reinterpret_cast<uint4 *>(s + shift + head + v * V) =
                *reinterpret_cast<const uint4 *>(base + head + v * V);
        for (int i = tail0 + threadIdx.x; i < n; i += blockDim.x) s[shift + i] = base[i];
        __syncthreads();
        const int outs = np * oh * ow;
        T *dst = y + p0 * oh * ow;
        for (int i = threadIdx.x; i < outs; i += blockDim.x) {
            const int wid = i % ow;
            const int t = i / ow;
            const int hid = t % oh, plane = t / oh;
            const T *win = s + shift + plane * plane_len + hid * sh * iw + wid * sw;
            float m = to_f32(win[0]);
            for (int fi = 0; fi < h; ++fi)
                for (int fj = 0; fj < w; ++fj) {
                    const float v = to_f32(win[fi * iw + fj]);
                    if (v > m) m = v;  // the first maximum wins; NaNs never win after the first cell
                }
            dst[i] = from_f32<T>(m);
        }
        __syncthreads();
    }
}

template <class T>
static int pool_forward(ag_device *dev, const T *x, T *y, int64_t planes, int ih, int iw, int oh,
                        int ow, int h, int w, int sh, int sw) {
    const int threads = 256;
    constexpr int V = Vec16<T>::N;
    const int64_t plane_bytes = (int64_t)ih * iw * (int64_t)sizeof(T);
    if (h == 2 && w == 2 && sh == 2 && sw == 2 && iw % V == 0 && aligned16(x)) {
        const int64_t items = planes * oh * (iw / V);
        max_pool2_2x2_kernel<T><<<grid_for(items, threads, dev->sm_count), threads, 0,
                                  dev->stream>>>(x, y, planes, ih, iw, oh, ow);
    } else if (h == 2 && w == 2 && sh == 2 && sw == 2 && (iw & 1) == 0 && (ih & 1) == 0 &&
               (reinterpret_cast<uintptr_t>(x) % (2 * sizeof(T))) == 0) {
        max_pool2_2x2_pair_kernel<T><<<grid_for(planes * oh * ow, threads, dev->sm_count), threads, 0,
                                       dev->stream>>>(x, y, planes, ih, iw, oh, ow);
    } else if (plane_bytes <= 40 * 1024 && planes >= dev->sm_count) {
        // a run of whole planes per CTA, about four CTAs per SM
        int per_cta = (int)((40 * 1024) / plane_bytes);
        const int64_t spread = ceil_div(planes, (int64_t)dev->sm_count * 4);
        if (per_cta > spread) per_cta = (int)(spread < 1 ? 1 : spread);
        const size_t smem = (size_t)per_cta * (size_t)plane_bytes + 16;
        const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(planes, per_cta),
                                                          (int64_t)dev->sm_count * 8);
        max_pool2_staged_kernel<T><<<grid, threads, smem, dev->stream>>>(x, y, planes, ih, iw, oh, ow,
                                                                         h, w, sh, sw, per_cta);
    } else {
        const int64_t items = planes * oh * ow;
        max_pool2_kernel<T><<<grid_for(items, threads, dev->sm_count), threads, 0, dev->stream>>>(
            x, y, planes, ih, iw, oh, ow, h, w, sh, sw);
    }
    AG_CHECK_LAUNCH();
    return AG_OK;
}

}  // namespace ag

using namespace ag;

#define AG_DISPATCH_FLOAT(dtype, T, ...)            \
    do {                                            \
        if ((dtype) == AG_F32) {                    \
            using T = float;                        \
            __VA_ARGS__                             \
        } else {                                    \
            using T = __nv_bfloat16;                \
            __VA_ARGS__                             \
        }                                           \
    } while (0)

extern "C" {

int ag_scaled_cast_u8(ag_device *dev, ag_dtype dtype, float alpha, const uint8_t *x, void *y,
                      int64_t n) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "scaled_cast to %d unimplemented", (int)dtype);
    AG_REQUIRE(n >= 0, AG_ERR_SHAPE, "negative length");
    if (n == 0) return AG_OK;
    AG_REQUIRE(x && y, AG_ERR_INVALID, "null tensor pointer");
    const int threads = 256;
    const unsigned grid = grid_for(ceil_div(n, 16), threads, dev->sm_count);
    AG_DISPATCH_FLOAT(dtype, T,
        scaled_cast_u8_kernel<T><<<grid, threads, 0, dev->stream>>>(x, (T *)y, n, alpha););
    AG_CHECK_LAUNCH();
    return AG_OK;
}

int ag_relu(ag_device *dev, ag_dtype dtype, const void *x, void *y, int64_t n) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "relu %d unimplemented", (int)dtype);
    AG_REQUIRE(n >= 0, AG_ERR_SHAPE, "negative length");
    if (n == 0) return AG_OK;
    AG_REQUIRE(x && y, AG_ERR_INVALID, "null tensor pointer");
    AG_DISPATCH_FLOAT(dtype, T, return map2<T>(dev, (const T *)x, (const T *)nullptr, (T *)y, n, ReluF{}););
}

int ag_relu_backward(ag_device *dev, ag_dtype dtype, const void *x, const void *dy, void *dx,
                     int64_t n) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "relu_backward %d unimplemented", (int)dtype);
    AG_REQUIRE(n >= 0, AG_ERR_SHAPE, "negative length");
    if (n == 0) return AG_OK;
    AG_REQUIRE(x && dy && dx, AG_ERR_INVALID, "null tensor pointer");
    AG_DISPATCH_FLOAT(dtype, T, return map2<T>(dev, (const T *)x, (const T *)dy, (T *)dx, n, ReluBackwardF{}););
}

int ag_scaled_add(ag_device *dev, ag_dtype dtype, float alpha, const void *x, void *y, int64_t n) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "scaled_add %d unimplemented", (int)dtype);
    AG_REQUIRE(n >= 0, AG_ERR_SHAPE, "negative length");
    if (n == 0) return AG_OK;
    AG_REQUIRE(x && y, AG_ERR_INVALID, "null tensor pointer");
    if (dtype == AG_F32)
        return map2<float>(dev, (const float *)x, (const float *)y, (float *)y, n,
                           ScaledAddF<float>{alpha});
    // alpha is cast to the element type first (ScalarElem::scalar_cast in the reference).
    float a = __bfloat162float(__float2bfloat16_rn(alpha));
    return map2<__nv_bfloat16>(dev, (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)y,
                               (__nv_bfloat16 *)y, n, ScaledAddF<__nv_bfloat16>{a});
}

int ag_max_pool2(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs, int64_t c, int64_t ih,
                 int64_t iw, int32_t h, int32_t w, int32_t sh, int32_t sw, void *y) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "max_pool2 %d unimplemented", (int)dtype);
    AG_REQUIRE(h > 0 && w > 0 && sh > 0 && sw > 0, AG_ERR_INVALID, "bad pool options");
    AG_REQUIRE(bs >= 0 && c >= 0 && ih >= h && iw >= w, AG_ERR_SHAPE,
               "pool window [%d,%d] does not fit input [%lld,%lld]", h, w, (long long)ih,
               (long long)iw);
    AG_REQUIRE(ih < (1 << 30) && iw < (1 << 30), AG_ERR_LIMIT, "image too large");
    const int oh = (int)((ih - h) / sh + 1), ow = (int)((iw - w) / sw + 1);
    if (bs * c == 0) return AG_OK;
    AG_REQUIRE(x && y, AG_ERR_INVALID, "null tensor pointer");
    AG_DISPATCH_FLOAT(dtype, T, return pool_forward<T>(dev, (const T *)x, (T *)y, bs * c, (int)ih, (int)iw, oh, ow, h, w, sh, sw););
}

// dx = max_pool2_backward(copy of x, dy); x == dx is the in-place form of the reference.
static int pool_backward(ag_device *dev, ag_dtype dtype, const void *x, void *dx, int64_t bs,
                         int64_t c, int64_t ih, int64_t iw, int32_t h, int32_t w, int32_t sh,
                         int32_t sw, const void *dy) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "max_pool2_backward %d unimplemented",
               (int)dtype);
    AG_REQUIRE(h > 0 && w > 0 && sh > 0 && sw > 0, AG_ERR_INVALID, "bad pool options");
    AG_REQUIRE(sh >= h && sw >= w, AG_ERR_UNSUPPORTED,
               "max_pool2_backward needs non-overlapping windows (stride >= size)");
    AG_REQUIRE(bs >= 0 && c >= 0 && ih >= h && iw >= w, AG_ERR_SHAPE,
               "pool window does not fit input");
    AG_REQUIRE(ih < (1 << 30) && iw < (1 << 30), AG_ERR_LIMIT, "image too large");
    const int oh = (int)((ih - h) / sh + 1), ow = (int)((iw - w) / sw + 1);
    const int64_t planes = bs * c;
    if (planes == 0) return AG_OK;
    AG_REQUIRE(x && dx && dy, AG_ERR_INVALID, "null tensor pointer");
    const int threads = 256;
    const int vlen = dtype == AG_F32 ? 4 : 8;
    if (h == 2 && w == 2 && sh == 2 && sw == 2 && iw % vlen == 0 &&
        (reinterpret_cast<uintptr_t>(dx) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
        ((ih & 1) == 0 || x == dx)) {  // out of place, a last row no window covers must be copied
        const unsigned grid2 = grid_for(planes * oh * (iw / vlen), threads, dev->sm_count);
        AG_DISPATCH_FLOAT(dtype, T,
            max_pool2_backward_2x2_kernel<T><<<grid2, threads, 0, dev->stream>>>(
                (const T *)x, (T *)dx, (const T *)dy, planes, (int)ih, (int)iw, oh, ow););
        AG_CHECK_LAUNCH();
        return AG_OK;
    }
    const size_t pair_bytes = 2 * dtype_size(dtype);
    if (h == 2 && w == 2 && sh == 2 && sw == 2 && (iw & 1) == 0 && (ih & 1) == 0 &&
        reinterpret_cast<uintptr_t>(dx) % pair_bytes == 0 &&
        reinterpret_cast<uintptr_t>(x) % pair_bytes == 0) {
        const unsigned gridp = grid_for(planes * oh * ow, threads, dev->sm_count);
        AG_DISPATCH_FLOAT(dtype, T,
            max_pool2_backward_2x2_pair_kernel<T><<<gridp, threads, 0, dev->stream>>>(
                (const T *)x, (T *)dx, (const T *)dy, planes, (int)ih, (int)iw, oh, ow););
        AG_CHECK_LAUNCH();
        return AG_OK;
    }
    const int64_t plane_bytes = ih * iw * (int64_t)dtype_size(dtype);
    if (plane_bytes <= 40 * 1024) {
        // a run of whole planes per CTA, about four CTAs per SM
        int per_cta = (int)((40 * 1024) / plane_bytes);
        const int64_t spread = ceil_div(planes, (int64_t)dev->sm_count * 4);
        if (per_cta > spread) per_cta = (int)(spread < 1 ? 1 : spread);
        const size_t smem = (size_t)per_cta * (size_t)plane_bytes + 16;
        const unsigned gridp = (unsigned)std::min<int64_t>(ceil_div(planes, per_cta),
                                                           (int64_t)dev->sm_count * 8);
        AG_DISPATCH_FLOAT(dtype, T,
            max_pool2_backward_staged_kernel<T><<<gridp, threads, smem, dev->stream>>>(
                (const T *)x, (T *)dx, (const T *)dy, planes, (int)ih, (int)iw, oh, ow, h, w, sh, sw, per_cta););
        AG_CHECK_LAUNCH();
        return AG_OK;
    }
    // planes too large to stage: copy first (when out of place), then the in-place kernel
    if (x != dx)
        AG_CUDA_TRY(cudaMemcpyAsync(dx, x, (size_t)(planes * ih * iw) * dtype_size(dtype),
                                    cudaMemcpyDeviceToDevice, dev->stream));
    const unsigned grid = grid_for(planes * oh * ow, threads, dev->sm_count);
    AG_DISPATCH_FLOAT(dtype, T,
        max_pool2_backward_kernel<T><<<grid, threads, 0, dev->stream>>>(
            (T *)dx, (const T *)dy, planes, (int)ih, (int)iw, oh, ow, h, w, sh, sw););
    AG_CHECK_LAUNCH();
    return AG_OK;
}

int ag_max_pool2_backward(ag_device *dev, ag_dtype dtype, void *dx, int64_t bs, int64_t c,
                          int64_t ih, int64_t iw, int32_t h, int32_t w, int32_t sh, int32_t sw,
                          const void *dy) {
    return pool_backward(dev, dtype, dx, dx, bs, c, ih, iw, h, w, sh, sw, dy);
}

int ag_max_pool2_backward_from_input(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                                     int64_t c, int64_t ih, int64_t iw, int32_t h, int32_t w,
                                     int32_t sh, int32_t sw, const void *dy, void *dx) {
    return pool_backward(dev, dtype, x, dx, bs, c, ih, iw, h, w, sh, sw, dy);
}

// Relu followed by a 2x2 / stride 2 pool over planes of even height and width, and the
// gradient of the pair at the Relu's input.
static int relu_pool_check(ag_device *dev, ag_dtype dtype, int64_t bs, int64_t c, int64_t ih,
                           int64_t iw, const void *a, const void *b, const void *d) {
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "relu_max_pool2 %d unimplemented", (int)dtype);
    AG_REQUIRE(bs >= 0 && c >= 0 && ih >= 2 && iw >= 2, AG_ERR_SHAPE,
               "pool window [2,2] does not fit input [%lld,%lld]", (long long)ih, (long long)iw);
    AG_REQUIRE((ih & 1) == 0 && (iw & 1) == 0, AG_ERR_UNSUPPORTED,
               "relu_max_pool2 needs even height and width");
    AG_REQUIRE(ih < (1 << 30) && iw < (1 << 30), AG_ERR_LIMIT, "image too large");
    if (bs * c == 0) return AG_OK;
    AG_REQUIRE(a && b && d, AG_ERR_INVALID, "null tensor pointer");
    const size_t pair_bytes = 2 * dtype_size(dtype);
    AG_REQUIRE(reinterpret_cast<uintptr_t>(a) % pair_bytes == 0 &&
                   reinterpret_cast<uintptr_t>(b) % pair_bytes == 0,
               AG_ERR_UNSUPPORTED, "relu_max_pool2 needs element-pair aligned tensors");
    return AG_OK;
}

int ag_relu_max_pool2_forward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs, int64_t c,
                              int64_t ih, int64_t iw, void *y) {
    AG_ENTER(dev);
    AG_TRY(relu_pool_check(dev, dtype, bs, c, ih, iw, x, x, y));
    const int64_t planes = bs * c;
    if (planes == 0) return AG_OK;
    const int oh = (int)(ih / 2), ow = (int)(iw / 2), threads = 256;
    const unsigned grid = grid_for(planes * oh * ow, threads, dev->sm_count);
    AG_DISPATCH_FLOAT(dtype, T,
        (max_pool2_2x2_pair_kernel<T, true><<<grid, threads, 0, dev->stream>>>(
            (const T *)x, (T *)y, planes, (int)ih, (int)iw, oh, ow)););
    AG_CHECK_LAUNCH();
    return AG_OK;
}

int ag_relu_max_pool2_backward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                               int64_t c, int64_t ih, int64_t iw, const void *dy, void *dx) {
    AG_ENTER(dev);
    AG_TRY(relu_pool_check(dev, dtype, bs, c, ih, iw, x, dx, dy));
    const int64_t planes = bs * c;
    if (planes == 0) return AG_OK;
    const int oh = (int)(ih / 2), ow = (int)(iw / 2), threads = 256;
    const unsigned grid = grid_for(planes * oh * ow, threads, dev->sm_count);
    AG_DISPATCH_FLOAT(dtype, T,
        (max_pool2_backward_2x2_pair_kernel<T, true><<<grid, threads, 0, dev->stream>>>(
            (const T *)x, (T *)dx, (const T *)dy, planes, (int)ih, (int)iw, oh, ow)););
    AG_CHECK_LAUNCH();
    return AG_OK;
}

int ag_bias_add(ag_device *dev, ag_dtype dtype, void *y, const void *bias, int64_t rows,
                int64_t cols, int64_t inner) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "add_assign %d unimplemented", (int)dtype);
    AG_REQUIRE(rows >= 0 && cols >= 0 && inner >= 0, AG_ERR_SHAPE, "negative dimension");
    const int64_t total = rows * cols * inner;
    if (total == 0) return AG_OK;
    AG_REQUIRE(y && bias, AG_ERR_INVALID, "null tensor pointer");
    const int threads = 256;
    const unsigned grid = grid_for(total, threads, dev->sm_count);
    AG_DISPATCH_FLOAT(dtype, T,
        bias_add_kernel<T><<<grid, threads, 0, dev->stream>>>((T *)y, (const T *)bias, total, cols, inner););
    AG_CHECK_LAUNCH();
    return AG_OK;
}

int ag_bias_grad(ag_device *dev, ag_dtype dtype, const void *x, int64_t rows, int64_t cols,
                 int64_t inner, float beta, void *y) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "sum_axis %d unimplemented", (int)dtype);
    AG_REQUIRE(rows >= 0 && cols >= 0 && inner >= 0, AG_ERR_SHAPE, "negative dimension");
    if (cols == 0) return AG_OK;
    AG_REQUIRE(y && (rows * inner == 0 || x), AG_ERR_INVALID, "null tensor pointer");
    AG_REQUIRE(cols < (1ll << 31), AG_ERR_LIMIT, "too many columns");
    AG_DISPATCH_FLOAT(dtype, T, return bias_grad_run<T>(dev, (const T *)x, rows, cols, inner, beta, (T *)y););
}

int ag_sgd_update(ag_device *dev, ag_dtype dtype, void *w, const void *g, int64_t n, float lr) {
    // w = cast_T(-lr) * g + w in T arithmetic: the reference routes plain SGD through scaled_add.
    return ag_scaled_add(dev, dtype, -lr, g, w, n);
}

int ag_sgd_update_momentum(ag_device *dev, ag_dtype dtype, void *w, const void *g, void *v,
                           int64_t n, float lr, float momentum) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "SGD %d unimplemented", (int)dtype);
    AG_REQUIRE(n >= 0, AG_ERR_SHAPE, "negative length");
    if (n == 0) return AG_OK;
    AG_REQUIRE(w && g && v, AG_ERR_INVALID, "null tensor pointer");
    const int threads = 256;
    const unsigned grid = grid_for(n, threads, dev->sm_count);
    AG_DISPATCH_FLOAT(dtype, T,
        sgd_momentum_kernel<T><<<grid, threads, 0, dev->stream>>>((T *)w, (const T *)g, (T *)v, n, lr, momentum););
    AG_CHECK_LAUNCH();
    return AG_OK;
}

}  // extern "C"
