// ag_gemm: argument checks and routing to the SIMT tile engine (f32, and bf16
// shapes the tensor-core kernel does not take) or the tcgen05 kernel (bf16).
#include "dense_small.cuh"
#include "gemm_simt_launch.cuh"
#include "gemm_tc.cuh"

namespace ag {

template <class T>
static bool aligned_for_vec(const T *p) {
    return (reinterpret_cast<uintptr_t>(p) % (4 * sizeof(T))) == 0;
}

template <class T, bool AK, bool BK_>
static int gemm_simt_typed(ag_device *dev, int m, int k, int n, float alpha, const T *a,
                           int64_t rsa, int64_t csa, const T *b, int64_t rsb, int64_t csb,
                           float beta, T *c, int64_t rsc, int64_t csc) {
    simt::StridedOperand<T, AK> A{a, rsa, csa, m, k, false};
    simt::StridedOperand<T, BK_> B{b, csb, rsb, n, k, false};
    if (AK)
        A.vec = (csa == 1) && (rsa % 4 == 0 || m == 1) && aligned_for_vec(a);
    else
        A.vec = (rsa == 1) && (csa % 4 == 0 || k == 1) && aligned_for_vec(a);
    if (BK_)
        B.vec = (rsb == 1) && (csb % 4 == 0 || n == 1) && aligned_for_vec(b);
    else
        B.vec = (csb == 1) && (rsb % 4 == 0 || k == 1) && aligned_for_vec(b);
    simt::StridedEpilogue<T> E{c, rsc, csc, alpha, beta, false, n};
    E.vec = (csc == 1) && (rsc % 4 == 0 || m == 1) && aligned_for_vec(c);
    return simt::gemm(dev, m, n, k, A, B, E, /*allow_split=*/true);
}

template <class T>
static int gemm_simt_dispatch(ag_device *dev, int m, int k, int n, float alpha, const T *a,
                              int64_t rsa, int64_t csa, const T *b, int64_t rsb, int64_t csb,
                              float beta, T *c, int64_t rsc, int64_t csc) {
    // Walk k fastest when the operand is contiguous along k.
    bool ak = (csa == 1 && rsa != 1) || (csa == 1 && m == 1);
    bool bk = (rsb == 1 && csb != 1) || (rsb == 1 && n == 1);
    if (ak && bk)
        return gemm_simt_typed<T, true, true>(dev, m, k, n, alpha, a, rsa, csa, b, rsb, csb, beta,
                                              c, rsc, csc);
    if (ak)
        return gemm_simt_typed<T, true, false>(dev, m, k, n, alpha, a, rsa, csa, b, rsb, csb, beta,
                                               c, rsc, csc);
    if (bk)
        return gemm_simt_typed<T, false, true>(dev, m, k, n, alpha, a, rsa, csa, b, rsb, csb, beta,
                                               c, rsc, csc);
    return gemm_simt_typed<T, false, false>(dev, m, k, n, alpha, a, rsa, csa, b, rsb, csb, beta, c,
                                            rsc, csc);
}

template <class T>
static int dense_forward_simt(ag_device *dev, const T *x, int bs, int inputs, const T *w,
                              int outputs, const T *bias, bool relu, T *y) {
    simt::StridedOperand<T, true> A{x, (int64_t)inputs, 1, bs, inputs, false};
    A.vec = (inputs % 4 == 0 || bs == 1) && aligned_for_vec(x);
    simt::StridedOperand<T, false> B{w, 1, (int64_t)outputs, outputs, inputs, false};
    B.vec = (outputs % 4 == 0 || inputs == 1) && aligned_for_vec(w);
    simt::BiasReluEpilogue<T> E{y, (int64_t)outputs, bias, relu};
    return simt::gemm(dev, bs, outputs, inputs, A, B, E, /*allow_split=*/true);
}

}  // namespace ag

using namespace ag;

extern "C" int ag_dense_forward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                                int64_t inputs, const void *w, int64_t outputs, const void *bias,
                                int fuse_relu, void *y) {
    AG_ENTER(dev);
    AG_REQUIRE(dtype == AG_F32 || dtype == AG_BF16, AG_ERR_DTYPE, "Dense %d not implemented",
               (int)dtype);
    AG_REQUIRE(bs >= 0 && inputs >= 0 && outputs >= 0, AG_ERR_SHAPE, "negative dimension");
    AG_REQUIRE(bs < (1ll << 31) && inputs < (1ll << 31) && outputs < (1ll << 31), AG_ERR_LIMIT,
               "dimension beyond 2^31");
    if (bs == 0 || outputs == 0) return AG_OK;
    AG_REQUIRE(y && (inputs == 0 || (x && w)), AG_ERR_INVALID, "null tensor pointer");
    if (dense_small::eligible(bs, inputs, outputs)) {
        if (dtype == AG_F32)
            return dense_small::forward<float>(dev, (const float *)x, (int)bs, (int)inputs,
                                               (const float *)w, (int)outputs, (const float *)bias,
                                               fuse_relu != 0, (float *)y);
        return dense_small::forward<__nv_bfloat16>(
            dev, (const __nv_bfloat16 *)x, (int)bs, (int)inputs, (const __nv_bfloat16 *)w,
            (int)outputs, (const __nv_bfloat16 *)bias, fuse_relu != 0, (__nv_bfloat16 *)y);
    }
    if (dtype == AG_F32)
        return dense_forward_simt<float>(dev, (const float *)x, (int)bs, (int)inputs,
                                         (const float *)w, (int)outputs, (const float *)bias,
                                         fuse_relu != 0, (float *)y);
    const __nv_bfloat16 *px = (const __nv_bfloat16 *)x, *pw = (const __nv_bfloat16 *)w;
    __nv_bfloat16 *py = (__nv_bfloat16 *)y;
    if (tc::gemm_bf16_eligible(bs, inputs, outputs, px, inputs, 1, pw, outputs, 1, py, outputs, 1)) {
        // Large products go to the tensor cores with bias and relu in the kernel's epilogue
        // (a bias that is not 16-byte aligned is added by a separate pass).
        const __nv_bfloat16 *pb = (const __nv_bfloat16 *)bias;
        const bool bias_fused = pb && (reinterpret_cast<uintptr_t>(pb) & 15) == 0;
        const bool relu_fused = fuse_relu && (!pb || bias_fused);
        tc::Epilogue epi{bias_fused ? pb : nullptr, relu_fused};
        AG_TRY(tc::gemm_bf16(dev, (int)bs, (int)inputs, (int)outputs, 1.f, px, inputs, 1, pw,
                             outputs, 1, 0.f, py, outputs, 1, &epi));
        if (pb && !bias_fused) AG_TRY(ag_bias_add(dev, dtype, y, bias, bs, outputs, 1));
        if (fuse_relu && !relu_fused) AG_TRY(ag_relu(dev, dtype, y, y, bs * outputs));
        return AG_OK;
    }
    return dense_forward_simt<__nv_bfloat16>(dev, px, (int)bs, (int)inputs, pw, (int)outputs,
                                             (const __nv_bfloat16 *)bias, fuse_relu != 0, py);
}

extern "C" int ag_dense_chain_forward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                                      int32_t n_layers, const int64_t *dims,
                                      const void *const *weights, const void *const *biases,
                                      const int32_t *relu, void *y) {
    AG_ENTER(dev);
    AG_REQUIRE(dtype == AG_F32 || dtype == AG_BF16, AG_ERR_DTYPE, "Dense %d not implemented",
               (int)dtype);
    AG_REQUIRE(n_layers >= 1 && dims && weights && relu, AG_ERR_INVALID, "null or empty chain");
    AG_REQUIRE(bs >= 0, AG_ERR_SHAPE, "negative batch");
    for (int i = 0; i <= n_layers; ++i)
        AG_REQUIRE(dims[i] > 0 && dims[i] < (1ll << 31), AG_ERR_SHAPE, "bad layer width");
    if (bs == 0) return AG_OK;
    AG_REQUIRE(x && y, AG_ERR_INVALID, "null tensor pointer");
    dense_small::ChainLayer layers[dense_small::kMaxChain];
    bool fused = n_layers <= dense_small::kMaxChain;
    if (fused) {
        for (int i = 0; i < n_layers; ++i) {
            AG_REQUIRE(weights[i] != nullptr, AG_ERR_INVALID, "null weight pointer");
            layers[i] = {weights[i], biases ? biases[i] : nullptr, (int)dims[i], (int)dims[i + 1],
                         relu[i]};
        }
        fused = dense_small::chain_eligible(bs, n_layers, layers);
    }
    if (fused) {
        if (dtype == AG_F32)
            return dense_small::chain_forward<float>(dev, (const float *)x, (int)bs, n_layers,
                                                     layers, (float *)y);
        return dense_small::chain_forward<__nv_bfloat16>(dev, (const __nv_bfloat16 *)x, (int)bs,
                                                         n_layers, layers, (__nv_bfloat16 *)y);
    }
    // Shapes the fused kernel does not take: layer by layer through the workspace.
    int64_t widest = 0;
    for (int i = 1; i < n_layers; ++i) widest = dims[i] > widest ? dims[i] : widest;
    void *tmp = nullptr;
    const size_t plane = (size_t)bs * (size_t)widest * dtype_size(dtype);
    if (n_layers > 1) AG_TRY(workspace(dev, 2 * plane + (64u << 20), &tmp));
    // keep clear of the split-k scratch at the start of the workspace
    char *ping = (char *)tmp + (64u << 20), *pong = ping + plane;
    const void *in = x;
    for (int i = 0; i < n_layers; ++i) {
        void *out = (i + 1 == n_layers) ? y : (void *)((i & 1) ? pong : ping);
        AG_TRY(ag_dense_forward(dev, dtype, in, bs, dims[i], weights[i], dims[i + 1],
                                biases ? biases[i] : nullptr, relu[i], out));
        in = out;
    }
    return AG_OK;
}

extern "C" int ag_dense_chain_forward_keep(ag_device *dev, ag_dtype dtype, const void *x,
                                           int64_t bs, int32_t n_layers, const int64_t *dims,
                                           const void *const *weights, const void *const *biases,
                                           const int32_t *relu, void *const *pre_out,
                                           void *const *act_out) {
    AG_ENTER(dev);
    AG_REQUIRE(dtype == AG_F32 || dtype == AG_BF16, AG_ERR_DTYPE, "Dense %d not implemented",
               (int)dtype);
    AG_REQUIRE(n_layers >= 1 && dims && weights && relu && pre_out && act_out, AG_ERR_INVALID,
               "null or empty chain");
    AG_REQUIRE(bs >= 0, AG_ERR_SHAPE, "negative batch");
    for (int i = 0; i <= n_layers; ++i)
        AG_REQUIRE(dims[i] > 0 && dims[i] < (1ll << 31), AG_ERR_SHAPE, "bad layer width");
    if (bs == 0) return AG_OK;
    AG_REQUIRE(x, AG_ERR_INVALID, "null tensor pointer");
    for (int i = 0; i < n_layers; ++i)
        AG_REQUIRE(weights[i] && pre_out[i] && (!relu[i] || act_out[i]), AG_ERR_INVALID,
                   "null weight or output pointer");
    dense_small::ChainLayer layers[dense_small::kMaxChain];
    bool fused = n_layers <= dense_small::kMaxChain;
    if (fused) {
        for (int i = 0; i < n_layers; ++i) {
            layers[i] = {weights[i], biases ? biases[i] : nullptr, (int)dims[i], (int)dims[i + 1],
                         relu[i]};
            layers[i].pre_out = pre_out[i];
            layers[i].act_out = relu[i] ? act_out[i] : nullptr;
        }
        fused = dense_small::chain_eligible(bs, n_layers, layers);
    }
    if (fused) {
        if (dtype == AG_F32)
            return dense_small::chain_forward<float>(dev, (const float *)x, (int)bs, n_layers,
                                                     layers, nullptr);
        return dense_small::chain_forward<__nv_bfloat16>(dev, (const __nv_bfloat16 *)x, (int)bs,
                                                         n_layers, layers, nullptr);
    }
    const void *in = x;
    for (int i = 0; i < n_layers; ++i) {
        AG_TRY(ag_dense_forward(dev, dtype, in, bs, dims[i], weights[i], dims[i + 1],
                                biases ? biases[i] : nullptr, 0, pre_out[i]));
        in = pre_out[i];
        if (relu[i]) {
            AG_TRY(ag_relu(dev, dtype, pre_out[i], act_out[i], bs * dims[i + 1]));
            in = act_out[i];
        }
    }
    return AG_OK;
}

extern "C" int ag_dense_chain_backward(ag_device *dev, ag_dtype dtype, int64_t bs, int32_t n_layers,
                                       const int64_t *dims, const void *const *layer_in,
                                       const void *const *weights, const void *const *gate,
                                       const void *dy, void *const *g, void *dx, void *const *dw,
                                       void *const *db) {
    AG_ENTER(dev);
    AG_REQUIRE(dtype == AG_F32 || dtype == AG_BF16, AG_ERR_DTYPE, "Dense %d not implemented",
               (int)dtype);
    AG_REQUIRE(n_layers >= 1 && n_layers <= 64 && dims && layer_in && weights && gate && g && dw,
               AG_ERR_INVALID, "null or empty chain");
    AG_REQUIRE(bs >= 0, AG_ERR_SHAPE, "negative batch");
    for (int i = 0; i <= n_layers; ++i)
        AG_REQUIRE(dims[i] > 0 && dims[i] < (1ll << 31), AG_ERR_SHAPE, "bad layer width");
    if (bs == 0) return AG_OK;
    AG_REQUIRE(dy, AG_ERR_INVALID, "null tensor pointer");
    const int L = n_layers;
    for (int i = 0; i < L; ++i) {
        AG_REQUIRE(layer_in[i] && weights[i] && dw[i], AG_ERR_INVALID, "null layer pointer");
        // g[i] is written for every layer but the last, and for the last when it is gated
        AG_REQUIRE(g[i] || (i == L - 1 && !gate[i]), AG_ERR_INVALID, "null gradient buffer");
    }
    // gradient at the last Dense's output
    const void *g_last = gate[L - 1] ? g[L - 1] : dy;

    // One kernel for the input gradients, one for all weight and bias gradients.
    const int n_steps = dx ? L : L - 1;
    bool fused = L <= dense_small::kMaxChain && bs <= 512 && n_steps >= 1;
    dense_small::ChainLayer steps[dense_small::kMaxChain];
    if (fused) {
        for (int i = 0; i < n_steps; ++i) {
            const int l = L - 1 - i;  // forward layer this step goes back through
            steps[i] = {weights[l], nullptr, (int)dims[l + 1], (int)dims[l], 0};
            steps[i].transposed = 1;
            steps[i].gate = l >= 1 ? gate[l - 1] : nullptr;
            steps[i].pre_out = (i + 1 < n_steps) ? g[l - 1] : nullptr;
        }
        fused = dense_small::chain_backward_eligible(bs, n_steps, steps);
    }
    if (fused) {
        void *y = dx ? dx : g[0];
        dense_small::WgradProblem pr[dense_small::kMaxChain];
        for (int l = 0; l < L; ++l)
            pr[l] = {layer_in[l], l == L - 1 ? g_last : g[l], dw[l], db ? db[l] : nullptr,
                     (int)dims[l], (int)dims[l + 1], 0, 0};
        if (dtype == AG_F32) {
            AG_TRY(dense_small::chain_backward_input<float>(
                dev, (const float *)dy, (int)bs, n_steps, steps, (const float *)gate[L - 1],
                (float *)(gate[L - 1] ? g[L - 1] : nullptr), (float *)y));
            return dense_small::chain_weight_grads<float>(dev, (int)bs, L, pr);
        }
        AG_TRY(dense_small::chain_backward_input<__nv_bfloat16>(
            dev, (const __nv_bfloat16 *)dy, (int)bs, n_steps, steps,
            (const __nv_bfloat16 *)gate[L - 1],
            (__nv_bfloat16 *)(gate[L - 1] ? g[L - 1] : nullptr), (__nv_bfloat16 *)y));
        return dense_small::chain_weight_grads<__nv_bfloat16>(dev, (int)bs, L, pr);
    }

    // Layer by layer: relu_backward, the two products and the column sum of every layer.
    const void *incoming = dy;
    for (int l = L - 1; l >= 0; --l) {
        const int64_t ins = dims[l], outs = dims[l + 1];
        const void *gl = incoming;
        if (gate[l]) {
            AG_TRY(ag_relu_backward(dev, dtype, gate[l], incoming, g[l], bs * outs));
            gl = g[l];
        }
        // dw = in^T . g
        AG_TRY(ag_gemm(dev, dtype, ins, bs, outs, 1.f, layer_in[l], 0, 1, ins, gl, 0, outs, 1, 0.f,
                       dw[l], 0, outs, 1));
        if (db && db[l]) AG_TRY(ag_bias_grad(dev, dtype, gl, bs, outs, 1, 0.f, db[l]));
        void *out = l >= 1 ? g[l - 1] : dx;
        if (out)  // g . w^T
            AG_TRY(ag_gemm(dev, dtype, bs, outs, ins, 1.f, gl, 0, outs, 1, weights[l], 0, 1, outs,
                           0.f, out, 0, ins, 1));
        incoming = out;
    }
    return AG_OK;
}

extern "C" int ag_gemm(ag_device *dev, ag_dtype dtype, int64_t m, int64_t k, int64_t n,
                       float alpha, const void *a, int64_t off_a, int64_t rsa, int64_t csa,
                       const void *b, int64_t off_b, int64_t rsb, int64_t csb, float beta,
                       void *c, int64_t off_c, int64_t rsc, int64_t csc) {
    AG_ENTER(dev);
    AG_REQUIRE(dtype == AG_F32 || dtype == AG_BF16, AG_ERR_DTYPE,
               "Dot unimplemented for dtype %d", (int)dtype);
    AG_REQUIRE(m >= 0 && k >= 0 && n >= 0, AG_ERR_SHAPE, "negative dimension m=%lld k=%lld n=%lld",
               (long long)m, (long long)k, (long long)n);
    AG_REQUIRE(m < (1ll << 31) && k < (1ll << 31) && n < (1ll << 31) && m * n < (1ll << 40),
               AG_ERR_LIMIT, "dimension beyond 2^31");
    if (m == 0 || n == 0) return AG_OK;
    AG_REQUIRE(c != nullptr && (k == 0 || (a != nullptr && b != nullptr)), AG_ERR_INVALID,
               "null operand pointer");
    AG_REQUIRE(off_a >= 0 && off_b >= 0 && off_c >= 0, AG_ERR_INVALID, "negative offset");
    // Small plain products (row-major contiguous operands, alpha = 1, beta = 0) share the
    // latency-oriented kernel with ag_dense_forward.
    if (alpha == 1.f && beta == 0.f && k > 0 && csa == 1 && rsa == k && csb == 1 && rsb == n &&
        csc == 1 && rsc == n && dense_small::eligible(m, k, n)) {
        if (dtype == AG_F32)
            return dense_small::forward<float>(dev, (const float *)a + off_a, (int)m, (int)k,
                                               (const float *)b + off_b, (int)n, nullptr, false,
                                               (float *)c + off_c);
        return dense_small::forward<__nv_bfloat16>(
            dev, (const __nv_bfloat16 *)a + off_a, (int)m, (int)k, (const __nv_bfloat16 *)b + off_b,
            (int)n, nullptr, false, (__nv_bfloat16 *)c + off_c);
    }
    if (dtype == AG_F32) {
        return gemm_simt_dispatch<float>(dev, (int)m, (int)k, (int)n, alpha,
                                         (const float *)a + off_a, rsa, csa,
                                         (const float *)b + off_b, rsb, csb, beta,
                                         (float *)c + off_c, rsc, csc);
    }
    const __nv_bfloat16 *pa = (const __nv_bfloat16 *)a + off_a;
    const __nv_bfloat16 *pb = (const __nv_bfloat16 *)b + off_b;
    __nv_bfloat16 *pc = (__nv_bfloat16 *)c + off_c;
    if (tc::gemm_bf16_eligible(m, k, n, pa, rsa, csa, pb, rsb, csb, pc, rsc, csc))
        return tc::gemm_bf16(dev, (int)m, (int)k, (int)n, alpha, pa, rsa, csa, pb, rsb, csb, beta,
                             pc, rsc, csc);
    return gemm_simt_dispatch<__nv_bfloat16>(dev, (int)m, (int)k, (int)n, alpha, pa, rsa, csa, pb,
                                             rsb, csb, beta, pc, rsc, csc);
}
