// bf16 tensor-core GEMM (tcgen05 / TMEM / TMA) entry points used by ag_gemm.
#pragma once

#include "common.cuh"

namespace ag {
namespace tc {

// True when the tcgen05 kernel can take the problem: operands contiguous along
// one index with 16-byte aligned bases and leading strides (TMA requirements),
// C row-major with 16-byte aligned rows, and a size worth a 128 x 256 tile.
bool gemm_bf16_eligible(int64_t m, int64_t k, int64_t n, const __nv_bfloat16 *a, int64_t rsa,
                        int64_t csa, const __nv_bfloat16 *b, int64_t rsb, int64_t csb,
                        const __nv_bfloat16 *c, int64_t rsc, int64_t csc);

// What a Dense layer does after the product, folded into the kernels' epilogues (only with
// alpha = 1, beta = 0): y = relu?(round(round(acc) + bias[col])), the two roundings of a
// product stored as bf16 followed by a bias add in bf16 (layer.rs:1134-1143, 1254-1267).
struct Epilogue {
    const __nv_bfloat16 *bias;  // [n] or null
    bool relu;
};

int gemm_bf16(ag_device *dev, int m, int k, int n, float alpha, const __nv_bfloat16 *a,
              int64_t rsa, int64_t csa, const __nv_bfloat16 *b, int64_t rsb, int64_t csb,
              float beta, __nv_bfloat16 *c, int64_t rsc, int64_t csc,
              const Epilogue *epi = nullptr);

// Paired-SM variant (cta_group::2, 256 x 256 tile per CTA pair): used for m, n >= 256
// unless the environment variable AG_TC2=0 selects the single-CTA kernel.
bool gemm_bf16_pair_enabled();
int gemm_bf16_pair(ag_device *dev, int m, int k, int n, float alpha, const __nv_bfloat16 *a,
                   int64_t rsa, int64_t csa, const __nv_bfloat16 *b, int64_t rsb, int64_t csb,
                   float beta, __nv_bfloat16 *c, int64_t rsc, int64_t csc,
                   const Epilogue *epi = nullptr);

}  // namespace tc
}  // namespace ag
