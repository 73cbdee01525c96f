// bf16 convolution on the tensor cores (tcgen05 implicit GEMM, see conv_tc.cu).
#pragma once

#include "common.cuh"

namespace ag {
namespace convtc {

// True when the tensor-core kernel takes the problem: stride 1, dilation 1, at
// least 32 output channels in the kernel's view (few input channels are zero-padded to 64), at least 4096
// output pixels.  Any padding up to filter - 1 is handled by the zero fill of
// out-of-range TMA coordinates.
bool eligible_forward(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
                      const ag_conv2_options *o);
bool eligible_backward_input(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
                             const ag_conv2_options *o);

// y = conv2(x, w) (+ bias) (relu), NCHW bf16.
int forward(ag_device *dev, const __nv_bfloat16 *x, int64_t bs, int64_t ic, int64_t ih, int64_t iw,
            const __nv_bfloat16 *w, int64_t oc, const __nv_bfloat16 *bias,
            const ag_conv2_options *o, bool relu, __nv_bfloat16 *y);

// dx = gradient of conv2(x, w) with respect to x given dy, NCHW bf16.
int backward_input(ag_device *dev, const __nv_bfloat16 *w, int64_t oc, int64_t ic,
                   const __nv_bfloat16 *dy, int64_t bs, int64_t ih, int64_t iw,
                   const ag_conv2_options *o, __nv_bfloat16 *dx);

// False when the environment disables the tensor-core kernels (AG_TC=0 or AG_CONV_TC=0).
bool tc_conv_enabled();

// Channels-last copy: x [bs][c][hw] -> out [bs][hw][cp], cp a multiple of 64,
// channels >= c zero.
int to_nhwc(ag_device *dev, const __nv_bfloat16 *x, int64_t bs, int64_t c, int64_t hw, int64_t cp,
            __nv_bfloat16 *out);

// True when the tensor-core weight-gradient kernel takes the problem: stride 1,
// dilation 1, at least 32 output channels, filter width up to 8, at least 4096
// output pixels.  Few input channels are zero-padded to 64.
bool eligible_backward_weight(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
                              const ag_conv2_options *o);

// dw = beta * dw + gradient of conv2(x, w) with respect to w given dy, bf16.
int backward_weight(ag_device *dev, const __nv_bfloat16 *x, int64_t bs, int64_t ic, int64_t ih,
                    int64_t iw, const __nv_bfloat16 *dy, int64_t oc, const ag_conv2_options *o,
                    float beta, __nv_bfloat16 *dw);

}  // namespace convtc
}  // namespace ag
