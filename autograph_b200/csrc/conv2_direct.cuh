// Direct convolution kernels for small channel counts (see conv2_direct.cu).
#pragma once

#include "common.cuh"

namespace ag {
namespace direct {

// True when the direct kernel can take the problem: default padding / stride /
// dilation, 5x5 or 3x3 filter, even output size, few channels.
bool eligible(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
              const ag_conv2_options *o);

// y = conv2(x, w) (+ bias) (relu) (2x2 max pool, stride 2).  With pool the
// output is [bs, oc, oh/2, ow/2], else [bs, oc, oh, ow].
template <class T>
int forward(ag_device *dev, const T *x, int64_t bs, int64_t ic, int64_t ih, int64_t iw, const T *w,
            int64_t oc, const T *bias, const ag_conv2_options *o, bool relu, bool pool, T *y,
            T *pre = nullptr);  // pre: optional copy of the convolution's output before relu / pool
                                // (fewer than 32 output channels only)

// dx = the gradient of conv2(x, w) with respect to x, given dy [bs, oc, oh, ow]
// and w [oc, ic, fh, fw]: the same kernel run on the transposed problem.
bool eligible_backward_input(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
                             const ag_conv2_options *o);
template <class T>
int backward_input(ag_device *dev, const T *w, int64_t oc, int64_t ic, const T *dy, int64_t bs,
                   int64_t ih, int64_t iw, const ag_conv2_options *o, T *dx);

// dw = beta * dw + the gradient of conv2(x, w) with respect to w: per-CTA partial
// sums over a group of images, then a fixed-order reduction (deterministic).
bool eligible_backward_weight(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
                              const ag_conv2_options *o);
template <class T>
int backward_weight(ag_device *dev, const T *x, int64_t bs, int64_t ic, int64_t ih, int64_t iw,
                    const T *dy, int64_t oc, const ag_conv2_options *o, float beta, T *dw);

}  // namespace direct
}  // namespace ag
