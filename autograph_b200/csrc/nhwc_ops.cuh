// Memory-bound bf16 kernels on channels-last activations [bs][h][w][cp] (cp a multiple of 8):
// what a run of Conv2 -> Relu -> MaxPool2 stages needs between its tensor-core convolutions,
// so that no activation of the run is ever rewritten from one layout to the other.
#pragma once

#include "common.cuh"

namespace ag {
namespace nhwc {

// The patches of an NCHW image as channels of a channels-last tensor: out[b][oy][ox][c] =
// x[b][ci][oy + fi][ox + fj] for c = (ci * fh + fi) * fw + fj < ic * fh * fw, zero above.  A
// convolution with few input channels is a 1 x 1 convolution of this tensor
// (im2col_conv2 of src/ops.rs:1011-1080 with the patch as the channel axis).
int im2col_channels(ag_device *dev, const __nv_bfloat16 *x, int64_t bs, int64_t ic, int64_t ih,
                    int64_t iw, int fh, int fw, int64_t oh, int64_t ow, int64_t cp,
                    __nv_bfloat16 *out);

// y[b][py][px][c] = max over the 2 x 2 window of relu(pre) (first maximum wins; an odd last
// row / column is not covered): Relu (layer.rs:1254-1298) then MaxPool2 (layer.rs:1193-1216).
int relu_pool(ag_device *dev, const __nv_bfloat16 *pre, int64_t bs, int64_t ih, int64_t iw, int64_t cp,
              __nv_bfloat16 *y);

// The gradient at `pre` of the same two layers given dy [bs][ih/2][iw/2][cp]: the pool's
// backward kernel run in place on a clone of the Relu's output (covered cells: dy at the first
// maximum, zero elsewhere; cells no window covers keep the Relu's output), gated by pre >= 0.
// `out` is addressed through its pitches in elements, so it may be the interior of a zero frame.
int relu_pool_backward(ag_device *dev, const __nv_bfloat16 *pre, const __nv_bfloat16 *dy, int64_t bs,
                       int64_t ih, int64_t iw, int64_t cp, __nv_bfloat16 *out, int64_t out_row_pitch,
                       int64_t out_image_pitch);

// Zeroes the frame of pad_h rows / pad_w columns around the interior of [bs][hp][wp][cp].
int zero_frame(ag_device *dev, __nv_bfloat16 *framed, int64_t bs, int64_t hp, int64_t wp, int pad_h,
               int pad_w, int64_t cp);

}  // namespace nhwc
}  // namespace ag
