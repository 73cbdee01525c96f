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

// The same copy into the middle of a zero frame of pad_h rows / pad_w columns on every side.
int to_nhwc_framed(ag_device *dev, const __nv_bfloat16 *x, int64_t bs, int64_t c, int64_t h,
                   int64_t w, int64_t cp, int pad_h, int pad_w, __nv_bfloat16 *out);

// Channels-last back to NCHW: in [bs][hw][cp] -> out [bs][c][hw].
int from_nhwc(ag_device *dev, const __nv_bfloat16 *in, int64_t bs, int64_t c, int64_t hw, int64_t cp,
              __nv_bfloat16 *out);

// A stride-1 correlation on channels-last data, in the kernel's view: c_in channels of
// in_h x in_w (zero padding pad_h / pad_w) into c_out channels of out_h x out_w with an fh x fw
// filter.  `transposed` reads the filter bank [w_oc][w_ic][fh][fw] as the input gradient
// does (channel axes swapped, taps reversed).  Channel counts in memory are rounded up to 64.
struct NhwcConv {
    int64_t bs, c_in, in_h, in_w;
    int64_t c_out, out_h, out_w;
    int fh, fw, pad_h, pad_w;
    bool transposed;
};
// True when the kernel that takes this problem reads the activation inside a zero frame
// ([bs][in_h + 2 pad_h][in_w + 2 pad_w][cp]) instead of relying on out-of-range fill.
bool nhwc_wants_frame(const NhwcConv &c);
int64_t nhwc_filter_scratch_bytes(const NhwcConv &c);
int correlate_nhwc(ag_device *dev, const NhwcConv &c, const __nv_bfloat16 *act_nhwc, bool framed,
                   const __nv_bfloat16 *w, int64_t w_oc, int64_t w_ic, const __nv_bfloat16 *bias,
                   bool relu, __nv_bfloat16 *wk, __nv_bfloat16 *out_nhwc);

// Resident-filter variant (conv_tc_halo.cu): plan (false when the shape does not fit: more
// than 128 output channels, a box of more than 256 rows, or too little shared memory) and run
// on the framed channels-last activation [bs][hp][wp][cp] and the repacked filter bank.
bool halo_plan(int64_t bs, int64_t cp, int64_t hp, int64_t wp, int64_t c_out, int fh, int fw,
               int *block_n, int *halo_rows, int *stages, int *smem_bytes);
int run_halo(ag_device *dev, const __nv_bfloat16 *act_rows, const __nv_bfloat16 *wk, int64_t bs,
             int64_t cp, int64_t hp, int64_t wp, int fh, int fw, int64_t c_out, int64_t out_h,
             int64_t out_w, const __nv_bfloat16 *bias, bool relu, __nv_bfloat16 *out_nhwc);

// True when the tensor-core weight-gradient kernel takes the problem: stride 1,
// dilation 1, at least 32 output channels, filter width up to 8, at least 4096
// output pixels.  Few input channels are zero-padded to 64.
bool eligible_backward_weight(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
                              const ag_conv2_options *o);

// dw = beta * dw + gradient of conv2(x, w) with respect to w given dy, bf16.
int backward_weight(ag_device *dev, const __nv_bfloat16 *x, int64_t bs, int64_t ic, int64_t ih,
                    int64_t iw, const __nv_bfloat16 *dy, int64_t oc, const ag_conv2_options *o,
                    float beta, __nv_bfloat16 *dw);

// The same on channels-last data: x [bs][ih][iw][cp]; dy is addressed through its pitches in
// elements (pixel = ocp channels; dy_row_pitch and dy_image_pitch let it sit inside a frame),
// all multiples of 8.
int backward_weight_nhwc(ag_device *dev, const __nv_bfloat16 *x_nhwc, int64_t bs, int64_t ic,
                         int64_t ih, int64_t iw, const __nv_bfloat16 *dy_nhwc, int64_t dy_row_pitch,
                         int64_t dy_image_pitch, int64_t oc, const ag_conv2_options *o, float beta,
                         __nv_bfloat16 *dw);

}  // namespace convtc
}  // namespace ag
