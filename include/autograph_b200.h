/*
 * autograph_b200 — C ABI of the B200 (sm_100a) backend for autograph's
 * dense-contraction path.
 *
 * Every operator entry point below stands where the reference has one krnl
 * dispatch site (`kernels::NAME::builder()?.specialize(..).build(device)?.dispatch(..)`).
 * The comment above each declaration names that site by file:line inside the
 * reference project.  Arguments mirror what the dispatch site passes: device
 * pointers to the caller's buffers, element offsets, element strides, sizes
 * and scalars.
 *
 * Conventions
 *  - Every function returns an ag_status (0 = ok, < 0 = error); the message of
 *    the most recent error on the calling thread is ag_last_error().  Nothing
 *    throws, aborts or traps the device.  (The reference returns
 *    anyhow::Result everywhere and bails on shape / type mismatches.)
 *  - The caller owns all tensor memory.  The library keeps no pointer after a
 *    call returns, except its own per-device workspace.
 *  - Calls on one ag_device run asynchronously, in submission order, on that
 *    device's CUDA stream (like krnl's device queue).  Only ag_download,
 *    ag_device_wait and the calls that return a host scalar synchronise.
 *  - Any host thread may call; calls on one ag_device are serialised inside.
 *  - dtype is AG_F32 or AG_BF16 for values, AG_U8/U16/U32 for class labels.
 *  - There is no CPU fallback: without a usable CUDA device every call fails
 *    with AG_ERR_CUDA.
 */
#ifndef AUTOGRAPH_B200_H
#define AUTOGRAPH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define AG_API __attribute__((visibility("default")))
#else
#define AG_API
#endif

typedef struct ag_device ag_device;
typedef struct ag_model ag_model;
typedef struct ag_comm ag_comm;

typedef enum ag_dtype { AG_F32 = 0, AG_BF16 = 1, AG_U8 = 2, AG_U16 = 3, AG_U32 = 4 } ag_dtype;

typedef enum ag_status {
    AG_OK = 0,
    AG_ERR_INVALID = -1,        /* null pointer, negative size, bad enum */
    AG_ERR_SHAPE = -2,          /* shape mismatch (reference: bail!("a_rows != c_rows ...")) */
    AG_ERR_DTYPE = -3,          /* unsupported scalar type */
    AG_ERR_CUDA = -4,           /* CUDA runtime / driver error, message has the CUDA string */
    AG_ERR_OOM = -5,            /* device allocation failed */
    AG_ERR_DEVICE_TIMEOUT = -6, /* a bounded device-side wait gave up */
    AG_ERR_UNSUPPORTED = -7,    /* valid request this build does not implement */
    AG_ERR_LIMIT = -8           /* size beyond a documented fixed limit */
} ag_status;

/* Convolution options; ≙ Im2ColConv2Options / ConvOptions<Ix2> (src/ops.rs:9-39,
 * src/learn/neural_network/layer.rs:54-145). */
typedef struct ag_conv2_options {
    int32_t filter[2];   /* fh, fw */
    int32_t padding[2];  /* ph, pw */
    int32_t stride[2];   /* sh, sw */
    int32_t dilation[2]; /* dh, dw */
} ag_conv2_options;

/* ---------------------------------------------------------------- runtime */

AG_API const char *ag_last_error(void);
AG_API const char *ag_version(void);
/* Diagnostic with no counterpart in the reference: number of GPU kernels this
 * library has launched in the calling process since it was loaded. */
AG_API int ag_kernel_launch_count(uint64_t *count);

/* ≙ iterating krnl devices (tests/integration_tests.rs:24-44). */
AG_API int ag_device_count(int *count);
/* ≙ Device::builder().index(i).build() (tests/integration_tests.rs:27-30).
 * Creates a non-blocking stream owned by the device object. */
AG_API int ag_device_create(int ordinal, ag_device **out);
/* Same, but work is submitted to a stream the caller owns (cudaStream_t). */
AG_API int ag_device_create_on_stream(int ordinal, void *cuda_stream, ag_device **out);
AG_API int ag_device_destroy(ag_device *dev);
/* ≙ device.wait() (src/tensor/linalg.rs:549). Also reports a device-side timeout flag. */
AG_API int ag_device_wait(ag_device *dev);
/* Diagnostic with no counterpart in the reference: exercises the bounded device-side wait
 * that every tcgen05 kernel of the library uses.  Enqueues one small kernel that waits on a
 * barrier nothing will ever complete; after limit_ns (at most one second) the wait gives up,
 * the kernel records status 199 and returns, and the next ag_device_wait reports
 * AG_ERR_DEVICE_TIMEOUT.  The GPU and the device object stay usable.  For tests of a host's
 * error handling. */
AG_API int ag_debug_expiring_wait(ag_device *dev, uint64_t limit_ns);
AG_API void *ag_device_stream(ag_device *dev);
AG_API int ag_device_ordinal(ag_device *dev);

/* ≙ Buffer allocation / transfer behind Tensor::into_device and into_array
 * (src/tensor.rs:1819-1833, 1923-1945). ag_upload is asynchronous with respect
 * to the host only when `host` is pinned memory; ag_download blocks until the
 * data is on the host. */
AG_API int ag_alloc(ag_device *dev, size_t bytes, void **dptr);
AG_API int ag_free(ag_device *dev, void *dptr);
AG_API int ag_host_alloc(size_t bytes, void **hptr); /* pinned host memory */
AG_API int ag_host_free(void *hptr);
AG_API int ag_upload(ag_device *dev, void *dptr, const void *host, size_t bytes);
AG_API int ag_download(ag_device *dev, void *host, const void *dptr, size_t bytes);
AG_API int ag_copy(ag_device *dev, void *dst, const void *src, size_t bytes);
AG_API int ag_fill_zero(ag_device *dev, void *dptr, size_t bytes);

/* ----------------------------------------------------------------- linalg */

/* C = alpha * A.B + beta * C.  ≙ fn gemm + kernels::gemm_<T>
 * (src/tensor/linalg.rs:249-360, 30-246), reached from Dot for TensorBase /
 * ScalarTensorBase (:362-468) and Variable2::dot (autograd.rs:607-627).
 * A is m x k, B is k x n, C is m x n; off_* are element offsets into the
 * buffers, rs* / cs* are row / column strides in elements (may describe a
 * transposed view; never a copy).  bf16 inputs are multiplied and accumulated
 * in f32 and the result is rounded once (linalg.rs:244).  beta == 0 never
 * reads C.  Large-k, small-output products are split along k with f32 partial
 * sums and a fixed reduction order (deterministic). */
AG_API int ag_gemm(ag_device *dev, ag_dtype dtype, int64_t m, int64_t k, int64_t n, float alpha,
                   const void *a, int64_t off_a, int64_t rsa, int64_t csa,
                   const void *b, int64_t off_b, int64_t rsb, int64_t csb,
                   float beta, void *c, int64_t off_c, int64_t rsc, int64_t csc);

/* The same product as ag_gemm for callers that cannot allocate device memory
 * (it has no counterpart in the reference).  Some hosts own all of a GPU's
 * memory themselves, or forbid driver allocations after start-up; ag_gemm does
 * not suit them because a product that is split along k keeps its partial sums
 * in a workspace grown with cudaMalloc, and creating an ag_device allocates too.
 * This entry point takes a device ordinal and a cudaStream_t instead of an
 * ag_device, keeps the partial sums in a fixed 4 MiB array inside the library
 * image (held by every GPU that loads the library, until the process exits) and
 * calls no allocating routine.  Limit: m * n <= 524288 output elements, else
 * AG_ERR_LIMIT.  The first call on a GPU looks up the array's device address;
 * make that first call before any stream capture.  All calls on a GPU share the
 * array: calls that overlap on the GPU (different streams, no ordering) race.
 * Always runs the SIMT engine (f32 accumulation; bf16 inputs allowed). */
AG_API int ag_gemm_static_scratch(int ordinal, void *cuda_stream, ag_dtype dtype, int64_t m,
                                  int64_t k, int64_t n, float alpha, const void *a, int64_t off_a,
                                  int64_t rsa, int64_t csa, const void *b, int64_t off_b,
                                  int64_t rsb, int64_t csb, float beta, void *c, int64_t off_c,
                                  int64_t rsc, int64_t csc);

/* y = x . w (+ bias) (then relu when fuse_relu != 0), all row-major contiguous:
 * ≙ Dense::forward (layer.rs:1134-1143: dot, then add_assign of the bias) with the
 * following Relu::forward (layer.rs:1254-1267) folded in.  x [bs, inputs],
 * w [inputs, outputs], bias [outputs] or NULL, y [bs, outputs].  Equals the
 * separate calls bit for bit. */
AG_API int ag_dense_forward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                            int64_t inputs, const void *w, int64_t outputs, const void *bias,
                            int fuse_relu, void *y);

/* A chain of Dense layers, each optionally followed by Relu, in one call:
 * y = L_n(..relu?(L_1(x))), L_i(v) = v . w_i (+ bias_i); ≙ the run of Dense::forward /
 * Relu::forward pairs at the end of a model's derived Forward (layer.rs:1134-1143,
 * 1254-1267; autograph_backend.rs:129-146).  dims has n_layers + 1 entries (input width,
 * then every output width); weights[i] is [dims[i], dims[i+1]] row-major; biases may be
 * NULL or hold NULL entries.  Small chains run as one kernel that keeps the
 * activations in shared memory; results equal the separate calls bit for bit. */
AG_API int ag_dense_chain_forward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                                  int32_t n_layers, const int64_t *dims,
                                  const void *const *weights, const void *const *biases,
                                  const int32_t *relu, void *y);

/* The same chain for a pass that records gradients: every layer's values are kept, because the
 * backward edges need them (Dense::forward keeps its input, layer.rs:1134-1143; Relu's edge gates
 * on its input, layer.rs:1283-1296).  pre_out[i] [bs, dims[i+1]] receives Dense i's output,
 * act_out[i] (read only where relu[i] != 0) the Relu's output; the chain's result is the last
 * of them.  One kernel for small chains, else layer by layer; values equal the separate calls. */
AG_API int ag_dense_chain_forward_keep(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                                       int32_t n_layers, const int64_t *dims,
                                       const void *const *weights, const void *const *biases,
                                       const int32_t *relu, void *const *pre_out,
                                       void *const *act_out);

/* Every backward edge of such a chain in one call (Variable2::dot's edges dX = dY.W^T and
 * dW = X^T.dY, autograd.rs:607-627; the bias edge's column sum, autograd.rs:490-542; Relu's
 * gate on its input, layer.rs:1283-1296).  layer_in[i] [bs, dims[i]] is Dense i's input,
 * gate[i] the Dense's own output when a Relu follows it (NULL otherwise), dy [bs, dims[n]] the
 * gradient at the chain's output.  g[i] [bs, dims[i+1]] receives the gradient at Dense i's
 * output (g[n-1] may be NULL when gate[n-1] is NULL: dy is that gradient); dx (may be NULL) the
 * gradient at the chain's input; dw[i] [dims[i], dims[i+1]] and db[i] (db or entries may be
 * NULL) the parameter gradients, overwritten.  Small chains at small batch run as two kernels;
 * anything else goes layer by layer through ag_relu_backward / ag_gemm / ag_bias_grad. */
AG_API int ag_dense_chain_backward(ag_device *dev, ag_dtype dtype, int64_t bs, int32_t n_layers,
                                   const int64_t *dims, const void *const *layer_in,
                                   const void *const *weights, const void *const *gate,
                                   const void *dy, void *const *g, void *dx, void *const *dw,
                                   void *const *db);

/* ------------------------------------------------------------ convolution */

/* y = conv2(x, w) (+ bias) (then relu when fuse_relu != 0), NCHW.
 * Replaces the sequence im2col_conv2 -> dot(Wmat^T) -> permute to NCHW ->
 * bias add of conv2 / conv2_im2col (src/learn/neural_network/layer.rs:930-1005);
 * fuse_relu folds the following Relu::forward (layer.rs:1254-1267).
 * x [bs,ic,ih,iw], w [oc,ic,fh,fw], bias [oc] or NULL, y [bs,oc,oh,ow] with
 * oh, ow from ag_conv2_output_shape. All tensors contiguous. */
AG_API int ag_conv2_forward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs, int64_t ic,
                            int64_t ih, int64_t iw, const void *w, int64_t oc, const void *bias,
                            const ag_conv2_options *opt, int fuse_relu, void *y);

/* Inference fusion of the chain Conv2::forward -> Relu::forward -> MaxPool2::forward
 * (layer.rs:1035-1047, 1254-1267, 1193-1216 -> ops.rs:1106-1141): y = max_pool2(relu?(conv2(x, w)
 * + bias)) with pool window (pool_h, pool_w) and stride = window.  Equals the three separate calls
 * bit for bit; y is [bs, oc, (oh-pool_h)/pool_h+1, (ow-pool_w)/pool_w+1].  The convolution output
 * is never written to memory when the direct kernel applies (default options, 5x5 / 3x3 filter,
 * few channels, 2x2 pool); other shapes run convolution and pool back to back. */
AG_API int ag_conv2_relu_max_pool2_forward(ag_device *dev, ag_dtype dtype, const void *x,
                                           int64_t bs, int64_t ic, int64_t ih, int64_t iw,
                                           const void *w, int64_t oc, const void *bias,
                                           const ag_conv2_options *opt, int fuse_relu,
                                           int32_t pool_h, int32_t pool_w, void *y);

/* One convolution stage of ag_conv_dense_chain_forward: y = max_pool2?(relu?(conv2(x, w) + bias)).
 * pool = {0, 0} means no pool; otherwise the window, with stride = window. */
typedef struct ag_conv_stage {
    const void *w;            /* [oc, ic, fh, fw] */
    const void *bias;         /* [oc] or NULL */
    int64_t oc;
    ag_conv2_options options;
    int32_t relu;
    int32_t pool[2];
} ag_conv_stage;

/* Conv2::forward -> Relu::forward -> MaxPool2::forward (2x2 window and stride) for a pass that
 * records gradients: pre [bs, oc, oh, ow] receives the convolution's output (+ bias), which the
 * Relu's and the pool's backward edges read (layer.rs:1283-1296, 1203-1212), y [bs, oc, oh/2, ow/2]
 * the pooled activations.  One kernel for the shapes the direct kernel takes (fewer than 32 output
 * channels), otherwise ag_conv2_forward followed by ag_relu_max_pool2_forward; the values are those
 * of the separate calls. */
AG_API int ag_conv2_relu_max_pool2_forward_keep(ag_device *dev, ag_dtype dtype, const void *x,
                                                int64_t bs, int64_t ic, int64_t ih, int64_t iw,
                                                const void *w, int64_t oc, const void *bias,
                                                const ag_conv2_options *opt, void *pre, void *y);

/* Inference fusion of a whole small network: n_conv stages of Conv2::forward -> Relu::forward ->
 * MaxPool2::forward (layer.rs:1035-1047, 1254-1267, 1193-1216), Flatten::forward
 * (layer.rs:1297-1309) and n_dense Dense::forward / Relu::forward pairs (layer.rs:1134-1143) --
 * the derived Forward of the reference's LeNet5 (benches/neural-network-benches/src/
 * autograph_backend.rs:129-146) -- as ONE kernel that keeps every activation in shared memory.
 * x [bs, ic, ih, iw]; dense arguments as in ag_dense_chain_forward (dims[0] must equal the
 * flattened size of the last stage); y [bs, dims[n_dense]].  Equals the layer-by-layer calls bit
 * for bit.  Only networks that fit the kernel are taken (default convolution options, one 5x5 or
 * 3x3 filter size, 2x2 pools, <= 16 input and <= 64 output channels per stage, dense layers with
 * <= 2048 inputs and <= 256 outputs, 8 images of every activation within one CTA's shared
 * memory); any other network returns AG_ERR_UNSUPPORTED without touching y, and the caller runs
 * the layers one by one. */
AG_API int ag_conv_dense_chain_forward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                                       int64_t ic, int64_t ih, int64_t iw, int32_t n_conv,
                                       const ag_conv_stage *stages, int32_t n_dense,
                                       const int64_t *dims, const void *const *weights,
                                       const void *const *biases, const int32_t *relu, void *y);

/* The same network on u8 images: the scaled_cast above (x = alpha * u8) is done while the images
 * are staged in shared memory, so a quarter of the bytes cross PCIe / HBM and no float copy of the
 * batch is ever written.  ≙ images_to_device_and_scale followed by the model's forward
 * (examples/neural-network-mnist/src/main.rs:236-243, 275-300).  Equals ag_scaled_cast_u8 followed
 * by ag_conv_dense_chain_forward bit for bit. */
AG_API int ag_conv_dense_chain_forward_u8(ag_device *dev, ag_dtype dtype, const uint8_t *x,
                                          float alpha, int64_t bs, int64_t ic, int64_t ih,
                                          int64_t iw, int32_t n_conv, const ag_conv_stage *stages,
                                          int32_t n_dense, const int64_t *dims,
                                          const void *const *weights, const void *const *biases,
                                          const int32_t *relu, void *y);

/* dx = col2im(dy . Wmat): replaces the input edge of conv2_im2col
 * (layer.rs:976-988) = dot + kernels::col2im_conv2_<T> (src/tensor/ops.rs:1602-1667).
 * dy [bs,oc,oh,ow] (NCHW, as the autograd edge receives it), dx [bs,ic,ih,iw]. */
AG_API int ag_conv2_backward_input(ag_device *dev, ag_dtype dtype, const void *w, int64_t oc,
                                   int64_t ic, const void *dy, int64_t bs, int64_t ih, int64_t iw,
                                   const ag_conv2_options *opt, void *dx);

/* dw = dy^T . im2col(x): replaces the weight edge of conv2_im2col (layer.rs:989-997).
 * dw [oc,ic,fh,fw] = beta * dw + gradient (beta = 1 accumulates, as
 * Node::backward_grad does for a second edge, autograd.rs:126-131). */
AG_API int ag_conv2_backward_weight(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                                    int64_t ic, int64_t ih, int64_t iw, const void *dy, int64_t oc,
                                    const ag_conv2_options *opt, float beta, void *dw);

/* Output size (i + 2p - d(f-1) - 1)/s + 1 (src/ops.rs:28-38). Fails with
 * AG_ERR_SHAPE when it is not positive. */
AG_API int ag_conv2_output_shape(int64_t ih, int64_t iw, const ag_conv2_options *opt, int64_t *oh,
                                 int64_t *ow);

/* ≙ kernels::im2col_conv2_<T> (src/tensor/ops.rs:831-888, 1536-1599).
 * x [bs,c,ih,iw] -> y [bs*oh*ow, c*fh*fw]; kept for trait / test parity. */
AG_API int ag_im2col_conv2(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs, int64_t c,
                           int64_t ih, int64_t iw, const ag_conv2_options *opt, void *y);

/* ≙ kernels::col2im_conv2_<T> (src/tensor/ops.rs:982-1037, 1602-1667).
 * x [bs*gh*gw, c*fh*fw] -> y [bs,c,oh,ow]; (gh, gw) is Col2ImConv2Options::shape
 * and the image size is (g-1)*s + d*(f-1) + 1 - 2p (src/ops.rs:67-78). Sums in f32. */
AG_API int ag_col2im_conv2(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs, int64_t c,
                           int64_t gh, int64_t gw, const ag_conv2_options *opt, void *y);

/* ---------------------------------------------------------------- pooling */

/* ≙ kernels::max_pool2_<T> (src/tensor/ops.rs:1106-1141, 1670-1702); host
 * semantics of :1040-1088 (first maximum wins). x [bs,c,ih,iw] ->
 * y [bs,c,(ih-h)/sh+1,(iw-w)/sw+1]. */
AG_API int ag_max_pool2(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs, int64_t c,
                        int64_t ih, int64_t iw, int32_t h, int32_t w, int32_t sh, int32_t sw,
                        void *y);

/* ≙ kernels::max_pool2_backward_<T> (src/tensor/ops.rs:1228-1275, 1705-1744)
 * with the host semantics of :1144-1207: dx must arrive holding a copy of the
 * forward input (layer.rs:1203-1212); each window is zeroed and receives dy at
 * its first maximum; cells no window covers keep their value.  Requires
 * non-overlapping windows (sh >= h and sw >= w), as in every use by the reference. */
AG_API int ag_max_pool2_backward(ag_device *dev, ag_dtype dtype, void *dx, int64_t bs, int64_t c,
                                 int64_t ih, int64_t iw, int32_t h, int32_t w, int32_t sh,
                                 int32_t sw, const void *dy);
/* The same result without the caller's copy: dx = max_pool2_backward(copy of x, dy) in one
 * pass (x is read, dx written; x == dx is the in-place form above).  ≙ the input edge of
 * MaxPool2::forward (layer.rs:1203-1212: clone the input, then max_pool2_backward on the clone). */
AG_API int ag_max_pool2_backward_from_input(ag_device *dev, ag_dtype dtype, const void *x,
                                            int64_t bs, int64_t c, int64_t ih, int64_t iw,
                                            int32_t h, int32_t w, int32_t sh, int32_t sw,
                                            const void *dy, void *dx);

/* Relu::forward followed by MaxPool2::forward with a 2x2 window and stride (layer.rs:1254-1298,
 * 1193-1216) as one pass over x [bs,c,ih,iw] (ih, iw even): y = max_pool2(relu(x)); the Relu's
 * output is not materialised.  AG_ERR_UNSUPPORTED for odd planes or tensors that are not
 * element-pair aligned. */
AG_API int ag_relu_max_pool2_forward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                                     int64_t c, int64_t ih, int64_t iw, void *y);
/* The two backward edges of that pair in one pass: dx = relu_backward(x, max_pool2_backward(copy of
 * relu(x), dy)) — the gradient lands on the first maximum of relu(x) in every window and passes
 * where x >= 0 (layer.rs:1203-1212, 1283-1296, 1526-1540). */
AG_API int ag_relu_max_pool2_backward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                                      int64_t c, int64_t ih, int64_t iw, const void *dy, void *dx);

/* ----------------------------------------------------------- input pipeline */

/* y = alpha * x with x u8 and y f32 / bf16: ≙ Tensor::scaled_cast (src/tensor/ops.rs:209-218 ->
 * assign, :295), the step that turns u8 images into network input
 * (examples/neural-network-mnist/src/main.rs:236-243, alpha = 1/255).  Cast and product are in
 * the output type: alpha is rounded to it first and the product is rounded once. */
AG_API int ag_scaled_cast_u8(ag_device *dev, ag_dtype dtype, float alpha, const uint8_t *x, void *y,
                             int64_t n);

/* ------------------------------------------------------------------- relu */

/* ≙ kernels::relu_<T> / relu_mut_<T> (layer.rs:1300-1369, 1546-1553): y = x >= 0 ? x : 0.
 * y may alias x (relu_mut). */
AG_API int ag_relu(ag_device *dev, ag_dtype dtype, const void *x, void *y, int64_t n);
/* ≙ kernels::relu_backward_<T> / relu_backward_mut_<T> (layer.rs:1413-1510, 1555-1563):
 * dx = x >= 0 ? dy : 0, x is the layer input. dx may alias dy. */
AG_API int ag_relu_backward(ag_device *dev, ag_dtype dtype, const void *x, const void *dy,
                            void *dx, int64_t n);

/* ------------------------------------------------------------ elementwise */

/* y = alpha * x + y, computed in the element type.
 * ≙ scaled_add -> kernels::assign_<X>_<Y> with BinaryOp::Add, contiguous case
 * (src/tensor/ops.rs:257-318, 1357-1400). */
AG_API int ag_scaled_add(ag_device *dev, ag_dtype dtype, float alpha, const void *x, void *y,
                         int64_t n);

/* y[r, c, i] += bias[c] for y viewed as [rows, cols, inner]; the broadcast
 * scaled_add behind Variable::add_assign (autograd.rs:571-599 -> ops.rs strided
 * assign kernels :1403-1490). inner = 1 for Dense, oh*ow for Conv2 (NCHW). */
AG_API int ag_bias_add(ag_device *dev, ag_dtype dtype, void *y, const void *bias, int64_t rows,
                       int64_t cols, int64_t inner);

/* y[c] = beta * y[c] + sum over r, i of x[r, c, i] for x viewed as [rows, cols, inner].
 * ≙ broadcast_backward -> sum_axis -> kernels::sum_axis<N>_<T>
 * (autograd.rs:490-542, src/tensor/reduce.rs:59-404, 578-833). f32 accumulation. */
AG_API int ag_bias_grad(ag_device *dev, ag_dtype dtype, const void *x, int64_t rows, int64_t cols,
                        int64_t inner, float beta, void *y);

/* -------------------------------------------------------------- criterion */

/* ≙ cross_entropy_loss_device + kernels::cross_entropy_loss_<X>_<T> + sum
 * (src/learn/criterion.rs:229-254, 299-324). x [bs,classes], t [bs] labels.
 * *loss_host receives the SUM over the batch (synchronises). */
AG_API int ag_cross_entropy_loss(ag_device *dev, ag_dtype dtype, ag_dtype label_dtype,
                                 const void *x, const void *t, int64_t bs, int64_t classes,
                                 float *loss_host);

/* The same loss left in device memory (*loss_dev, one f32) without synchronising, so
 * that a whole training step can be enqueued (and captured in a CUDA graph) before
 * the host reads the value. ≙ the same kernels as ag_cross_entropy_loss. */
AG_API int ag_cross_entropy_loss_device(ag_device *dev, ag_dtype dtype, ag_dtype label_dtype,
                                        const void *x, const void *t, int64_t bs, int64_t classes,
                                        float *loss_dev);

/* ag_cross_entropy_loss_device together with the gradient its backward edge would produce for an
 * output gradient dy (ag_cross_entropy_loss_backward(.., dy, dx)): one kernel for up to 1024 rows,
 * where loss and gradient share the row maxima and sums; two launches beyond.  For steps whose
 * loss is always differentiated with the seed gradient 1 (Node::backward, autograd.rs:224-235). */
AG_API int ag_cross_entropy_loss_device_grad(ag_device *dev, ag_dtype dtype, ag_dtype label_dtype,
                                             const void *x, const void *t, int64_t bs,
                                             int64_t classes, float *loss_dev, float dy, void *dx);

/* ≙ kernels::cross_entropy_loss_backward_<X>_<T>
 * (src/learn/neural_network/criterion.rs:79-137, 154-184):
 * dx = (dy / bs) * (softmax(x) - onehot(t)). */
AG_API int ag_cross_entropy_loss_backward(ag_device *dev, ag_dtype dtype, ag_dtype label_dtype,
                                          const void *x, const void *t, int64_t bs,
                                          int64_t classes, float dy, void *dx);

/* ≙ kernels::accuracy_<X>_<T> + sum (src/learn/criterion.rs:100-128, 271-296):
 * counts rows whose target logit is strictly greater than every other logit
 * (synchronises). */
AG_API int ag_accuracy(ag_device *dev, ag_dtype dtype, ag_dtype label_dtype, const void *x,
                       const void *t, int64_t bs, int64_t classes, uint64_t *correct_host);

/* -------------------------------------------------------------- optimizer */

/* ≙ SGD::update without momentum (optimizer.rs:419-424): w = cast_T(-lr) * g + w in T. */
AG_API int ag_sgd_update(ag_device *dev, ag_dtype dtype, void *w, const void *g, int64_t n,
                         float lr);
/* ≙ kernels::sgd_update_with_momentum_<T> (optimizer.rs:430-500, 509-545):
 * v = m*v + g; w -= lr*v in f32, stored back in T. */
AG_API int ag_sgd_update_momentum(ag_device *dev, ag_dtype dtype, void *w, const void *g, void *v,
                                  int64_t n, float lr, float momentum);

/* --------------------------------------------------- neural-network layer
 * Host-side mirror of the reference's Layer / Forward objects for the
 * benchmark networks (benches/neural-network-benches/src/autograph_backend.rs:16-163):
 * a model is a chain of Conv2 / Relu / MaxPool2 / Flatten / Dense layers with
 * resident parameters, run through define-by-run autograd on the device. */

typedef enum ag_layer_kind {
    AG_LAYER_CONV2 = 0,   /* a = inputs, b = outputs, c = fh, d = fw, bias */
    AG_LAYER_RELU = 1,
    AG_LAYER_MAXPOOL2 = 2, /* c = h, d = w (stride = filter, layer.rs:535-539) */
    AG_LAYER_FLATTEN = 3,
    AG_LAYER_DENSE = 4    /* a = inputs, b = outputs, bias; c = 0, or 1 + the index of an earlier
                           * Dense layer of the same shape whose parameters this layer shares
                           * (one Parameter feeding two layers: its gradients are summed,
                           * autograd.rs:126-131) */
} ag_layer_kind;

typedef struct ag_layer_spec {
    int32_t kind;
    int32_t a, b, c, d;
    int32_t bias;
} ag_layer_spec;

/* ≙ LeNet5::new / the layer builders (autograph_backend.rs:104-163,
 * layer.rs:330-397, 452-504). Parameters are drawn from U(-a, a),
 * a = sqrt(2 / fan_in), from a generator seeded with `seed`. */
AG_API int ag_model_create(ag_device *dev, ag_dtype dtype, const ag_layer_spec *layers,
                           int32_t n_layers, uint64_t seed, ag_model **out);
AG_API int ag_model_create_lenet5(ag_device *dev, ag_dtype dtype, uint64_t seed, ag_model **out);
AG_API int ag_model_destroy(ag_model *model);
/* ≙ Layer::try_for_each_parameter (layer.rs:597-640): number of parameter
 * tensors, and the element count of each. */
AG_API int ag_model_parameter_count(ag_model *model, int32_t *count);
AG_API int ag_model_parameter_len(ag_model *model, int32_t index, int64_t *len);
/* Copy one parameter tensor from / to host memory holding `dtype` elements. */
AG_API int ag_model_set_parameter(ag_model *model, int32_t index, const void *host);
AG_API int ag_model_get_parameter(ag_model *model, int32_t index, void *host);
/* Gradient of the last training step (before the update consumed it). */
AG_API int ag_model_get_gradient(ag_model *model, int32_t index, void *host);
/* ≙ SGD::builder().momentum(m).build() (optimizer.rs:353-357); momentum < 0 = plain SGD.
 * Clears the velocity state. */
AG_API int ag_model_set_sgd(ag_model *model, float momentum);
/* The optimizer state of one parameter: SGD's "velocity" tensor (optimizer.rs:366-383), which
 * the reference stores in the parameter (ParameterBase::optim_state, autograd.rs:647-656) and
 * writes into checkpoints.  Host memory holding the model's dtype; same length as the
 * parameter. */
AG_API int ag_model_get_velocity(ag_model *model, int32_t index, void *host);
AG_API int ag_model_set_velocity(ag_model *model, int32_t index, const void *host);
/* Scale applied to gradients before the update (1/world for data parallel). */
AG_API int ag_model_set_grad_scale(ag_model *model, float scale);

/* ≙ LeNet5Classifier::infer (autograph_backend.rs:44-69): host input
 * [bs, c, h, w] of `dtype` elements -> device, forward, logits back to host
 * (blocking). */
AG_API int ag_model_infer(ag_model *model, const void *x_host, int64_t bs, int64_t c, int64_t h,
                          int64_t w, void *logits_host);
/* Pipelined form of ag_model_infer for a caller that keeps two batches in flight (a serving loop):
 * _enqueue copies the pinned batch to the device on the copy engine's own stream and enqueues the
 * network behind it (logits land in the pinned logits_host); it returns at once with a ticket
 * (0 or 1).  _wait blocks until that ticket's logits are in host memory.  At most two tickets are
 * in flight; while one batch computes, the next one crosses PCIe, so the steady-state rate is
 * that of the transfer alone.  Both buffers must be pinned (AG_ERR_INVALID otherwise) and must not
 * be touched until the ticket has been waited for.
 * ≙ two LeNet5Classifier::infer calls (autograph_backend.rs:44-69) overlapped. */
AG_API int ag_model_infer_enqueue(ag_model *model, const void *x_host, int64_t bs, int64_t c,
                                  int64_t h, int64_t w, void *logits_host, int32_t *ticket);
AG_API int ag_model_infer_wait(ag_model *model, int32_t ticket);

/* The same from u8 images, as the reference's MNIST example feeds its model
 * (examples/neural-network-mnist/src/main.rs:236-243): x = alpha * u8 in the model's dtype, then
 * the forward pass.  A one-kernel network reads the u8 images itself (from pinned host memory:
 * a quarter of the PCIe bytes of the float path); any other network runs ag_scaled_cast_u8 on the
 * device first.  Blocking. */
AG_API int ag_model_infer_u8(ag_model *model, const uint8_t *x_host, int64_t bs, int64_t c,
                             int64_t h, int64_t w, float alpha, void *logits_host);
/* Forward only, device-resident input and output (no host copies, no sync). */
AG_API int ag_model_forward_device(ag_model *model, const void *x_dev, int64_t bs, int64_t c,
                                   int64_t h, int64_t w, void *logits_dev);
/* ≙ LeNet5Classifier::train (autograph_backend.rs:70-85): init grads, forward,
 * cross_entropy_loss, backward, optimizer update. Labels are u8. *loss_host =
 * summed loss of the batch. */
AG_API int ag_model_train_step(ag_model *model, const void *x_host, const uint8_t *t_host,
                               int64_t bs, int64_t c, int64_t h, int64_t w, float lr,
                               float *loss_host);
/* The same step split in two for data-parallel training: gradients of this
 * rank's shard are left in one flat f32/bf16 bucket (device pointer and
 * element count returned) so that the caller can all-reduce it; apply then
 * runs the optimizer over the bucket. */
AG_API int ag_model_train_forward_backward(ag_model *model, const void *x_dev,
                                           const uint8_t *t_dev, int64_t bs, int64_t c, int64_t h,
                                           int64_t w, float *loss_host, void **grad_bucket,
                                           int64_t *grad_len);
AG_API int ag_model_apply_update(ag_model *model, float lr);
/* ag_model_train_forward_backward accepts loss_host == NULL: the step is then only enqueued (no
 * synchronisation), so the caller's all-reduce and ag_model_apply_update can be enqueued behind it
 * while it runs; this call waits for the stream and returns that step's loss (the one host read
 * per step that the reference's training loop makes, autograph_backend.rs:70-85). */
AG_API int ag_model_last_loss(ag_model *model, float *loss_host);

/* ------------------------------------------------------------ data parallel
 * The reference has no multi-device code.  Its networks shard by batch (every image is
 * independent, parameters are replicated), and because the loss gradient is scaled by the
 * local batch size (src/learn/neural_network/criterion.rs:84) a data-parallel step is: every
 * rank's forward / backward, ONE sum all-reduce of the flat gradient bucket, a factor
 * 1 / world, the optimizer (optimizer.rs:389-428).  A communicator spans up to 16 GPUs of
 * one box.  NCCL is looked up at run time (AG_ERR_UNSUPPORTED when it cannot be loaded). */

/* One process drives all GPUs: devs[r] is rank r's device object (its stream carries the
 * rank's collectives, so they are ordered with its kernels).  ≙ ncclCommInitAll. */
AG_API int ag_comm_create(ag_device *const *devs, int n, ag_comm **out);
/* One process per GPU: rank 0 calls ag_comm_unique_id (128 bytes), hands the id to the other
 * ranks by any means, and every rank calls ag_comm_create_rank.  ≙ ncclCommInitRank. */
AG_API int ag_comm_unique_id(void *id_out, size_t bytes);
AG_API int ag_comm_create_rank(ag_device *dev, int world, int rank, const void *unique_id,
                               size_t id_bytes, ag_comm **out);
AG_API int ag_comm_destroy(ag_comm *comm);
/* Number of ranks, and whether the GPUs can address one another's memory (what
 * ag_model_allreduce_update needs). */
AG_API int ag_comm_world(ag_comm *comm, int *world, int *fused_available);
/* Limit, in seconds, of ag_comm_wait and of the device-side wait of
 * ag_model_allreduce_update (default 2). */
AG_API int ag_comm_set_timeout(ag_comm *comm, double seconds);

/* buf (n elements of dtype, on rank's GPU) = sum over all ranks, in place, enqueued on the
 * rank's stream.  With one process per GPU each process calls it for its rank.  With one
 * process for all GPUs either one host thread per rank calls it, or one thread calls
 * ag_allreduce_sum_all with every rank's buffer. */
AG_API int ag_allreduce_sum(ag_comm *comm, int rank, ag_dtype dtype, void *buf, int64_t n);
AG_API int ag_allreduce_sum_all(ag_comm *comm, ag_dtype dtype, void *const *bufs, int64_t n);
/* Waits for rank's stream without blocking inside the driver: polls the stream and NCCL's
 * asynchronous error state, and gives up after the communicator's timeout
 * (AG_ERR_DEVICE_TIMEOUT; the rank's NCCL communicator is then aborted, because a collective
 * whose peer never joins cannot complete). */
AG_API int ag_comm_wait(ag_comm *comm, int rank);

/* The data-parallel tail of a training step as ONE kernel per GPU: sum all-reduce of the
 * model's gradient bucket over NVLink (each GPU reads its peers' buckets with plain loads
 * and adds them in rank order, so all replicas compute the same bits), the factor set by
 * ag_model_set_grad_scale, and the SGD update (≙ criterion.rs:84 + SGD::update,
 * optimizer.rs:389-428).  Same result as ag_allreduce_sum on the bucket followed by
 * ag_model_apply_update.  Enqueued on the model's stream; returns without waiting.  Buckets of
 * more than 512 KiB return AG_ERR_LIMIT (use the two calls above).  A rank whose peers do not
 * arrive within the communicator's timeout leaves its parameters untouched and reports
 * AG_ERR_DEVICE_TIMEOUT at the next ag_device_wait / ag_comm_wait. */
AG_API int ag_model_allreduce_update(ag_model *model, ag_comm *comm, int rank, float lr);

#ifdef __cplusplus
}
#endif
#endif /* AUTOGRAPH_B200_H */
