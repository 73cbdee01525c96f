/*
 * CPU oracle for the dense-contraction path of autograph (TEST INFRASTRUCTURE).
 *
 * This file restates, in plain C, the host-side algorithms of the reference
 * project so that the CUDA kernels can be checked against them.  It is a
 * checker and a timed CPU baseline only: nothing in the shipped library links
 * or calls it.
 *
 * Parity status: the reference is Rust and cannot be built where this code
 * is developed, so the oracle is pinned on the generator-defined integer
 * vectors of the reference's own tests (tests/integration_tests.rs), whose
 * results are exact in f32, and cross-checked against independent numpy /
 * torch-f64 implementations.  Beyond those vectors the bit pattern of the
 * reference's host GEMM (third-party ndarray 0.15.6 / matrixmultiply, not
 * vendored) is "parity unpinned"; tolerances apply there.
 *
 * All tensors are passed as f32 arrays.  bf16 tensors are represented by f32
 * values that are exactly representable in bf16; functions take a `bf16`
 * flag and round their result to bf16 (round-to-nearest-even, like the `half`
 * crate) where the reference stores a bf16.
 *
 * Each function cites the reference file:line it follows (paths are relative
 * to the reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ---- bf16 rounding (half crate bf16::from_f32: round to nearest even) ---- */
static inline float bf16_round(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) { /* NaN: keep quiet NaN */
        u = (u | 0x00400000u) & 0xffff0000u;
    } else {
        uint32_t lsb = (u >> 16) & 1u;
        u += 0x7fffu + lsb;
        u &= 0xffff0000u;
    }
    memcpy(&x, &u, 4);
    return x;
}

ORC_API void orc_round_bf16(float *x, int64_t n) {
    for (int64_t i = 0; i < n; ++i) x[i] = bf16_round(x[i]);
}

/* scaled_cast of u8 images (src/tensor/ops.rs:209-218 -> assign, :295: y = alpha * x.cast()):
 * the cast and the product are in the output type, so for bf16 alpha is first rounded to
 * bf16 and the product rounded once (examples/neural-network-mnist/src/main.rs:196-199). */
ORC_API void orc_scaled_cast_u8(const unsigned char *x, float *y, int64_t n, float alpha, int bf16) {
    if (bf16) alpha = bf16_round(alpha);
    for (int64_t i = 0; i < n; ++i) {
        float v = alpha * (float)x[i];
        y[i] = bf16 ? bf16_round(v) : v;
    }
}

/* Overrides OMP_NUM_THREADS (launchers such as torchrun set it to 1). */
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------
 * GEMM: C = alpha * A.B + beta * C on strided 2-D views.
 * Contract of fn gemm (src/tensor/linalg.rs:249-360) and host Dot
 * (src/tensor/linalg.rs:362-423).  Strides are in elements.
 * acc: 0 = f32 accumulation in k order, 1 = f64 accumulation (tolerance
 * checker), 2 = accumulate in bf16 (every multiply and add rounded to bf16:
 * what the reference's generic host loop does for bf16 tensors).
 * beta == 0 never reads C (src/tensor/linalg.rs:215-218).
 * ---------------------------------------------------------------------- */
ORC_API void orc_gemm(int64_t m, int64_t k, int64_t n, float alpha,
                      const float *a, int64_t rsa, int64_t csa,
                      const float *b, int64_t rsb, int64_t csb,
                      float beta, float *c, int64_t rsc, int64_t csc,
                      int acc, int bf16) {
#pragma omp parallel for schedule(static) if (m * n * k > 100000)
    for (int64_t i = 0; i < m; ++i) {
        for (int64_t j = 0; j < n; ++j) {
            float r;
            if (acc == 1) {
                double s = 0.0;
                for (int64_t p = 0; p < k; ++p)
                    s += (double)a[i * rsa + p * csa] * (double)b[p * rsb + j * csb];
                double v = (double)alpha * s;
                if (beta != 0.f) v += (double)beta * (double)c[i * rsc + j * csc];
                r = (float)v;
            } else if (acc == 2) {
                float s = 0.f;
                for (int64_t p = 0; p < k; ++p)
                    s = bf16_round(s + bf16_round(a[i * rsa + p * csa] * b[p * rsb + j * csb]));
                float v = bf16_round(alpha * s);
                if (beta != 0.f) v = bf16_round(v + bf16_round(beta * c[i * rsc + j * csc]));
                r = v;
            } else {
                float s = 0.f;
                for (int64_t p = 0; p < k; ++p)
                    s += a[i * rsa + p * csa] * b[p * rsb + j * csb];
                float v = alpha * s;
                if (beta != 0.f) v += beta * c[i * rsc + j * csc];
                r = v;
            }
            c[i * rsc + j * csc] = bf16 ? bf16_round(r) : r;
        }
    }
}

/* Blocked, threaded f32 GEMM standing in for the matrixmultiply crate that
 * ndarray::linalg::general_mat_mul forwards to (src/tensor/linalg.rs:394-402).
 * Used for the timed CPU baseline; C is row-major contiguous [m,n]. */
ORC_API void orc_gemm_f32_fast(int64_t m, int64_t k, int64_t n,
                               const float *a, int64_t rsa, int64_t csa,
                               const float *b, int64_t rsb, int64_t csb,
                               float *c) {
    enum { MB = 64, KB = 256 };
#pragma omp parallel
    {
        float *bpack = (float *)malloc(sizeof(float) * KB * (size_t)n);
        float *apack = (float *)malloc(sizeof(float) * MB * KB);
#pragma omp for schedule(dynamic)
        for (int64_t i0 = 0; i0 < m; i0 += MB) {
            int64_t mb = (m - i0 < MB) ? (m - i0) : MB;
            for (int64_t i = 0; i < mb; ++i)
                memset(c + (i0 + i) * n, 0, sizeof(float) * (size_t)n);
            for (int64_t p0 = 0; p0 < k; p0 += KB) {
                int64_t kb = (k - p0 < KB) ? (k - p0) : KB;
                for (int64_t p = 0; p < kb; ++p)
                    for (int64_t j = 0; j < n; ++j)
                        bpack[p * n + j] = b[(p0 + p) * rsb + j * csb];
                for (int64_t i = 0; i < mb; ++i)
                    for (int64_t p = 0; p < kb; ++p)
                        apack[i * kb + p] = a[(i0 + i) * rsa + (p0 + p) * csa];
                for (int64_t i = 0; i < mb; ++i) {
                    float *crow = c + (i0 + i) * n;
                    for (int64_t p = 0; p < kb; ++p) {
                        float av = apack[i * kb + p];
                        const float *brow = bpack + p * n;
                        for (int64_t j = 0; j < n; ++j) crow[j] += av * brow[j];
                    }
                }
            }
        }
        free(bpack);
        free(apack);
    }
}

/* ------------------------------------------------------------------------
 * Convolution geometry (src/ops.rs:27-38; layer.rs ConvOptions::output_shape)
 * ---------------------------------------------------------------------- */
typedef struct {
    int fh, fw, ph, pw, sh, sw, dh, dw;
} conv_opt;

static inline int conv_out(int i, int f, int p, int s, int d) {
    return (i + 2 * p - d * (f - 1) - 1) / s + 1;
}

ORC_API void orc_conv2_output_shape(int ih, int iw, const int *opt, int *oh, int *ow) {
    *oh = conv_out(ih, opt[0], opt[2], opt[4], opt[6]);
    *ow = conv_out(iw, opt[1], opt[3], opt[5], opt[7]);
}

/* Naive forward convolution: the reference's own ground truth
 * conv2_direct_naive (tests/integration_tests.rs:1127-1174).
 * x [bs,ic,ih,iw], w [oc,ic,fh,fw] -> y [bs,oc,oh,ow]; opt = {fh,fw,ph,pw,sh,sw,dh,dw}.
 * acc64 != 0 accumulates in f64 (checker); else in f32 in the test's loop order. */
ORC_API void orc_conv2_naive(const float *x, const float *w, float *y, int bs, int ic, int ih,
                             int iw, int oc, const int *o, int acc64, int bf16) {
    int fh = o[0], fw = o[1], ph = o[2], pw = o[3], sh = o[4], sw = o[5], dh = o[6], dw = o[7];
    int oh = conv_out(ih, fh, ph, sh, dh), ow = conv_out(iw, fw, pw, sw, dw);
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < bs; ++b)
        for (int co = 0; co < oc; ++co)
            for (int hy = 0; hy < oh; ++hy)
                for (int wy = 0; wy < ow; ++wy) {
                    double s64 = 0.0;
                    float s32 = 0.f;
                    for (int ci = 0; ci < ic; ++ci)
                        for (int fi = 0; fi < fh; ++fi) {
                            int hx = -ph + sh * hy + dh * fi;
                            if (hx < 0 || hx >= ih) continue;
                            for (int fj = 0; fj < fw; ++fj) {
                                int wx = -pw + sw * wy + dw * fj;
                                if (wx < 0 || wx >= iw) continue;
                                float xv = x[((size_t)(b * ic + ci) * ih + hx) * iw + wx];
                                float wv = w[((size_t)(co * ic + ci) * fh + fi) * fw + fj];
                                s64 += (double)xv * (double)wv;
                                s32 += xv * wv;
                            }
                        }
                    float r = acc64 ? (float)s64 : s32;
                    y[((size_t)(b * oc + co) * oh + hy) * ow + wy] = bf16 ? bf16_round(r) : r;
                }
}

/* Naive backward-input: conv2_direct_backward_input_naive
 * (tests/integration_tests.rs:1253-1301), written as a gather per dx element. */
ORC_API void orc_conv2_backward_input_naive(const float *w, const float *dy, float *dx, int bs,
                                            int ic, int ih, int iw, int oc, const int *o,
                                            int acc64, int bf16) {
    int fh = o[0], fw = o[1], ph = o[2], pw = o[3], sh = o[4], sw = o[5], dh = o[6], dw = o[7];
    int oh = conv_out(ih, fh, ph, sh, dh), ow = conv_out(iw, fw, pw, sw, dw);
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < bs; ++b)
        for (int ci = 0; ci < ic; ++ci)
            for (int hx = 0; hx < ih; ++hx)
                for (int wx = 0; wx < iw; ++wx) {
                    double s64 = 0.0;
                    float s32 = 0.f;
                    for (int co = 0; co < oc; ++co)
                        for (int fi = 0; fi < fh; ++fi) {
                            int th = hx + ph - dh * fi;
                            if (th < 0 || th % sh != 0) continue;
                            int hy = th / sh;
                            if (hy >= oh) continue;
                            for (int fj = 0; fj < fw; ++fj) {
                                int tw = wx + pw - dw * fj;
                                if (tw < 0 || tw % sw != 0) continue;
                                int wy = tw / sw;
                                if (wy >= ow) continue;
                                float wv = w[((size_t)(co * ic + ci) * fh + fi) * fw + fj];
                                float g = dy[((size_t)(b * oc + co) * oh + hy) * ow + wy];
                                s64 += (double)wv * (double)g;
                                s32 += wv * g;
                            }
                        }
                    float r = acc64 ? (float)s64 : s32;
                    dx[((size_t)(b * ic + ci) * ih + hx) * iw + wx] = bf16 ? bf16_round(r) : r;
                }
}

/* Naive backward-weight: conv2_direct_backward_weight_naive
 * (tests/integration_tests.rs:1377-1423). */
ORC_API void orc_conv2_backward_weight_naive(const float *x, const float *dy, float *dwt, int bs,
                                             int ic, int ih, int iw, int oc, const int *o,
                                             int acc64, int bf16) {
    int fh = o[0], fw = o[1], ph = o[2], pw = o[3], sh = o[4], sw = o[5], dh = o[6], dw = o[7];
    int oh = conv_out(ih, fh, ph, sh, dh), ow = conv_out(iw, fw, pw, sw, dw);
#pragma omp parallel for collapse(2) schedule(static)
    for (int co = 0; co < oc; ++co)
        for (int ci = 0; ci < ic; ++ci)
            for (int fi = 0; fi < fh; ++fi)
                for (int fj = 0; fj < fw; ++fj) {
                    double s64 = 0.0;
                    float s32 = 0.f;
                    for (int b = 0; b < bs; ++b)
                        for (int hy = 0; hy < oh; ++hy) {
                            int hx = -ph + sh * hy + fi * dh;
                            if (hx < 0 || hx >= ih) continue;
                            for (int wy = 0; wy < ow; ++wy) {
                                int wx = -pw + sw * wy + fj * dw;
                                if (wx < 0 || wx >= iw) continue;
                                float xv = x[((size_t)(b * ic + ci) * ih + hx) * iw + wx];
                                float g = dy[((size_t)(b * oc + co) * oh + hy) * ow + wy];
                                s64 += (double)xv * (double)g;
                                s32 += xv * g;
                            }
                        }
                    float r = acc64 ? (float)s64 : s32;
                    dwt[((size_t)(co * ic + ci) * fh + fi) * fw + fj] = bf16 ? bf16_round(r) : r;
                }
}

/* Host direct convolution for f32 with default options, restating the
 * accumulation order of conv2_direct_host_f32
 * (src/learn/neural_network/layer/conv_direct.rs:760-946): images are spread
 * over threads (:844-849); for every output element the sum runs over
 * (input-channel block of 8, fi, fj, channel inside the block) with fused
 * multiply-add (:796-823, built with +fma).  No padding/stride/dilation. */
ORC_API void orc_conv2_direct_f32(const float *x, const float *w, float *y, int bs, int ic, int ih,
                                  int iw, int oc, int fh, int fw) {
    int oh = ih - fh + 1, ow = iw - fw + 1;
#pragma omp parallel for schedule(static)
    for (int b = 0; b < bs; ++b) {
        const float *xb = x + (size_t)b * ic * ih * iw;
        float *yb = y + (size_t)b * oc * oh * ow;
        for (int co = 0; co < oc; ++co) {
            float *yc = yb + (size_t)co * oh * ow;
            for (int i = 0; i < oh * ow; ++i) yc[i] = 0.f;
            for (int cb = 0; cb < ic; cb += 8)
                for (int hy = 0; hy < oh; ++hy) {
                    float *yr = yc + hy * ow;
                    for (int fi = 0; fi < fh; ++fi)
                        for (int fj = 0; fj < fw; ++fj)
                            for (int ci = cb; ci < ic && ci < cb + 8; ++ci) {
                                float wv = w[((size_t)(co * ic + ci) * fh + fi) * fw + fj];
                                const float *xr = xb + ((size_t)ci * ih + hy + fi) * iw + fj;
                                for (int wy = 0; wy < ow; ++wy) yr[wy] = fmaf(xr[wy], wv, yr[wy]);
                            }
                }
        }
    }
}

/* Gradient with respect to the input of the host direct convolution, restating the
 * accumulation order of conv2_direct_backward_input_host_f32
 * (src/learn/neural_network/layer/conv_direct.rs:948-1156): images are spread over threads
 * (:1083-1089); the gradient starts at zero (:1140) and every element is updated in place, in
 * this loop order: block of 8 output channels (:1098-1103), row of dy (:1106), tile of TWY
 * positions along that row (:1108-1126; TWY = min(7, ow), or min(8, ow) when there is a single
 * input channel, :1134-1139), filter row, filter column (:975-976), channel inside the block
 * (:982), with fused multiply-add (:987).  Default options only. */
ORC_API void orc_conv2_direct_backward_input_f32(const float *w, const float *dy, float *dx, int bs,
                                                 int ic, int ih, int iw, int oc, int fh, int fw) {
    int oh = ih - fh + 1, ow = iw - fw + 1;
    int twy_max = (ic == 1) ? 8 : 7;
    if (twy_max > ow) twy_max = ow;
#pragma omp parallel for schedule(static)
    for (int b = 0; b < bs; ++b) {
        float *dxb = dx + (size_t)b * ic * ih * iw;
        const float *dyb = dy + (size_t)b * oc * oh * ow;
        for (size_t i = 0; i < (size_t)ic * ih * iw; ++i) dxb[i] = 0.f;
        for (int ci = 0; ci < ic; ++ci) {   /* the lanes of an input-channel block are independent */
            float *dxc = dxb + (size_t)ci * ih * iw;
            for (int cyb = 0; cyb < oc; cyb += 8)
                for (int hy = 0; hy < oh; ++hy)
                    for (int wy0 = 0; wy0 < ow; wy0 += twy_max) {
                        int twy = ow - wy0 < twy_max ? ow - wy0 : twy_max;
                        for (int fi = 0; fi < fh; ++fi)
                            for (int fj = 0; fj < fw; ++fj)
                                for (int co = cyb; co < oc && co < cyb + 8; ++co) {
                                    float wv = w[((size_t)(co * ic + ci) * fh + fi) * fw + fj];
                                    const float *g = dyb + ((size_t)co * oh + hy) * ow + wy0;
                                    float *d = dxc + (size_t)(hy + fi) * iw + wy0 + fj;
                                    for (int t = 0; t < twy; ++t) d[t] = fmaf(g[t], wv, d[t]);
                                }
                    }
        }
    }
}

/* Gradient with respect to the weight, restating conv2_direct_backward_weight_host_f32
 * (conv_direct.rs:1158-1346): the batch is dealt out to threads_bs partial sums, image bid
 * going to partial bid % threads_bs (:1194-1201); a partial adds its images in ascending order
 * and, per image, walks the rows and columns of dy with fused multiply-add (:1241-1264); the
 * partials are then added in order, starting from zero (:1318-1343; a single partial is the
 * result as it is, :1313-1317).  threads_bs = min(threads / threads_c, bs) with threads_c =
 * min(threads, groups of output-channel blocks x input-channel blocks) (:1286-1291): the result
 * depends on the number of threads the reference runs with, which is a parameter here. */
ORC_API void orc_conv2_direct_backward_weight_f32(const float *x, const float *dy, float *dw, int bs,
                                                  int ic, int ih, int iw, int oc, int fh, int fw,
                                                  int threads) {
    int oh = ih - fh + 1, ow = iw - fw + 1;
    int oc_blocks = (oc + 7) / 8, ic_blocks = ic == 1 ? 1 : (ic + 7) / 8;
    int tby = oc_blocks < 4 ? oc_blocks : 4;
    int oc_groups = (oc_blocks + tby - 1) / tby;
    if (threads < 1) threads = 1;
    int threads_c = threads < oc_groups * ic_blocks ? threads : oc_groups * ic_blocks;
    int threads_bs = threads / threads_c;
    if (threads_bs > bs) threads_bs = bs;
    if (threads_bs < 1) threads_bs = 1;
    size_t plane = (size_t)oc * ic * fh * fw;
    float *tmp = (float *)calloc((size_t)threads_bs * plane, sizeof(float));
#pragma omp parallel for schedule(static)
    for (int tb = 0; tb < threads_bs; ++tb) {
        float *acc = tmp + (size_t)tb * plane;
        for (int b = tb; b < bs; b += threads_bs)
            for (int co = 0; co < oc; ++co)
                for (int ci = 0; ci < ic; ++ci)
                    for (int fi = 0; fi < fh; ++fi)
                        for (int fj = 0; fj < fw; ++fj) {
                            float a = acc[((size_t)(co * ic + ci) * fh + fi) * fw + fj];
                            for (int hy = 0; hy < oh; ++hy) {
                                const float *xr = x + (((size_t)b * ic + ci) * ih + hy + fi) * iw + fj;
                                const float *g = dy + (((size_t)b * oc + co) * oh + hy) * ow;
                                for (int wy = 0; wy < ow; ++wy) a = fmaf(xr[wy], g[wy], a);
                            }
                            acc[((size_t)(co * ic + ci) * fh + fi) * fw + fj] = a;
                        }
    }
    if (threads_bs == 1) {
        for (size_t i = 0; i < plane; ++i) dw[i] = tmp[i];
    } else {
        for (size_t i = 0; i < plane; ++i) {
            float s = 0.f;
            for (int tb = 0; tb < threads_bs; ++tb) s += tmp[(size_t)tb * plane + i];
            dw[i] = s;
        }
    }
    free(tmp);
}

/* im2col, host version (src/tensor/ops.rs:741-813): rows (b,oh,ow), columns
 * (c,fi,fj), zero outside the image. */
ORC_API void orc_im2col_conv2(const float *x, float *y, int bs, int c, int ih, int iw,
                              const int *o) {
    int fh = o[0], fw = o[1], ph = o[2], pw = o[3], sh = o[4], sw = o[5], dh = o[6], dw = o[7];
    int oh = conv_out(ih, fh, ph, sh, dh), ow = conv_out(iw, fw, pw, sw, dw);
#pragma omp parallel for schedule(static)
    for (int b = 0; b < bs; ++b)
        for (int hy = 0; hy < oh; ++hy)
            for (int wy = 0; wy < ow; ++wy)
                for (int ci = 0; ci < c; ++ci)
                    for (int fi = 0; fi < fh; ++fi)
                        for (int fj = 0; fj < fw; ++fj) {
                            int hx = -ph + fi * dh + sh * hy;
                            int wx = -pw + fj * dw + sw * wy;
                            float v = 0.f;
                            if (hx >= 0 && hx < ih && wx >= 0 && wx < iw)
                                v = x[((size_t)(b * c + ci) * ih + hx) * iw + wx];
                            y[(((((size_t)b * oh + hy) * ow + wy) * c + ci) * fh + fi) * fw + fj] = v;
                        }
}

/* col2im, host version (src/tensor/ops.rs:891-964): scatter-add of patch
 * matrix rows into the image, in (c, hid, wid, fi, fj) order, accumulating in
 * the element type (f32; for bf16 each add is rounded to bf16 as the generic
 * host code does).  gh,gw = patch grid ("shape" in Col2ImConv2Options),
 * image size = (g-1)*s + d*(f-1) + 1 - 2p (src/ops.rs:67-78).
 * device_acc != 0 instead follows the device kernel (ops.rs:1602-1667): one
 * f32 sum per image element, rounded once. */
ORC_API void orc_col2im_conv2(const float *x, float *y, int bs, int c, int gh, int gw,
                              const int *o, int bf16, int device_acc) {
    int fh = o[0], fw = o[1], ph = o[2], pw = o[3], sh = o[4], sw = o[5], dh = o[6], dw = o[7];
    int oh = (gh - 1) * sh + dh * (fh - 1) + 1 - 2 * ph;
    int ow = (gw - 1) * sw + dw * (fw - 1) + 1 - 2 * pw;
#pragma omp parallel for schedule(static)
    for (int b = 0; b < bs; ++b) {
        float *yb = y + (size_t)b * c * oh * ow;
        for (size_t i = 0; i < (size_t)c * oh * ow; ++i) yb[i] = 0.f;
        for (int ci = 0; ci < c; ++ci)
            for (int hid = 0; hid < gh; ++hid)
                for (int wid = 0; wid < gw; ++wid)
                    for (int fi = 0; fi < fh; ++fi)
                        for (int fj = 0; fj < fw; ++fj) {
                            int hy = -ph + fi * dh + sh * hid;
                            int wy = -pw + fj * dw + sw * wid;
                            if (hy < 0 || hy >= oh || wy < 0 || wy >= ow) continue;
                            float v = x[(((((size_t)b * gh + hid) * gw + wid) * c + ci) * fh + fi) * fw + fj];
                            float *dst = &yb[((size_t)ci * oh + hy) * ow + wy];
                            float s = *dst + v;
                            *dst = (bf16 && !device_acc) ? bf16_round(s) : s;
                        }
        if (bf16 && device_acc)
            for (size_t i = 0; i < (size_t)c * oh * ow; ++i) yb[i] = bf16_round(yb[i]);
    }
}

/* max_pool2 host (src/tensor/ops.rs:1040-1088): floor output size
 * (src/ops.rs:92-102), strict '>' so the first maximum wins. */
ORC_API void orc_max_pool2(const float *x, float *y, int bs, int c, int ih, int iw, int h, int w,
                           int sh, int sw) {
    int oh = (ih - h) / sh + 1, ow = (iw - w) / sw + 1;
#pragma omp parallel for schedule(static)
    for (int bc = 0; bc < bs * c; ++bc)
        for (int hid = 0; hid < oh; ++hid)
            for (int wid = 0; wid < ow; ++wid) {
                float m = 0.f;
                for (int fi = 0; fi < h; ++fi)
                    for (int fj = 0; fj < w; ++fj) {
                        float v = x[((size_t)bc * ih + fi + sh * hid) * iw + fj + sw * wid];
                        if ((fi == 0 && fj == 0) || v > m) m = v;
                    }
                y[((size_t)bc * oh + hid) * ow + wid] = m;
            }
}

/* max_pool2_backward host (src/tensor/ops.rs:1144-1207): dx arrives holding a
 * copy of x (layer.rs:1203-1212).  Per window in row-major order: find the
 * first maximum of the current contents, zero the window, add dy at the
 * argmax.  Cells no window covers keep x's value. */
ORC_API void orc_max_pool2_backward(float *dx, const float *dy, int bs, int c, int ih, int iw,
                                    int h, int w, int sh, int sw) {
    int oh = (ih - h) / sh + 1, ow = (iw - w) / sw + 1;
#pragma omp parallel for schedule(static)
    for (int bc = 0; bc < bs * c; ++bc) {
        float *d = dx + (size_t)bc * ih * iw;
        for (int hid = 0; hid < oh; ++hid)
            for (int wid = 0; wid < ow; ++wid) {
                float m = 0.f;
                int hm = 0, wm = 0;
                for (int fi = 0; fi < h; ++fi)
                    for (int fj = 0; fj < w; ++fj) {
                        int hx = fi + sh * hid, wx = fj + sw * wid;
                        float v = d[hx * iw + wx];
                        if ((fi == 0 && fj == 0) || v > m) {
                            m = v;
                            hm = hx;
                            wm = wx;
                        }
                        d[hx * iw + wx] = 0.f;
                    }
                d[hm * iw + wm] += dy[((size_t)bc * oh + hid) * ow + wid];
            }
    }
}

/* relu / relu_backward (src/learn/neural_network/layer.rs:1526-1540):
 * x >= 0 ? x : 0 (so -0.0 passes, NaN -> 0); backward gates on the layer
 * input and passes dy at x == 0. */
ORC_API void orc_relu(const float *x, float *y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = (x[i] >= 0.f) ? x[i] : 0.f;
}

ORC_API void orc_relu_backward(const float *x, const float *dy, float *dx, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dx[i] = (x[i] >= 0.f) ? dy[i] : 0.f;
}

/* scaled_add: y = alpha*x + y computed in the element type
 * (src/tensor/ops.rs:295; BinaryOp::Add src/tensor/ops.rs:1285-1330). */
ORC_API void orc_scaled_add(float alpha, const float *x, float *y, int64_t n, int bf16) {
    for (int64_t i = 0; i < n; ++i) {
        if (bf16)
            y[i] = bf16_round(bf16_round(alpha * x[i]) + y[i]);
        else
            y[i] = alpha * x[i] + y[i];
    }
}

/* Bias add: y[r, c] += bias[c], the broadcast scaled_add behind
 * Variable::add_assign (src/learn/neural_network/autograd.rs:571-599). */
ORC_API void orc_bias_add(float *y, const float *bias, int64_t rows, int64_t cols, int64_t inner,
                          int bf16) {
    /* y viewed as [rows, cols, inner]; bias indexed by the middle axis
     * (inner = 1 for Dense, oh*ow for Conv2's NCHW output). */
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c)
            for (int64_t i = 0; i < inner; ++i) {
                float *p = &y[(r * cols + c) * inner + i];
                float s = *p + bias[c];
                *p = bf16 ? bf16_round(s) : s;
            }
}

/* Column sum used for the bias gradient: broadcast_backward -> sum_axis
 * (autograd.rs:490-542, src/tensor/reduce.rs:59-113).  x viewed as
 * [rows, cols, inner]; y[c] = beta*y[c] + sum over rows and inner; f32
 * accumulation for bf16 inputs (reduce.rs kernels accumulate 16-bit types in f32). */
ORC_API void orc_sum_axis_keep_mid(const float *x, float *y, int64_t rows, int64_t cols,
                                   int64_t inner, float beta, int acc64, int bf16) {
    for (int64_t c = 0; c < cols; ++c) {
        double s64 = 0.0;
        float s32 = 0.f;
        for (int64_t r = 0; r < rows; ++r)
            for (int64_t i = 0; i < inner; ++i) {
                float v = x[(r * cols + c) * inner + i];
                s64 += v;
                s32 += v;
            }
        float r = acc64 ? (float)s64 : s32;
        if (beta != 0.f) r += beta * y[c];
        y[c] = bf16 ? bf16_round(r) : r;
    }
}

/* cross_entropy_loss_host (src/learn/criterion.rs:205-226): sum over rows of
 * ln(sum exp(x-m)) - (x_t - m), all in f32. */
ORC_API float orc_cross_entropy_loss(const float *x, const uint32_t *t, int64_t bs, int64_t classes) {
    float y = 0.f;
    for (int64_t r = 0; r < bs; ++r) {
        const float *row = x + r * classes;
        float m = row[0];
        for (int64_t i = 0; i < classes; ++i) m = fmaxf(m, row[i]);
        float s = 0.f;
        for (int64_t i = 0; i < classes; ++i) s += expf(row[i] - m);
        y += logf(s) - (row[t[r]] - m);
    }
    return y;
}

/* cross_entropy_loss_backward host (src/learn/neural_network/criterion.rs:79-103):
 * dx = (dy/bs) * (softmax(x) - onehot(t)). */
ORC_API void orc_cross_entropy_loss_backward(const float *x, const uint32_t *t, float dy, float *dx,
                                             int64_t bs, int64_t classes, int bf16) {
    dy /= (float)bs;
    for (int64_t r = 0; r < bs; ++r) {
        const float *row = x + r * classes;
        float m = row[0];
        for (int64_t i = 0; i < classes; ++i) m = fmaxf(m, row[i]);
        float s = 0.f;
        for (int64_t i = 0; i < classes; ++i) s += expf(row[i] - m);
        for (int64_t i = 0; i < classes; ++i) {
            float tt = (i == (int64_t)t[r]) ? 1.f : 0.f;
            float v = dy * (expf(row[i] - m) / s - tt);
            dx[r * classes + i] = bf16 ? bf16_round(v) : v;
        }
    }
}

/* accuracy_host (src/learn/criterion.rs:30-47): a row counts only if the
 * target logit is strictly greater than every other logit. */
ORC_API int64_t orc_accuracy(const float *x, const uint32_t *t, int64_t bs, int64_t classes) {
    int64_t correct = 0;
    for (int64_t r = 0; r < bs; ++r) {
        const float *row = x + r * classes;
        float xt = row[t[r]];
        int ok = 1;
        for (int64_t i = 0; i < classes; ++i)
            if (i != (int64_t)t[r] && !(xt > row[i])) {
                ok = 0;
                break;
            }
        correct += ok;
    }
    return correct;
}

/* SGD (src/learn/neural_network/optimizer.rs:389-428): without momentum
 * w = cast_T(-lr) * g + w in the parameter type (:420-423); with momentum
 * v = m*v + g; w -= lr*v in f32, stored back in T (:446-459, :509-512). */
ORC_API void orc_sgd_update(float *w, const float *g, int64_t n, float lr, int bf16) {
    float alpha = bf16 ? bf16_round(-lr) : -lr;
    orc_scaled_add(alpha, g, w, n, bf16);
}

ORC_API void orc_sgd_update_momentum(float *w, const float *g, float *v, int64_t n, float lr,
                                     float mom, int bf16) {
    for (int64_t i = 0; i < n; ++i) {
        float vv = mom * v[i] + g[i];
        float ww = w[i] - lr * vv;
        v[i] = bf16 ? bf16_round(vv) : vv;
        w[i] = bf16 ? bf16_round(ww) : ww;
    }
}
