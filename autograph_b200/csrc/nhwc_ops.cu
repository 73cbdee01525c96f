// Channels-last helpers of the convolution stages (see nhwc_ops.cuh).  Every thread moves
// 16 bytes (8 channels of one pixel); consecutive threads take consecutive channel groups of a
// pixel and then consecutive pixels, so every access of a warp is one contiguous run.
#include "nhwc_ops.cuh"

namespace ag {
namespace nhwc {

namespace {

struct Vec8 {
    uint4 raw;
    __device__ __forceinline__ float get(int i) const {
        const uint32_t w = (&raw.x)[i >> 1];
        return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
    }
    __device__ __forceinline__ void set_pair(int j, float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        (&raw.x)[j] = *reinterpret_cast<uint32_t *>(&h);
    }
};

// FH, FW > 0: the filter size is a compile-time constant (the divisions below become shifts
// and multiplies; with run-time divisors the kernel is bound by them, 173 us against the 25 us
// its 126 MB of stores take at the wide stack's first layer).
template <int FH, int FW>
__global__ void im2col_channels_kernel(const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ out,
                                       int ic, int ih, int iw, int fh_rt, int fw_rt, int oh, int ow, int cp,
                                       uint32_t per_image) {
    const int fh = FH > 0 ? FH : fh_rt, fw = FW > 0 ? FW : fw_rt;
    const uint32_t groups = (uint32_t)cp / 8;
    const int taps = fh * fw, k = ic * taps;
    const int64_t plane = (int64_t)ih * iw;
    const int64_t b = blockIdx.y;   // one image per grid row: 32-bit index arithmetic inside it
    out += b * (int64_t)per_image * 8;
    // The stride of the loop is a multiple of the groups per pixel, so a thread keeps its channel
    // group: the eight source offsets relative to the pixel are computed once.
    const uint32_t first = blockIdx.x * blockDim.x + threadIdx.x;
    const int g = (int)(first % groups);
    int off[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const int c = g * 8 + e;
        const int ci = c / taps, r = c - ci * taps;
        const int fi = r / fw, fj = r - fi * fw;
        off[e] = c < k ? (int)(ci * plane) + fi * iw + fj : -1;
    }
    const unsigned short *img = reinterpret_cast<const unsigned short *>(x) + b * ic * plane;
    for (uint32_t i = first; i < per_image; i += gridDim.x * blockDim.x) {
        const uint32_t t = i / groups;
        const uint32_t oy = t / (uint32_t)ow, ox = t - oy * (uint32_t)ow;
        uint32_t wds[4] = {0u, 0u, 0u, 0u};
        if (g * 8 < k) {
            const unsigned short *px = img + oy * (uint32_t)iw + ox;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const unsigned short v = off[e] >= 0 ? __ldg(px + off[e]) : (unsigned short)0;
                wds[e >> 1] |= (uint32_t)v << ((e & 1) * 16);
            }
        }
        reinterpret_cast<uint4 *>(out)[i] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
    }
}

__global__ void relu_pool_kernel(const __nv_bfloat16 *__restrict__ pre, __nv_bfloat16 *__restrict__ y,
                                 int ih, int iw, int ph, int pw, int cp, int64_t total) {
    const int groups = cp / 8;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int g = (int)(i % groups);
        int64_t t = i / groups;
        const int px = (int)(t % pw);
        t /= pw;
        const int py = (int)(t % ph);
        const int64_t b = t / ph;
        const __nv_bfloat16 *p = pre + ((b * ih + 2 * py) * (int64_t)iw + 2 * px) * cp + g * 8;
        Vec8 a0, a1, b0, b1, o;
        a0.raw = *reinterpret_cast<const uint4 *>(p);
        a1.raw = *reinterpret_cast<const uint4 *>(p + cp);
        b0.raw = *reinterpret_cast<const uint4 *>(p + (int64_t)iw * cp);
        b1.raw = *reinterpret_cast<const uint4 *>(p + (int64_t)iw * cp + cp);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float m[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int e = 2 * j + h;
                float v0 = a0.get(e), v1 = a1.get(e), v2 = b0.get(e), v3 = b1.get(e);
                v0 = v0 >= 0.f ? v0 : 0.f; v1 = v1 >= 0.f ? v1 : 0.f;
                v2 = v2 >= 0.f ? v2 : 0.f; v3 = v3 >= 0.f ? v3 : 0.f;
                float mm = v0;   // window order (0,0),(0,1),(1,0),(1,1)
                if (v1 > mm) mm = v1;
                if (v2 > mm) mm = v2;
                if (v3 > mm) mm = v3;
                m[h] = mm;
            }
            o.set_pair(j, m[0], m[1]);
        }
        reinterpret_cast<uint4 *>(y)[i] = o.raw;
    }
}

// One thread per (image, window position of the grid that covers every cell, channel group).
__global__ void relu_pool_backward_kernel(const __nv_bfloat16 *__restrict__ pre,
                                          const __nv_bfloat16 *__restrict__ dy, __nv_bfloat16 *__restrict__ out,
                                          int ih, int iw, int ph, int pw, int cp, int64_t row_pitch,
                                          int64_t image_pitch, int64_t total) {
    const int groups = cp / 8;
    const int wh = (ih + 1) / 2, ww = (iw + 1) / 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int g = (int)(i % groups);
        int64_t t = i / groups;
        const int wx = (int)(t % ww);
        t /= ww;
        const int wy = (int)(t % wh);
        const int64_t b = t / wh;
        const int y0 = 2 * wy, x0 = 2 * wx;
        const bool has_r1 = y0 + 1 < ih, has_c1 = x0 + 1 < iw;
        const __nv_bfloat16 *p = pre + ((b * ih + y0) * (int64_t)iw + x0) * cp + g * 8;
        __nv_bfloat16 *q = out + b * image_pitch + y0 * row_pitch + (int64_t)x0 * cp + g * 8;
        Vec8 v[4], o[4];
        const uint4 zero = make_uint4(0, 0, 0, 0);
        v[0].raw = *reinterpret_cast<const uint4 *>(p);
        v[1].raw = has_c1 ? *reinterpret_cast<const uint4 *>(p + cp) : zero;
        v[2].raw = has_r1 ? *reinterpret_cast<const uint4 *>(p + (int64_t)iw * cp) : zero;
        v[3].raw = (has_r1 && has_c1) ? *reinterpret_cast<const uint4 *>(p + (int64_t)iw * cp + cp) : zero;
        if (wy < ph && wx < pw) {   // a whole window
            Vec8 gr;
            gr.raw = *reinterpret_cast<const uint4 *>(dy + ((b * ph + wy) * (int64_t)pw + wx) * cp + g * 8);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float r[4][2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int e = 2 * j + h;
                    float a[4];
                    bool pass[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float x = v[c].get(e);
                        pass[c] = x >= 0.f;          // Relu's gate
                        a[c] = pass[c] ? x : 0.f;    // Relu's output, which the pool saw
                    }
                    float m = a[0];
                    int am = 0;
                    if (a[1] > m) { m = a[1]; am = 1; }
                    if (a[2] > m) { m = a[2]; am = 2; }
                    if (a[3] > m) { m = a[3]; am = 3; }
                    const float gv = __fadd_rn(0.f, gr.get(e));
#pragma unroll
                    for (int c = 0; c < 4; ++c) r[c][h] = (am == c && pass[c]) ? gv : 0.f;
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) o[c].set_pair(j, r[c][0], r[c][1]);
            }
        } else {                    // cells no window covers keep the Relu's output
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float x0v = v[c].get(2 * j), x1v = v[c].get(2 * j + 1);
                    o[c].set_pair(j, x0v >= 0.f ? x0v : 0.f, x1v >= 0.f ? x1v : 0.f);
                }
        }
        *reinterpret_cast<uint4 *>(q) = o[0].raw;
        if (has_c1) *reinterpret_cast<uint4 *>(q + cp) = o[1].raw;
        if (has_r1) *reinterpret_cast<uint4 *>(q + row_pitch) = o[2].raw;
        if (has_r1 && has_c1) *reinterpret_cast<uint4 *>(q + row_pitch + cp) = o[3].raw;
    }
}

__global__ void zero_frame_kernel(__nv_bfloat16 *framed, int hp, int wp, int pad_h, int pad_w, int cp,
                                  int64_t cells_per_image, int64_t total) {
    const int groups = cp / 8;
    const int64_t band = (int64_t)pad_h * wp;   // cells of the top (and of the bottom) rows
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int g = (int)(i % groups);
        int64_t t = i / groups;
        const int64_t cell = t % cells_per_image;
        const int64_t b = t / cells_per_image;
        int y, x;
        if (cell < band) {
            y = (int)(cell / wp);
            x = (int)(cell % wp);
        } else if (cell < 2 * band) {
            const int64_t r = cell - band;
            y = hp - pad_h + (int)(r / wp);
            x = (int)(r % wp);
        } else {
            const int64_t r = cell - 2 * band;
            y = pad_h + (int)(r / (2 * pad_w));
            const int k = (int)(r % (2 * pad_w));
            x = k < pad_w ? k : wp - 2 * pad_w + k;
        }
        *reinterpret_cast<uint4 *>(framed + ((b * hp + y) * (int64_t)wp + x) * cp + g * 8) =
            make_uint4(0, 0, 0, 0);
    }
}

inline unsigned grid_for(ag_device *dev, int64_t total) {
    const int64_t want = ceil_div(total, 256);
    const int64_t cap = (int64_t)dev->sm_count * 32;
    return (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int im2col_channels(ag_device *dev, const __nv_bfloat16 *x, int64_t bs, int64_t ic, int64_t ih,
                    int64_t iw, int fh, int fw, int64_t oh, int64_t ow, int64_t cp,
                    __nv_bfloat16 *out) {
    AG_REQUIRE(cp % 8 == 0 && ic * fh * fw <= cp && aligned16(out), AG_ERR_INVALID,
               "im2col_channels: bad channel pitch or alignment");
    AG_REQUIRE(oh == ih - fh + 1 && ow == iw - fw + 1 && oh > 0 && ow > 0, AG_ERR_SHAPE,
               "im2col_channels: output shape does not match");
    const int64_t per_image = oh * ow * (cp / 8);
    AG_REQUIRE(per_image < (int64_t(1) << 31) && bs <= 65535 && ic * ih * iw < (int64_t(1) << 31), AG_ERR_LIMIT,
               "im2col_channels: image too large");
    AG_REQUIRE(256 % (cp / 8) == 0, AG_ERR_UNSUPPORTED, "im2col_channels: channel pitch must be 64, 128 or 256");
    if (bs == 0) return AG_OK;
    // eight pixels per thread, so that the offsets a thread computes up front are used eight times
    const int64_t want = ceil_div(per_image, 256 * 8);
    const dim3 grid((unsigned)(want > 4096 ? 4096 : want), (unsigned)bs);
    if (fh == 3 && fw == 3)
        im2col_channels_kernel<3, 3><<<grid, 256, 0, dev->stream>>>(
            x, out, (int)ic, (int)ih, (int)iw, fh, fw, (int)oh, (int)ow, (int)cp, (uint32_t)per_image);
    else if (fh == 5 && fw == 5)
        im2col_channels_kernel<5, 5><<<grid, 256, 0, dev->stream>>>(
            x, out, (int)ic, (int)ih, (int)iw, fh, fw, (int)oh, (int)ow, (int)cp, (uint32_t)per_image);
    else
        im2col_channels_kernel<0, 0><<<grid, 256, 0, dev->stream>>>(
            x, out, (int)ic, (int)ih, (int)iw, fh, fw, (int)oh, (int)ow, (int)cp, (uint32_t)per_image);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

int relu_pool(ag_device *dev, const __nv_bfloat16 *pre, int64_t bs, int64_t ih, int64_t iw, int64_t cp,
              __nv_bfloat16 *y) {
    AG_REQUIRE(cp % 8 == 0 && aligned16(pre) && aligned16(y), AG_ERR_INVALID,
               "relu_pool: bad channel pitch or alignment");
    AG_REQUIRE(ih >= 2 && iw >= 2, AG_ERR_SHAPE, "relu_pool: window larger than input");
    const int64_t ph = ih / 2, pw = iw / 2;
    const int64_t total = bs * ph * pw * (cp / 8);
    if (total == 0) return AG_OK;
    relu_pool_kernel<<<grid_for(dev, total), 256, 0, dev->stream>>>(pre, y, (int)ih, (int)iw, (int)ph,
                                                                   (int)pw, (int)cp, total);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

int relu_pool_backward(ag_device *dev, const __nv_bfloat16 *pre, const __nv_bfloat16 *dy, int64_t bs,
                       int64_t ih, int64_t iw, int64_t cp, __nv_bfloat16 *out, int64_t out_row_pitch,
                       int64_t out_image_pitch) {
    AG_REQUIRE(cp % 8 == 0 && out_row_pitch % 8 == 0 && out_image_pitch % 8 == 0 && aligned16(pre) &&
                   aligned16(dy) && aligned16(out),
               AG_ERR_INVALID, "relu_pool_backward: bad pitch or alignment");
    AG_REQUIRE(ih >= 2 && iw >= 2, AG_ERR_SHAPE, "relu_pool_backward: window larger than input");
    const int64_t total = bs * ((ih + 1) / 2) * ((iw + 1) / 2) * (cp / 8);
    if (total == 0) return AG_OK;
    relu_pool_backward_kernel<<<grid_for(dev, total), 256, 0, dev->stream>>>(
        pre, dy, out, (int)ih, (int)iw, (int)(ih / 2), (int)(iw / 2), (int)cp, out_row_pitch,
        out_image_pitch, total);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

int zero_frame(ag_device *dev, __nv_bfloat16 *framed, int64_t bs, int64_t hp, int64_t wp, int pad_h,
               int pad_w, int64_t cp) {
    AG_REQUIRE(cp % 8 == 0 && aligned16(framed), AG_ERR_INVALID, "zero_frame: bad pitch or alignment");
    const int64_t cells = 2 * (int64_t)pad_h * wp + 2 * (int64_t)pad_w * (hp - 2 * pad_h);
    const int64_t total = bs * cells * (cp / 8);
    if (total <= 0) return AG_OK;
    zero_frame_kernel<<<grid_for(dev, total), 256, 0, dev->stream>>>(framed, (int)hp, (int)wp, pad_h,
                                                                    pad_w, (int)cp, cells, total);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

}  // namespace nhwc
}  // namespace ag
