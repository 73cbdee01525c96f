// Direct weight gradient of a convolution with small channel counts and default
// options (no padding, stride 1, dilation 1):
//   dw[co][ci][fi][fj] = sum over (b, hy, wy) of dy[b][co][hy][wy] * x[b][ci][hy+fi][wy+fj]
// The reduction runs over the whole batch, the output is tiny (LeNet5: 150 and
// 2400 values), so a GEMM formulation leaves the GPU almost empty.  Here a CTA
// takes a group of images, stages one image of x and dy at a time in shared
// memory, and every thread owns the FW gradients of one (co, ci, fi) filter row
// for a slice of dy's rows.  Slices are combined in shared memory, CTAs through a
// [CTA][oc*ic*FH*FW] scratch plane and a second kernel; every sum has a fixed
// order, so the result does not depend on scheduling.
#include "conv2_direct.cuh"
#include "conv2_direct_device.cuh"

namespace ag {
namespace direct {

struct WgradParams {
    int bs, ic, ih, iw, oc;
    int group;   // images per CTA
    int slices;  // row slices per filter row (threads per item)
    int items;   // oc * ic * FH
};

// grid.x = ceil(bs / group), blockDim.x >= items * slices.
// dynamic shared memory: float xs[ic][ih][iw]; float dys[oc][oh][ow]; float red[slices][items*FW]
template <class T, int FH, int FW>
__global__ void __launch_bounds__(1024)
    conv2_wgrad_kernel(const T *__restrict__ x, const T *__restrict__ dy, float *__restrict__ partial,
                       const WgradParams p) {
    extern __shared__ __align__(16) float smem[];
    const int oh = p.ih - FH + 1, ow = p.iw - FW + 1;
    const int x_elems = p.ic * p.ih * p.iw, dy_elems = p.oc * oh * ow;
    float *xs = smem;
    float *dys = xs + ((x_elems + 3) & ~3);
    float *red = dys + ((dy_elems + 3) & ~3);
    const int b0 = blockIdx.x * p.group;
    const int nimg = min(p.group, p.bs - b0);

    const int tid = threadIdx.x;
    const int item = tid / p.slices, slice = tid - item * p.slices;
    const bool active = item < p.items;
    // item = (co, ci, fi), fi fastest
    const int fi = item % FH, cc = item / FH;
    const int ci = cc % p.ic, co = cc / p.ic;
    const int row0 = (int)((int64_t)oh * slice / p.slices);
    const int row1 = (int)((int64_t)oh * (slice + 1) / p.slices);

    float acc[FW];
#pragma unroll
    for (int j = 0; j < FW; ++j) acc[j] = 0.f;

    for (int g = 0; g < nimg; ++g) {
        __syncthreads();  // the previous image is no longer read
        const T *xg = x + (int64_t)(b0 + g) * x_elems;
        const T *dyg = dy + (int64_t)(b0 + g) * dy_elems;
        stage_contiguous<T>(xg, xs, x_elems);  // 4 elements per load where aligned
        stage_contiguous<T>(dyg, dys, dy_elems);
        __syncthreads();
        if (!active) continue;
        for (int hy = row0; hy < row1; ++hy) {
            const float *xr = xs + (ci * p.ih + hy + fi) * p.iw;
            const float *dr = dys + (co * oh + hy) * ow;
            float win[FW];
#pragma unroll
            for (int j = 0; j < FW - 1; ++j) win[j + 1] = xr[j];
            for (int wy = 0; wy < ow; ++wy) {
#pragma unroll
                for (int j = 0; j < FW - 1; ++j) win[j] = win[j + 1];
                win[FW - 1] = xr[wy + FW - 1];
                const float d = dr[wy];
#pragma unroll
                for (int j = 0; j < FW; ++j) acc[j] = fmaf(d, win[j], acc[j]);
            }
        }
    }

    // combine the row slices in slice order
    float *out = partial + (int64_t)blockIdx.x * p.items * FW;
    if (p.slices == 1) {
        if (active) {
#pragma unroll
            for (int j = 0; j < FW; ++j) out[item * FW + j] = acc[j];
        }
        return;
    }
    if (active) {
#pragma unroll
        for (int j = 0; j < FW; ++j) red[slice * p.items * FW + item * FW + j] = acc[j];
    }
    __syncthreads();
    for (int i = tid; i < p.items * FW; i += blockDim.x) {
        float s = 0.f;
        for (int z = 0; z < p.slices; ++z) s += red[z * p.items * FW + i];
        out[i] = s;
    }
}

// dw[i] = beta * dw[i] + sum over CTAs of partial[cta][i].  A CTA takes 32 outputs; its eight
// warps each add every eighth plane (loads of one warp are independent, so the planes' L2
// latencies overlap), and the eight sums are added in warp order: a fixed order.
template <class T>
__global__ void __launch_bounds__(256)
    conv2_wgrad_reduce_kernel(const float *__restrict__ partial, int planes, int len, float beta,
                              T *__restrict__ dw) {
    __shared__ float part[8][32];
    const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int i = blockIdx.x * 32 + lane;
    float s = 0.f;
    if (i < len) {
        int z = grp;
        for (; z + 56 < planes; z += 64) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = partial[(int64_t)(z + 8 * j) * len + i];
#pragma unroll
            for (int j = 0; j < 8; ++j) s += v[j];
        }
        for (; z < planes; z += 8) s += partial[(int64_t)z * len + i];
    }
    part[grp][lane] = s;
    __syncthreads();
    if (grp == 0 && i < len) {
        float t = part[0][lane];
#pragma unroll
        for (int g = 1; g < 8; ++g) t += part[g][lane];
        if (beta != 0.f) t = fmaf(beta, to_f32(dw[i]), t);
        dw[i] = from_f32<T>(t);
    }
}

static int wgrad_slices(int items, int oh) {
    int s = 256 / items;
    if (s < 1) s = 1;
    if (s > oh) s = oh;
    if (s > 16) s = 16;
    return s;
}

static size_t wgrad_smem(int64_t ic, int64_t ih, int64_t iw, int64_t oc, int fh, int fw, int slices) {
    const int64_t oh = ih - fh + 1, ow = iw - fw + 1;
    const int64_t xs = (ic * ih * iw + 3) & ~3ll, dys = (oc * oh * ow + 3) & ~3ll;
    const int64_t red = slices > 1 ? (int64_t)slices * oc * ic * fh * fw : 0;
    return (size_t)(xs + dys + red) * 4;
}

bool eligible_backward_weight(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int64_t oc,
                              const ag_conv2_options *o) {
    if (o->padding[0] || o->padding[1] || o->stride[0] != 1 || o->stride[1] != 1 ||
        o->dilation[0] != 1 || o->dilation[1] != 1)
        return false;
    const int fh = o->filter[0], fw = o->filter[1];
    if (!((fh == 5 && fw == 5) || (fh == 3 && fw == 3))) return false;
    if (ih < fh || iw < fw || bs <= 0 || ic <= 0 || oc <= 0) return false;
    const int64_t items = oc * ic * fh;
    if (items > 1024) return false;
    const int slices = wgrad_slices((int)items, (int)(ih - fh + 1));
    return wgrad_smem(ic, ih, iw, oc, fh, fw, slices) <= 96 * 1024;
}

template <class T, int FH, int FW>
static int launch_wgrad(ag_device *dev, const T *x, const T *dy, const WgradParams &p, size_t smem,
                        float beta, T *dw) {
    auto kernel = conv2_wgrad_kernel<T, FH, FW>;
    if (smem > 48 * 1024)
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    const int len = p.items * FW;
    const int ctas = (int)ceil_div(p.bs, p.group);
    void *ws = nullptr;
    AG_TRY(workspace(dev, sizeof(float) * (size_t)ctas * (size_t)len, &ws));
    const int threads = ((p.items * p.slices + 31) / 32) * 32;
    kernel<<<ctas, threads, smem, dev->stream>>>(x, dy, (float *)ws, p);
    AG_CHECK_LAUNCH();
    conv2_wgrad_reduce_kernel<T><<<(unsigned)ceil_div(len, 32), 256, 0, dev->stream>>>(
        (const float *)ws, ctas, len, beta, dw);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

template <class T>
int backward_weight(ag_device *dev, const T *x, int64_t bs, int64_t ic, int64_t ih, int64_t iw,
                    const T *dy, int64_t oc, const ag_conv2_options *o, float beta, T *dw) {
    const int fh = o->filter[0], fw = o->filter[1];
    WgradParams p;
    p.bs = (int)bs; p.ic = (int)ic; p.ih = (int)ih; p.iw = (int)iw; p.oc = (int)oc;
    p.items = (int)(oc * ic * fh);
    p.slices = wgrad_slices(p.items, (int)(ih - fh + 1));
    // About two CTAs per SM; each adds one plane to the second pass.
    p.group = (int)ceil_div(bs, 2 * (int64_t)dev->sm_count);
    if (p.group < 1) p.group = 1;
    const size_t smem = wgrad_smem(ic, ih, iw, oc, fh, fw, p.slices);
    if (fh == 5) return launch_wgrad<T, 5, 5>(dev, x, dy, p, smem, beta, dw);
    return launch_wgrad<T, 3, 3>(dev, x, dy, p, smem, beta, dw);
}

template int backward_weight<float>(ag_device *, const float *, int64_t, int64_t, int64_t, int64_t,
                                    const float *, int64_t, const ag_conv2_options *, float, float *);
template int backward_weight<__nv_bfloat16>(ag_device *, const __nv_bfloat16 *, int64_t, int64_t,
                                            int64_t, int64_t, const __nv_bfloat16 *, int64_t,
                                            const ag_conv2_options *, float, __nv_bfloat16 *);

}  // namespace direct
}  // namespace ag
