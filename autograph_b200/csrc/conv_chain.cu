// A whole small network in one kernel: one or two (Conv2 -> Relu -> MaxPool2)
// stages, Flatten, and a chain of Dense (-> Relu) layers -- the shape of LeNet5.
//
// At batch 1000 each layer of such a network is a few microseconds of work, so a
// layer-by-layer run is bound by launch gaps, by the tail of every grid and by
// the round trips of the activations through L2.  Here a CTA owns up to 8 images from
// the input to the logits: the images and both filter banks are staged in shared
// memory once, the activations of every layer stay in shared memory, and only the
// dense weights are streamed (from L2) while the logits are the only thing
// written back.  When the images live in pinned host memory, the CTAs that have
// received theirs compute while the others still wait for PCIe.
//
// The arithmetic is that of the stand-alone kernels (conv2_direct_device.cuh,
// dense_small_device.cuh), including the rounding to the tensor type at every
// layer boundary, so the result equals the layer-by-layer calls bit for bit.
#include "conv2_direct.cuh"
#include "conv2_direct_device.cuh"
#include "conv_chain.cuh"
#include "dense_small_device.cuh"

#include <cstdlib>

namespace ag {
namespace conv_chain {

using dense_small::ROWS;

// Phase timestamps for the profile summaries: a library built with -DAG_PHASE_STAMPS records
// %globaltimer at every phase boundary of the first 1024 CTAs (thread 0) and exports
// ag_debug_chain_stamps to read them.  Not part of normal builds.
#ifdef AG_PHASE_STAMPS
constexpr int kStampSlots = 8;
static __device__ unsigned long long g_stamps[1024 * kStampSlots];
__device__ __forceinline__ void stamp(int i) {
    if (threadIdx.x == 0 && blockIdx.x < 1024) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_stamps[blockIdx.x * kStampSlots + i] = t;
    }
}
#define AG_STAMP(i) stamp(i)
#else
#define AG_STAMP(i)
#endif

}  // namespace conv_chain
}  // namespace ag

#include "conv_chain_lenet.cuh"
#include "conv_chain_lenet_tc.cuh"

namespace ag {
namespace conv_chain {

struct StagePlan {
    const void *w, *bias;
    direct::Params p;  // kernel view of the stage (group = ROWS)
    int w_off, bias_off;  // float offsets into shared memory
    int out_h, out_w;     // after the optional pool
};

struct Plan {
    int bs, n_conv;
    int group;  // images per CTA (<= ROWS)
    const uint8_t *x8;  // when set: u8 images, scaled by alpha while they are staged
    float alpha;
    StagePlan st[kMaxConv];
    int in_off, mid_off;  // staged input images; output of stage 0 when there are two stages
    int xa_off, xb_off, red_off;
    dense_small::ChainParams chain;
};

// Output of a conv stage as the next stage's image: [g][oc][h][w].
struct ImageOut {
    float *dst;
    int oc, h, w;
    __device__ __forceinline__ void pooled(int g, int c, int py, int px, float v) const {
        dst[((g * oc + c) * h + py) * w + px] = v;
    }
    __device__ __forceinline__ void plain(int g, int c, int y, int x, float v) const {
        pooled(g, c, y, x, v);
    }
};

// Output of the last conv stage, flattened (c, h, w) into the dense chain's
// input layout [k][ROWS].
struct FlatOut {
    float *xa;
    int h, w;
    __device__ __forceinline__ void pooled(int g, int c, int py, int px, float v) const {
        xa[((c * h + py) * w + px) * ROWS + g] = v;
    }
    __device__ __forceinline__ void plain(int g, int c, int y, int x, float v) const {
        pooled(g, c, y, x, v);
    }
};

template <class T, int F>
__global__ void __launch_bounds__(512, 1)
    conv_chain_kernel(const T *__restrict__ x, T *__restrict__ y, const Plan pl) {
    extern __shared__ __align__(16) float smem[];
    const int b0 = blockIdx.x * pl.group;
    const int nimg = min(pl.group, pl.bs - b0);
    const direct::Params &p0 = pl.st[0].p;
    const int img_elems = p0.ic * p0.ih * p0.iw;
    float *xa = smem + pl.xa_off;
    AG_STAMP(0);

    if (pl.x8 != nullptr) {
        // scaled_cast on the way in: alpha * u8 in T (alpha rounded to T, one rounding of the product)
        const float a = to_f32(from_f32<T>(pl.alpha));
        const uint8_t *src = pl.x8 + (int64_t)b0 * img_elems;
        float *dst = smem + pl.in_off;
        const int total = nimg * img_elems;
        const int nvec = (reinterpret_cast<uintptr_t>(src) & 3) == 0 ? total / 4 : 0;
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
            const uint32_t q = reinterpret_cast<const uint32_t *>(src)[i];
            float4 v;
            v.x = to_f32(from_f32<T>(a * (float)(q & 0xffu)));
            v.y = to_f32(from_f32<T>(a * (float)((q >> 8) & 0xffu)));
            v.z = to_f32(from_f32<T>(a * (float)((q >> 16) & 0xffu)));
            v.w = to_f32(from_f32<T>(a * (float)(q >> 24)));
            reinterpret_cast<float4 *>(dst)[i] = v;
        }
        for (int i = nvec * 4 + threadIdx.x; i < total; i += blockDim.x)
            dst[i] = to_f32(from_f32<T>(a * (float)src[i]));
    } else {
        direct::stage_contiguous<T>(x + (int64_t)b0 * img_elems, smem + pl.in_off, nimg * img_elems);
    }
    for (int s = 0; s < pl.n_conv; ++s) {
        const StagePlan &sp = pl.st[s];
        direct::stage_filters<T>(reinterpret_cast<const T *>(sp.w),
                                 reinterpret_cast<const T *>(sp.bias), smem + sp.w_off,
                                 smem + sp.bias_off, sp.p.oc, sp.p.ocp, sp.p.ic * F * F);
    }
    if (nimg < ROWS) {
        // rows without an image still flow through the dense layers: give them zeros
        const int k0 = pl.chain.s[0].K;
        for (int i = threadIdx.x; i < k0 * ROWS; i += blockDim.x) xa[i] = 0.f;
    }
    __syncthreads();
    AG_STAMP(1);

    const float *img = smem + pl.in_off;
    for (int s = 0; s < pl.n_conv; ++s) {
        const StagePlan &sp = pl.st[s];
        if (s + 1 < pl.n_conv) {
            ImageOut out{smem + pl.mid_off, sp.p.oc, sp.out_h, sp.out_w};
            direct::compute_items<T, F, F>(img, smem + sp.w_off, smem + sp.bias_off,
                                           sp.bias != nullptr, sp.p, nimg, out);
            img = smem + pl.mid_off;
        } else {
            FlatOut out{xa, sp.out_h, sp.out_w};
            direct::compute_items<T, F, F>(img, smem + sp.w_off, smem + sp.bias_off,
                                           sp.bias != nullptr, sp.p, nimg, out);
        }
        __syncthreads();
        AG_STAMP(2 + s);
    }
    dense_small::chain_layers<T>(xa, smem + pl.xb_off, smem + pl.red_off, pl.chain, b0, nimg, y);
    AG_STAMP(7);
}

static bool default_options(const ag_conv2_options &o) {
    return !o.padding[0] && !o.padding[1] && o.stride[0] == 1 && o.stride[1] == 1 &&
           o.dilation[0] == 1 && o.dilation[1] == 1;
}

// Fills `pl`; returns the dynamic shared memory in bytes, or 0 when the network
// does not fit the kernel.
static size_t make_plan(Plan *pl, int64_t bs, int64_t ic, int64_t ih, int64_t iw, int n_conv,
                        const ag_conv_stage *stages, int n_dense,
                        const dense_small::ChainLayer *layers) {
    if (n_conv < 1 || n_conv > kMaxConv || n_dense < 1 || n_dense > dense_small::kMaxChain) return 0;
    if (bs <= 0 || bs > (int64_t)ROWS * 65535 * 32) return 0;
    const int f = stages[0].options.filter[0];
    int off = 0;
    auto take = [&](int64_t floats) {
        const int at = off;
        off += (int)((floats + 3) & ~3ll);
        return at;
    };
    pl->bs = (int)bs;
    pl->n_conv = n_conv;
    pl->in_off = take((int64_t)ROWS * ic * ih * iw);
    pl->mid_off = 0;
    int64_t c = ic, h = ih, w = iw;
    for (int s = 0; s < n_conv; ++s) {
        const ag_conv_stage &cs = stages[s];
        if (!default_options(cs.options) || cs.options.filter[0] != f || cs.options.filter[1] != f)
            return 0;
        if (!direct::eligible(ROWS, c, h, w, cs.oc, &cs.options)) return 0;
        const bool pool = cs.pool[0] != 0 || cs.pool[1] != 0;
        if (pool && (cs.pool[0] != 2 || cs.pool[1] != 2)) return 0;
        StagePlan &sp = pl->st[s];
        sp.w = cs.w;
        sp.bias = cs.bias;
        sp.p.bs = (int)bs; sp.p.ic = (int)c; sp.p.ih = (int)h; sp.p.iw = (int)w;
        sp.p.oc = (int)cs.oc;
        sp.p.ocp = ((int)cs.oc + 1) & ~1;
        sp.p.group = ROWS;
        sp.p.relu = cs.relu != 0;
        sp.p.pool = pool;
        sp.p.split = 1;
        sp.w_off = take((int64_t)c * f * f * sp.p.ocp);
        sp.bias_off = take(sp.p.ocp);
        const int64_t oh = h - f + 1, ow = w - f + 1;
        sp.out_h = (int)(pool ? oh / 2 : oh);
        sp.out_w = (int)(pool ? ow / 2 : ow);
        c = cs.oc; h = sp.out_h; w = sp.out_w;
        if (s + 1 < n_conv) pl->mid_off = take((int64_t)ROWS * c * h * w);
    }
    if (c * h * w != layers[0].inputs) return 0;
    for (int i = 0; i < n_dense; ++i) {
        if (!dense_small::eligible(ROWS, layers[i].inputs, layers[i].outputs)) return 0;
        if (i > 0 && layers[i].inputs != layers[i - 1].outputs) return 0;
    }
    dense_small::plan_chain(&pl->chain, (int)bs, n_dense, layers);
    pl->xa_off = take((int64_t)pl->chain.max_k * ROWS);
    pl->xb_off = take((int64_t)pl->chain.max_k * ROWS);
    pl->red_off = take(pl->chain.red_floats);
    const size_t bytes = (size_t)off * sizeof(float);
    return bytes <= 200 * 1024 ? bytes : 0;
}

bool eligible(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int n_conv,
              const ag_conv_stage *stages, int n_dense, const dense_small::ChainLayer *layers) {
    Plan pl;
    const int f = (n_conv >= 1) ? stages[0].options.filter[0] : 0;
    if (f != 5 && f != 3) return false;
    return make_plan(&pl, bs, ic, ih, iw, n_conv, stages, n_dense, layers) != 0;
}

template <class T, int F>
static int launch(ag_device *dev, const T *x, T *y, const Plan &pl, size_t smem) {
    auto kernel = conv_chain_kernel<T, F>;
    if (smem > 48 * 1024)
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    kernel<<<(unsigned)ceil_div(pl.bs, pl.group), 512, smem, dev->stream>>>(x, y, pl);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

// Launches the kernel specialised for LeNet5's geometry, or returns AG_ERR_UNSUPPORTED when
// the network is not of that geometry.  flat_out != null: stop after the flatten.
template <class T>
static int launch_lenet(ag_device *dev, const T *x, const uint8_t *x8, float alpha, int64_t bs,
                        int64_t ic, int64_t ih, int64_t iw, int n_conv, const ag_conv_stage *stages,
                        int n_dense, const dense_small::ChainLayer *layers, T *y, T *flat_out) {
    lenet::Plan lp;
    const ag_dtype dtype = sizeof(T) == 4 ? AG_F32 : AG_BF16;
    const size_t lsmem =
        lenet::make_plan(&lp, dtype, bs, ic, ih, iw, n_conv, stages, n_dense, layers, flat_out);
    if (lsmem == 0) return AG_ERR_UNSUPPORTED;
    int64_t group = ceil_div(bs, (int64_t)dev->sm_count);
    lp.group = (int)(group < 1 ? 1 : (group > lenet::kGroup ? lenet::kGroup : group));
    lp.status = dev->status_dev;
    auto kernel = lenet::lenet_chain_kernel<T>;
    static bool attr_set[64] = {};
    if (dev->ordinal >= 64 || !attr_set[dev->ordinal]) {
        AG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lsmem));
        if (dev->ordinal < 64) attr_set[dev->ordinal] = true;
    }
    // launched so that it may overlap the tail of a preceding launch of the same kernel
    // (the kernel itself waits for its predecessor before it reads or writes memory)
    cudaLaunchConfig_t cfg = {};
    int64_t ctas = ceil_div(bs, (int64_t)lp.group);
    // the group-walking form: 16-byte aligned images and groups, one CTA per SM
    lp.persist = lp.persist && x8 == nullptr && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                 (lp.group * 784 * sizeof(T)) % 16 == 0 && ctas > dev->sm_count;
    if (lp.persist) ctas = dev->sm_count;
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(lenet::kThreads);
    cfg.dynamicSmemBytes = lsmem;
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    AG_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, x, x8, alpha, y, lp));
    AG_CHECK_LAUNCH();
    return AG_OK;
}

template <class T>
int forward(ag_device *dev, const T *x, const uint8_t *x8, float alpha, int64_t bs, int64_t ic,
            int64_t ih, int64_t iw, int n_conv, const ag_conv_stage *stages, int n_dense,
            const dense_small::ChainLayer *layers, T *y) {
    // A network with LeNet5's geometry runs the kernel specialised for it (AG_CHAIN_GENERIC=1
    // keeps the generic kernel, for comparisons).
    static const bool generic_only = [] {
        const char *e = getenv("AG_CHAIN_GENERIC");
        return e && e[0] == '1';
    }();
    // Large batches of a LeNet5-geometry network: the kernel stops after the flatten and the
    // dense layers run as products over the whole batch (ag_dense_forward: tensor cores for
    // bf16, the SIMT tile engine for f32).  Inside the one-kernel form every CTA streams all
    // dense weights for its 7 images; over the whole batch they are read once per 128-row tile.
    static const int64_t split_batch = [] {
        const char *e = getenv("AG_CHAIN_SPLIT_BATCH");
        return e ? (int64_t)atoll(e) : (int64_t)5120;
    }();
    if (!generic_only && split_batch > 0 && bs >= split_batch) {
        const ag_dtype dtype = sizeof(T) == 4 ? AG_F32 : AG_BF16;
        int64_t widest = layers[0].inputs;
        for (int i = 0; i < n_dense; ++i) widest = layers[i].outputs > widest ? layers[i].outputs : widest;
        void *scratch = nullptr;
        // [bs, 256] after the flatten, then two buffers the layers alternate between
        const size_t plane = (size_t)bs * (size_t)widest * sizeof(T);
        AG_TRY(staging(dev, 3 * plane, &scratch));
        T *flat = reinterpret_cast<T *>(scratch);
        const int r = launch_lenet<T>(dev, x, x8, alpha, bs, ic, ih, iw, n_conv, stages, n_dense, layers, y, flat);
        if (r == AG_OK) {
            const T *in = flat;
            for (int i = 0; i < n_dense; ++i) {
                T *out = i + 1 == n_dense
                             ? y
                             : reinterpret_cast<T *>(reinterpret_cast<char *>(scratch) + (1 + (i & 1)) * plane);
                AG_TRY(ag_dense_forward(dev, dtype, in, bs, layers[i].inputs, layers[i].w, layers[i].outputs,
                                        layers[i].bias, layers[i].relu, out));
                in = out;
            }
            return AG_OK;
        }
        if (r != AG_ERR_UNSUPPORTED) return r;
    }
    if constexpr (sizeof(T) == 2) {
        // bf16: the variant whose second convolution runs on the tensor cores.  Off unless
        // AG_LENET_TC=1 (read per call): correct, but slower than the FFMA kernel below, because
        // a tcgen05.mma with N = 16, K = 16 occupies the tensor core about as long as one with
        // N = 256, and this layer cannot fill more of it (measured: 10 us against 7 us for the
        // phase, 29.7 against 22.7 us for the step).
        const char *tc_env = getenv("AG_LENET_TC");
        const bool tc_off = !(tc_env && tc_env[0] == '1');
        lenet_tc::Plan tp;
        size_t tsmem = 0;
        if (!generic_only && !tc_off &&
            (tsmem = lenet_tc::make_plan(&tp, bs, ic, ih, iw, n_conv, stages, n_dense, layers)) != 0) {
            int64_t group = ceil_div(bs, (int64_t)dev->sm_count);
            tp.group = (int)(group < 1 ? 1 : (group > lenet::kGroup ? lenet::kGroup : group));
            tp.status = dev->status_dev;
            static bool attr_set = false;
            if (!attr_set) {
                AG_CUDA_TRY(cudaFuncSetAttribute(lenet_tc::lenet_chain_tc_kernel,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tsmem));
                attr_set = true;
            }
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)ceil_div(bs, (int64_t)tp.group));
            cfg.blockDim = dim3(lenet::kThreads);
            cfg.dynamicSmemBytes = tsmem;
            cfg.stream = dev->stream;
            cudaLaunchAttribute attr;
            attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr.val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = &attr;
            cfg.numAttrs = 1;
            AG_CUDA_TRY(cudaLaunchKernelEx(&cfg, lenet_tc::lenet_chain_tc_kernel, x, x8, alpha, y, tp));
            AG_CHECK_LAUNCH();
            return AG_OK;
        }
    }
    if (!generic_only) {
        const int r = launch_lenet<T>(dev, x, x8, alpha, bs, ic, ih, iw, n_conv, stages, n_dense, layers, y,
                                      nullptr);
        if (r != AG_ERR_UNSUPPORTED) return r;
    }
    Plan pl;
    pl.x8 = x8;
    pl.alpha = alpha;
    const size_t smem = make_plan(&pl, bs, ic, ih, iw, n_conv, stages, n_dense, layers);
    AG_REQUIRE(smem != 0, AG_ERR_UNSUPPORTED, "this network does not fit the fused kernel");
    // Images per CTA: a batch that does not fill the GPU at 8 per CTA is spread over all
    // SMs instead (fewer rounds of convolution work items per CTA, one wave of CTAs).
    int64_t group = ceil_div(bs, (int64_t)dev->sm_count);
    pl.group = (int)(group < 1 ? 1 : (group > ROWS ? ROWS : group));
    if (stages[0].options.filter[0] == 5) return launch<T, 5>(dev, x, y, pl, smem);
    return launch<T, 3>(dev, x, y, pl, smem);
}

template int forward<float>(ag_device *, const float *, const uint8_t *, float, int64_t, int64_t,
                            int64_t, int64_t, int, const ag_conv_stage *, int,
                            const dense_small::ChainLayer *, float *);
template int forward<__nv_bfloat16>(ag_device *, const __nv_bfloat16 *, const uint8_t *, float,
                                    int64_t, int64_t, int64_t, int64_t, int, const ag_conv_stage *,
                                    int, const dense_small::ChainLayer *, __nv_bfloat16 *);

}  // namespace conv_chain
}  // namespace ag

using namespace ag;

static int conv_dense_chain_entry(ag_device *dev, ag_dtype dtype, const void *x, const uint8_t *x8,
                                  float alpha, int64_t bs, int64_t ic, int64_t ih, int64_t iw,
                                  int32_t n_conv, const ag_conv_stage *stages, int32_t n_dense,
                                  const int64_t *dims, const void *const *weights,
                                  const void *const *biases, const int32_t *relu, void *y) {
    AG_ENTER(dev);
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "conv_dense_chain %d not implemented",
               (int)dtype);
    AG_REQUIRE(bs >= 0 && ic > 0 && ih > 0 && iw > 0, AG_ERR_SHAPE, "bad input shape");
    AG_REQUIRE(n_conv >= 1 && n_conv <= conv_chain::kMaxConv && stages, AG_ERR_UNSUPPORTED,
               "1..%d convolution stages are supported", conv_chain::kMaxConv);
    AG_REQUIRE(n_dense >= 1 && n_dense <= dense_small::kMaxChain && dims && weights,
               AG_ERR_UNSUPPORTED, "1..%d dense layers are supported", dense_small::kMaxChain);
    dense_small::ChainLayer layers[dense_small::kMaxChain];
    for (int i = 0; i < n_dense; ++i) {
        AG_REQUIRE(dims[i] > 0 && dims[i + 1] > 0 && dims[i] < (1 << 30) && dims[i + 1] < (1 << 30),
                   AG_ERR_SHAPE, "bad dense width");
        AG_REQUIRE(weights[i] != nullptr, AG_ERR_INVALID, "null weight pointer");
        layers[i] = {weights[i], biases ? biases[i] : nullptr, (int)dims[i], (int)dims[i + 1],
                     relu ? relu[i] : 0};
    }
    for (int s = 0; s < n_conv; ++s)
        AG_REQUIRE(stages[s].w != nullptr && stages[s].oc > 0, AG_ERR_INVALID, "bad conv stage");
    if (bs == 0) return AG_OK;
    AG_REQUIRE((x || x8) && y, AG_ERR_INVALID, "null tensor pointer");
    if (dtype == AG_F32)
        return conv_chain::forward<float>(dev, (const float *)x, x8, alpha, bs, ic, ih, iw, n_conv,
                                          stages, n_dense, layers, (float *)y);
    return conv_chain::forward<__nv_bfloat16>(dev, (const __nv_bfloat16 *)x, x8, alpha, bs, ic, ih,
                                              iw, n_conv, stages, n_dense, layers,
                                              (__nv_bfloat16 *)y);
}

#ifdef AG_PHASE_STAMPS
extern "C" __attribute__((visibility("default"))) int ag_debug_chain_stamps(unsigned long long *host,
                                                                            size_t count) {
    const size_t n = count < 1024 * conv_chain::kStampSlots ? count : 1024 * conv_chain::kStampSlots;
    AG_CUDA_TRY(cudaMemcpyFromSymbol(host, conv_chain::g_stamps, n * sizeof(unsigned long long)));
    return AG_OK;
}
#endif

extern "C" int ag_conv_dense_chain_forward(ag_device *dev, ag_dtype dtype, const void *x, int64_t bs,
                                           int64_t ic, int64_t ih, int64_t iw, int32_t n_conv,
                                           const ag_conv_stage *stages, int32_t n_dense,
                                           const int64_t *dims, const void *const *weights,
                                           const void *const *biases, const int32_t *relu,
                                           void *y) {
    AG_REQUIRE(x != nullptr || bs == 0, AG_ERR_INVALID, "null tensor pointer");
    return conv_dense_chain_entry(dev, dtype, x, nullptr, 0.f, bs, ic, ih, iw, n_conv, stages,
                                  n_dense, dims, weights, biases, relu, y);
}

extern "C" int ag_conv_dense_chain_forward_u8(ag_device *dev, ag_dtype dtype, const uint8_t *x,
                                              float alpha, int64_t bs, int64_t ic, int64_t ih,
                                              int64_t iw, int32_t n_conv,
                                              const ag_conv_stage *stages, int32_t n_dense,
                                              const int64_t *dims, const void *const *weights,
                                              const void *const *biases, const int32_t *relu,
                                              void *y) {
    AG_REQUIRE(x != nullptr || bs == 0, AG_ERR_INVALID, "null tensor pointer");
    return conv_dense_chain_entry(dev, dtype, nullptr, x, alpha, bs, ic, ih, iw, n_conv, stages,
                                  n_dense, dims, weights, biases, relu, y);
}
