// One or two (Conv2 -> Relu -> MaxPool2) stages, Flatten and a chain of small
// Dense layers as one kernel (see conv_chain.cu).
#pragma once

#include "common.cuh"
#include "dense_small.cuh"

namespace ag {
namespace conv_chain {

constexpr int kMaxConv = 2;

// True when the whole network fits the fused kernel: default convolution
// options, one 5x5 or 3x3 filter size for every stage, 2x2 / stride-2 pools,
// few channels, dense layers small enough for the latency-oriented chain, and
// everything a CTA needs for 8 images within its shared memory.
bool eligible(int64_t bs, int64_t ic, int64_t ih, int64_t iw, int n_conv,
              const ag_conv_stage *stages, int n_dense, const dense_small::ChainLayer *layers);

// Reads x, or (x8 != null) u8 images that are scaled by alpha while they are staged.
template <class T>
int forward(ag_device *dev, const T *x, const uint8_t *x8, float alpha, int64_t bs, int64_t ic,
            int64_t ih, int64_t iw, int n_conv, const ag_conv_stage *stages, int n_dense,
            const dense_small::ChainLayer *layers, T *y);

}  // namespace conv_chain
}  // namespace ag
