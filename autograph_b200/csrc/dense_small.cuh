// Small row-major products y = x . w (+ bias) (relu): the Dense layers of
// LeNet5-sized networks at small batch (see dense_small.cu).
#pragma once

#include "common.cuh"

namespace ag {
namespace dense_small {

// True when the latency-oriented kernel should take y[m,n] = x[m,k] . w[k,n]
// (all row-major contiguous): few rows, narrow output, moderate k.
bool eligible(int64_t m, int64_t k, int64_t n);

template <class T>
int forward(ag_device *dev, const T *x, int m, int k, const T *w, int n, const T *bias, bool relu,
            T *y);

// A chain of up to kMaxChain small dense layers (each followed by an optional
// relu) run by one kernel: the 8 rows a CTA owns pass from layer to layer
// through shared memory, so the intermediate activations never leave the SM.
constexpr int kMaxChain = 4;
struct ChainLayer {
    const void *w;     // [inputs, outputs]
    const void *bias;  // [outputs] or null
    int inputs, outputs;
    int relu;
    // Optional copies for a training pass: the layer's output before the relu
    // ([m, outputs]) and after it.
    void *pre_out = nullptr;
    void *act_out = nullptr;
};
bool chain_eligible(int64_t m, int n_layers, const ChainLayer *layers);
// y may be null when every value wanted leaves through pre_out / act_out.
template <class T>
int chain_forward(ag_device *dev, const T *x, int m, int n_layers, const ChainLayer *layers, T *y);

}  // namespace dense_small
}  // namespace ag
