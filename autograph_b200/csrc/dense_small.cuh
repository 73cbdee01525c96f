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
    // A backward step v -> v . w^T: w is the forward layer's [outputs, inputs] matrix read
    // transposed, and the result is zeroed where gate[m, outputs] < 0.
    int transposed = 0;
    const void *gate = nullptr;
};
bool chain_eligible(int64_t m, int n_layers, const ChainLayer *layers);
// y may be null when every value wanted leaves through pre_out / act_out.
template <class T>
int chain_forward(ag_device *dev, const T *x, int m, int n_layers, const ChainLayer *layers, T *y);

// The input gradients of a chain in one kernel.  steps[i] are backward steps (transposed = 1)
// from the last layer to the first; step i's result goes to steps[i].pre_out (the last
// step's to y).  dy [m, steps[0].inputs]; with gate_last the incoming gradient is first
// zeroed where gate_last < 0 and that value stored to g_last.
bool chain_backward_eligible(int64_t m, int n_steps, const ChainLayer *steps);
template <class T>
int chain_backward_input(ag_device *dev, const T *dy, int m, int n_steps, const ChainLayer *steps,
                         const T *gate_last, T *g_last, T *y);

// dw_i = in_i^T . g_i and db_i = column sums of g_i for up to kMaxChain layers in one launch
// (in_i [m, rows_i], g_i [m, cols_i], dw_i [rows_i, cols_i]; db_i may be null).
struct WgradProblem {
    const void *in, *g;
    void *dw, *db;
    int rows, cols;
    int tile0, tiles_n;  // filled by the launcher
};
template <class T>
int chain_weight_grads(ag_device *dev, int m, int n, WgradProblem *problems);

}  // namespace dense_small
}  // namespace ag
