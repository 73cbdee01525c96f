"""Oracle composition of the benchmark networks (TEST INFRASTRUCTURE).

Chains the oracle's operators in the order the reference's derived
``Forward`` does (benches/neural-network-benches/src/autograph_backend.rs:88-163
for LeNet5) and runs the reverse pass edge by edge the way
``Node::backward_grad`` does (src/learn/neural_network/autograd.rs:239-261).

A network is a list of layer specs shared with the product's host code:
    ("conv", inputs, outputs, (fh, fw), bias)   Conv2, default padding/stride/dilation
    ("relu",) ("pool", (h, w)) ("flatten",)
    ("dense", inputs, outputs, bias[, tie])  tie = index of an earlier dense layer of the
                                             same shape whose parameters this layer shares
"""
from __future__ import annotations

import numpy as np

from . import (accuracy, bias_add, bias_grad, conv2_backward_input_naive,
               conv2_backward_weight_naive, conv2_direct_backward_input_f32,
               conv2_direct_backward_weight_f32, conv2_direct_f32, conv2_naive, cross_entropy_loss,
               cross_entropy_loss_backward, gemm, gemm_f32_fast, max_pool2, max_pool2_backward,
               relu, relu_backward, round_bf16, sgd_update, sgd_update_momentum)

LENET5 = [
    ("conv", 1, 6, (5, 5), False), ("relu",), ("pool", (2, 2)),
    ("conv", 6, 16, (5, 5), False), ("relu",), ("pool", (2, 2)),
    ("flatten",),
    ("dense", 256, 128, False), ("relu",),
    ("dense", 128, 84, False), ("relu",),
    ("dense", 84, 10, True),
]

WIDE_STACK = [
    ("conv", 3, 64, (3, 3), False), ("relu",), ("pool", (2, 2)),
    ("conv", 64, 128, (3, 3), False), ("relu",), ("pool", (2, 2)),
    ("flatten",),
    ("dense", 128 * 14 * 14, 512, False), ("relu",),
    ("dense", 512, 10, True),
]


def init_params(spec, seed: int, bf16: bool = False):
    """Default initialiser of the reference (layer.rs:345-389, 463-503):
    U(-a, a), a = sqrt(2 / fan_in), bias drawn with the same a; bf16 = RNE of the
    f32 draw.  The reference draws from an unseedable thread_rng, so only the
    distribution can be matched; the stream here is numpy's default_rng(seed + i)
    for the i-th parameter tensor."""
    params = []
    idx = 0
    for layer in spec:
        if layer[0] == "conv":
            _, ic, oc, (fh, fw), bias = layer
            a = np.float32(np.sqrt(np.float32(2.0) / np.float32(ic * fh * fw)))
            shapes = [(oc, ic, fh, fw)] + ([(oc,)] if bias else [])
        elif layer[0] == "dense":
            if len(layer) > 4:
                continue  # shares an earlier layer's parameters
            _, ins, outs, bias = layer
            a = np.float32(np.sqrt(np.float32(2.0) / np.float32(ins)))
            shapes = [(ins, outs)] + ([(outs,)] if bias else [])
        else:
            continue
        for shp in shapes:
            rng = np.random.default_rng(seed + idx)
            w = rng.uniform(-a, a, size=shp).astype(np.float32)
            params.append(round_bf16(w) if bf16 else w)
            idx += 1
    return params


def _param_index(spec):
    """Index of the first parameter of every layer (a tied dense layer points at its owner's)."""
    pidx, i = [], 0
    for layer in spec:
        if layer[0] == "dense" and len(layer) > 4:
            pidx.append(pidx[layer[4]])
            continue
        pidx.append(i)
        if layer[0] == "conv":
            i += 1 + int(layer[4])
        elif layer[0] == "dense":
            i += 1 + int(layer[3])
    return pidx


def _dot(a, b, acc, bf16, fast):
    if fast and not bf16:
        return gemm_f32_fast(a, b)
    return gemm(a, b, acc=acc, bf16=bf16)


def forward(spec, params, x, *, bf16=False, acc="f32", keep=False, fast=False):
    """Returns logits (and the per-layer inputs when keep=True).

    acc="f32" follows the reference's host arithmetic (direct conv for f32);
    acc="f64" is the high-precision checker used for tolerance tests.
    fast=True uses the threaded GEMM (CPU-baseline timing)."""
    pidx = _param_index(spec)
    saved = []
    h = np.ascontiguousarray(x, np.float32)
    for li, layer in enumerate(spec):
        kind = layer[0]
        saved.append(h if keep else None)
        if kind == "conv":
            w = params[pidx[li]]
            if acc == "f32" and not bf16:
                h = conv2_direct_f32(h, w)
            else:
                h = conv2_naive(h, w, acc64=(acc == "f64"), bf16=bf16)
            if layer[4]:
                h = bias_add(h, params[pidx[li] + 1], bf16=bf16)
        elif kind == "dense":
            w = params[pidx[li]]
            h = _dot(h, w, acc, bf16, fast)
            if layer[3]:
                h = bias_add(h, params[pidx[li] + 1], bf16=bf16)
        elif kind == "relu":
            h = relu(h)
        elif kind == "pool":
            h = max_pool2(h, layer[1])
        elif kind == "flatten":
            h = h.reshape(h.shape[0], -1)
    return (h, saved) if keep else h


def backward(spec, params, saved, dlogits, *, bf16=False, acc="f32"):
    """Gradients of every parameter, in parameter order."""
    grads = [None] * len(params)
    pidx = _param_index(spec)
    a64 = acc == "f64"

    def deliver(i, g):
        # a second gradient arriving at a parameter is added to the first, in the element
        # type (Node::backward_grad, autograd.rs:126-131)
        if grads[i] is None:
            grads[i] = g
        else:
            s = grads[i].astype(np.float32) + g.astype(np.float32)
            grads[i] = round_bf16(s) if bf16 else s

    g = dlogits
    for li in range(len(spec) - 1, -1, -1):
        layer = spec[li]
        kind = layer[0]
        xin = saved[li]
        if kind == "dense":
            w = params[pidx[li]]
            if layer[3]:
                deliver(pidx[li] + 1, bias_grad(g, acc64=a64, bf16=bf16))
            deliver(pidx[li], gemm(xin.T, g, acc=acc, bf16=bf16))         # dW = X^T . dY
            g = gemm(g, w.T, acc=acc, bf16=bf16)                          # dX = dY . W^T
        elif kind == "conv":
            w = params[pidx[li]]
            if layer[4]:
                deliver(pidx[li] + 1, bias_grad(g, acc64=a64, bf16=bf16))
            host_f32 = acc == "f32" and not bf16   # the reference's host path: direct kernels
            if host_f32:
                deliver(pidx[li], conv2_direct_backward_weight_f32(xin, g, layer[3]))
            else:
                deliver(pidx[li], conv2_backward_weight_naive(xin, g, layer[3], acc64=a64, bf16=bf16))
            if li > 0:  # the network input has no node: no dX for the first layer
                if host_f32:
                    g = conv2_direct_backward_input_f32(w, g, xin.shape[2:])
                else:
                    g = conv2_backward_input_naive(w, g, xin.shape[2:], acc64=a64, bf16=bf16)
        elif kind == "relu":
            g = relu_backward(xin, g)
        elif kind == "pool":
            g = max_pool2_backward(xin, g, layer[1])
        elif kind == "flatten":
            g = g.reshape(xin.shape)
    return grads


def train_step(spec, params, x, t, lr, *, momentum=None, velocity=None, bf16=False, acc="f32"):
    """One step as in LeNet5Classifier::train (autograph_backend.rs:70-85).
    Returns (loss, grads, new_params, new_velocity)."""
    logits, saved = forward(spec, params, x, bf16=bf16, acc=acc, keep=True)
    loss = cross_entropy_loss(logits, t)
    dlogits = cross_entropy_loss_backward(logits, t, 1.0, bf16=bf16)
    grads = backward(spec, params, saved, dlogits, bf16=bf16, acc=acc)
    new_params, new_vel = [], []
    for i, (w, g) in enumerate(zip(params, grads)):
        if momentum is None:
            new_params.append(sgd_update(w, g, lr, bf16=bf16))
        else:
            v = velocity[i] if velocity is not None else np.zeros_like(w)
            w2, v2 = sgd_update_momentum(w, g, v, lr, momentum, bf16=bf16)
            new_params.append(w2)
            new_vel.append(v2)
    return loss, grads, new_params, (new_vel if momentum is not None else None)


__all__ = ["LENET5", "WIDE_STACK", "init_params", "forward", "backward", "train_step", "accuracy"]
