"""Generates tests/golden/golden_vectors.npz.

The reference keeps no data files: its tests build inputs from closed-form
integer cycles and compare the device against an independent host
implementation (tests/integration_tests.rs).  The reference itself is Rust and
cannot be run where this repository is developed, so this script rebuilds the
same inputs from the generator definitions and computes the expected outputs
with implementations that share no code with the oracle or the CUDA kernels:
numpy integer / float64 arithmetic and torch float64 conv2d / max_pool2d /
autograd.  Because the inputs are small integers the float32 results are exact.

Run from the repository root:  python tests/golden/gen_golden.py
"""
from __future__ import annotations

import itertools
import json
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

OUT = Path(__file__).resolve().parent / "golden_vectors.npz"


def cycle(lo, hi, n):
    """lo, lo+1, ..., hi-1 repeated, n values (Rust `(lo..hi).cycle().take(n)`)."""
    return (np.arange(n) % (hi - lo) + lo).astype(np.float32)


def dot_cases(store):
    # tensor_dot_<T>_m{n}_k{n}_n{n}_{nn,tn,nt,tt}, gen_array = cycle 1..9 (integration_tests.rs:272-305)
    names = []
    for n in [2, 4, 5, 8, 16, 32, 64, 128]:
        for ta, tb in itertools.product("nt", "nt"):
            a = cycle(1, 10, n * n).reshape(n, n)
            b = cycle(1, 10, n * n).reshape(n, n)
            av = a.T if ta == "t" else a
            bv = b.T if tb == "t" else b
            c = (av.astype(np.int64) @ bv.astype(np.int64)).astype(np.float32)
            name = f"dot_n{n}_{ta}{tb}"
            store[name] = c
            names.append(name)
    return names


def conv_option_grid():
    # integration_tests.rs:884-923
    filters = [(1, 1), (3, 3), (5, 5), (7, 7), (1, 3), (3, 5), (1, 7)]
    opts = [dict()]
    opts += [dict(padding=p) for p in [(0, 1), (1, 1)]]
    opts += [dict(stride=s) for s in [(1, 2), (2, 2)]]
    opts += [dict(dilation=d) for d in [(1, 2), (2, 2)]]
    bio = [(1, 1, 1)] + [t for x in (2, 3, 13) for t in ((x, 1, 1), (1, x, 1), (1, 1, x))]
    outs = [(oh, ow) for oh in (1, 2, 3, 5) for ow in (1, 2, 3, 5)]   # all 16 output shapes
    for f in filters:
        for o in opts:
            yield f, o, bio, outs


def fingerprint(a):
    """(sum, position-weighted sum) of an integer-valued array as exact int64: two numbers
    that stand for the whole tensor where the full grid would make the fixture too large."""
    v = np.rint(np.asarray(a, np.float64)).astype(np.int64).ravel()
    wts = (np.arange(v.size, dtype=np.int64) * 2654435761 % 1000003) + 1
    return [int(v.sum()), int((v * wts).sum())]


def input_shape(oh, ow, f, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    ih = dilation[0] * (f[0] - 1) + 1 + stride[0] * (oh - 1) - 2 * padding[0]
    iw = dilation[1] * (f[1] - 1) + 1 + stride[1] * (ow - 1) - 2 * padding[1]
    return (ih, iw) if ih > 0 and iw > 0 else None


def conv_cases(store):
    """conv2 forward / backward-input / backward-weight on cycle 1..=10 inputs
    (integration_tests.rs:1182-1497), expected from torch float64."""
    cases = []
    grid, prints = [], []
    idx = 0
    for f, o, bio, outs in conv_option_grid():
        for (bs, ic, oc), (oh, ow) in itertools.product(bio, outs):
            hw = input_shape(oh, ow, f, **o)
            if hw is None:
                continue
            ih, iw = hw
            idx += 1
            kw = dict(padding=o.get("padding", (0, 0)), stride=o.get("stride", (1, 1)),
                      dilation=o.get("dilation", (1, 1)))
            x = cycle(1, 11, bs * ic * ih * iw).reshape(bs, ic, ih, iw)
            w = cycle(1, 11, oc * ic * f[0] * f[1]).reshape(oc, ic, f[0], f[1])
            xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
            wt = torch.tensor(w, dtype=torch.float64, requires_grad=True)
            y = F.conv2d(xt, wt, **kw)
            assert tuple(y.shape[2:]) == (oh, ow), (y.shape, oh, ow, f, o)
            dy = cycle(1, 11, y.numel()).reshape(tuple(y.shape))
            y.backward(torch.tensor(dy, dtype=torch.float64))
            # every case of the grid: its shape and the fingerprints of the three results
            grid.append([bs, ic, ih, iw, oc, f[0], f[1], *kw["padding"], *kw["stride"],
                         *kw["dilation"]])
            prints.append([fingerprint(y.detach().numpy()), fingerprint(xt.grad.numpy()),
                           fingerprint(wt.grad.numpy())])
            if idx % 9 != 0:   # full expected tensors for a deterministic ninth of the grid
                continue
            name = f"conv_{len(cases)}"
            store[name + "_y"] = y.detach().numpy().astype(np.float32)
            store[name + "_dx"] = xt.grad.numpy().astype(np.float32)
            store[name + "_dw"] = wt.grad.numpy().astype(np.float32)
            cases.append(dict(name=name, x_shape=[bs, ic, ih, iw], oc=oc, filter=list(f),
                              padding=list(kw["padding"]), stride=list(kw["stride"]),
                              dilation=list(kw["dilation"])))
    store["conv_grid"] = np.asarray(grid, np.int32)
    store["conv_grid_fp"] = np.asarray(prints, np.int64)
    return cases


def im2col_cases(store):
    """im2col x = 1..len; col2im dy = 1..len (integration_tests.rs:1499-1552).
    Expected im2col from torch unfold; expected col2im from torch fold (float64)."""
    cases = []
    grid, prints = [], []
    idx = 0
    for f, o, bio, outs in conv_option_grid():
        for (bs, c, oc), (oh, ow) in itertools.product(bio, outs):
            if oc != 1:
                continue
            hw = input_shape(oh, ow, f, **o)
            if hw is None:
                continue
            ih, iw = hw
            idx += 1
            kw = dict(padding=o.get("padding", (0, 0)), stride=o.get("stride", (1, 1)),
                      dilation=o.get("dilation", (1, 1)))
            n = bs * c * ih * iw
            x = np.arange(1, n + 1, dtype=np.float64).reshape(bs, c, ih, iw)
            cols = F.unfold(torch.tensor(x), kernel_size=f, **kw)       # [bs, c*fh*fw, oh*ow]
            im = cols.permute(0, 2, 1).reshape(bs * oh * ow, c * f[0] * f[1])
            dy = np.arange(1, im.numel() + 1, dtype=np.float64).reshape(tuple(im.shape))
            dcols = torch.tensor(dy).reshape(bs, oh * ow, -1).permute(0, 2, 1)
            # image size of the reference's col2im: (g-1)*s + d*(f-1) + 1 - 2p
            oh_img = (oh - 1) * kw["stride"][0] + kw["dilation"][0] * (f[0] - 1) + 1 - 2 * kw["padding"][0]
            ow_img = (ow - 1) * kw["stride"][1] + kw["dilation"][1] * (f[1] - 1) + 1 - 2 * kw["padding"][1]
            img = F.fold(dcols, output_size=(oh_img, ow_img), kernel_size=f, **kw)
            grid.append([bs, c, ih, iw, oh, ow, f[0], f[1], *kw["padding"], *kw["stride"],
                         *kw["dilation"]])
            prints.append([fingerprint(im.numpy()), fingerprint(img.numpy())])
            if idx % 9 != 0:
                continue
            name = f"im2col_{len(cases)}"
            store[name + "_y"] = im.numpy().astype(np.float32)
            store[name + "_dx"] = img.numpy().astype(np.float32)
            cases.append(dict(name=name, x_shape=[bs, c, ih, iw], grid=[oh, ow], filter=list(f),
                              padding=list(kw["padding"]), stride=list(kw["stride"]),
                              dilation=list(kw["dilation"])))
    store["im2col_grid"] = np.asarray(grid, np.int32)
    store["im2col_grid_fp"] = np.asarray(prints, np.int64)
    return cases


def pool_cases(store):
    """max_pool2 x = cycle 0..9, dy = 0..len (integration_tests.rs:1038-1061, 1554-1628).
    Expected from numpy window loops with first-max-wins."""
    cases = []
    for shape in [(1, 1, 4, 4), (1, 1, 12, 12), (2, 3, 4, 4), (1, 1, 24, 24), (2, 2, 5, 7)]:
        bs, c, ih, iw = shape
        x = cycle(0, 10, bs * c * ih * iw).reshape(shape)
        oh, ow = ih // 2, iw // 2
        y = np.zeros((bs, c, oh, ow), np.float32)
        dy = np.arange(bs * c * oh * ow, dtype=np.float32).reshape(bs, c, oh, ow)
        dx = x.copy()
        for b, ch, i, j in itertools.product(range(bs), range(c), range(oh), range(ow)):
            win = x[b, ch, 2 * i:2 * i + 2, 2 * j:2 * j + 2]
            flat = win.reshape(-1)
            k = int(np.argmax(flat))  # numpy argmax returns the first maximum
            y[b, ch, i, j] = flat[k]
            dx[b, ch, 2 * i:2 * i + 2, 2 * j:2 * j + 2] = 0
            dx[b, ch, 2 * i + k // 2, 2 * j + k % 2] = dy[b, ch, i, j]
        name = f"pool_{len(cases)}"
        store[name + "_y"] = y
        store[name + "_dx"] = dx
        cases.append(dict(name=name, shape=list(shape)))
    return cases


def relu_cases(store):
    """relu x = cycle -10..9; relu_backward x = cycle -1,0, dy = 0..len
    (integration_tests.rs:1062-1078, 1630-1695)."""
    cases = []
    for shape in [(1, 8), (15, 20)]:
        n = shape[0] * shape[1]
        x = cycle(-10, 10, n).reshape(shape)
        xb = cycle(-1, 1, n).reshape(shape)
        dy = np.arange(n, dtype=np.float32).reshape(shape)
        name = f"relu_{len(cases)}"
        store[name + "_y"] = np.where(x >= 0, x, 0).astype(np.float32)
        store[name + "_dx"] = np.where(xb >= 0, dy, 0).astype(np.float32)
        cases.append(dict(name=name, shape=list(shape)))
    return cases


def criterion_cases(store):
    """cross_entropy_loss(_backward) x = cycle 0..9, t = cycle 0..classes; accuracy
    x = (0..classes).cycle().skip(classes/2+1) (integration_tests.rs:767-827, 1091-1125).
    Expected from float64 numpy."""
    cases = []
    for bs, classes in [(1, 8), (31, 16), (1000, 100)]:
        x = cycle(0, 10, bs * classes).reshape(bs, classes).astype(np.float64)
        t = (np.arange(bs) % classes).astype(np.int64)
        m = x.max(1, keepdims=True)
        e = np.exp(x - m)
        s = e.sum(1, keepdims=True)
        loss = float((np.log(s[:, 0]) - (x[np.arange(bs), t] - m[:, 0])).sum())
        onehot = np.zeros_like(x)
        onehot[np.arange(bs), t] = 1
        dx = (1.0 / bs) * (e / s - onehot)
        xa = ((np.arange(bs * classes) + classes // 2 + 1) % classes).astype(np.float64)
        xa = xa.reshape(bs, classes)
        xt = xa[np.arange(bs), t]
        others = np.where(onehot > 0, -np.inf, xa)
        correct = int((xt > others.max(1)).sum())
        name = f"ce_{len(cases)}"
        store[name + "_dx"] = dx.astype(np.float32)
        cases.append(dict(name=name, bs=bs, classes=classes, loss=loss, correct=correct))
    return cases


def misc_cases(store):
    """scaled_add alpha=2, x = cycle 1..9, y = cycle 11..19 (integration_tests.rs:425-452);
    sum_axis cycle 1..15 (:667-698) used here as bias-gradient column sums."""
    cases = []
    for n in [7, 64, 300, 15, 294]:
        x = cycle(1, 10, n)
        y = cycle(11, 20, n)
        name = f"axpy_{n}"
        store[name] = (2 * x + y).astype(np.float32)
        cases.append(dict(name=name, n=n))
    sums = []
    for rows, cols, inner in [(4, 3, 1), (11, 5, 1), (33, 10, 1), (3, 4, 25), (100, 10, 1)]:
        x = cycle(1, 16, rows * cols * inner).reshape(rows, cols, inner)
        name = f"colsum_{rows}_{cols}_{inner}"
        store[name] = x.astype(np.float64).sum(axis=(0, 2)).astype(np.float32)
        sums.append(dict(name=name, rows=rows, cols=cols, inner=inner))
    return cases, sums


def main():
    store = {}
    meta = {}
    meta["dot"] = dot_cases(store)
    meta["conv"] = conv_cases(store)
    meta["im2col"] = im2col_cases(store)
    meta["pool"] = pool_cases(store)
    meta["relu"] = relu_cases(store)
    meta["criterion"] = criterion_cases(store)
    meta["axpy"], meta["colsum"] = misc_cases(store)
    store["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(OUT, **store)
    print(OUT, OUT.stat().st_size, "bytes;", {k: len(v) for k, v in meta.items()})


if __name__ == "__main__":
    main()
