"""The reference's serde layout for tensors and layer stacks, so that parameters can move
between autograph and this backend.

serde is format-agnostic: a type describes itself as a tree of structs, tuples, sequences and
primitives, and a serializer (serde_json, bincode, ...) prints that tree.  This module builds
the tree the reference builds and offers its serde_json form.

* Tensor / ScalarTensor (src/tensor.rs:1200-1249, 2180-2228):
  ``struct Tensor { dim: D, buffer: Buffer }``; ``dim`` is ndarray's ``Dim`` (a tuple of
  usize); ``Buffer`` is krnl's tuple struct ``Buffer(scalar type name, element count, data)``
  whose data is the raw little-endian bytes taken eight at a time as u64 and byte-swapped
  (``u64::to_be``), i.e. each item is the big-endian reading of eight data bytes.  This
  layout is pinned by the reference's own token test (src/tensor.rs:2240-2262), which
  ``tests/test_serde_format.py`` replays.  krnl is not vendored in the reference, so what it
  does with a tail of fewer than eight bytes is not pinned: zero padding is assumed here.
* Parameter (src/learn/neural_network/autograd.rs:638-656): ``{ value: ScalarTensor }`` plus
  ``optim_state`` only when an optimizer state exists (skipped when none; gradients are never
  stored).  The state (src/learn/neural_network/optimizer.rs:102-131, 166-172) is
  ``State { name, key_values: [(key, Value)] }`` (the type id is skipped) with
  ``Value::Tensor(TensorValue { tensor, parameter_device, parameter_type })``; SGD with momentum
  keeps one entry, ``"velocity"`` (optimizer.rs:366-383).  serde_json prints the enum as
  ``{"Tensor": {...}}`` and the pair as a two-element array.
* Layers (src/learn/neural_network/layer.rs:834-848, 1069-1073, 1150-1155, 1222-1251):
  ``Conv { weight, padding, stride, dilation, bias }``, ``Dense { weight, bias }``,
  ``MaxPool { filter, stride }``; ``Relu``, ``Flatten`` and ``Identity`` are unit structs
  (serde_json prints ``null``).  A model is the user's struct of such fields in declaration
  order.
"""
from __future__ import annotations

import json

import numpy as np

_NAMES = {"uint8": "U8", "int8": "I8", "uint16": "U16", "int16": "I16", "uint32": "U32",
          "int32": "I32", "uint64": "U64", "int64": "I64", "float16": "F16", "float32": "F32",
          "float64": "F64"}
_DTYPES = {v: np.dtype(k) for k, v in _NAMES.items()}


def _scalar_name(a: np.ndarray, bf16: bool) -> str:
    if bf16:
        if a.dtype != np.uint16:
            raise TypeError("bf16 data is passed as its uint16 bit pattern")
        return "BF16"
    try:
        return _NAMES[a.dtype.name]
    except KeyError:
        raise TypeError(f"no serde scalar type for {a.dtype}") from None


def buffer_items(a: np.ndarray) -> list[int]:
    """The u64 items of krnl's Buffer: big-endian reading of every eight data bytes."""
    raw = np.ascontiguousarray(a).astype(a.dtype.newbyteorder("<"), copy=False).tobytes()
    raw += b"\0" * (-len(raw) % 8)
    return [int.from_bytes(raw[i:i + 8], "big") for i in range(0, len(raw), 8)]


def tensor_tokens(a: np.ndarray, bf16: bool = False) -> list[tuple]:
    """The serde_test token stream of a tensor (the form the reference's test asserts)."""
    items = buffer_items(a)
    toks = [("Struct", "Tensor", 2), ("Str", "dim"), ("Tuple", a.ndim)]
    toks += [("U64", int(d)) for d in a.shape]
    toks += [("TupleEnd",), ("Str", "buffer"), ("TupleStruct", "Buffer", 3),
             ("Str", _scalar_name(a, bf16)), ("U64", int(a.size)), ("Seq", len(items))]
    toks += [("U64", v) for v in items]
    toks += [("SeqEnd",), ("TupleStructEnd",), ("StructEnd",)]
    return toks


def tensor_to_value(a: np.ndarray, bf16: bool = False) -> dict:
    """serde_json's value for a tensor: structs are objects, tuples and sequences arrays."""
    return {"dim": [int(d) for d in a.shape],
            "buffer": [_scalar_name(a, bf16), int(a.size), buffer_items(a)]}


def tensor_from_value(v: dict) -> tuple[np.ndarray, bool]:
    """Inverse of tensor_to_value: (array, is_bf16); bf16 comes back as its uint16 bits."""
    name, count, items = v["buffer"]
    bf16 = name == "BF16"
    dtype = np.dtype(np.uint16) if bf16 else _DTYPES[name]
    raw = b"".join(int(x).to_bytes(8, "big") for x in items)
    need = int(count) * dtype.itemsize
    if len(raw) < need:
        raise ValueError("buffer shorter than its element count")
    a = np.frombuffer(raw[:need], dtype=dtype.newbyteorder("<")).astype(dtype)
    dim = tuple(int(d) for d in v["dim"])
    if int(np.prod(dim, dtype=np.int64)) != int(count):
        raise ValueError("dim does not match the element count")
    return a.reshape(dim), bf16


def _f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return (u >> 16).astype(np.uint16)  # values handed over are already bf16-representable


def _bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def _tensor(a: np.ndarray, bf16: bool) -> dict:
    data = _f32_to_bf16_bits(a) if bf16 else np.ascontiguousarray(a, np.float32)
    return tensor_to_value(data, bf16)


def sgd_state_to_value(velocity: np.ndarray, bf16: bool) -> dict:
    """SGD's per-parameter state as the reference serialises it (momentum in use)."""
    return {"name": "SGD",
            "key_values": [["velocity", {"Tensor": {"tensor": _tensor(velocity, bf16),
                                                    "parameter_device": True,
                                                    "parameter_type": True}}]]}


def sgd_state_from_value(v):
    """The velocity array of an optim_state value, or None when it holds none."""
    if not v:
        return None
    for key, value in v.get("key_values", []):
        if key == "velocity" and "Tensor" in value:
            a, is_bf16 = tensor_from_value(value["Tensor"]["tensor"])
            return (_bf16_bits_to_f32(a) if is_bf16 else a.astype(np.float32)).ravel()
    return None


def _param(a: np.ndarray, bf16: bool, velocity=None) -> dict:
    out = {"value": _tensor(a, bf16)}
    if velocity is not None:   # skipped when there is no state (skip_serializing_if)
        out["optim_state"] = sgd_state_to_value(np.asarray(velocity, np.float32).reshape(a.shape), bf16)
    return out


def model_to_value(spec, params, field_names, bf16: bool = False, velocities=None) -> dict:
    """A layer stack as the reference would serialise the user's model struct.

    spec: the layer list used to build an ``autograph_b200.Model`` (tuples such as
    ("conv", ic, oc, (fh, fw), bias), ("relu",), ("pool", (h, w)), ("flatten",),
    ("dense", inputs, outputs, bias)); params: the parameter arrays in the model's order
    (float32; for a bf16 model the bf16-representable values); field_names: one name per layer;
    velocities: SGD's velocity per parameter (same order) when momentum is in use, else None.
    """
    if len(field_names) != len(spec):
        raise ValueError("one field name per layer")
    out, it = {}, iter(params)
    vit = iter(velocities) if velocities is not None else None
    vel = lambda: next(vit) if vit is not None else None
    for name, layer in zip(field_names, spec):
        kind = layer[0]
        if kind == "conv":
            _, ic, oc, (fh, fw), bias = layer
            w = np.asarray(next(it), np.float32).reshape(oc, ic, fh, fw)
            b = np.asarray(next(it), np.float32).reshape(oc) if bias else None
            out[name] = {"weight": _param(w, bf16, vel()), "padding": [0, 0], "stride": [1, 1],
                         "dilation": [1, 1], "bias": _param(b, bf16, vel()) if bias else None}
        elif kind == "dense":
            if len(layer) > 4:
                raise ValueError("a layer that shares another layer's parameters has no "
                                 "counterpart in the reference's format")
            _, ins, outs, bias = layer
            w = np.asarray(next(it), np.float32).reshape(ins, outs)
            b = np.asarray(next(it), np.float32).reshape(outs) if bias else None
            out[name] = {"weight": _param(w, bf16, vel()),
                         "bias": _param(b, bf16, vel()) if bias else None}
        elif kind == "pool":
            out[name] = {"filter": [int(layer[1][0]), int(layer[1][1])],
                         "stride": [int(layer[1][0]), int(layer[1][1])]}
        elif kind in ("relu", "flatten", "identity"):
            out[name] = None
        else:
            raise ValueError(f"unknown layer kind {kind}")
    return out


def model_from_value(value: dict, with_state: bool = False):
    """The parameter arrays (float32, flattened, in field order: weight then bias) of a stack
    written by model_to_value or by the reference.  with_state: also the list of SGD velocities
    (None where a parameter carries no state)."""
    params, states = [], []
    for layer in value.values():
        if not isinstance(layer, dict):
            continue
        for key in ("weight", "bias"):
            p = layer.get(key)
            if p is None:
                continue
            a, is_bf16 = tensor_from_value(p["value"])
            params.append((_bf16_bits_to_f32(a) if is_bf16 else a.astype(np.float32)).ravel())
            states.append(sgd_state_from_value(p.get("optim_state")))
    return (params, states) if with_state else params


def dumps(value) -> str:
    return json.dumps(value, separators=(",", ":"))


def loads(text: str):
    return json.loads(text)
