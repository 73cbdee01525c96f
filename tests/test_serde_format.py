"""CPU: the serde layout of tensors and layer stacks (autograph_b200/serde_format.py) against
the reference's own token test (src/tensor.rs:2240-2262) and as a round trip."""
import numpy as np
import pytest

from autograph_b200 import serde_format as sf


def test_tensor_tokens_match_the_reference_test():
    """tensor_serde in the reference: Tensor::from(vec![1u32, 2, 3, 4]) must produce exactly
    these tokens; the two u64 items are the data cast to u64 and byte-swapped."""
    data = np.array([1, 2, 3, 4], np.uint32)
    items = data.view("<u8")                       # bytemuck::cast_slice(data) as u64
    be = [int.from_bytes(int(v).to_bytes(8, "little"), "big") for v in items]   # u64::to_be
    want = [("Struct", "Tensor", 2), ("Str", "dim"), ("Tuple", 1), ("U64", 4), ("TupleEnd",),
            ("Str", "buffer"), ("TupleStruct", "Buffer", 3), ("Str", "U32"), ("U64", 4),
            ("Seq", 2), ("U64", be[0]), ("U64", be[1]), ("SeqEnd",), ("TupleStructEnd",),
            ("StructEnd",)]
    assert sf.tensor_tokens(data) == want
    # the same numbers spelled out: bytes 01 00 00 00 02 00 00 00 read big-endian
    assert be[0] == 0x0100000002000000 and be[1] == 0x0300000004000000


@pytest.mark.parametrize("dtype", [np.float32, np.uint8, np.uint16, np.int64, np.float64])
@pytest.mark.parametrize("shape", [(4,), (3, 5), (2, 1, 3, 3), (7,)])
def test_tensor_round_trip(dtype, shape):
    rng = np.random.default_rng(5)
    a = (rng.standard_normal(shape) * 50).astype(dtype)
    v = sf.loads(sf.dumps(sf.tensor_to_value(a)))
    b, is_bf16 = sf.tensor_from_value(v)
    assert not is_bf16 and b.dtype == a.dtype and np.array_equal(a, b)
    assert v["dim"] == list(shape) and v["buffer"][1] == a.size


def test_model_round_trip_f32_and_bf16():
    import autograph_b200 as ag
    rng = np.random.default_rng(6)
    shapes = [(6, 1, 5, 5), (16, 6, 5, 5), (256, 128), (128, 84), (84, 10), (10,)]
    params = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    names = ["conv1", "relu1", "pool1", "conv2", "relu2", "pool2", "flatten", "dense1", "relu3",
             "dense2", "relu4", "dense3"]
    v = sf.model_to_value(ag.LENET5_SPEC, params, names)
    assert list(v) == names and v["relu1"] is None and v["flatten"] is None
    assert v["pool1"] == {"filter": [2, 2], "stride": [2, 2]}
    assert v["conv1"]["bias"] is None and v["conv1"]["padding"] == [0, 0]
    assert v["conv1"]["weight"]["value"]["dim"] == [6, 1, 5, 5]
    assert v["dense3"]["bias"]["value"]["buffer"][0] == "F32"
    back = sf.model_from_value(sf.loads(sf.dumps(v)))
    assert len(back) == 6 and all(np.array_equal(a.ravel(), b) for a, b in zip(params, back))
    # bf16: values that are bf16-representable survive exactly, stored as 2 bytes each
    pb = [(p.view(np.uint32) & 0xffff0000).view(np.float32) for p in params]
    vb = sf.model_to_value(ag.LENET5_SPEC, pb, names, bf16=True)
    assert vb["dense1"]["weight"]["value"]["buffer"][0] == "BF16"
    assert len(vb["dense1"]["weight"]["value"]["buffer"][2]) == 256 * 128 * 2 // 8
    back = sf.model_from_value(vb)
    assert all(np.array_equal(a.ravel(), b) for a, b in zip(pb, back))


def test_optimizer_state_layout_and_round_trip():
    """Parameter { value, optim_state } with SGD's velocity (autograd.rs:647-656,
    optimizer.rs:102-131, 166-172, 366-383): State { name, key_values: [("velocity",
    Value::Tensor(TensorValue { tensor, parameter_device, parameter_type }))] }."""
    import autograph_b200 as ag
    rng = np.random.default_rng(7)
    shapes = [(6, 1, 5, 5), (16, 6, 5, 5), (256, 128), (128, 84), (84, 10), (10,)]
    params = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    vel = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    names = ["conv1", "relu1", "pool1", "conv2", "relu2", "pool2", "flatten", "dense1", "relu3",
             "dense2", "relu4", "dense3"]
    v = sf.loads(sf.dumps(sf.model_to_value(ag.LENET5_SPEC, params, names, velocities=vel)))
    st = v["dense3"]["bias"]["optim_state"]
    assert st["name"] == "SGD" and len(st["key_values"]) == 1
    key, value = st["key_values"][0]
    assert key == "velocity" and list(value) == ["Tensor"]
    tv = value["Tensor"]
    assert list(tv) == ["tensor", "parameter_device", "parameter_type"]
    assert tv["parameter_device"] is True and tv["parameter_type"] is True
    assert tv["tensor"]["dim"] == [10] and tv["tensor"]["buffer"][0] == "F32"
    back, states = sf.model_from_value(v, with_state=True)
    assert all(np.array_equal(a.ravel(), b) for a, b in zip(params, back))
    assert all(np.array_equal(a.ravel(), b) for a, b in zip(vel, states))
    # no optimizer state: the field is absent, as skip_serializing_if leaves it
    plain = sf.model_to_value(ag.LENET5_SPEC, params, names)
    assert "optim_state" not in plain["dense1"]["weight"]
    assert sf.model_from_value(plain, with_state=True)[1] == [None] * 6
