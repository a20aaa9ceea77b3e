"""Rotary embeddings without a GPU: the oracle against the closed forms the reference's own tests
hold (crates/dash-mag/tests/rope.rs), the host mirror's tables and refusals, and the C ABI's
refusals before anything is launched."""
import ctypes
import math

import numpy as np
import pytest
import torch

from dashmag_b200 import _lib
from dashmag_b200.attention import AttentionError
from dashmag_b200.rope import Rope
from oracle import attention_oracle
from oracle import rope_oracle as R


def test_it_is_transformers_rotation():
    """crates/dash-mag/tests/rope.rs:9-29: x cos + rotate_half(x) sin, angles worked out in f64."""
    dim, base = 4, np.float32(10000.0)
    cos, sin = R.tables(dim, base, 8, "f32")
    x = attention_oracle.seeded((1, 2, 1, 6), 1)
    y = R.apply_range(x, 3, cos, sin, dim, "f32")
    want = []
    for t, position in enumerate(range(3, 5)):
        row = x[0, t, 0]
        rotated = [-row[2], -row[3], row[0], row[1]]
        for j in range(4):
            frequency = np.float32(1.0) / np.float32(math.pow(float(base), float(np.float32(2 * (j % 2)) / np.float32(dim))))
            angle = float(np.float32(position) * frequency)
            want.append(np.float32(row[j] * np.float32(math.cos(angle)) + rotated[j] * np.float32(math.sin(angle))))
        want.extend(row[4:])
    assert np.max(np.abs(y.reshape(-1) - np.array(want, dtype=np.float32))) <= 1e-6


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
def test_a_position_at_a_time_is_the_range_s_row(dtype):
    """crates/dash-mag/tests/rope.rs:31-43."""
    cos, sin = R.tables(8, 10000.0, 16, dtype)
    x = R.round_to(attention_oracle.seeded((1, 4, 3, 16), 2), dtype)
    whole = R.apply_range(x, 5, cos, sin, 8, dtype)
    for t in range(4):
        one = R.apply_at(x[:, t], [5 + t], cos, sin, 8, dtype)
        assert np.array_equal(one, whole[:, t])
    assert np.array_equal(R.round_to(whole, dtype), whole), "the result holds values of the dtype"


def test_bf16_rounding_is_torch_s():
    x = attention_oracle.seeded((4096,), 3) * np.float32(1.2345)
    assert np.array_equal(R.round_to(x, "bf16"), torch.from_numpy(x).to(torch.bfloat16).float().numpy())
    assert np.array_equal(R.round_to(x, "f16"), torch.from_numpy(x).to(torch.float16).float().numpy())


def test_the_inverse_is_the_transpose():
    """<rotate(x), g> = <x, rotate^T(g)> in f32, up to f32's rounding."""
    cos, sin = R.tables(16, 10000.0, 32, "f32")
    x, g = attention_oracle.seeded((2, 7, 3, 24), 4), attention_oracle.seeded((2, 7, 3, 24), 5)
    a = np.sum(R.apply_range(x, 9, cos, sin, 16, "f32").astype(np.float64) * g)
    b = np.sum(x.astype(np.float64) * R.apply_range(g, 9, cos, sin, 16, "f32", inverse=True))
    assert abs(a - b) <= 1e-4 * max(1.0, abs(a))


def test_packed_sequences_are_rotated_one_by_one():
    cos, sin = R.tables(8, 10000.0, 32, "bf16")
    x = R.round_to(attention_oracle.seeded((20, 2, 8), 6), "bf16")
    cu = [0, 5, 5, 17]
    y = R.apply_packed(x, cu, 2, cos, sin, 8, "bf16")
    assert np.array_equal(y[0:5], R.apply_range(x[None, 0:5], 2, cos, sin, 8, "bf16")[0])
    assert np.array_equal(y[5:17], R.apply_range(x[None, 5:17], 2, cos, sin, 8, "bf16")[0])
    assert np.array_equal(y[17:], x[17:]), "tokens of no sequence pass unchanged"


@pytest.mark.parametrize("dtype,torch_dtype", [("f32", torch.float32), ("bf16", torch.bfloat16), ("f16", torch.float16)])
def test_the_host_mirror_builds_the_oracle_s_tables(dtype, torch_dtype):
    rope = Rope(64, 10000.0, 300, torch_dtype, device="cpu")
    cos, sin = R.tables(64, 10000.0, 300, dtype)
    assert np.array_equal(rope.cos.float().numpy(), cos) and np.array_equal(rope.sin.float().numpy(), sin)
    assert rope.len() == 300 and not rope.is_empty()


def test_it_refuses_what_it_does_not_hold():
    """crates/dash-mag/tests/rope.rs:45-58, 78-90, 93-108."""
    rope = Rope(8, 10000.0, 4, torch.float32, device="cpu")
    with pytest.raises(AttentionError, match="7 features; an even number is rotated"):
        Rope(7, 10000.0, 4, torch.float32, device="cpu")
    with pytest.raises(AttentionError, match="is not floating"):
        Rope(4, 10000.0, 8, torch.int32, device="cpu")
    x = torch.zeros(1, 4, 1, 16)
    with pytest.raises(AttentionError, match=r"Rope: positions 1\.\.5 of 4"):
        rope.apply_range(x, range(1, 5))                       # past the table
    with pytest.raises(AttentionError, match=r"Rope: positions 0\.\.3 of 4"):
        rope.apply_range(x, range(0, 3))                       # not T positions
    with pytest.raises(AttentionError, match="8 features to rotate"):
        rope.apply_range(torch.zeros(1, 4, 1, 6), range(0, 4))  # too narrow
    with pytest.raises(AttentionError, match="under a rotation of"):
        rope.apply_range(x.to(torch.bfloat16), range(0, 4))
    token = torch.zeros(2, 1, 16)
    with pytest.raises(AttentionError, match="positions of torch.float32"):
        rope.apply_at(token, torch.tensor([1.0, 3.0]))
    with pytest.raises(AttentionError, match="positions of torch.bool"):
        rope.apply_at(token, torch.tensor([True, False]))
    with pytest.raises(AttentionError, match="positions of torch.int32"):
        rope.apply_at(token, torch.tensor([1, 2, 3], dtype=torch.int32))


def test_the_c_abi_refuses_before_it_launches():
    lib = _lib.lib()
    p = _lib.RopeParams()
    p.tokens, p.d, p.heads_a, p.start, p.period = 8, 16, 2, 0, 8
    p.stride_a = (ctypes.c_int64 * 2)(32, 16)
    call = lambda tables: lib.dash_rope_apply(ctypes.byref(tables), ctypes.byref(p), None, None, None, None, None)
    assert call(_lib.RopeTables(0, 7, 8, None, None)) == _lib.INVALID and _lib.last_error() == "Rope: 7 features; an even number is rotated"
    assert call(_lib.RopeTables(0, 32, 8, None, None)) == _lib.INVALID and _lib.last_error() == "Rope: 32 features to rotate, of 16"
    assert call(_lib.RopeTables(5, 8, 8, None, None)) == _lib.INVALID and "is not floating" in _lib.last_error()
    assert call(_lib.RopeTables(0, 8, 4, ctypes.c_void_p(256), ctypes.c_void_p(512))) == _lib.INVALID
    assert _lib.last_error() == "Rope: positions 0..8 of 4 for 8 tokens"
    assert call(_lib.RopeTables(0, 8, 8, ctypes.c_void_p(256), ctypes.c_void_p(512))) == _lib.INVALID
    assert _lib.last_error() == "rope_apply: a tensor pointer is null"
    p.tokens = 0
    assert call(_lib.RopeTables(0, 8, 8, ctypes.c_void_p(256), ctypes.c_void_p(512))) == _lib.OK   # nothing to do
