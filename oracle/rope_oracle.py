"""CPU restatement of the reference's rotary position embedding - TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU leg may import this file; the library never
does.  It follows crates/dash-mag/src/rope.rs: the tables of ``Rope::new`` (:43-56) and the
rotation of ``Rope::rotate`` (:94-107), which the reference builds from whole-tensor operations
of the tensors' dtype - so every product and the sum is rounded once to that dtype, and this file
rounds in the same three places.

Pinned against the reference's own tests (crates/dash-mag/tests/rope.rs), which hold no stored
vectors but closed forms: the f64 rotation of ``it_is_transformers_rotation`` (:9-29) and the
row-by-row identity of ``a_position_at_a_time_is_the_range_s_row`` (:31-43); both are restated in
tests/test_rope_cpu.py.  The one unpinned detail is ``f32::powf`` in the frequencies (:44-46),
taken here as numpy's float32 power.
"""
from __future__ import annotations

import numpy as np

DTYPES = ("f32", "bf16", "f16")


def round_to(x, dtype: str) -> np.ndarray:
    """float32 values rounded (to nearest, ties to even) to ``dtype`` and widened back."""
    x = np.asarray(x, dtype=np.float32)
    if dtype == "f32":
        return x
    if dtype == "f16":
        return x.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        bits = x.view(np.uint32).astype(np.uint64)
        rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
        out = rounded.astype(np.uint32).view(np.float32)
        return np.where(np.isnan(x), x, out).astype(np.float32)
    raise ValueError(dtype)


def tables(dim: int, base: float, length: int, dtype: str):
    """``Rope::new`` (rope.rs:43-56): frequencies ``1 / base^(2i / dim)`` in f32, the angle
    ``position * frequency`` in f32, its cosine and sine in f64 rounded to f32 and then to
    ``dtype``.  Returns (cos, sin), each ``[length, dim]`` float32 holding ``dtype`` values."""
    if dim == 0 or dim % 2:
        raise ValueError(f"Rope: {dim} features; an even number is rotated")
    half = dim // 2
    exponent = (2 * np.arange(half)).astype(np.float32) / np.float32(dim)
    frequencies = (np.float32(1.0) / np.power(np.float32(base), exponent, dtype=np.float32)).astype(np.float32)
    j = np.arange(dim) % half
    angle = (np.arange(length, dtype=np.float32)[:, None] * frequencies[j][None, :]).astype(np.float32)
    cos = np.cos(angle.astype(np.float64)).astype(np.float32)
    sin = np.sin(angle.astype(np.float64)).astype(np.float32)
    return round_to(cos, dtype), round_to(sin, dtype)


def rotate(x, cos, sin, dim: int, dtype: str, inverse: bool = False) -> np.ndarray:
    """``Rope::rotate`` (rope.rs:94-107) on ``x [..., D]`` with ``cos`` / ``sin`` broadcastable to
    ``[..., dim]``: ``x cos + rotate_half(x) sin`` over the first ``dim`` features, every product
    and the sum rounded to ``dtype``; the features behind pass unchanged.  ``inverse`` is the
    transpose, which the gradient goes through: the gradient times each table, the second part
    un-rotated, the two added."""
    x = np.asarray(x, dtype=np.float32)
    half = dim // 2
    turned = x[..., :dim]
    if not inverse:
        rotated = np.concatenate([-turned[..., half:], turned[..., :half]], axis=-1)
        out = round_to(round_to(turned * cos, dtype) + round_to(rotated * sin, dtype), dtype)
    else:
        r = round_to(turned * sin, dtype)
        back = np.concatenate([r[..., half:], -r[..., :half]], axis=-1)
        out = round_to(round_to(turned * cos, dtype) + back, dtype)
    return np.concatenate([out, x[..., dim:]], axis=-1)


def apply_range(x, start: int, cos, sin, dim: int, dtype: str, inverse: bool = False) -> np.ndarray:
    """``Rope::apply_range`` (rope.rs:110-135): ``x [B,T,H,D]`` at positions ``start..start+T``."""
    t = x.shape[1]
    if start + t > cos.shape[0]:
        raise ValueError(f"Rope: positions {start}..{start + t} of {cos.shape[0]} for {list(x.shape)}")
    return rotate(x, cos[start:start + t].reshape(1, t, 1, dim), sin[start:start + t].reshape(1, t, 1, dim), dim, dtype, inverse)


def apply_at(x, positions, cos, sin, dim: int, dtype: str, inverse: bool = False) -> np.ndarray:
    """``Rope::apply_at`` (rope.rs:141-165): ``x [B,H,D]``, one token per sequence, at ``positions [B]``."""
    positions = np.asarray(positions)
    b = x.shape[0]
    return rotate(x, cos[positions].reshape(b, 1, dim), sin[positions].reshape(b, 1, dim), dim, dtype, inverse)


def apply_packed(x, cu_seqlens, start: int, cos, sin, dim: int, dtype: str, inverse: bool = False) -> np.ndarray:
    """``x [tokens,H,D]`` of sequences packed back to back (offsets ``cu_seqlens``), each rotated as
    ``apply_range`` would rotate it alone from ``start``; tokens of no sequence pass unchanged."""
    out = np.array(x, dtype=np.float32, copy=True)
    for s in range(len(cu_seqlens) - 1):
        a, b = int(cu_seqlens[s]), int(cu_seqlens[s + 1])
        a, b = min(a, x.shape[0]), min(b, x.shape[0])
        if b > a:
            out[a:b] = apply_range(out[None, a:b], start, cos, sin, dim, dtype, inverse)[0]
    return out
