"""Rotary position embeddings over device tensors, as dash-mag exposes them.

Mirrors ``Rope`` of crates/dash-mag/src/rope.rs: the same constructor (features rotated, base,
positions held, dtype), ``apply_range`` and ``apply_at`` with the same meaning and the same
refusals, tables computed on the host once exactly as ``Rope::new`` computes them (:43-56) and the
rotation itself a call through the C ABI (``dash_rope_apply``), whose kernel keeps the roundings
of the reference's whole-tensor form.  On top of the reference's two methods: a pair of tensors
rotated in one launch (a layer's query and key), sequences packed back to back, the transpose
for the gradient, and the appending decoding step with the rotation in front
(``attention_decode_append_rope``).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch

from . import _lib
from .attention import (AttentionError, AttentionOptions, _check_device, _DTYPES, _index_bytes, _ptr, _raise, _stream,
                        _workspace, make_decode_params)


class Rope:
    """The rotation of positions ``0..len`` over the first ``dim`` features of a head
    (crates/dash-mag/src/rope.rs:11-24)."""

    def __init__(self, dim: int, base: float, len: int, dtype: torch.dtype, device="cuda"):
        if dim == 0 or dim % 2:
            raise AttentionError(f"Rope: {dim} features; an even number is rotated")
        if dtype not in _DTYPES:
            raise AttentionError(f"Rope: {dtype} is not floating")
        self.dim, self.base, self._len, self.dtype = dim, float(base), len, dtype
        # Rope::new (:43-56): frequencies and angles in f32, cosine and sine in f64, rounded to f32
        # and then to the dtype.
        half = dim // 2
        exponent = (2 * np.arange(half)).astype(np.float32) / np.float32(dim)
        frequencies = (np.float32(1.0) / np.power(np.float32(base), exponent, dtype=np.float32)).astype(np.float32)
        angle = (np.arange(len, dtype=np.float32)[:, None] * frequencies[np.arange(dim) % half][None, :]).astype(np.float32)
        cos = np.cos(angle.astype(np.float64)).astype(np.float32)
        sin = np.sin(angle.astype(np.float64)).astype(np.float32)
        self.cos = torch.from_numpy(cos).to(dtype).to(device)
        self.sin = torch.from_numpy(sin).to(dtype).to(device)

    def len(self) -> int:
        """The last position this holds, plus one."""
        return self._len

    def __len__(self) -> int:
        return self._len

    def is_empty(self) -> bool:
        return self._len == 0

    # ------------------------------------------------------------------------------------------
    def tables(self) -> _lib.RopeTables:
        return _lib.RopeTables(int(_DTYPES[self.dtype]), self.dim, self._len, _ptr(self.cos), _ptr(self.sin))

    def _check_features(self, x: torch.Tensor) -> int:
        """rope.rs:76-92."""
        if x.dtype != self.dtype:
            raise AttentionError(f"Rope: {x.dtype} under a rotation of {self.dtype}")
        d = x.shape[-1] if x.dim() else 0
        if d < self.dim:
            raise AttentionError(f"Rope: {self.dim} features to rotate, of {list(x.shape)}")
        return d

    def _run(self, tokens: int, x: torch.Tensor, other: Optional[torch.Tensor], inverse: bool, **where):
        d = self._check_features(x)
        tensors = [x] if other is None else [x, other]
        if other is not None and self._check_features(other) != d:
            raise AttentionError(f"Rope: {list(x.shape)} and {list(other.shape)} rotated together must have one head dimension")
        _check_device("Rope", self.cos, *tensors)
        tensors = [t if t.stride(-1) == 1 else t.contiguous() for t in tensors]
        outs = [torch.empty_like(t, memory_format=torch.contiguous_format) for t in tensors]
        tensors = [t.contiguous() for t in tensors]
        p = _lib.RopeParams()
        p.tokens, p.d, p.inverse = tokens, d, int(inverse)
        p.heads_a = tensors[0].shape[-2]
        p.stride_a = (ctypes.c_int64 * 2)(p.heads_a * d, d)
        if other is not None:
            p.heads_b = tensors[1].shape[-2]
            p.stride_b = (ctypes.c_int64 * 2)(p.heads_b * d, d)
        keep = []
        if "positions" in where:
            positions = where["positions"]
            p.positions, p.positions_elem_bytes = _ptr(positions), positions.element_size()
            keep.append(positions)
        elif "cu_seqlens" in where:
            cu = where["cu_seqlens"]
            p.cu_seqlens, p.cu_seqlens_len, p.index_elem_bytes = _ptr(cu), cu.numel(), _index_bytes(cu, "Rope: the offsets")
            p.start = where.get("start", 0)
            keep.append(cu)
        else:
            p.start, p.period = where["start"], where["period"]
        tables = self.tables()
        with torch.cuda.device(x.device):   # the library launches on the current device
            rc = _lib.lib().dash_rope_apply(ctypes.byref(tables), ctypes.byref(p), _ptr(tensors[0]), _ptr(outs[0]),
                                            _ptr(tensors[1]) if other is not None else None,
                                            _ptr(outs[1]) if other is not None else None, _stream(x.device))
        if rc != _lib.OK:
            _raise(rc)
        return outs[0] if other is None else (outs[0], outs[1])

    def apply_range(self, x: torch.Tensor, positions: range, other: Optional[torch.Tensor] = None, inverse: bool = False):
        """``x [B,T,H,D]`` at the positions ``positions`` of every sequence, ``T`` of them
        (rope.rs:110-135).  With ``other`` (same ``B``, ``T``, ``D``; its own heads) both are rotated
        in one launch and returned as a pair; ``inverse`` rotates a gradient back."""
        shape = x.shape
        if x.dim() != 4 or shape[1] != len(positions) or positions.stop > self._len or positions.step != 1:
            raise AttentionError(f"Rope: positions {positions.start}..{positions.stop} of {self._len} for {list(shape)}")
        if other is not None and (other.dim() != 4 or other.shape[:2] != shape[:2]):
            raise AttentionError(f"Rope: {list(other.shape)} beside {list(shape)}")
        return self._run(shape[0] * shape[1], x, other, inverse, start=positions.start, period=shape[1])

    def apply_at(self, x: torch.Tensor, positions: torch.Tensor, other: Optional[torch.Tensor] = None, inverse: bool = False):
        """``x [B,H,D]``, one token per sequence, at ``positions [B]``, integer (rope.rs:141-165).
        A position past the tables is the caller's to avoid, as in the reference; here it gives
        NaN, not an out-of-bounds read."""
        shape = x.shape
        integer = positions.dtype in (torch.int32, torch.int64)
        if not integer or x.dim() != 3 or tuple(positions.shape) != (shape[0],):
            raise AttentionError(f"Rope: positions of {positions.dtype} {list(positions.shape)} for {list(shape)}")
        if other is not None and (other.dim() != 3 or other.shape[0] != shape[0]):
            raise AttentionError(f"Rope: {list(other.shape)} beside {list(shape)}")
        return self._run(shape[0], x, other, inverse, positions=positions.contiguous())

    def apply_packed(self, x: torch.Tensor, cu_seqlens: torch.Tensor, start: int = 0, other: Optional[torch.Tensor] = None,
                     inverse: bool = False):
        """``x [tokens,H,D]`` (or ``[1,tokens,H,D]``) of sequences packed back to back with the
        attention mask's offsets ``cu_seqlens``: every sequence is rotated from position ``start``
        on, as ``apply_range`` would rotate it alone; tokens of no sequence pass unchanged."""
        lead = x.dim() == 4
        if lead and x.shape[0] != 1 or x.dim() not in (3, 4):
            raise AttentionError(f"Rope: packed tokens are [tokens, H, D], got {list(x.shape)}")
        tokens = x.shape[1] if lead else x.shape[0]
        return self._run(tokens, x, other, inverse, cu_seqlens=cu_seqlens.contiguous(), start=start)


def attention_decode_append_rope(rope: Rope, query, new_key, new_value, key, value, cache_lengths,
                                 options: AttentionOptions = AttentionOptions(), positions: Optional[torch.Tensor] = None):
    """The appending decoding step with the rotation in front: ``query [B,Hq,D]`` and ``new_key
    [B,Hkv,D]`` are rotated at ``cache_lengths[b]`` (or ``positions[b]``), the rotated key and
    ``new_value`` go into the caches at ``cache_lengths[b]`` and the query sees the keys up to and
    including them - ``Rope::apply_at`` twice, ``put_along_axis_owned`` twice and
    ``attention_decode`` in the reference's caller (crates/dash-mag/tests/step.rs:200-217 is the
    prefill form of the same sequence), one call here."""
    op = "attention_decode_append_rope"
    if cache_lengths is None:
        raise AttentionError(f"{op}: the lengths are needed: they say where each sequence's new row goes")
    p, keep = make_decode_params(query, key, value, cache_lengths, options)
    _check_device(op, query, key, value, new_key, new_value, rope.cos, positions, *keep)
    want = (key.shape[0], key.shape[2], key.shape[3])
    for name, t in (("new_key", new_key), ("new_value", new_value)):
        if tuple(t.shape) != want or t.dtype != key.dtype:
            raise AttentionError(f"{op}: {name} must be {list(want)} of the cache's dtype, got {list(t.shape)} {t.dtype}")
    rope._check_features(query)
    if positions is not None and (positions.dtype not in (torch.int32, torch.int64) or tuple(positions.shape) != (query.shape[0],)):
        raise AttentionError(f"Rope: positions of {positions.dtype} {list(positions.shape)} for {list(query.shape)}")
    new_key, new_value = new_key.contiguous(), new_value.contiguous()
    if query.stride(-1) != 1:
        query = query.contiguous()
        p.q_stride = (ctypes.c_int64 * 3)(*query.stride())
    lib = _lib.lib()
    out = torch.empty(query.shape, dtype=query.dtype, device=query.device)
    ws = _workspace(lib.dash_attn_decode_append_rope_workspace(ctypes.byref(p)), query.device)
    tables = rope.tables()
    with torch.cuda.device(query.device):   # the library launches on the current device
        rc = lib.dash_attn_decode_append_rope(ctypes.byref(p), ctypes.byref(tables),
                                              _ptr(positions.contiguous()) if positions is not None else None,
                                              positions.element_size() if positions is not None else 0,
                                              _ptr(query), _ptr(new_key), _ptr(new_value), _ptr(key), _ptr(value), _ptr(out),
                                              _ptr(ws), 0 if ws is None else ws.numel(), _stream(query.device))
    if rc != _lib.OK:
        _raise(rc)
    return out
