"""The attention contract as plain data.

Mirrors crates/dash-contract/src/attention.rs:71-183 (``Window``, ``AttentionOptions``,
``AttentionMask``) and crates/dash-contract/src/lib.rs (``DType``): same names, same defaults,
same meaning, so that a call written against the reference reads the same here.
"""
from __future__ import annotations

import dataclasses
import enum
import math
import struct
from typing import Any, Optional

#: ``usize::MAX`` in the reference: that side of the window is unbounded.
UNBOUNDED = None


class DType(enum.IntEnum):
    """The float dtypes queries, keys and values may share (the values are the C ABI's codes)."""
    F32 = 0
    BF16 = 1
    F16 = 2


@dataclasses.dataclass(frozen=True)
class Window:
    """A sliding window around each query's position: no key more than ``left`` positions before
    it or ``right`` after it; ``None`` leaves that side unbounded
    (crates/dash-contract/src/attention.rs:71-80)."""
    left: Optional[int] = UNBOUNDED
    right: Optional[int] = UNBOUNDED


@dataclasses.dataclass(frozen=True)
class AttentionOptions:
    """crates/dash-contract/src/attention.rs:82-160: attention over every key, scaled by
    ``1 / sqrt(D)``, with a backward pass that gives the same bits on every run, unless said
    otherwise."""
    causal: bool = False
    scale: Optional[float] = None
    window: Optional[Window] = None
    deterministic: bool = True

    @staticmethod
    def causal_() -> "AttentionOptions":
        return AttentionOptions(causal=True)

    def with_causal(self, causal: bool) -> "AttentionOptions":
        return dataclasses.replace(self, causal=causal)

    def with_scale(self, scale: float) -> "AttentionOptions":
        return dataclasses.replace(self, scale=scale)

    def with_window(self, left: Optional[int], right: Optional[int]) -> "AttentionOptions":
        return dataclasses.replace(self, window=Window(left, right))

    def with_deterministic(self, deterministic: bool) -> "AttentionOptions":
        return dataclasses.replace(self, deterministic=deterministic)

    def scale_for(self, d: int) -> float:
        """``(1 / sqrt(d) as f64) as f32`` unless a scale is given (:157-159)."""
        if self.scale is not None:
            return struct.unpack("f", struct.pack("f", self.scale))[0]
        return struct.unpack("f", struct.pack("f", 1.0 / math.sqrt(d)))[0] if d > 0 else 1.0

    def reach(self) -> tuple:
        """How far a query sees before and after its position (``None``: no bound); causality
        bounds the right side at 0 (crates/dash-ops/src/attention.rs:231-242)."""
        left, right = (None, None) if self.window is None else (self.window.left, self.window.right)
        return left, (0 if self.causal else right)


@dataclasses.dataclass(frozen=True)
class AttentionMask:
    """Which keys each query may see beside causality and the window
    (crates/dash-contract/src/attention.rs:162-183): ``none()``, ``key_padding(mask [B,Tk])`` with
    true where a key is left out, or ``packed(cu_seqlens_q, cu_seqlens_k)`` (``[S+1]`` each, B = 1).
    The tensors are the caller's own (torch tensors on the device for the library, NumPy arrays or
    lists for the host-side adapter)."""
    kind: str = "none"
    key_padding_mask: Any = None
    cu_seqlens_q: Any = None
    cu_seqlens_k: Any = None

    @staticmethod
    def none() -> "AttentionMask":
        return AttentionMask()

    @staticmethod
    def key_padding(mask) -> "AttentionMask":
        return AttentionMask("key_padding", key_padding_mask=mask)

    @staticmethod
    def packed(cu_seqlens_q, cu_seqlens_k) -> "AttentionMask":
        return AttentionMask("packed", cu_seqlens_q=cu_seqlens_q, cu_seqlens_k=cu_seqlens_k)
