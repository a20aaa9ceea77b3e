"""The conformance adapter for this library: host tensors in, host tensors out.

Plays the part of dash-ops' test adapter (crates/dash-ops/tests/common/adapter.rs:594-705) behind
dash-conformance's ``Adapter`` trait (crates/dash-conformance/src/lib.rs:176-215): inputs arrive as
float32 NumPy arrays with the dtype the case runs in, gradients are those of
``sum(out * grad)`` with the cotangent rounded to the output's dtype, and everything comes back as
float32 arrays together with the dtype the library returned it in.
"""
import dataclasses
from typing import Optional

import numpy as np
import torch

from dashmag_b200 import attention as A
from dashmag_b200.contract import AttentionMask, AttentionOptions, DType

TORCH = {DType.F32: torch.float32, DType.BF16: torch.bfloat16, DType.F16: torch.float16}
FROM_TORCH = {v: k for k, v in TORCH.items()}


@dataclasses.dataclass
class Attention:
    """crates/dash-conformance/src/lib.rs:453-470."""
    q: np.ndarray
    k: np.ndarray
    v: np.ndarray
    dtype: DType
    mask: AttentionMask = AttentionMask.none()
    options: AttentionOptions = AttentionOptions()
    grad: Optional[np.ndarray] = None


@dataclasses.dataclass
class AttentionOut:
    out: np.ndarray
    lse: np.ndarray
    grads: Optional[tuple]
    dtypes: list


@dataclasses.dataclass
class AttentionDecode:
    """crates/dash-conformance/src/lib.rs:493-506."""
    q: np.ndarray
    k: np.ndarray
    v: np.ndarray
    dtype: DType
    lengths: Optional[list] = None
    options: AttentionOptions = AttentionOptions()


class Unsupported(Exception):
    pass


class B200Adapter:
    def __init__(self, device="cuda:0"):
        self.device = torch.device(device)

    def describe(self) -> str:
        return f"dashmag_b200 on {torch.cuda.get_device_name(self.device)}"

    def has(self, dtype: DType) -> bool:
        return dtype in TORCH

    def _dev(self, x, dtype):
        return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(self.device).to(TORCH[dtype])

    def _mask(self, mask: AttentionMask) -> AttentionMask:
        if mask.kind == "key_padding":
            return AttentionMask.key_padding(torch.from_numpy(np.asarray(mask.key_padding_mask, dtype=bool)).to(self.device))
        if mask.kind == "packed":
            cq = torch.tensor(np.asarray(mask.cu_seqlens_q), dtype=torch.int32, device=self.device)
            ck = torch.tensor(np.asarray(mask.cu_seqlens_k), dtype=torch.int32, device=self.device)
            return AttentionMask.packed(cq, ck)
        return AttentionMask.none()

    @staticmethod
    def _host(t):
        return t.detach().to(torch.float32).cpu().numpy()

    def attention(self, call: Attention) -> AttentionOut:
        q, k, v = (self._dev(x, call.dtype) for x in (call.q, call.k, call.v))
        mask = self._mask(call.mask)
        try:
            out, lse = A.attention_with_lse(q, k, v, mask, call.options)
            grads, dtypes = None, [FROM_TORCH[out.dtype], FROM_TORCH[lse.dtype]]
            if call.grad is not None:
                # The cotangent rounded to the output's dtype (crates/dash-conformance/src/lib.rs:52-57).
                g = self._dev(call.grad, call.dtype)
                dq, dk, dv = A.attention_backward(q, k, v, out, lse, g, mask, call.options)
                grads = (self._host(dq), self._host(dk), self._host(dv))
                dtypes += [FROM_TORCH[dq.dtype], FROM_TORCH[dk.dtype], FROM_TORCH[dv.dtype]]
        except A.Unsupported as e:
            raise Unsupported(str(e))
        torch.cuda.synchronize(self.device)
        return AttentionOut(self._host(out), self._host(lse), grads, dtypes)

    def attention_decode(self, call: AttentionDecode) -> np.ndarray:
        q, k, v = (self._dev(x, call.dtype) for x in (call.q, call.k, call.v))
        lengths = None
        if call.lengths is not None:
            lengths = torch.tensor(list(call.lengths), dtype=torch.int64, device=self.device)
        try:
            out = A.attention_decode(q, k, v, lengths, call.options)
        except A.Unsupported as e:
            raise Unsupported(str(e))
        torch.cuda.synchronize(self.device)
        assert out.dtype == TORCH[call.dtype]
        return self._host(out)
