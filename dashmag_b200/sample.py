"""Sampling the next token over device tensors, as dash-ops exposes it.

Mirrors ``sample`` of crates/dash-ops/src/sample.rs with ``SampleOptions`` of
crates/dash-contract/src/sample.rs:98-150 (same fields, same defaults, ``greedy()``,
``is_greedy()``): logits ``[B, V]`` in, ``Sampled`` (tokens and the three log-probabilities) out,
the computation a call through the C ABI (``dash_sample``) on the current CUDA stream.
"""
from __future__ import annotations

import ctypes
import dataclasses
from typing import Sequence

import torch

from . import _lib
from .attention import AttentionError, _check_device, _DTYPES, _ptr, _raise, _stream, _workspace


@dataclasses.dataclass(frozen=True)
class SampleOptions:
    """crates/dash-contract/src/sample.rs:98-150."""
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0
    offset: int = 0
    masked: Sequence[int] = ()

    @staticmethod
    def greedy() -> "SampleOptions":
        return SampleOptions(temperature=0.0)

    def is_greedy(self) -> bool:
        return self.temperature == 0.0


@dataclasses.dataclass
class Sampled:
    """Tokens ``[B]`` and their log-probabilities ``[B]`` f32 under the model's distribution, the
    model's at the temperature, and the one drawn from."""
    tokens: torch.Tensor
    logprob: torch.Tensor
    tempered_logprob: torch.Tensor
    sampling_logprob: torch.Tensor


def make_sample_params(logits: torch.Tensor, options: SampleOptions, token_dtype=torch.int64):
    if logits.dim() != 2:
        raise AttentionError(f"sample: logits must be [B, V], got {list(logits.shape)}")
    if logits.dtype not in _DTYPES:
        raise AttentionError(f"sample: logits must be f32, bf16 or f16, got {logits.dtype}")
    p = _lib.SampleParams()
    p.dtype = int(_DTYPES[logits.dtype])
    p.b, p.v = logits.shape
    p.row_stride = logits.stride(0) if logits.shape[0] > 1 else logits.shape[1]
    p.temperature, p.top_k, p.top_p = options.temperature, options.top_k, options.top_p
    p.seed, p.offset = options.seed, options.offset
    ids = (ctypes.c_uint32 * max(len(options.masked), 1))(*options.masked)
    p.masked, p.masked_len = ctypes.cast(ids, ctypes.POINTER(ctypes.c_uint32)), len(options.masked)
    p.token_elem_bytes = 8 if token_dtype == torch.int64 else 4
    return p, ids


def sample(logits: torch.Tensor, options: SampleOptions = SampleOptions(), token_dtype=torch.int64) -> Sampled:
    """One token per row of ``logits [B, V]`` (crates/dash-ops/src/sample.rs ``sample``)."""
    if logits.dim() == 2 and logits.stride(1) != 1:
        logits = logits.contiguous()
    p, keep = make_sample_params(logits, options, token_dtype)
    _check_device("sample", logits)
    b, dev = logits.shape[0], logits.device
    out = Sampled(torch.empty(b, dtype=token_dtype, device=dev), *(torch.empty(b, dtype=torch.float32, device=dev) for _ in range(3)))
    lib = _lib.lib()
    ws = _workspace(lib.dash_sample_workspace(ctypes.byref(p)), dev)
    with torch.cuda.device(dev):   # the library launches on the current device
        rc = lib.dash_sample(ctypes.byref(p), _ptr(logits), _ptr(out.tokens), _ptr(out.logprob), _ptr(out.tempered_logprob),
                             _ptr(out.sampling_logprob), _ptr(ws), 0 if ws is None else ws.numel(), _stream(dev))
    if rc != _lib.OK:
        _raise(rc)
    return out
