"""The attention entry points over device tensors, as dash-ops exposes them.

Mirrors the public functions of crates/dash-ops/src/attention.rs:648-806 - ``attention``,
``attention_with_lse``, ``attention_backward``, ``attention_decode`` and the ``causal_*`` forms -
with the same argument order, the same meaning and the same refusals.  Tensors are torch CUDA
tensors used purely as device buffers (torch plays the part Burn plays for the reference:
allocation, streams); every computation is a call through the C ABI of ``include/dash_attn.h``
on the current CUDA stream.  Outputs are allocated here, contiguous, as the reference's launch
glue does (crates/dash-ops/src/attention/cube.rs:573-580).

Where dash-ops panics (shapes that do not fit together) these raise :class:`AttentionError` with
the same message; a well-formed call the library does not take raises :class:`Unsupported`
(dash-conformance's ``Unsupported``, crates/dash-conformance/src/lib.rs:170-172).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from .contract import AttentionMask, AttentionOptions, DType


class AttentionError(ValueError):
    """The shapes of a call do not fit together: where dash-ops panics."""


class Unsupported(NotImplementedError):
    """A well-formed call this library does not take."""


_DTYPES = {torch.float32: DType.F32, torch.bfloat16: DType.BF16, torch.float16: DType.F16}


def _raise(code: int) -> None:
    message = _lib.last_error()
    if code == _lib.UNSUPPORTED:
        raise Unsupported(message)
    if code in (_lib.INVALID, _lib.WORKSPACE):
        raise AttentionError(message)
    raise RuntimeError(message)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None or t.numel() == 0 else ctypes.c_void_p(t.data_ptr())


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _on(device):
    """Makes the tensors' device the current one for the call: the library launches on the current
    device, and the caller's may be another (one process driving several GPUs)."""
    return torch.cuda.device(device)


def _strides(t: torch.Tensor, n: int):
    return (ctypes.c_int64 * n)(*t.stride())


def _index_bytes(t: torch.Tensor, what: str) -> int:
    if t.dtype == torch.int32:
        return 4
    if t.dtype == torch.int64:
        return 8
    raise AttentionError(f"{what} holds 4- or 8-byte integers, got {t.dtype}")


def _check_device(op: str, *tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise Unsupported(f"{op}: tensors must be on a CUDA device; this library has no CPU path")


def make_params(op: str, query, key, value, mask: AttentionMask, options: AttentionOptions,
                output=None, grad_output=None) -> Tuple[_lib.Params, list]:
    """``dash_attn_params`` for a call, and the tensors it points to (kept alive by the caller)."""
    if query.dim() != 4:
        raise AttentionError(f"{op}: query is [B, Tq, Hq, D]")
    if key.dim() != 4:
        raise AttentionError(f"{op}: key is [B, Tk, Hkv, D]")
    if value.dim() != 4:
        raise AttentionError(f"{op}: key and value must have one shape")
    if query.dtype not in _DTYPES:
        raise AttentionError(f"{op}: the dtype must be f32, bf16 or f16, got {query.dtype}")
    if key.dtype != query.dtype or value.dtype != query.dtype:
        raise AttentionError(f"{op}: queries, keys and values share one dtype")
    p = _lib.Params()
    keep = []
    p.dtype = int(_DTYPES[query.dtype])
    p.b, p.tq, p.hq, p.d = query.shape
    p.k_b, p.tk, p.hkv, p.k_d = key.shape
    if value.shape[0] != key.shape[0]:
        raise AttentionError(f"{op}: key and value must have one shape")
    _, p.v_tk, p.v_hkv, p.v_d = value.shape
    p.q_stride, p.k_stride, p.v_stride = _strides(query, 4), _strides(key, 4), _strides(value, 4)
    if output is not None:
        p.o_stride = _strides(output, 4)
    if grad_output is not None:
        p.do_stride = _strides(grad_output, 4)
    if mask.kind == "key_padding":
        kp = mask.key_padding_mask
        if kp.dim() != 2:
            raise AttentionError(f"{op}: the key padding mask is [B, Tk] = [{p.b}, {p.tk}]")
        if kp.dtype in (torch.bool, torch.uint8, torch.int8):
            p.key_padding_elem_bytes = 1
        elif kp.dtype == torch.int32:
            p.key_padding_elem_bytes = 4
        else:
            raise AttentionError(f"{op}: the key padding mask holds 1-byte booleans or 4-byte integers")
        p.mask_kind = _lib.MASK_KEY_PADDING
        p.key_padding = kp.data_ptr()
        p.key_padding_shape = (ctypes.c_int32 * 2)(*kp.shape)
        p.key_padding_stride = (ctypes.c_int64 * 2)(*kp.stride())
        keep.append(kp)
    elif mask.kind == "packed":
        cq, ck = mask.cu_seqlens_q, mask.cu_seqlens_k
        if cq.dim() != 1 or ck.dim() != 1 or cq.dtype != ck.dtype:
            raise AttentionError(
                f"{op}: cu_seqlens_q and cu_seqlens_k are [S + 1], one S, got {list(cq.shape)}, {list(ck.shape)}")
        p.mask_kind = _lib.MASK_PACKED
        p.index_elem_bytes = _index_bytes(cq, f"{op}: cu_seqlens")
        cq, ck = cq.contiguous(), ck.contiguous()
        p.cu_seqlens_q, p.cu_seqlens_k = cq.data_ptr(), ck.data_ptr()
        p.cu_seqlens_q_len, p.cu_seqlens_k_len = cq.shape[0], ck.shape[0]
        keep += [cq, ck]
    else:
        p.mask_kind = _lib.MASK_NONE
    p.causal = int(options.causal)
    if options.window is not None:
        p.has_window = 1
        p.window_left = -1 if options.window.left is None else int(options.window.left)
        p.window_right = -1 if options.window.right is None else int(options.window.right)
    if options.scale is not None:
        p.has_scale, p.scale = 1, float(options.scale)
    p.deterministic = int(options.deterministic)
    return p, keep


def _workspace(nbytes: int, device) -> Optional[torch.Tensor]:
    return torch.empty(nbytes, dtype=torch.uint8, device=device) if nbytes else None


def attention_with_lse(query, key, value, mask: AttentionMask = AttentionMask.none(),
                       options: AttentionOptions = AttentionOptions()):
    """crates/dash-ops/src/attention.rs:660-682: the output ``[B,Tq,Hq,D]`` in the queries' dtype
    and the natural log-sum-exp ``[B,Tq,Hq]`` in f32 (``-inf`` for a query that sees no key)."""
    op = "attention"
    p, keep = make_params(op, query, key, value, mask, options)
    _check_device(op, query, key, value, *keep)
    lib = _lib.lib()
    b, tq, hq, d = query.shape
    out = torch.empty((b, tq, hq, d), dtype=query.dtype, device=query.device)
    lse = torch.empty((b, tq, hq), dtype=torch.float32, device=query.device)
    ws = _workspace(lib.dash_attn_forward_workspace(ctypes.byref(p)), query.device)
    with _on(query.device):
        rc = lib.dash_attn_forward(ctypes.byref(p), _ptr(query), _ptr(key), _ptr(value), _ptr(out), _ptr(lse),
                                   _ptr(ws), 0 if ws is None else ws.numel(), _stream(query.device))
    if rc != _lib.OK:
        _raise(rc)
    return out, lse


def attention(query, key, value, mask: AttentionMask = AttentionMask.none(),
              options: AttentionOptions = AttentionOptions()):
    """crates/dash-ops/src/attention.rs:648-656."""
    return attention_with_lse(query, key, value, mask, options)[0]


def attention_backward(query, key, value, output, lse, grad_output, mask: AttentionMask = AttentionMask.none(),
                       options: AttentionOptions = AttentionOptions()):
    """crates/dash-ops/src/attention.rs:689-724: the gradients of ``query``, ``key`` and ``value``,
    each in its input's shape and dtype, from the forward's ``output`` and ``lse`` and the
    gradient of the output."""
    op = "attention_backward"
    p, keep = make_params(op, query, key, value, mask, options, output, grad_output)
    if tuple(output.shape) != tuple(query.shape):
        raise AttentionError("attention_backward: output")
    if tuple(grad_output.shape) != tuple(query.shape):
        raise AttentionError("attention_backward: grad")
    if tuple(lse.shape) != tuple(query.shape[:3]):
        raise AttentionError("attention_backward: lse")
    if output.dtype != query.dtype or grad_output.dtype != query.dtype or lse.dtype != torch.float32:
        raise AttentionError("attention_backward: output and grad in the queries' dtype, lse in f32")
    _check_device(op, query, key, value, output, lse, grad_output, *keep)
    lib = _lib.lib()
    lse = lse.contiguous()
    dq = torch.empty(query.shape, dtype=query.dtype, device=query.device)
    dk = torch.empty(key.shape, dtype=key.dtype, device=query.device)
    dv = torch.empty(value.shape, dtype=value.dtype, device=query.device)
    ws = _workspace(lib.dash_attn_backward_workspace(ctypes.byref(p)), query.device)
    with _on(query.device):
        rc = lib.dash_attn_backward(ctypes.byref(p), _ptr(query), _ptr(key), _ptr(value), _ptr(output), _ptr(lse),
                                    _ptr(grad_output), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(ws),
                                    0 if ws is None else ws.numel(), _stream(query.device))
    if rc != _lib.OK:
        _raise(rc)
    return dq, dk, dv


def make_decode_params(query, key, value, cache_lengths, options: AttentionOptions):
    op = "attention_decode"
    if query.dim() != 3:
        raise AttentionError(f"{op}: query is [B, Hq, D]")
    if key.dim() != 4:
        raise AttentionError(f"{op}: key is [B, S, Hkv, D]")
    if value.dim() != 4:
        raise AttentionError("attention: key and value must have one shape")
    if query.dtype not in _DTYPES:
        raise AttentionError(f"{op}: the dtype must be f32, bf16 or f16, got {query.dtype}")
    if key.dtype != query.dtype or value.dtype != query.dtype:
        raise AttentionError(f"{op}: queries, keys and values share one dtype")
    p = _lib.DecodeParams()
    keep = []
    p.dtype = int(_DTYPES[query.dtype])
    p.b, p.hq, p.d = query.shape
    p.k_b, p.s, p.hkv, p.k_d = key.shape
    p.v_b, p.v_s, p.v_hkv, p.v_d = value.shape
    p.q_stride = _strides(query, 3)
    p.k_stride, p.v_stride = _strides(key, 4), _strides(value, 4)
    if cache_lengths is not None:
        if cache_lengths.dim() != 1:
            raise AttentionError(f"{op}: the cache lengths are [B] = [{p.b}]")
        cache_lengths = cache_lengths.contiguous()
        p.lengths = cache_lengths.data_ptr()
        p.lengths_len = cache_lengths.shape[0]
        p.lengths_elem_bytes = _index_bytes(cache_lengths, f"{op}: the cache lengths")
        keep.append(cache_lengths)
    if options.window is not None:
        p.has_window = 1
        p.window_left = -1 if options.window.left is None else int(options.window.left)
    if options.scale is not None:
        p.has_scale, p.scale = 1, float(options.scale)
    return p, keep


def attention_decode(query, key, value, cache_lengths=None, options: AttentionOptions = AttentionOptions()):
    """crates/dash-ops/src/attention.rs:732-760: ``query`` ``[B,Hq,D]`` against the cache
    ``[B,S,Hkv,D]`` (a slice of a longer cache is read in place); ``cache_lengths`` ``[B]`` int or
    ``None`` for all ``S``; of the options the scale and the window's ``left`` apply."""
    op = "attention_decode"
    p, keep = make_decode_params(query, key, value, cache_lengths, options)
    _check_device(op, query, key, value, *keep)
    lib = _lib.lib()
    out = torch.empty(query.shape, dtype=query.dtype, device=query.device)
    ws = _workspace(lib.dash_attn_decode_workspace(ctypes.byref(p)), query.device)
    with _on(query.device):
        rc = lib.dash_attn_decode(ctypes.byref(p), _ptr(query), _ptr(key), _ptr(value), _ptr(out), _ptr(ws),
                                  0 if ws is None else ws.numel(), _stream(query.device))
    if rc != _lib.OK:
        _raise(rc)
    return out


def attention_decode_append(query, new_key, new_value, key, value, cache_lengths, options: AttentionOptions = AttentionOptions()):
    """The decoding step that first appends: ``new_key`` / ``new_value`` ``[B,Hkv,D]`` are written
    into the caches ``[B,S,Hkv,D]`` (in place) at position ``cache_lengths[b]`` and the query sees
    the keys up to and including them - the reference's ``put_along_axis_owned`` on the cache
    (crates/dash-mag/src/tensor.rs:732-744) followed by ``attention_decode`` with the lengths plus
    one (crates/dash-ops/src/attention.rs:732-760), in the decoding step's own launches.
    ``cache_lengths`` are the lengths before the step; a full cache gets no row."""
    op = "attention_decode_append"
    if cache_lengths is None:
        raise ValueError(f"{op}: the lengths are needed: they say where each sequence's new row goes")
    p, keep = make_decode_params(query, key, value, cache_lengths, options)
    _check_device(op, query, key, value, new_key, new_value, *keep)
    want = (key.shape[0], key.shape[2], key.shape[3])
    for name, t in (("new_key", new_key), ("new_value", new_value)):
        if tuple(t.shape) != want or t.dtype != key.dtype:
            raise ValueError(f"{op}: {name} must be {list(want)} of the cache's dtype, got {list(t.shape)} {t.dtype}")
    new_key, new_value = new_key.contiguous(), new_value.contiguous()
    lib = _lib.lib()
    out = torch.empty(query.shape, dtype=query.dtype, device=query.device)
    ws = _workspace(lib.dash_attn_decode_workspace(ctypes.byref(p)), query.device)
    with _on(query.device):
        rc = lib.dash_attn_decode_append(ctypes.byref(p), _ptr(query), _ptr(new_key), _ptr(new_value), _ptr(key), _ptr(value),
                                         _ptr(out), _ptr(ws), 0 if ws is None else ws.numel(), _stream(query.device))
    if rc != _lib.OK:
        _raise(rc)
    return out


def causal_attention(query, key, value, scale: float):
    """crates/dash-ops/src/attention.rs:764-772."""
    return attention(query, key, value, AttentionMask.none(), AttentionOptions.causal_().with_scale(scale))


def causal_attention_with_lse(query, key, value, scale: float):
    """crates/dash-ops/src/attention.rs:775-783."""
    return attention_with_lse(query, key, value, AttentionMask.none(), AttentionOptions.causal_().with_scale(scale))


def causal_attention_backward(query, key, value, output, lse, grad_output, scale: float):
    """crates/dash-ops/src/attention.rs:786-806."""
    return attention_backward(query, key, value, output, lse, grad_output, AttentionMask.none(),
                              AttentionOptions.causal_().with_scale(scale))


def kernels_take(query, key, value, mask=AttentionMask.none(), options=AttentionOptions(), backward=False) -> int:
    """Which kernels a call would run: 0 generic, 1 tensor-core (the analogue of dash-ops'
    ``kernels_take``, crates/dash-ops/src/attention.rs:814-821)."""
    p, keep = make_params("attention", query, key, value, mask, options, query, query)
    rc = _lib.lib().dash_attn_kernels_take(ctypes.byref(p), _ptr(query), _ptr(key), _ptr(value), int(backward))
    if rc < 0:
        _raise(-rc)
    return rc
