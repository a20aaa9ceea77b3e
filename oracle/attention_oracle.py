"""CPU oracle for the attention path: TEST INFRASTRUCTURE, not product code.

Two restatements of the reference's CPU algorithm (crates/dash-ops/src/attention/reference.rs:
materialised scores and mask per head, expanded key-value heads, guarded softmax, plain products):

* the C library built from ``attention_oracle.c`` (``forward``, ``backward``, ``decode``), in
  double (``precise=True``, the parity oracle) or in float as the reference's Flex path computes
  (``precise=False``, the timed CPU baseline);
* a NumPy twin (``numpy_forward``, ``numpy_backward``, ``numpy_decode``) in float64, written from
  the contract's closed form (one visible key interval per query,
  crates/dash-contract/src/attention.rs:33-59) rather than from the boolean mask, so that the two
  check each other.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.  Arguments are
NumPy float32 arrays in the contract's layouts (q, o, do ``[B,Tq,Hq,D]``; k, v ``[B,Tk,Hkv,D]``;
lse ``[B,Tq,Hq]``; decode q ``[B,Hq,D]``, cache ``[B,S,Hkv,D]``).  ``window=(left, right)`` with
``None`` (or a negative number) for an unbounded side.
"""
from __future__ import annotations

import ctypes
import math
import pathlib
import subprocess

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent
LIB_PATH = HERE / "_build" / "liboracle_attention.so"


class _Params(ctypes.Structure):
    _fields_ = [
        ("b", ctypes.c_int32), ("tq", ctypes.c_int32), ("tk", ctypes.c_int32),
        ("hq", ctypes.c_int32), ("hkv", ctypes.c_int32), ("d", ctypes.c_int32),
        ("mask_kind", ctypes.c_int32),
        ("key_padding", ctypes.c_void_p),
        ("cu_q", ctypes.c_void_p), ("cu_k", ctypes.c_void_p),
        ("seqs", ctypes.c_int32), ("causal", ctypes.c_int32),
        ("window_left", ctypes.c_int64), ("window_right", ctypes.c_int64),
        ("scale", ctypes.c_float),
    ]


def build(force: bool = False) -> pathlib.Path:
    """Compiles the C oracle with the committed Makefile when the library is missing or stale."""
    sources = [HERE / "attention_oracle.c", HERE / "attention_oracle_body.inc", HERE / "Makefile"]
    stale = (not LIB_PATH.exists()) or any(s.stat().st_mtime > LIB_PATH.stat().st_mtime for s in sources)
    if force or stale:
        subprocess.run(["make", "-C", str(HERE), "-B"], check=True, capture_output=True)
    return LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        _lib = ctypes.CDLL(str(LIB_PATH))
        _lib.oracle_threads.restype = ctypes.c_int
    return _lib


def threads() -> int:
    return int(lib().oracle_threads())


def set_threads(n: int) -> None:
    lib().oracle_set_threads(ctypes.c_int(n))


def default_scale(d: int) -> float:
    """crates/dash-contract/src/attention.rs:157-159: (1 / sqrt(d) in f64) rounded to f32."""
    return float(np.float32(1.0 / math.sqrt(d))) if d > 0 else 1.0


def _side(x) -> int:
    return -1 if x is None or x < 0 else int(x)


def _f32(x) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _params(q, k, key_padding, cu_q, cu_k, causal, window, scale):
    b, tq, hq, d = q.shape
    _, tk, hkv, _ = k.shape
    keep = []
    p = _Params()
    p.b, p.tq, p.tk, p.hq, p.hkv, p.d = b, tq, tk, hq, hkv, d
    p.mask_kind = 0
    if key_padding is not None:
        kp = np.ascontiguousarray(np.asarray(key_padding) != 0, dtype=np.uint8).reshape(b, tk)
        keep.append(kp)
        p.mask_kind, p.key_padding = 1, _ptr(kp)
    elif cu_q is not None:
        cq = np.ascontiguousarray(cu_q, dtype=np.int64)
        ck = np.ascontiguousarray(cu_k, dtype=np.int64)
        keep += [cq, ck]
        p.mask_kind, p.cu_q, p.cu_k, p.seqs = 2, _ptr(cq), _ptr(ck), len(cq) - 1
    p.causal = int(bool(causal))
    p.window_left, p.window_right = _side(window[0]), _side(window[1])
    p.scale = default_scale(d) if scale is None else float(scale)
    return p, keep


def forward(q, k, v, *, key_padding=None, cu_q=None, cu_k=None, causal=False, window=(None, None),
            scale=None, precise=True):
    """(o, lse) as float32 arrays."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    p, keep = _params(q, k, key_padding, cu_q, cu_k, causal, window, scale)
    o = np.empty(q.shape, np.float32)
    lse = np.empty(q.shape[:3], np.float32)
    fn = lib().oracle_attention_forward_f64 if precise else lib().oracle_attention_forward_f32
    fn(ctypes.byref(p), _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse))
    del keep
    return o, lse


def backward(q, k, v, o, lse, dout, *, key_padding=None, cu_q=None, cu_k=None, causal=False,
             window=(None, None), scale=None, precise=True):
    """(dq, dk, dv) as float32 arrays."""
    q, k, v, o, lse, dout = (_f32(x) for x in (q, k, v, o, lse, dout))
    p, keep = _params(q, k, key_padding, cu_q, cu_k, causal, window, scale)
    dq, dk, dv = np.empty(q.shape, np.float32), np.empty(k.shape, np.float32), np.empty(v.shape, np.float32)
    fn = lib().oracle_attention_backward_f64 if precise else lib().oracle_attention_backward_f32
    fn(ctypes.byref(p), _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(dout), _ptr(dq), _ptr(dk), _ptr(dv))
    del keep
    return dq, dk, dv


def decode(q, k, v, *, lengths=None, window_left=None, scale=None, precise=True):
    """The decoding step's output ``[B,Hq,D]`` as float32."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    b, hq, d = q.shape
    _, s, hkv, _ = k.shape
    out = np.zeros(q.shape, np.float32)
    ln = None if lengths is None else np.ascontiguousarray(lengths, dtype=np.int64)
    fn = lib().oracle_attention_decode_f64 if precise else lib().oracle_attention_decode_f32
    fn(ctypes.c_int32(b), ctypes.c_int32(s), ctypes.c_int32(hq), ctypes.c_int32(hkv), ctypes.c_int32(d),
       _ptr(q), _ptr(k), _ptr(v), _ptr(ln), ctypes.c_int64(_side(window_left)),
       ctypes.c_float(default_scale(d) if scale is None else float(scale)), _ptr(out))
    return out


# --------------------------------------------------------------------------------------------
# NumPy twin, from the closed form: each query sees one interval of keys, less the padded ones.
# --------------------------------------------------------------------------------------------

def visible_intervals(tq, tk, *, cu_q=None, cu_k=None, causal=False, window=(None, None)):
    """``lo, hi`` (int64 ``[Tq]``): query i sees keys ``lo[i] <= j < hi[i]`` (``hi <= lo``: none).

    Not packed: position ``i + Tk - Tq``; packed: ``i_local + Lk - Lq`` inside its own sequence,
    nothing outside ``[cu[0], cu[S])`` (crates/dash-contract/src/attention.rs:33-54).
    """
    big = tq + tk + 1
    left = big if _side(window[0]) < 0 else min(_side(window[0]), big)
    right = 0 if causal else (big if _side(window[1]) < 0 else min(_side(window[1]), big))
    lo = np.full(tq, tk, np.int64)
    hi = np.zeros(tq, np.int64)
    if cu_q is None:
        for i in range(tq):
            pos = i + tk - tq
            lo[i], hi[i] = max(0, pos - left), min(tk, pos + right + 1)
    else:
        cu_q, cu_k = np.asarray(cu_q, np.int64), np.asarray(cu_k, np.int64)
        for s in range(len(cu_q) - 1):
            q0, q1 = int(cu_q[s]), int(cu_q[s + 1])
            k0, k1 = int(cu_k[s]), int(cu_k[s + 1])
            for i in range(max(q0, 0), min(q1, tq)):
                pos = (i - q0) + (k1 - k0) - (q1 - q0)
                lo[i] = max(k0 + max(0, pos - left), 0)
                hi[i] = min(k0 + min(k1 - k0, pos + right + 1), tk)
    empty = hi <= lo
    lo[empty], hi[empty] = tk, 0
    return lo, hi


def _visible(b, tq, tk, key_padding, **kw):
    lo, hi = visible_intervals(tq, tk, **kw)
    j = np.arange(tk)[None, :]
    vis = (j >= lo[:, None]) & (j < hi[:, None])
    vis = np.broadcast_to(vis[None], (b, tq, tk)).copy()
    if key_padding is not None:
        vis &= ~(np.asarray(key_padding).reshape(b, 1, tk) != 0)
    return vis


def numpy_forward(q, k, v, *, key_padding=None, cu_q=None, cu_k=None, causal=False,
                  window=(None, None), scale=None):
    q, k, v = (np.asarray(x, np.float64) for x in (q, k, v))
    b, tq, hq, d = q.shape
    _, tk, hkv, _ = k.shape
    scale = default_scale(d) if scale is None else float(np.float32(scale))
    o = np.zeros((b, tq, hq, d))
    lse = np.full((b, tq, hq), -np.inf)
    if q.size == 0 or tk == 0:
        return o.astype(np.float32), lse.astype(np.float32)
    vis = _visible(b, tq, tk, key_padding, cu_q=cu_q, cu_k=cu_k, causal=causal, window=window)
    g = hq // hkv
    for h in range(hq):
        s = np.einsum("bid,bjd->bij", q[:, :, h], k[:, :, h // g]) * scale
        s = np.where(vis, s, -np.inf)
        m = s.max(-1, keepdims=True)
        m = np.where(np.isfinite(m), m, 0.0)
        e = np.exp(s - m)
        z = e.sum(-1, keepdims=True)
        o[:, :, h] = np.einsum("bij,bjd->bid", e / np.where(z == 0, 1.0, z), v[:, :, h // g])
        with np.errstate(divide="ignore"):
            lse[:, :, h] = (m + np.log(z))[..., 0]
    return o.astype(np.float32), lse.astype(np.float32)


def numpy_backward(q, k, v, o, lse, dout, *, key_padding=None, cu_q=None, cu_k=None, causal=False,
                   window=(None, None), scale=None):
    q, k, v, o, lse, dout = (np.asarray(x, np.float64) for x in (q, k, v, o, lse, dout))
    b, tq, hq, d = q.shape
    _, tk, hkv, _ = k.shape
    scale = default_scale(d) if scale is None else float(np.float32(scale))
    dq, dk, dv = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    if q.size == 0 or tk == 0:
        return dq.astype(np.float32), dk.astype(np.float32), dv.astype(np.float32)
    vis = _visible(b, tq, tk, key_padding, cu_q=cu_q, cu_k=cu_k, causal=causal, window=window)
    g = hq // hkv
    for h in range(hq):
        kh, vh = k[:, :, h // g], v[:, :, h // g]
        s = np.einsum("bid,bjd->bij", q[:, :, h], kh) * scale
        l = np.where(np.isneginf(lse[:, :, h]), np.inf, lse[:, :, h])[..., None]
        p = np.where(vis, np.exp(np.where(vis, s, 0.0) - l), 0.0)
        dv[:, :, h // g] += np.einsum("bij,bid->bjd", p, dout[:, :, h])
        dp = np.einsum("bid,bjd->bij", dout[:, :, h], vh)
        delta = (dout[:, :, h] * o[:, :, h]).sum(-1, keepdims=True)
        ds = p * (dp - delta)
        dq[:, :, h] = np.einsum("bij,bjd->bid", ds, kh) * scale
        dk[:, :, h // g] += np.einsum("bij,bid->bjd", ds, q[:, :, h]) * scale
    return dq.astype(np.float32), dk.astype(np.float32), dv.astype(np.float32)


def numpy_decode(q, k, v, *, lengths=None, window_left=None, scale=None):
    q, k, v = (np.asarray(x, np.float64) for x in (q, k, v))
    b, hq, d = q.shape
    _, s, hkv, _ = k.shape
    scale = default_scale(d) if scale is None else float(np.float32(scale))
    out = np.zeros((b, hq, d))
    g = hq // hkv
    for bi in range(b):
        n = s if lengths is None else int(min(max(int(lengths[bi]), 0), s))
        if n == 0:
            continue
        first = 0 if _side(window_left) < 0 else max(0, n - 1 - _side(window_left))
        for h in range(hq):
            sc = k[bi, first:n, h // g] @ q[bi, h] * scale
            e = np.exp(sc - sc.max())
            out[bi, h] = (e / e.sum()) @ v[bi, first:n, h // g]
    return out.astype(np.float32)


def seeded(shape, seed: int) -> np.ndarray:
    """Deterministic bf16-representable values in about [-2, 2], the reference tests' generator
    (crates/dash-conformance/src/attention.rs:433-452)."""
    out = np.empty(int(np.prod(shape)), np.float32)
    lib().oracle_seeded(_ptr(out), ctypes.c_int64(out.size), ctypes.c_uint64(seed))
    return out.reshape(shape)


def coins(n: int, p: float, seed: int) -> np.ndarray:
    """Deterministic booleans, true with probability ``p``
    (crates/dash-ops/tests/attention_masks.rs:373-384)."""
    out = np.empty(n, np.uint8)
    lib().oracle_coins(_ptr(out), ctypes.c_int64(n), ctypes.c_float(p), ctypes.c_uint64(seed))
    return out.astype(bool)
