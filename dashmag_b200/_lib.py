"""ctypes binding of ``include/dash_attn.h``: the structs, the prototypes and the loader.

The library is the product; there is no fallback.  If ``libdash_attn_b200.so`` is missing this
module raises at import time of the first call, naming the build command.
"""
from __future__ import annotations

import ctypes
import os
import pathlib

HERE = pathlib.Path(__file__).resolve().parent
#: The built library; DASH_ATTN_LIBRARY names another build of the same sources (for experiments).
LIB_PATH = pathlib.Path(os.environ.get("DASH_ATTN_LIBRARY", HERE / "csrc" / "libdash_attn_b200.so"))

OK, INVALID, UNSUPPORTED, WORKSPACE, CUDA = 0, 1, 2, 3, 4
MASK_NONE, MASK_KEY_PADDING, MASK_PACKED = 0, 1, 2
PROBES = {
    "kernel_launches": 0,
    "backward_runs": 1,
    "input_copies": 2,
    "atomic_runs": 3,
    "tensor_core_runs": 4,
    "generic_runs": 5,
    "tensor_map_encodes": 6,
}

i32, i64, f32, vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p


class Params(ctypes.Structure):
    """``dash_attn_params``."""
    _fields_ = [
        ("dtype", i32),
        ("b", i32), ("tq", i32), ("tk", i32), ("hq", i32), ("hkv", i32), ("d", i32),
        ("v_tk", i32), ("v_hkv", i32), ("v_d", i32),
        ("k_b", i32), ("k_d", i32),
        ("q_stride", i64 * 4), ("k_stride", i64 * 4), ("v_stride", i64 * 4),
        ("o_stride", i64 * 4), ("do_stride", i64 * 4),
        ("mask_kind", i32),
        ("key_padding", vp),
        ("key_padding_elem_bytes", i32),
        ("key_padding_shape", i32 * 2),
        ("key_padding_stride", i64 * 2),
        ("cu_seqlens_q", vp), ("cu_seqlens_k", vp),
        ("cu_seqlens_q_len", i32), ("cu_seqlens_k_len", i32),
        ("index_elem_bytes", i32),
        ("causal", i32),
        ("has_window", i32),
        ("window_left", i64), ("window_right", i64),
        ("has_scale", i32),
        ("scale", f32),
        ("deterministic", i32),
    ]


class DecodeParams(ctypes.Structure):
    """``dash_attn_decode_params``."""
    _fields_ = [
        ("dtype", i32),
        ("b", i32), ("s", i32), ("hq", i32), ("hkv", i32), ("d", i32),
        ("k_b", i32), ("k_d", i32), ("v_b", i32), ("v_s", i32), ("v_hkv", i32), ("v_d", i32),
        ("q_stride", i64 * 3),
        ("k_stride", i64 * 4), ("v_stride", i64 * 4),
        ("lengths", vp),
        ("lengths_len", i32),
        ("lengths_elem_bytes", i32),
        ("has_window", i32),
        ("window_left", i64),
        ("has_scale", i32),
        ("scale", f32),
    ]


class RopeTables(ctypes.Structure):
    """``dash_rope_tables``."""
    _fields_ = [("dtype", i32), ("dim", i32), ("len", i64), ("cos", vp), ("sin", vp)]


class RopeParams(ctypes.Structure):
    """``dash_rope_params``."""
    _fields_ = [
        ("tokens", i64),
        ("d", i32),
        ("heads_a", i32), ("heads_b", i32),
        ("stride_a", i64 * 2), ("stride_b", i64 * 2),
        ("inverse", i32),
        ("positions", vp),
        ("positions_elem_bytes", i32),
        ("cu_seqlens", vp),
        ("cu_seqlens_len", i32),
        ("index_elem_bytes", i32),
        ("start", i64), ("period", i64),
    ]


class SampleParams(ctypes.Structure):
    """``dash_sample_params``."""
    _fields_ = [
        ("dtype", i32),
        ("b", i32), ("v", i32),
        ("row_stride", i64),
        ("temperature", f32),
        ("top_k", i64),
        ("top_p", f32),
        ("seed", ctypes.c_uint64), ("offset", ctypes.c_uint64),
        ("masked", ctypes.POINTER(ctypes.c_uint32)),
        ("masked_len", i32),
        ("token_elem_bytes", i32),
    ]


#: Every symbol ``include/dash_attn.h`` declares, with (restype, argtypes).
PROTOTYPES = {
    "dash_attn_forward_workspace": (ctypes.c_size_t, [ctypes.POINTER(Params)]),
    "dash_attn_backward_workspace": (ctypes.c_size_t, [ctypes.POINTER(Params)]),
    "dash_attn_decode_workspace": (ctypes.c_size_t, [ctypes.POINTER(DecodeParams)]),
    "dash_attn_forward": (ctypes.c_int, [ctypes.POINTER(Params), vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]),
    "dash_attn_backward": (ctypes.c_int, [ctypes.POINTER(Params), vp, vp, vp, vp, vp, vp, vp, vp, vp, vp,
                                          ctypes.c_size_t, vp]),
    "dash_attn_decode": (ctypes.c_int, [ctypes.POINTER(DecodeParams), vp, vp, vp, vp, vp, ctypes.c_size_t, vp]),
    "dash_attn_decode_append": (ctypes.c_int, [ctypes.POINTER(DecodeParams), vp, vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]),
    "dash_rope_apply": (ctypes.c_int, [ctypes.POINTER(RopeTables), ctypes.POINTER(RopeParams), vp, vp, vp, vp, vp]),
    "dash_attn_decode_append_rope_workspace": (ctypes.c_size_t, [ctypes.POINTER(DecodeParams)]),
    "dash_attn_decode_append_rope": (ctypes.c_int, [ctypes.POINTER(DecodeParams), ctypes.POINTER(RopeTables), vp, i32,
                                                    vp, vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]),
    "dash_sample_workspace": (ctypes.c_size_t, [ctypes.POINTER(SampleParams)]),
    "dash_sample": (ctypes.c_int, [ctypes.POINTER(SampleParams), vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]),
    "dash_attn_decode_static": (ctypes.c_int, [ctypes.POINTER(DecodeParams), vp, vp, vp, vp, vp]),
    "dash_attn_kernels_take": (ctypes.c_int, [ctypes.POINTER(Params), vp, vp, vp, ctypes.c_int]),
    "dash_attn_device_status": (ctypes.c_int, [ctypes.c_int]),
    "dash_attn_last_error": (ctypes.c_char_p, []),
    "dash_attn_probe": (ctypes.c_uint64, [ctypes.c_int]),
    "dash_attn_force_generic": (None, [ctypes.c_int]),
    "dash_attn_force_tensor": (None, [ctypes.c_int]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises if it has not been built: nothing else can run the path."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m dashmag_b200.build` "
                "(nvcc, sm_100a). There is no fallback path."
            )
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def last_error() -> str:
    return lib().dash_attn_last_error().decode()


def probe(name: str) -> int:
    return int(lib().dash_attn_probe(PROBES[name]))
