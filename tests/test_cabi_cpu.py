"""The C ABI without a GPU: the library loads, exports every symbol ``include/dash_attn.h``
declares, and refuses ill-formed calls with the reference's wording before touching a device
(crates/dash-ops/src/attention.rs:551-638)."""
import ctypes
import pathlib
import re

import pytest
import torch

from dashmag_b200 import _lib
from dashmag_b200 import attention as A
from dashmag_b200.contract import AttentionMask, AttentionOptions

HEADER = pathlib.Path(__file__).resolve().parent.parent / "include" / "dash_attn.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(dash_(?:attn|rope|sample)[a-z_]*)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    names = declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in dash_attn.h but not exported"
    assert set(names) == set(_lib.PROTOTYPES), "the ctypes prototypes cover the header exactly"


def test_struct_sizes_match_the_header():
    """Compiles a two-line C program's worth of truth: sizeof through the C compiler."""
    import subprocess, tempfile
    src = f'#include "{HEADER}"\n#include <stdio.h>\nint main(){{printf("%zu %zu %zu %zu", sizeof(dash_attn_params), sizeof(dash_attn_decode_params), sizeof(dash_rope_tables), sizeof(dash_rope_params));}}'
    with tempfile.TemporaryDirectory() as tmp:
        c = pathlib.Path(tmp) / "s.c"
        c.write_text(src)
        exe = pathlib.Path(tmp) / "s"
        subprocess.run(["/usr/bin/gcc", str(c), "-o", str(exe)], check=True)
        a, b, c, d = map(int, subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split())
    assert ctypes.sizeof(_lib.Params) == a and ctypes.sizeof(_lib.DecodeParams) == b
    assert ctypes.sizeof(_lib.RopeTables) == c and ctypes.sizeof(_lib.RopeParams) == d


def forward_refusal(q, k, v, mask=AttentionMask.none(), options=AttentionOptions()):
    p, keep = A.make_params("attention", q, k, v, mask, options)
    rc = _lib.lib().dash_attn_forward(ctypes.byref(p), None, None, None, None, None, None, 0, None)
    return rc, _lib.last_error()


def t(*shape, dtype=torch.float32):
    return torch.zeros(*shape, dtype=dtype)


@pytest.mark.parametrize("q,k,v,message", [
    (t(2, 5, 4, 64), t(2, 7, 2, 64), t(2, 7, 2, 32), "attention: key and value must have one shape"),
    (t(2, 5, 4, 64), t(3, 7, 2, 64), t(3, 7, 2, 64), "attention: query and key must have one batch size"),
    (t(2, 5, 4, 64), t(2, 7, 2, 32), t(2, 7, 2, 32), "attention: query and key must have one head dimension"),
    (t(2, 5, 4, 64), t(2, 7, 3, 64), t(2, 7, 3, 64),
     "attention: the query heads (4) must be a multiple of the key-value heads (3)"),
])
def test_shape_refusals_carry_the_reference_wording(q, k, v, message):
    rc, text = forward_refusal(q, k, v)
    assert rc == _lib.INVALID and text == message


def test_mask_refusals():
    q, k = t(2, 5, 4, 64), t(2, 7, 2, 64)
    rc, text = forward_refusal(q, k, k, AttentionMask.key_padding(torch.zeros(2, 6, dtype=torch.bool)))
    assert rc == _lib.INVALID and text == "attention: the key padding mask is [B, Tk] = [2, 7]"
    cu = torch.tensor([0, 3, 5], dtype=torch.int32)
    rc, text = forward_refusal(q, k, k, AttentionMask.packed(cu, cu))
    assert rc == _lib.INVALID and text == "attention: packed sequences lie along the time, B = 1"
    q1, k1 = t(1, 5, 4, 64), t(1, 7, 2, 64)
    rc, text = forward_refusal(q1, k1, k1, AttentionMask.packed(cu, torch.tensor([0, 7], dtype=torch.int32)))
    assert rc == _lib.INVALID
    assert text == "attention: cu_seqlens_q and cu_seqlens_k are [S + 1], one S, got [3], [2]"


def test_unsupported_is_not_invalid():
    q, k = t(1, 5, 2, 512), t(1, 7, 2, 512)
    rc, text = forward_refusal(q, k, k)
    assert rc == _lib.UNSUPPORTED and "head dimension 512" in text


def test_rank_and_dtype_refusals_before_the_library():
    with pytest.raises(A.AttentionError, match=r"attention: query is \[B, Tq, Hq, D\]"):
        A.make_params("attention", t(5, 4, 64), t(2, 7, 2, 64), t(2, 7, 2, 64), AttentionMask.none(), AttentionOptions())
    with pytest.raises(A.AttentionError, match="dtype must be f32, bf16 or f16"):
        A.make_params("attention", t(2, 5, 4, 64, dtype=torch.float64), t(2, 7, 2, 64, dtype=torch.float64),
                      t(2, 7, 2, 64, dtype=torch.float64), AttentionMask.none(), AttentionOptions())
    with pytest.raises(A.Unsupported, match="no CPU path"):
        A.attention(t(2, 5, 4, 64), t(2, 7, 2, 64), t(2, 7, 2, 64))


def test_decode_refusals():
    lib = _lib.lib()
    p, _ = A.make_decode_params(t(3, 4, 64), t(3, 50, 2, 64), t(3, 50, 2, 64), torch.zeros(2, dtype=torch.int64), AttentionOptions())
    rc = lib.dash_attn_decode(ctypes.byref(p), None, None, None, None, None, 0, None)
    assert rc == _lib.INVALID and _lib.last_error() == "attention_decode: the cache lengths are [B] = [3]"
    p, _ = A.make_decode_params(t(3, 4, 64), t(3, 50, 3, 64), t(3, 50, 3, 64), None, AttentionOptions())
    rc = lib.dash_attn_decode(ctypes.byref(p), None, None, None, None, None, 0, None)
    assert rc == _lib.INVALID and "must be a multiple of the key-value heads (3)" in _lib.last_error()
    with pytest.raises(A.AttentionError, match=r"attention_decode: query is \[B, Hq, D\]"):
        A.make_decode_params(t(3, 1, 4, 64), t(3, 50, 2, 64), t(3, 50, 2, 64), None, AttentionOptions())


def test_decode_append_refusals():
    """The appending step needs the lengths (they say where the row goes) and both new rows, and
    otherwise refuses what attention_decode refuses, under its own name."""
    lib = _lib.lib()
    p, _ = A.make_decode_params(t(3, 4, 64), t(3, 50, 2, 64), t(3, 50, 2, 64), None, AttentionOptions())
    rc = lib.dash_attn_decode_append(ctypes.byref(p), None, None, None, None, None, None, None, 0, None)
    assert rc == _lib.INVALID and _lib.last_error().startswith("attention_decode_append: the lengths are needed")
    p, _ = A.make_decode_params(t(3, 4, 64), t(3, 50, 2, 64), t(3, 50, 2, 64), torch.zeros(3, dtype=torch.int64), AttentionOptions())
    rc = lib.dash_attn_decode_append(ctypes.byref(p), None, None, None, None, None, None, None, 0, None)
    assert rc == _lib.INVALID and _lib.last_error() == "attention_decode_append: a new row is null"
    p, _ = A.make_decode_params(t(3, 4, 64), t(3, 50, 2, 64), t(3, 50, 2, 64), torch.zeros(2, dtype=torch.int64), AttentionOptions())
    rc = lib.dash_attn_decode_append(ctypes.byref(p), None, ctypes.c_void_p(256), ctypes.c_void_p(256), None, None, None, None, 0, None)
    assert rc == _lib.INVALID and _lib.last_error() == "attention_decode_append: the cache lengths are [B] = [3]"


def test_workspace_queries_are_pure_functions_of_the_shape():
    lib = _lib.lib()
    q, k = t(1, 300, 8, 128, dtype=torch.bfloat16), t(1, 300, 2, 128, dtype=torch.bfloat16)
    p, _ = A.make_params("attention", q, k, k, AttentionMask.none(), AttentionOptions.causal_(), q, q)
    assert lib.dash_attn_backward_workspace(ctypes.byref(p)) >= 4 * 300 * 8
    pd, _ = A.make_decode_params(t(64, 32, 128, dtype=torch.bfloat16), torch.empty(0).new_empty((64, 32768, 8, 128), dtype=torch.bfloat16, device="meta"),
                                 torch.empty(0).new_empty((64, 32768, 8, 128), dtype=torch.bfloat16, device="meta"), None, AttentionOptions())
    need = lib.dash_attn_decode_workspace(ctypes.byref(pd))
    assert need == lib.dash_attn_decode_workspace(ctypes.byref(pd)) and need > 0
    # a workspace that is too small is refused before any launch
    rc = lib.dash_attn_decode(ctypes.byref(pd), ctypes.c_void_p(256), ctypes.c_void_p(256), ctypes.c_void_p(256),
                              ctypes.c_void_p(256), ctypes.c_void_p(256), 16, None)
    assert rc == _lib.WORKSPACE and "workspace holds 16 bytes" in _lib.last_error()


def test_probe_counters_start_readable():
    for name in _lib.PROBES:
        assert _lib.probe(name) >= 0
    assert _lib.probe("input_copies") == 0
