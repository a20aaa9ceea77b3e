"""The decoding step for callers that cannot provide a workspace (``dash_attn_decode_static``).

Some users of the library are handed raw device pointers and nothing else - a shim under a tensor
runtime whose memory pool owns all device memory, a serving loop that has promised not to allocate
once it runs - so they cannot call ``cudaMalloc`` or ask anyone for scratch.  For them the split
pass keeps its partial outputs in an array inside the library.  This test calls that entry point
through the C ABI exactly as such a caller would (inputs and output only) and holds it to the
regular entry point's result on the same inputs, twice in a row with different inputs and shapes,
because the array is shared between calls and keeps the previous call's contents.

The file sorts last on purpose: a run that stops at the first failure has by then run every other
test.  It passes alone in a fresh process as well as after the others.
"""
import ctypes

import numpy as np
import pytest
import torch

from dashmag_b200 import _lib
from dashmag_b200 import attention as A
from dashmag_b200.contract import AttentionOptions
from oracle import attention_oracle as oracle

pytestmark = pytest.mark.gpu

# One rounding of the bf16 output plus f32 noise: the two entry points may cut the cache into
# different splits, which changes the order of the f32 sums and nothing else (the bound the other
# decode tests use against the oracle).
BF16_ROUNDING = 2.0 ** -8


def decode_static(q, k, v, lengths, options):
    p, keep = A.make_decode_params(q, k, v, lengths, options)
    out = torch.full(q.shape, float("nan"), dtype=q.dtype, device=q.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
    rc = _lib.lib().dash_attn_decode_static(ctypes.byref(p), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), stream)
    assert rc == _lib.OK, _lib.last_error()
    return out


def case(b, s, hq, hkv, d, lengths, seed, dev):
    q, k, v = (torch.from_numpy(oracle.seeded(shape, seed + i)).to(dev).to(torch.bfloat16)
               for i, shape in enumerate([(b, hq, d), (b, s, hkv, d), (b, s, hkv, d)]))
    return q, k, v, torch.tensor(lengths, dtype=torch.int32, device=dev)


def test_static_scratch_decode_matches_the_workspace_entry_point_twice_in_a_row():
    dev = torch.device("cuda:0")
    calls = [
        # a long cache first, so that the second, smaller call finds the array full of stale partials
        (case(4, 6000, 8, 2, 128, [6000, 1, 0, 3333], 900, dev), AttentionOptions()),
        (case(3, 700, 4, 2, 64, [700, 129, 64], 910, dev), AttentionOptions().with_window(100, 0)),
    ]
    for (q, k, v, lengths), options in calls:
        got = decode_static(q, k, v, lengths, options)
        want = A.attention_decode(q, k, v, lengths, options)
        torch.cuda.synchronize()
        got, want = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert np.all(np.isfinite(got)), "the output was not written everywhere"
        slack = BF16_ROUNDING * np.abs(want) * 1.02 + 2e-6 * np.abs(want).max()
        assert np.all(np.abs(got - want) <= slack), f"max difference {np.max(np.abs(got - want)):.3e}"
        reference = oracle.decode(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(),
                                  lengths=lengths.cpu().numpy(), window_left=None if options.window is None else options.window.left)
        slack = BF16_ROUNDING * np.abs(reference) * 1.02 + 2e-6 * np.abs(reference).max()
        assert np.all(np.abs(got - reference) <= slack)
        empty = (lengths.cpu().numpy() <= 0)
        assert np.all(got[empty] == 0.0)


def test_static_scratch_decode_cuts_fewer_longer_splits_when_the_planned_ones_do_not_fit():
    """64 sequences x 32 query heads on one key-value head, D = 128, a cache of 4096: the plan is 32
    splits of 128 keys, of which only 15 fit the array (64 * 32 * 129 + 64 floats each), so the call
    doubles the chunk to 512 keys and runs 8 splits - the multi-unit path of the tensor-core split
    pass at a chunk the planner itself never picks for this shape."""
    dev = torch.device("cuda:0")
    b, s, hq, hkv, d = 64, 4096, 32, 1, 128
    gen = torch.Generator(device=dev).manual_seed(77)
    q = torch.randn((b, hq, d), generator=gen, device=dev).to(torch.bfloat16)
    k = torch.randn((b, s, hkv, d), generator=gen, device=dev).to(torch.bfloat16)
    v = torch.randn((b, s, hkv, d), generator=gen, device=dev).to(torch.bfloat16)
    lengths = torch.randint(1, s + 1, (b,), generator=gen, device=dev, dtype=torch.int32)
    lengths[0], lengths[1] = s, 1
    got = decode_static(q, k, v, lengths, AttentionOptions())
    want = A.attention_decode(q, k, v, lengths, AttentionOptions())
    torch.cuda.synchronize()
    got, want = got.float().cpu().numpy(), want.float().cpu().numpy()
    # Two roundings of f32 results that differ in their last bits (8 splits against 32) may land on
    # neighbouring bf16 values: one whole step between the two, half a step from each to the oracle.
    slack = 2 * BF16_ROUNDING * np.abs(want) * 1.02 + 2e-6 * np.abs(want).max()
    assert np.all(np.abs(got - want) <= slack), f"max difference {np.max(np.abs(got - want)):.3e}"
    rows = [0, 1, 17, 63]   # the oracle on a few sequences: the whole batch is 8 G products
    sub = lambda t: t[rows].float().cpu().numpy()
    reference = oracle.decode(sub(q), sub(k), sub(v), lengths=lengths[rows].cpu().numpy())
    slack = BF16_ROUNDING * np.abs(reference) * 1.02 + 2e-6 * np.abs(reference).max()
    assert np.all(np.abs(got[rows] - reference) <= slack)


def test_static_scratch_decode_refuses_what_does_not_fit():
    """B * Hq * (D + 1) floats of partials per split must fit the 4 Mi-float array."""
    meta = lambda *shape: torch.empty(shape, dtype=torch.bfloat16, device="meta")
    p, _ = A.make_decode_params(meta(4096, 64, 256), meta(4096, 16, 8, 256), meta(4096, 16, 8, 256), None, AttentionOptions())
    rc = _lib.lib().dash_attn_decode_static(ctypes.byref(p), 256, 256, 256, 256, None)
    assert rc == _lib.UNSUPPORTED
    assert "exceed the library's" in _lib.last_error() and "dash_attn_decode with a workspace" in _lib.last_error()
