"""The attention node under automatic differentiation and the routing of a tracked decoding step
(crates/dash-ops/src/attention.rs:377-542), as dash-ops' own tests hold them
(crates/dash-ops/tests/attention.rs: gradients through ``sum(out * grad)`` against the reference's)."""
import numpy as np
import pytest
import torch

import cases as K
import records as R
from dashmag_b200 import _lib, autodiff
from dashmag_b200 import attention as A
from dashmag_b200.contract import AttentionMask, AttentionOptions
from oracle import attention_oracle as oracle
from test_kernels_gpu import OWN, oracle_results
from dashmag_b200.contract import DType

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(x, dtype, grad=False):
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(DEV).to(dtype)
    return t.requires_grad_(grad)


def device_mask(mask: AttentionMask) -> AttentionMask:
    if mask.kind == "packed":
        cq = torch.tensor(np.asarray(mask.cu_seqlens_q), dtype=torch.int32, device=DEV)
        ck = torch.tensor(np.asarray(mask.cu_seqlens_k), dtype=torch.int32, device=DEV)
        return AttentionMask.packed(cq, ck)
    if mask.kind == "key_padding":
        return AttentionMask.key_padding(torch.from_numpy(np.asarray(mask.key_padding_mask, dtype=bool)).to(DEV))
    return mask


@pytest.mark.parametrize("case", [K.tensor_core_cases()[6], K.tiled_cases()[8], K.tensor_core_cases(64)[1]],
                         ids=["packed causal D128", "key padding", "causal ragged D64"])
def test_gradients_through_the_node_are_the_written_out_backward(case):
    """sum(out * grad).backward() gives the oracle's gradients; the node saved exactly the inputs, the
    output and the log-sum-exp, and ran the library's backward once."""
    q, k, v = (dev(x, torch.bfloat16, True) for x in (case.q, case.k, case.v))
    g = dev(case.grad, torch.bfloat16)
    mask = device_mask(case.mask)
    runs = _lib.probe("backward_runs")
    out, lse = autodiff.attention_with_lse(q, k, v, mask, case.options)
    assert out.requires_grad and not lse.requires_grad
    node = out.grad_fn
    saved = node.saved_tensors
    assert len(saved) == 5 and [t.data_ptr() for t in saved[:3]] == [q.data_ptr(), k.data_ptr(), v.data_ptr()]
    assert node.mask is mask and node.options is case.options
    assert torch.equal(saved[3], out.detach()) and torch.equal(saved[4], lse)
    (out.float() * g.float()).sum().backward()
    assert _lib.probe("backward_runs") == runs + 1
    host = lambda t: t.detach().float().cpu().numpy()
    R.check(f"autodiff {case.name}", [host(out), host(lse), host(q.grad), host(k.grad), host(v.grad)], oracle_results(case), OWN[DType.BF16])
    # only what is tracked gets a gradient
    q2, k2 = dev(case.q, torch.bfloat16, True), dev(case.k, torch.bfloat16)
    out2 = autodiff.attention(q2, k2, dev(case.v, torch.bfloat16), mask, case.options)
    (out2.float() * g.float()).sum().backward()
    assert torch.equal(q2.grad, q.grad) and k2.grad is None


def test_untracked_call_records_nothing():
    case = K.tensor_core_cases()[0]
    q, k, v = (dev(x, torch.bfloat16) for x in (case.q, case.k, case.v))
    out, lse = autodiff.attention_with_lse(q, k, v, AttentionMask.none(), case.options)
    assert out.grad_fn is None and not out.requires_grad
    with torch.no_grad():
        out2 = autodiff.attention(q.clone().requires_grad_(True), k, v, AttentionMask.none(), case.options)
    assert out2.grad_fn is None and torch.equal(out, out2)


@pytest.mark.parametrize("dtype,d", [(torch.float32, 64), (torch.bfloat16, 128)], ids=["f32 D64", "bf16 D128"])
def test_tracked_decode_without_lengths_is_the_training_forward_with_one_query(dtype, d):
    """attention.rs:498-515: Tq = 1, causality off; the bits of the training forward on [B,1,Hq,D],
    and the gradients of its node, carried back to [B,Hq,D]."""
    b, s, hq, hkv = 3, 200, 8, 2
    qh, kh, vh, gh = oracle.seeded((b, hq, d), 700), oracle.seeded((b, s, hkv, d), 701), oracle.seeded((b, s, hkv, d), 702), oracle.seeded((b, hq, d), 703)
    for options in (AttentionOptions(), AttentionOptions().with_window(37, 0), AttentionOptions.causal_()):
        q, k, v = dev(qh, dtype, True), dev(kh, dtype, True), dev(vh, dtype, True)
        launches = _lib.probe("kernel_launches")
        out = autodiff.attention_decode(q, k, v, None, options)
        assert out.shape == (b, hq, d) and out.grad_fn is not None
        plain, _ = A.attention_with_lse(q.detach().reshape(b, 1, hq, d), k.detach(), v.detach(), AttentionMask.none(), options.with_causal(False))
        assert torch.equal(out.detach(), plain.reshape(b, hq, d)), "the tracked step is the training forward's bits"
        step = A.attention_decode(q.detach(), k.detach(), v.detach(), None, options)
        tol = 1e-6 if dtype == torch.float32 else 2.0 ** -7
        assert float((out.detach().float() - step.float()).abs().max()) <= tol * max(1.0, float(step.float().abs().max()))
        (out.float() * dev(gh, dtype).float()).sum().backward()
        left = None if options.window is None else options.window.left
        wo, wl = oracle.forward(qh.reshape(b, 1, hq, d), kh, vh, window=(left, None))
        wdq, wdk, wdv = oracle.backward(qh.reshape(b, 1, hq, d), kh, vh, wo, wl, gh.reshape(b, 1, hq, d), window=(left, None))
        bound = 1e-5 if dtype == torch.float32 else 8e-3
        for name, got, want in (("dq", q.grad.reshape(b, 1, hq, d), wdq), ("dk", k.grad, wdk), ("dv", v.grad, wdv)):
            err = R.errors(got.float().cpu().numpy(), want)[1]
            print(f"tracked decode {dtype} {options} {name}: relative {err:.3e}")
            assert err <= bound
        assert _lib.probe("kernel_launches") > launches


def test_tracked_decode_with_lengths_is_the_recorded_reference():
    """attention.rs:516-517: per-sequence lengths have no training path; the recorded reference gives
    the decoding kernels' result and gradients to every input."""
    b, s, hq, hkv, d = 4, 90, 4, 2, 64
    qh, kh, vh = oracle.seeded((b, hq, d), 710), oracle.seeded((b, s, hkv, d), 711), oracle.seeded((b, s, hkv, d), 712)
    lengths = [90, 17, 0, 1]
    lt = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    for options in (AttentionOptions(), AttentionOptions().with_window(9, 0)):
        q, k, v = dev(qh, torch.float32, True), dev(kh, torch.float32, True), dev(vh, torch.float32, True)
        out = autodiff.attention_decode(q, k, v, lt, options)
        left = None if options.window is None else options.window.left
        want = oracle.decode(qh, kh, vh, lengths=lengths, window_left=left)
        assert np.max(np.abs(out.detach().cpu().numpy() - want)) <= 2e-6
        kernels = A.attention_decode(q.detach(), k.detach(), v.detach(), lt, options)
        assert float((out.detach() - kernels).abs().max()) <= 2e-6
        out.square().sum().backward()
        assert q.grad is not None and k.grad is not None and v.grad is not None
        assert torch.all(q.grad[2] == 0) and torch.all(k.grad[1, 17:] == 0), "nothing flows to what a sequence does not hold"
    # untracked: the kernels themselves
    plain = autodiff.attention_decode(dev(qh, torch.float32), dev(kh, torch.float32), dev(vh, torch.float32), lt, AttentionOptions())
    assert plain.grad_fn is None
