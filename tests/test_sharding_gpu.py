"""The multi-GPU partition of the training passes, every rank's share run one after another on ONE
GPU: the shares of ``sharding.training_plan`` (head slices read in place through strides; bins of
sequences gathered into packed tensors of their own when the heads run out) put back together are
the whole call - to the bit where a share is a head slice (the same tiles run), and to the rounding of
the dtype where a bin of sequences is packed anew (its tiles then cut the sequences elsewhere, so the
sums run in another order).  The units are independent: nothing but the partition is under test."""
import numpy as np
import pytest
import torch

from dashmag_b200 import attention as A
from dashmag_b200 import sharding
from dashmag_b200.contract import AttentionMask, AttentionOptions

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def normal(shape, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randn(shape, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)


def run(q, k, v, g, lengths, options):
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32, device=DEV)
    mask = AttentionMask.packed(cu, cu)
    o, lse = A.attention_with_lse(q, k, v, mask, options)
    return (o, lse) + tuple(A.attention_backward(q, k, v, o, lse, g, mask, options))


@pytest.mark.parametrize("world,hkv,window", [(2, 4, None), (8, 4, 300), (4, 1, None), (8, 8, None)],
                         ids=["2 ranks x 2 heads", "8 ranks: 4 heads x 2 sequence bins, window", "4 ranks share one head", "a head a rank"])
def test_the_ranks_shares_put_together_are_the_whole_call(world, hkv, window):
    lengths = [700, 130, 1, 515, 260, 390, 128, 333]
    t, group, d = sum(lengths), 2, 128
    q, k, v, g = normal((1, t, hkv * group, d), 1), normal((1, t, hkv, d), 2), normal((1, t, hkv, d), 3), normal((1, t, hkv * group, d), 4)
    options = AttentionOptions.causal_() if window is None else AttentionOptions.causal_().with_window(window, 0)
    whole = run(q, k, v, g, lengths, options)
    parts = [torch.full_like(x, float("nan")) for x in whole]
    starts = np.concatenate([[0], np.cumsum(lengths)])
    plan = sharding.training_plan(lengths, hkv, group, world, window)
    for rank, entry in enumerate(plan):
        seqs, kv, qh = entry
        mine, qr, kr, vr, gr = sharding.training_share(entry, lengths, q, k, v, g)
        if qr.numel() == 0:
            continue
        if list(seqs) == list(range(len(lengths))):
            assert qr.data_ptr() == q[:, :, qh].data_ptr(), "a head share is a view of the caller's tensor"
        o, lse, dq, dk, dv = run(qr, kr, vr, gr, mine, options)
        at = 0
        for s_ in seqs:   # scatter the share's sequences back to their places
            a, b = int(starts[s_]), int(starts[s_ + 1])
            n = b - a
            parts[0][:, a:b, qh] = o[:, at:at + n]
            parts[1][:, a:b, qh] = lse[:, at:at + n]
            parts[2][:, a:b, qh] = dq[:, at:at + n]
            parts[3][:, a:b, kv] = dk[:, at:at + n]
            parts[4][:, a:b, kv] = dv[:, at:at + n]
            at += n
    torch.cuda.synchronize()
    bins = any(list(seqs) != list(range(len(lengths))) for seqs, _, _ in plan)
    for name, got, want in zip("o lse dq dk dv".split(), parts, whole):
        assert not torch.isnan(got.float()).any(), f"{name}: some unit was given to no rank"
        if not bins:
            assert torch.equal(got, want), f"{name}: the shares do not rebuild the whole call"
        else:
            got, want = got.float(), want.float()
            # o: its own rounding (neighbouring bf16 values) plus P rounded against other step boundaries (2^-9 of
            # each weight); lse: f32 rounding; the gradients: both results lie within the parity bound of the exact
            # gradient (dQ 7.7e-3, dK 4.6e-3, dV 5.0e-3 of the largest value, tests/test_full_size_gpu.py), so they
            # lie within twice that of each other
            if name == "o":
                bound = 2.0 ** -7 * want.abs() + 1e-3 * float(want.abs().max())
            elif name == "lse":
                bound = 1e-6 * want.abs().clamp_min(1.0)
            else:
                bound = torch.full_like(want, 2 * {"dq": 7.7e-3, "dk": 4.6e-3, "dv": 5.0e-3}[name] * float(want.abs().max()))
            finite = torch.isfinite(want)
            assert torch.equal(torch.isfinite(got), finite), name
            assert bool(((got - want).abs()[finite] <= bound[finite]).all()), f"{name}: a bin of sequences differs from the whole call"
