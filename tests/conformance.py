"""The attention bodies of dash-conformance, restated over the Python adapter
(crates/dash-conformance/src/attention.rs): every record against torch, a call without gradients,
and decoding against attention with one query.  Each returns what it measured and how many calls
ran; a call the adapter refuses is recorded as skipped, and the caller asserts that none was."""
import numpy as np

import records as R
from adapter import Attention, AttentionDecode, Unsupported
from dashmag_b200.contract import AttentionMask, AttentionOptions, DType
from oracle import attention_oracle as oracle

# crates/dash-conformance/src/attention.rs:70-108, each in the order o, lse, dq, dk, dv.
FLEX_F32 = {"causal": [3e-7, 1.1e-7, 5e-7, 3.5e-7, 3.5e-7], "masks": [3.2e-7, 1.2e-7, 3.2e-7, 4.1e-7, 3.5e-7]}
CUBE_F32 = {"causal": [3.2e-7, 1.1e-7, 8.5e-7, 4.6e-7, 4.1e-7], "masks": [5.5e-7, 1.4e-7, 5.3e-7, 4.3e-7, 3.4e-7]}
AUTOTUNE_F32 = {"causal": [1e-6, 2e-7, 1e-6, 1e-6, 1e-6], "masks": [1e-6, 2e-7, 1e-6, 1e-6, 1e-6]}
BF16 = {"causal": [3.4e-3, 2.5e-7, 4.7e-3, 4e-3, 4.2e-3], "masks": [3.2e-3, 1.2e-7, 4.3e-3, 4.4e-3, 3.6e-3]}
F16 = {"causal": [4.6e-4, 1.7e-7, 4.7e-4, 3.6e-4, 4e-4], "masks": [3.9e-4, 1.2e-7, 7.4e-4, 6.9e-4, 6.4e-4]}


class Outcome:
    """crates/dash-conformance/src/lib.rs:508-567."""

    def __init__(self):
        self.ran, self.skipped, self.value = 0, [], None

    def all_ran(self):
        assert not self.skipped, f"{len(self.skipped)} calls skipped, {self.ran} ran: {self.skipped}"
        assert self.ran > 0, "no call ran"
        return self.value


def _run(outcome, label, fn, call):
    try:
        result = fn(call)
    except Unsupported as e:
        print(f"skipped: does not run {label}: {e}")
        outcome.skipped.append(f"{label}: {e}")
        return None
    outcome.ran += 1
    return result


def matches_torch(adapter, label, dtype: DType, deterministic: bool, bounds) -> Outcome:
    """:352-394."""
    outcome = Outcome()
    worst = {"causal": [0.0] * 5, "masks": [0.0] * 5}
    empty = compared = 0
    for rec in R.records():
        case = f"{label} {rec.name}"
        call = Attention(rec.q, rec.k, rec.v, dtype, rec.mask, rec.options.with_deterministic(deterministic), rec.grad)
        got = _run(outcome, case, adapter.attention, call)
        if got is None:
            continue
        assert got.dtypes == [dtype, DType.F32, dtype, dtype, dtype], (
            f"{case}: the output and gradients in the inputs' dtype, the log-sum-exp in f32")
        which = "causal" if rec.causal_set else "masks"
        actual = [got.out, got.lse, *got.grads]
        errs = R.check(case, actual, rec.expected, bounds[which])
        worst[which] = [max(a, b) for a, b in zip(worst[which], errs)]
        empty += R.check_empty_rows(case, got.out, got.grads[0], rec.expected[1])
        compared += 1
    assert compared == 0 or empty > 0, "no record has a query that sees no key"
    outcome.value = worst
    return outcome


def without_gradients(adapter, label, bounds) -> Outcome:
    """:399-429."""
    outcome = Outcome()
    for name in ["padding_causal_b2_gqa2x1_d64_t26", "packed_causal_gqa2x1_d64"]:
        rec = R.Record(name)
        case = f"{label} no gradient {name}"
        got = _run(outcome, case, adapter.attention, Attention(rec.q, rec.k, rec.v, DType.F32, rec.mask, rec.options))
        if got is None:
            continue
        assert got.grads is None
        R.check_empty_rows(case, got.out, None, rec.expected[1])
        for i, actual in enumerate([got.out, got.lse]):
            abs_err, rel = R.errors(actual, rec.expected[i])
            print(f"{case} {R.PARTS[i]}: max abs {abs_err:.3e}, relative {rel:.3e} (tolerance {bounds['masks'][i]:.1e})")
            assert rel <= bounds["masks"][i]
    return outcome


def decoding_is_attention_with_one_query(adapter, label, bounds) -> Outcome:
    """:484-565: bounds are absolute differences, [without lengths, with lengths]."""
    outcome = Outcome()
    b, s, hq, hkv, d = 3, 50, 4, 2, 64
    q = oracle.seeded((b, 1, hq, d), 400)
    k = oracle.seeded((b, s, hkv, d), 401)
    v = oracle.seeded((b, s, hkv, d), 402)
    step_q = q.reshape(b, hq, d)
    for options in [AttentionOptions(), AttentionOptions().with_window(7, 0)]:
        case = f"{label} decode {options}"
        step = _run(outcome, case, adapter.attention_decode, AttentionDecode(step_q, k, v, DType.F32, None, options))
        if step is None:
            continue
        assert step.shape == (b, hq, d), "decoding returns [B, Hq, D]"
        full = _run(outcome, case, adapter.attention,
                    Attention(q, k, v, DType.F32, AttentionMask.none(), options.with_causal(True)))
        if full is None:
            continue
        diff = float(np.max(np.abs(step - full.out.reshape(b, hq, d))))
        print(f"{case}: decode against attention, max abs {diff:.3e}")
        assert diff <= bounds[0], f"{case}: decode and attention differ by {diff}"
    lengths = [50, 17, 1]
    options = AttentionOptions().with_window(9, 0)
    case = f"{label} decode, lengths {lengths}, window 9"
    step = _run(outcome, case, adapter.attention_decode, AttentionDecode(step_q, k, v, DType.F32, lengths, options))
    if step is not None:
        for bi, n in enumerate(lengths):
            full = _run(outcome, case, adapter.attention,
                        Attention(q[bi:bi + 1], k[bi:bi + 1, :n], v[bi:bi + 1, :n], DType.F32, AttentionMask.none(), options))
            if full is None:
                continue
            diff = float(np.max(np.abs(step[bi] - full.out.reshape(hq, d))))
            print(f"{case}: sequence {bi} of {n} keys, max abs {diff:.3e}")
            assert diff <= bounds[1], f"{case}: sequence {bi} of {n} keys: decode differs by {diff}"
    return outcome
