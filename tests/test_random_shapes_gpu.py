"""A seeded sweep of shapes over the tensor-core kernels (bf16, D = 128 and D = 64, and the D = 256 forward): sizes and masks drawn at
random so that tile boundaries, sequence boundaries, windows and padding fall in places nobody
chose, every case against the f64 oracle and run twice for identical bits (the pipelines hand
tiles between warps through barriers; a lost ordering shows as a run-to-run difference)."""
import numpy as np
import pytest

import cases as K
import records as R
from dashmag_b200.contract import AttentionMask, AttentionOptions, DType
from oracle import attention_oracle as oracle
from adapter import B200Adapter
from test_kernels_gpu import oracle_results, run_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def adapter():
    return B200Adapter()


def random_cases(count, seed, d=128):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(count):
        hkv = int(rng.choice([1, 2, 3]))
        group = int(rng.choice([1, 2, 3, 4]))
        kind = int(rng.integers(0, 4))            # none, causal, window, causal + window
        options = AttentionOptions.causal_() if kind in (1, 3) else AttentionOptions()
        if kind >= 2:
            left = int(rng.integers(0, 300))
            options = options.with_window(left, 0 if kind == 3 else int(rng.integers(0, 200)))
        masking = int(rng.integers(0, 3))         # none, key padding, packed
        if masking == 2:
            n = int(rng.integers(1, 6))
            ql = [int(x) for x in rng.integers(0, 330, size=n)]
            kl = ql if rng.random() < 0.6 else [int(x) for x in rng.integers(0, 330, size=n)]
            if sum(ql) == 0 or sum(kl) == 0:
                ql, kl = [129], [129]
            b, tq, tk = 1, sum(ql) + int(rng.integers(0, 3)), sum(kl) + int(rng.integers(0, 3))
            mask = AttentionMask.packed(K.offsets(ql), K.offsets(kl))
        else:
            b = int(rng.integers(1, 4))
            tq, tk = int(rng.integers(1, 700)), int(rng.integers(1, 700))
            if d != 128:   # the tensor-core kernels take this head dimension from 128 queries and keys on
                tq, tk = max(tq, 128), max(tk, 128)
            if rng.random() < 0.5:
                tk = tq
            mask = AttentionMask.none()
            if masking == 1:
                mask = AttentionMask.key_padding(oracle.coins(b * tk, float(rng.uniform(0.05, 0.6)), 900 + i).reshape(b, tk))
        if d != 128 and masking == 2:
            tq, tk = max(tq, 128), max(tk, 128)   # tokens past the last offset belong to no sequence
        out.append(K.seeded(f"random {i}: d{d} b{b} hq{hkv * group} hkv{hkv} tq{tq} tk{tk} kind{kind} mask{masking}",
                            [b, hkv * group, hkv, tq, tk, d], mask, options, 1000 + 7 * i))
    return out


CASES = random_cases(40, 20261125) + random_cases(20, 20261126, d=64) + random_cases(12, 20261127, d=256)
# o, lse, dq, dk, dv relative to each result's largest value: the bounds of the fixed shapes
# (test_kernels_gpu.OWN) with a tenth more room for dk, whose sums of values rounded to bf16 (P, dS:
# 2^-9 each) grow with the number of terms at shapes drawn at random.  Largest errors measured over
# the 72 cases: 4.35e-3, 2.8e-7, 4.95e-3, 4.99e-3, 4.54e-3; a wrong tile, mask or ordering is off by
# orders of magnitude more.
SWEEP = [4.6e-3, 4.4e-7, 7.7e-3, 5.3e-3, 5.0e-3]


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_random_shape(adapter, case):
    a = run_case(adapter, case, DType.BF16)
    R.check(f"bf16 {case.name}", [a.out, a.lse, *a.grads], oracle_results(case), SWEEP)
    b = run_case(adapter, case, DType.BF16)
    for x, y in zip([a.out, a.lse, *a.grads], [b.out, b.lse, *b.grads]):
        assert np.array_equal(x, y, equal_nan=True), "two runs of the same call differ"
