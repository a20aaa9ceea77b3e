"""The sampler without a GPU: the oracle against the known answers and closed forms the
reference's tests hold (crates/dash-ops/src/sample/philox.rs, crates/dash-ops/tests/sample.rs),
and the C ABI's refusals (crates/dash-ops/src/sample.rs:300-342) before anything is launched."""
import ctypes
import math
import pathlib
import subprocess
import tempfile

import numpy as np
import pytest
import torch

from dashmag_b200 import _lib
from dashmag_b200.attention import AttentionError
from dashmag_b200.sample import SampleOptions, make_sample_params
from oracle import sample_oracle as S

HEADER = pathlib.Path(__file__).resolve().parent.parent / "include" / "dash_attn.h"


def test_philox_gives_random123s_known_answers():
    """philox.rs ``philox_gives_random123s_known_answers``: the three published vectors."""
    cases = [([0] * 4, [0] * 2, [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]),
             ([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2, [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]),
             ([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0],
              [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1])]
    for counter, key, want in cases:
        assert S.philox4x32_10(np.array(counter, dtype=np.uint64), key).tolist() == want


def test_gumbel_variates_against_f64():
    """sample.rs "Random numbers": g = -ln(-ln u), u = (x + 1/2) / 2^32, within 6e-6 (tests/sample.rs GUMBEL)."""
    words = np.array([0, 1, 2, 1000, 2 ** 20, 2 ** 30, 2 ** 31 - 1, 2 ** 31, 2 ** 31 + 1, 3 * 2 ** 30, 2 ** 32 - 2 ** 26,
                      2 ** 32 - 2 ** 25 - 1, 2 ** 32 - 1000, 2 ** 32 - 2, 2 ** 32 - 1], dtype=np.uint64)
    rng = np.random.default_rng(5)
    words = np.concatenate([words, rng.integers(0, 2 ** 32, size=4000, dtype=np.uint64)]).astype(np.uint32)
    got = S.gumbel_of_inputs(S.gumbel_input(words)).astype(np.float64)
    u = (words.astype(np.float64) + 0.5) / 2.0 ** 32
    want = -np.log(-np.log1p(-(1.0 - u)))
    assert np.max(np.abs(got - want)) <= 6e-6
    assert got.min() >= -3.14 and got.max() <= 22.9


def test_sums_are_trees():
    x = np.random.default_rng(1).random((3, 1001)).astype(np.float32)
    assert np.allclose(S.tree_sum(x), x.astype(np.float64).sum(axis=1), rtol=3e-7)
    assert np.allclose(S.tree_cumsum(x), np.cumsum(x.astype(np.float64), axis=1), rtol=5e-7)


def exact_kept(z, top_k, top_p, tau, masked):
    """The definition in f64 (contract sample.rs:28-40): the ids P keeps."""
    u = [i for i in range(len(z)) if i not in masked]
    zs = sorted((z[i] for i in u), reverse=True)
    k_set = u if top_k == 0 or top_k >= len(u) else [i for i in u if z[i] >= zs[top_k - 1]]
    if top_p >= 1.0:
        return sorted(k_set)
    m = max(z[i] for i in u)
    w = {i: math.exp((z[i] - m) * tau) for i in k_set}
    total = sum(w.values())
    for v in sorted({z[i] for i in k_set}, reverse=True):
        if sum(w[j] for j in k_set if z[j] >= v) >= top_p * total:
            return sorted(i for i in k_set if z[i] >= v)
    return sorted(k_set)


@pytest.mark.parametrize("top_k,top_p,temperature,masked", [
    (0, 1.0, 1.0, ()), (3, 1.0, 1.0, ()), (2, 1.0, 0.7, ()), (0, 0.5, 1.0, ()), (0, 0.0, 1.0, ()), (0, 1e-6, 1.0, ()),
    (4, 0.7, 1.3, ()), (2, 1.0, 1.0, (7, 3)), (0, 0.8, 1.2, (1, 5)), (8, 1.0, 1.0, ()), (100, 0.99, 0.5, (0,))])
def test_the_definition_keeps_what_it_says(top_k, top_p, temperature, masked):
    """Every token the oracle draws over many offsets lies in the kept set; with ties at the cut."""
    z = np.array([2.0, 1.0, 1.0, 0.5, 0.5, 0.5, -1.0, 3.0, -np.inf, 0.0], dtype=np.float32)
    tau = float(S.inverse_temperature(temperature))
    kept = exact_kept([float(x) for x in z], top_k, top_p, tau, set(masked))
    drawn = set()
    for offset in range(40):
        tokens, lp, tp, sp = S.sample(np.tile(z, (16, 1)), temperature, top_k, top_p, 3, offset, masked)
        drawn |= set(tokens.tolist())
        w = np.exp((z.astype(np.float64) - z[kept].max()) * tau)
        want_sp = np.log(w[tokens] / w[kept].sum())
        assert np.max(np.abs(sp - want_sp)) <= 1e-6
    assert drawn <= set(kept) and (len(kept) > 3 or drawn == set(kept))


def test_identities_hold_bit_for_bit():
    """sample.rs:62-68: tempered is logprob at temperature 1, sampling is tempered where nothing is cut."""
    z = np.random.default_rng(2).normal(size=(6, 300)).astype(np.float32) * 4
    t, lp, tp, sp = S.sample(z, 1.0, 0, 1.0, 9, 1)
    assert np.array_equal(lp.view(np.uint32), tp.view(np.uint32)) and np.array_equal(tp.view(np.uint32), sp.view(np.uint32))
    t, lp, tp, sp = S.sample(z, 0.8, 0, 1.0, 9, 1)
    assert np.array_equal(tp.view(np.uint32), sp.view(np.uint32)) and not np.array_equal(lp, tp)
    t, lp, tp, sp = S.sample(z, 1.0, 300, 1.0, 9, 1)          # k >= |U| cuts nothing
    assert np.array_equal(tp.view(np.uint32), sp.view(np.uint32))
    t, lp, tp, sp = S.sample(z, 0.0)
    assert np.array_equal(t, np.argmax(z, axis=1)) and not tp.any() and not sp.any()
    z[2] = -np.inf
    t, lp, tp, sp = S.sample(z, 1.0, 5, 0.9, 9, 1, masked=(0, 1))
    assert t[2] == 2 and np.isnan(lp[2]) and np.isnan(tp[2]) and np.isnan(sp[2])


def test_struct_size_and_refusals():
    src = f'#include "{HEADER}"\n#include <stdio.h>\nint main(){{printf("%zu", sizeof(dash_sample_params));}}'
    with tempfile.TemporaryDirectory() as tmp:
        c = pathlib.Path(tmp) / "s.c"
        c.write_text(src)
        subprocess.run(["/usr/bin/gcc", str(c), "-o", str(pathlib.Path(tmp) / "s")], check=True)
        size = int(subprocess.run([str(pathlib.Path(tmp) / "s")], capture_output=True, text=True, check=True).stdout)
    assert ctypes.sizeof(_lib.SampleParams) == size
    lib = _lib.lib()

    def refusal(logits, options):
        p, keep = make_sample_params(logits, options)
        rc = lib.dash_sample(ctypes.byref(p), None, None, None, None, None, None, 0, None)
        return rc, _lib.last_error()

    z = torch.zeros(2, 10)
    assert refusal(torch.zeros(2, 0), SampleOptions()) == (_lib.INVALID, "sample: the vocabulary is empty")
    assert refusal(z, SampleOptions(temperature=-1.0)) == (_lib.INVALID, "sample: the temperature must be finite and >= 0, got -1")
    assert refusal(z, SampleOptions(temperature=float("inf")))[0] == _lib.INVALID
    assert refusal(z, SampleOptions(top_p=1.5)) == (_lib.INVALID, "sample: top_p must be within 0..=1, got 1.5")
    assert refusal(z, SampleOptions(masked=(3, 10))) == (_lib.INVALID, "sample: masked token id 10 is outside the vocabulary of 10")
    assert refusal(z, SampleOptions(masked=tuple(range(10)) + (3,))) == (_lib.INVALID, "sample: every token of the vocabulary is masked")
    assert refusal(z, SampleOptions()) == (_lib.INVALID, "sample: a tensor pointer is null")
    assert refusal(torch.zeros(0, 10), SampleOptions())[0] == _lib.OK
    with pytest.raises(AttentionError, match=r"logits must be \[B, V\]"):
        make_sample_params(torch.zeros(2, 3, 4), SampleOptions())
