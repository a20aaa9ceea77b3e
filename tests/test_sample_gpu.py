"""The sampling kernel against the oracle (the reference's own CPU form restated), as
crates/dash-ops/tests/sample.rs holds the reference's kernel to it: the same tokens, the three
log-probabilities within KERNEL_REFERENCE = 4e-6, identities and repeats bit for bit, draws that
follow the kept set's distribution."""
import numpy as np
import pytest
import torch

from dashmag_b200.sample import SampleOptions, sample
from oracle import sample_oracle as S
from oracle.rope_oracle import round_to

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TORCH = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
KERNEL_REFERENCE = 4e-6


def logits_of(b, v, dtype, seed, scale=3.0):
    z = np.random.default_rng(seed).normal(size=(b, v)).astype(np.float32) * np.float32(scale)
    return round_to(z, dtype)


def run(z, dtype, options, token_dtype=torch.int64):
    out = sample(torch.from_numpy(z).to(DEV).to(TORCH[dtype]), options, token_dtype)
    torch.cuda.synchronize()
    return (out.tokens.cpu().numpy().astype(np.int64), out.logprob.cpu().numpy(), out.tempered_logprob.cpu().numpy(),
            out.sampling_logprob.cpu().numpy())


def oracle_of(z, o):
    return S.sample(z, o.temperature, o.top_k, o.top_p, o.seed, o.offset, o.masked)


def close(a, b, bound=KERNEL_REFERENCE):
    both_nan = np.isnan(a) & np.isnan(b)
    return np.all(both_nan | (np.abs(a - b) <= bound * np.maximum(1.0, np.abs(b))))


OPTIONS = [
    ("plain", SampleOptions(seed=1, offset=2)),
    ("greedy", SampleOptions.greedy()),
    ("temperature 0.7", SampleOptions(temperature=0.7, seed=3)),
    ("top-k 50", SampleOptions(top_k=50, seed=4, offset=2 ** 33 + 5)),
    ("top-p 0.9", SampleOptions(top_p=0.9, seed=2 ** 40 + 7)),
    ("top-k 20, top-p 0.8, T 1.3", SampleOptions(temperature=1.3, top_k=20, top_p=0.8, seed=6)),
    ("top-p 0", SampleOptions(top_p=0.0, seed=7)),
    ("top-p 1e-6", SampleOptions(top_p=1e-6, seed=8)),
    ("masked", SampleOptions(masked=(0, 3, 2, 3), seed=9)),
    ("masked, top-k 3, T 0.5", SampleOptions(temperature=0.5, top_k=3, masked=(1, 4), seed=10)),
    ("cold", SampleOptions(temperature=1e-6, seed=11)),
]


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("dims", [(3, 5), (4, 1000), (2, 32003), (2, 151936)], ids=lambda d: f"{d[0]}x{d[1]}")
@pytest.mark.parametrize("name,options", OPTIONS, ids=[o[0] for o in OPTIONS])
def test_kernel_against_the_reference_form(name, options, dims, dtype):
    z = logits_of(*dims, dtype, 100 + dims[1])
    got, want = run(z, dtype, options), oracle_of(z, options)
    # The same tokens - but for a draw decided inside the last places of f32 (the device's and the
    # host's logarithms differ by an ulp): there the two scores must be that close.
    for r in np.nonzero(got[0] != want[0])[0]:
        tau = float(S.inverse_temperature(options.temperature))
        g = S.gumbel_of_inputs(S.row_inputs(options.seed, options.offset, int(r), dims[1]))
        score = (z[r] - z[r].max()) * tau + g
        assert abs(score[got[0][r]] - score[want[0][r]]) <= 4e-6 * max(1.0, abs(score[want[0][r]])), f"row {r}: {got[0][r]} vs {want[0][r]}"
    same = got[0] == want[0]
    for k in (1, 2, 3):
        assert close(got[k][same], want[k][same]), f"{name} output {k}: {got[k]} vs {want[k]}"
    again = run(z, dtype, options)
    for a, b in zip(got, again):
        assert np.array_equal(a, b, equal_nan=True), "two runs differ"


def test_identities_hold_bit_for_bit():
    """crates/dash-contract/src/sample.rs:62-68."""
    z = logits_of(8, 5000, "bf16", 7)
    bits = lambda x: x.view(np.uint32)
    t, lp, tp, sp = run(z, "bf16", SampleOptions(seed=5))
    assert np.array_equal(bits(lp), bits(tp)) and np.array_equal(bits(tp), bits(sp))
    t, lp, tp, sp = run(z, "bf16", SampleOptions(temperature=0.8, seed=5))
    assert np.array_equal(bits(tp), bits(sp)) and not np.array_equal(lp, tp)
    t, lp, tp, sp = run(z, "bf16", SampleOptions(top_k=5000, seed=5))
    assert np.array_equal(bits(lp), bits(sp))
    t, lp, tp, sp = run(z, "bf16", SampleOptions.greedy())
    assert np.array_equal(t, np.argmax(z, axis=1)) and not tp.any() and not sp.any()


def test_offsets_rows_and_seeds_draw_independently():
    z = np.tile(logits_of(1, 2000, "f32", 3, scale=1.0), (64, 1))
    a = run(z, "f32", SampleOptions(seed=1, offset=0))[0]
    assert len(set(a.tolist())) > 40, "the rows of one call draw different numbers"
    b = run(z, "f32", SampleOptions(seed=1, offset=1))[0]
    c = run(z, "f32", SampleOptions(seed=2, offset=0))[0]
    assert np.sum(a != b) >= 56 and np.sum(a != c) >= 56
    assert np.array_equal(run(z, "f32", SampleOptions(seed=1, offset=0), torch.int32)[0], a)


def test_a_row_without_a_finite_logit():
    z = logits_of(3, 40, "f32", 4)
    z[1] = -np.inf
    t, lp, tp, sp = run(z, "f32", SampleOptions(top_k=3, top_p=0.5, masked=(0, 1), seed=2))
    assert t[1] == 2 and np.isnan(lp[1]) and np.isnan(tp[1]) and np.isnan(sp[1])
    assert not np.isnan(lp[[0, 2]]).any()
    z[0, 5] = -np.inf   # a token the model rules out is never drawn
    for offset in range(20):
        assert 5 not in run(np.tile(z[:1], (32, 1)), "f32", SampleOptions(seed=3, offset=offset))[0]


@pytest.mark.parametrize("name,options,kept", [
    ("all", SampleOptions(seed=21), list(range(8))),
    ("T 0.6", SampleOptions(temperature=0.6, seed=22), list(range(8))),
    ("top-k 3 with a tie", SampleOptions(top_k=3, seed=23), [0, 1, 2, 3]),
    ("top-p 0.6", SampleOptions(top_p=0.6, seed=24), None),
    ("masked", SampleOptions(masked=(0,), top_k=2, seed=25), [1, 2, 3]),
])
def test_draws_follow_the_kept_distribution(name, options, kept):
    """tests/sample.rs ``check_distribution``: chi-square of 40 000 draws against the exact
    probabilities over the kept set, at a level a seeded test passes or fails for good."""
    z = np.array([2.0, 1.5, 1.0, 1.0, 0.5, 0.0, -1.0, -2.0], dtype=np.float32)
    n = 40000
    tokens, lp, tp, sp = run(np.tile(z, (n, 1)), "f32", options)
    tau = 1.0 / options.temperature
    counts = np.bincount(tokens, minlength=8)
    drawn = np.nonzero(counts)[0].tolist()
    if kept is None:
        kept = drawn
    assert drawn == kept, f"{name}: drew {drawn}"
    w = np.exp(z[kept].astype(np.float64) * tau)
    prob = w / w.sum()
    chi2 = float(np.sum((counts[kept] - n * prob) ** 2 / (n * prob)))
    df = len(kept) - 1
    bound = df * (1 - 2 / (9 * df) + 3.719016 * np.sqrt(2 / (9 * df))) ** 3 if df > 0 else 1e-9   # Wilson-Hilferty at 1 - 1e-4
    assert chi2 <= bound, f"{name}: chi-square {chi2:.1f} over {df} degrees of freedom (bound {bound:.1f})"
    assert np.max(np.abs(sp - np.log(prob[[kept.index(t) for t in tokens]]))) <= 2e-6


@pytest.mark.parametrize("dims", [(1, 1), (3, 2), (1, 151936), (200, 700)], ids=lambda d: f"{d[0]}x{d[1]}")
def test_smallest_and_widest_calls(dims):
    """One token, two tokens, one row over a cluster of eight blocks, more rows than multiprocessors."""
    z = logits_of(*dims, "bf16", 55)
    for options in (SampleOptions(seed=4), SampleOptions(temperature=0.8, top_k=2, top_p=0.7, seed=4), SampleOptions.greedy()):
        got, want = run(z, "bf16", options), oracle_of(z, options)
        assert np.array_equal(got[0], want[0])
        for k in (1, 2, 3):
            assert close(got[k], want[k])


def test_rows_of_a_wider_buffer():
    """The rows' stride is the caller's: logits that are a slice of a wider tensor are read in place."""
    wide = logits_of(5, 3000, "f16", 56)
    z = np.ascontiguousarray(wide[:, :2048])
    t = torch.from_numpy(wide).to(DEV).to(torch.float16)[:, :2048]
    assert t.stride(0) == 3000
    options = SampleOptions(temperature=0.9, top_p=0.95, seed=11, offset=3)
    out = sample(t, options)
    want = oracle_of(z, options)
    assert np.array_equal(out.tokens.cpu().numpy(), want[0]) and close(out.sampling_logprob.cpu().numpy(), want[3])


def random_calls(count, seed):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(count):
        v = int(rng.choice([7, 64, 257, 1000, 4099, 20000]))
        b = int(rng.integers(1, 6))
        dtype = str(rng.choice(["f32", "bf16", "f16"]))
        masked = tuple(int(x) for x in rng.choice(v, size=int(rng.integers(0, min(v - 1, 6))), replace=False))
        options = SampleOptions(temperature=float(rng.choice([0.0, 0.3, 0.7, 1.0, 1.5, 4.0])), top_k=int(rng.choice([0, 1, 2, 5, 40, v, v + 3])),
                                top_p=float(rng.choice([1.0, 0.99, 0.9, 0.5, 0.1, 0.0])), seed=int(rng.integers(0, 2 ** 62)),
                                offset=int(rng.integers(0, 2 ** 40)), masked=masked)
        scale = float(rng.choice([0.5, 3.0, 10.0]))
        ties = bool(rng.random() < 0.3)
        out.append((f"call {i}: {b}x{v} {dtype} T{options.temperature} k{options.top_k} p{options.top_p} m{len(masked)} scale{scale}{' ties' if ties else ''}",
                    b, v, dtype, options, scale, ties, 5000 + i))
    return out


CALLS = random_calls(60, 20261125)


@pytest.mark.parametrize("name,b,v,dtype,options,scale,ties,seed", CALLS, ids=[c[0] for c in CALLS])
def test_random_calls(name, b, v, dtype, options, scale, ties, seed):
    """A seeded sweep over sizes, dtypes, options and masked ids nobody chose; rows of few distinct values put
    whole groups of ties at the cuts."""
    z = logits_of(b, v, dtype, seed, scale)
    if ties:
        z = round_to(np.round(z * 2) / 2, dtype)
    if v > 10 and seed % 3 == 0:
        z[0, 3:9] = -np.inf   # tokens the model rules out
    got, want = run(z, dtype, options), oracle_of(z, options)
    for r in np.nonzero(got[0] != want[0])[0]:
        tau = float(S.inverse_temperature(options.temperature)) if options.temperature > 0 else 1.0
        g = S.gumbel_of_inputs(S.row_inputs(options.seed, options.offset, int(r), v))
        with np.errstate(invalid="ignore"):
            score = (z[r] - np.max(np.delete(z[r], list(options.masked)))) * tau + g
        assert options.temperature > 0 and abs(score[got[0][r]] - score[want[0][r]]) <= 4e-6 * max(1.0, abs(score[want[0][r]])), f"row {r}: {got[0][r]} vs {want[0][r]}"
    same = got[0] == want[0]
    for k in (1, 2, 3):
        assert close(got[k][same], want[k][same]), f"output {k}: {got[k]} vs {want[k]}"
