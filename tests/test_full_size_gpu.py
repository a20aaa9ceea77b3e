"""The benchmark configurations at their full sizes, where the CPU oracle cannot hold the whole
call: checked through what does not depend on size - single sequences and sampled rows against the
oracle restricted to what they see, exact linearity in the output's gradient, a padded batch against
the same sequences packed, head shards against the whole call."""
import numpy as np
import pytest
import torch

import bench
from dashmag_b200 import attention as A
from dashmag_b200 import sharding
from dashmag_b200.contract import AttentionMask, AttentionOptions
from oracle import attention_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# bf16 results against the f64 oracle: o, lse, dq, dk, dv relative to each part's largest value
# (the bounds of test_kernels_gpu.OWN: one rounding of the dtype plus the rounded P / dS; measured on
# the sequences checked below: 2.7e-3, 1.3e-7, 3.8e-3, 3.4e-3, 3.1e-3).
TOL = [4.2e-3, 4.4e-7, 7.7e-3, 4.6e-3, 5.0e-3]
# A single sampled query is normalised by the largest value of its own row only, which sits well
# under the tensor's: P rounded to bf16 (2^-9 of sum p|v| / l, up to twice the row's largest output
# over ~100 keys) plus the output's own rounding (2^-9).
ROW_TOL = 8.0e-3


def normal(shape, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randn(shape, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)


def host(t):
    return t.float().cpu().numpy()


def rel(got, want):
    return float(np.max(np.abs(got - want)) / max(float(np.max(np.abs(want))), 1e-30))


def packed_case(lens, hq, hkv, seed, window=None):
    t, d = int(sum(lens)), 128
    q, k, v, g = normal((1, t, hq, d), seed), normal((1, t, hkv, d), seed + 1), normal((1, t, hkv, d), seed + 2), normal((1, t, hq, d), seed + 3)
    cu_host = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    cu = torch.tensor(cu_host, dtype=torch.int32, device=DEV)
    options = AttentionOptions.causal_() if window is None else AttentionOptions.causal_().with_window(window, 0)
    return q, k, v, g, cu_host, AttentionMask.packed(cu, cu), options


def check_one_sequence(name, s, cu, q, k, v, g, results, window):
    """Sequence s of the packed call against the oracle run on that sequence alone."""
    a, b = int(cu[s]), int(cu[s + 1])
    sl = lambda x: host(x[:, a:b])
    wo, wl = oracle.forward(sl(q), sl(k), sl(v), causal=True, window=(window, None))
    want = [wo, wl, *oracle.backward(sl(q), sl(k), sl(v), wo, wl, sl(g), causal=True, window=(window, None))]
    for part, got, w, tol in zip("o lse dq dk dv".split(), results, want, TOL):
        err = rel(sl(got), w)
        print(f"{name} sequence {s} ({b - a} tokens) {part}: relative {err:.3e} (tolerance {tol:.1e})")
        assert err <= tol, f"{name} {part}: {err:.3e} > {tol:.1e}"


def check_sampled_rows(name, rows, cu, q, k, v, o, lse, window):
    """Single queries against the oracle over exactly the keys each sees."""
    for i in rows:
        s = int(np.searchsorted(cu, i, side="right") - 1)
        lo = int(cu[s]) if window is None else max(int(cu[s]), i - window)
        wo, wl = oracle.numpy_forward(host(q[:, i:i + 1]), host(k[:, lo:i + 1]), host(v[:, lo:i + 1]))
        eo, el = rel(host(o[:, i:i + 1]), wo), rel(host(lse[:, i:i + 1]), wl)
        assert eo <= ROW_TOL and el <= TOL[1], f"{name} row {i} (keys {lo}..{i}): o {eo:.3e}, lse {el:.3e}"


def run(q, k, v, g, mask, options):
    o, lse = A.attention_with_lse(q, k, v, mask, options)
    return (o, lse) + tuple(A.attention_backward(q, k, v, o, lse, g, mask, options))


def test_config2_packed_causal_gqa_full_size():
    c = bench.TRAIN
    lens = bench.seq_lengths(c["seqs"], c["lo"], c["hi"], c["total"], seed=0)
    q, k, v, g, cu, mask, options = packed_case(lens, c["hq"], c["hkv"], seed=10)
    assert A.kernels_take(q, k, v, mask, options) == 1 and A.kernels_take(q, k, v, mask, options, backward=True) == 1
    res = run(q, k, v, g, mask, options)
    check_one_sequence("config 2", int(np.argmin(lens)), cu, q, k, v, g, res, None)
    longest = int(np.argmax(lens))
    rows = [int(cu[longest]), int(cu[longest]) + 127, int(cu[longest]) + 128, int(cu[longest + 1]) - 1, c["total"] - 1]
    check_sampled_rows("config 2", rows, cu, q, k, v, res[0], res[1], None)
    # Linearity: doubling dO doubles every gradient exactly (a power of two scales every term).
    twice = A.attention_backward(q, k, v, res[0], res[1], g * 2, mask, options)
    for a, b in zip(res[2:], twice):
        assert torch.equal(a.float() * 2, b.float())
    # and the same call again gives the same bits
    again = run(q, k, v, g, mask, options)
    assert all(torch.equal(a, b) for a, b in zip(res, again))


def test_config4_sliding_window_packed_and_padded_full_size():
    """Config 4 both ways the contract can express it: packed offsets with the window in the
    options, and the same sequences as a right-padded batch with a key-padding mask."""
    lens = bench.seq_lengths(16, 1024, 8192, 65536, seed=4)
    window, hq, hkv, d = 4096, 16, 4, 128
    q, k, v, g, cu, mask, options = packed_case(lens, hq, hkv, seed=40, window=window)
    res = run(q, k, v, g, mask, options)
    check_one_sequence("config 4", int(np.argmin(lens)), cu, q, k, v, g, res, window)
    longest = int(np.argmax(lens))
    assert lens[longest] > window + 200
    a = int(cu[longest])
    rows = [a, a + window, a + window + 1, a + window + 130, int(cu[longest + 1]) - 1]
    check_sampled_rows("config 4", rows, cu, q, k, v, res[0], res[1], window)
    del res
    # The padded batch: B = 16, T = max length rounded up, real tokens first.
    tmax = int(-(-int(lens.max()) // 128) * 128)
    pad = lambda x, heads: torch.zeros((16, tmax, heads, d), dtype=x.dtype, device=DEV)
    qb, kb, vb, gb = pad(q, hq), pad(k, hkv), pad(v, hkv), pad(g, hq)
    padding = torch.ones((16, tmax), dtype=torch.bool, device=DEV)
    for s, n in enumerate(lens):
        n, a = int(n), int(cu[s])
        qb[s, :n], kb[s, :n], vb[s, :n], gb[s, :n] = q[0, a:a + n], k[0, a:a + n], v[0, a:a + n], g[0, a:a + n]
        padding[s, :n] = False
    packed = run(q, k, v, g, mask, options)
    # Tq = Tk = tmax: the bottom-right alignment is the identity, so query i is key i as in the packed form.
    batch = run(qb, kb, vb, gb, AttentionMask.key_padding(padding), options)
    for s in (int(np.argmin(lens)), longest, 7):
        n, a = int(lens[s]), int(cu[s])
        for part, p_, b_, tol in zip("o lse dq dk dv".split(), packed, batch, TOL):
            err = rel(host(b_[s:s + 1, :n]), host(p_[:, a:a + n]))
            assert err <= 2 * tol + 1e-6, f"config 4 padded vs packed, sequence {s} {part}: {err:.3e}"
    # padded queries see real keys (padding hides keys, not queries) but padded KEYS get no gradient
    s = int(np.argmin(lens))
    assert torch.all(batch[3][s, int(lens[s]):] == 0) and torch.all(batch[4][s, int(lens[s]):] == 0)


def test_config3_decode_full_size():
    c = bench.DECODE
    rng = np.random.default_rng(77)
    lengths_host = rng.integers(c["lo"], c["hi"] + 1, size=c["b"])
    lengths = torch.tensor(lengths_host, dtype=torch.int32, device=DEV)
    shape = (c["b"], c["s"], c["hkv"], c["d"])
    kc = torch.empty(shape, dtype=torch.bfloat16, device=DEV)
    vc = torch.empty(shape, dtype=torch.bfloat16, device=DEV)
    for i, t in enumerate((kc, vc)):
        for b0 in range(0, c["b"], 8):
            t[b0:b0 + 8] = normal((8,) + shape[1:], 300 + 10 * i + b0)
    q = normal((c["b"], c["hq"], c["d"]), 299)
    for left in (None, 4096):
        options = AttentionOptions() if left is None else AttentionOptions().with_window(left, 0)
        out = A.attention_decode(q, kc, vc, lengths, options)
        for b in (int(np.argmin(lengths_host)), int(np.argmax(lengths_host)), 5):
            n = int(lengths_host[b])
            want = oracle.decode(host(q[b:b + 1]), host(kc[b:b + 1, :n]), host(vc[b:b + 1, :n]), window_left=left)
            got = host(out[b:b + 1])
            slack = 2.0 ** -8 * np.abs(want) * 1.02 + 2e-6 * np.abs(want).max()
            assert np.all(np.abs(got - want) <= slack), f"config 3 sequence {b} ({n} keys, window {left})"
            # the decoding step is attention with one query after every key of the sequence
            one = A.attention(q[b:b + 1].unsqueeze(1), kc[b:b + 1, :n], vc[b:b + 1, :n], AttentionMask.none(), options.with_causal(True))
            assert rel(host(one.reshape(1, c["hq"], c["d"])), want) <= TOL[0]
    del kc, vc


def test_config5_one_kv_head_group_of_the_long_sequence():
    """What one of eight GPUs computes of config 5: T = 131072, one key-value head and its eight
    query heads.  Sampled queries against the oracle over the keys they see; sampled keys' gradients
    from the closed form with the (checked) log-sum-exp and output."""
    t, hq, hkv, d = 131072, 8, 1, 128
    q, k, v, g = normal((1, t, hq, d), 50), normal((1, t, hkv, d), 51), normal((1, t, hkv, d), 52), normal((1, t, hq, d), 53)
    options = AttentionOptions.causal_()
    o, lse = A.attention_with_lse(q, k, v, AttentionMask.none(), options)
    cu = np.array([0, t])
    check_sampled_rows("config 5", [0, 1, 127, 128, 65535, 65536, t - 129, t - 1], cu, q, k, v, o, lse, None)
    dq, dk, dv = A.attention_backward(q, k, v, o, lse, g, AttentionMask.none(), options)
    scale = 1.0 / np.sqrt(d)
    # keys near the end are seen by few queries: dV_j = sum_i P_ij dO_i, dK_j = scale sum_i dS_ij Q_i
    for j in (t - 1, t - 2, t - 70, t - 130):
        rows = slice(j, t)
        qf, gf, of = (host(x[0, rows]).astype(np.float64) for x in (q, g, o))          # [n, Hq, D]
        kj, vj = host(k[0, j, 0]).astype(np.float64), host(v[0, j, 0]).astype(np.float64)
        p = np.exp(np.einsum("nhd,d->nh", qf, kj) * scale - host(lse[0, rows]).astype(np.float64))
        delta = (gf * of).sum(-1)
        ds = p * (np.einsum("nhd,d->nh", gf, vj) - delta)
        want_dv = np.einsum("nh,nhd->d", p, gf)
        want_dk = np.einsum("nh,nhd->d", ds, qf) * scale
        for name, got, want in (("dv", host(dv[0, j, 0]), want_dv), ("dk", host(dk[0, j, 0]), want_dk)):
            err = float(np.max(np.abs(got - want)) / max(np.max(np.abs(want)), 1e-30))
            assert err <= 1.2e-2, f"config 5 key {j} {name}: {err:.3e}"
    # the first query's gradient has one term: dQ_0 = scale dS_00 K_0 with P_00 = 1
    q0 = host(dq[0, 0]).astype(np.float64)
    ds0 = (host(g[0, 0]).astype(np.float64) @ host(v[0, 0, 0]).astype(np.float64)) - (host(g[0, 0]).astype(np.float64) * host(o[0, 0]).astype(np.float64)).sum(-1)
    want = ds0[:, None] * host(k[0, 0, 0]).astype(np.float64)[None] * scale
    assert np.max(np.abs(q0 - want)) <= 8e-3 * max(np.max(np.abs(want)), 1e-3) + 1e-3


def test_head_shards_equal_the_whole_call_to_the_bit():
    """The multi-GPU partition: a rank's key-value heads computed alone (read in place through
    strides) are the same bits as those heads of the whole call - units never interact."""
    lens = [700, 1300, 48, 2048]
    q, k, v, g, cu, mask, options = packed_case(lens, 8, 4, seed=60)
    whole = run(q, k, v, g, mask, options)
    for rank in range(2):
        lq, lk, lv = sharding.shard_heads(q, k, v, rank, 2)
        kv, qh = sharding.head_shards(4, 2, 2)[rank]
        part = run(lq, lk, lv, g[:, :, qh], mask, options)
        assert torch.equal(part[0], whole[0][:, :, qh]) and torch.equal(part[1], whole[1][:, :, qh])
        assert torch.equal(part[2], whole[2][:, :, qh])
        assert torch.equal(part[3], whole[3][:, :, kv]) and torch.equal(part[4], whole[4][:, :, kv])
