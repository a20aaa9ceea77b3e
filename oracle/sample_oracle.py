"""CPU restatement of the reference's token sampler - TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU leg may import this file; the library never
does.  It follows the definition in crates/dash-contract/src/sample.rs:1-96 as the reference's own
CPU form computes it (crates/dash-ops/src/sample/reference.rs): f32 throughout, the cuts from the
row sorted in descending order (:141-196), every sum a balanced tree of pairs (``tree_sum``
:198-214, ``tree_cumsum`` :216-231), the Gumbel variates from Philox4x32-10 words
(crates/dash-ops/src/sample/philox.rs) in the two-branch form of ``gumbel_of_inputs`` (:255-285).

Pinned by the known answers the reference's tests hold: Random123's three Philox4x32-10 vectors
(philox.rs ``philox_gives_random123s_known_answers``) and the definition's closed forms (kept
sets, identities between the three log-probabilities, greedy = argmax), restated in
tests/test_sample_cpu.py.
"""
from __future__ import annotations

import numpy as np

M0, M1 = 0xD2511F53, 0xCD9E8D57
W0, W1 = 0x9E3779B9, 0xBB67AE85
F32_MAX = np.float32(3.4028234663852886e38)


def philox4x32_10(counter, key) -> np.ndarray:
    """``counter [..., 4]`` and ``key [2]`` (uint32) -> the four words ``[..., 4]`` (philox.rs)."""
    c = [np.asarray(counter, dtype=np.uint64)[..., i] & 0xFFFFFFFF for i in range(4)]
    k0, k1 = int(key[0]) & 0xFFFFFFFF, int(key[1]) & 0xFFFFFFFF
    mask = np.uint64(0xFFFFFFFF)
    for rnd in range(10):
        if rnd > 0:
            k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
        p0 = np.uint64(M0) * c[0]
        p1 = np.uint64(M1) * c[2]
        c = [(p1 >> np.uint64(32)) ^ c[1] ^ np.uint64(k0), p1 & mask, (p0 >> np.uint64(32)) ^ c[3] ^ np.uint64(k1), p0 & mask]
    return np.stack(c, axis=-1).astype(np.uint32)


def gumbel_input(x) -> np.ndarray:
    """philox.rs ``gumbel_input``: ``a = (2y + 1) / 2^33`` as f32, negative for the upper half."""
    x = np.asarray(x, dtype=np.uint32)
    upper = (x >> np.uint32(31)) == 1
    y = np.where(upper, ~x, x).astype(np.uint32)
    a = (((y << np.uint32(1)) | np.uint32(1)).astype(np.float32) * np.float32(2.0 ** -33)).astype(np.float32)
    return np.where(upper, -a, a).astype(np.float32)


def row_inputs(seed: int, offset: int, row: int, v: int) -> np.ndarray:
    """philox.rs ``row_inputs``: counter ``(i / 4, row, offset lo, offset hi)``, word ``i % 4``."""
    key = (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    groups = (v + 3) // 4
    counter = np.zeros((groups, 4), dtype=np.uint64)
    counter[:, 0] = np.arange(groups)
    counter[:, 1] = row
    counter[:, 2] = offset & 0xFFFFFFFF
    counter[:, 3] = (offset >> 32) & 0xFFFFFFFF
    return gumbel_input(philox4x32_10(counter, key).reshape(-1)[:v])


def gumbel_of_inputs(c) -> np.ndarray:
    """reference.rs:255-285 in f32: ``E = -ln a`` below one half; above, ``-ln_1p(-a)`` as
    ``a (6 - a) / (6 - 4a)`` for ``a <= 2^-6`` and ``-ln(w) a / (1 - w)``, ``w = 1 - a``, beyond;
    ``g = -ln E``."""
    f = np.float32
    c = np.asarray(c, dtype=np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        upper = c < 0
        a = np.abs(c)
        e_lower = -np.log(a, dtype=np.float32)
        e_small = (a * ((f(6.0) - a) / (f(6.0) + a * f(-4.0)))).astype(np.float32)
        w = (f(1.0) - a).astype(np.float32)
        one_less_w = (f(1.0) - w).astype(np.float32)
        e_large = ((-np.log(w, dtype=np.float32)) * (a / one_less_w)).astype(np.float32)
        e_upper = np.where(a <= f(2.0 ** -6), e_small, e_large)
        e = np.where(upper, e_upper, e_lower).astype(np.float32)
        return (-np.log(e, dtype=np.float32)).astype(np.float32)


def tree_sum(x) -> np.ndarray:
    """reference.rs:198-214: each row summed in pairs, the pairs' sums in pairs, ... (an odd
    length takes a zero).  ``x [B, V]`` f32 -> ``[B]``."""
    x = np.asarray(x, dtype=np.float32)
    while x.shape[1] > 1:
        if x.shape[1] % 2:
            x = np.concatenate([x, np.zeros((x.shape[0], 1), dtype=np.float32)], axis=1)
        x = (x[:, 0::2] + x[:, 1::2]).astype(np.float32)
    return x[:, 0]


def tree_cumsum(x) -> np.ndarray:
    """reference.rs:216-231: Hillis and Steele's inclusive scan, f32."""
    x = np.array(x, dtype=np.float32)
    shift = 1
    v = x.shape[1]
    while shift < v:
        shifted = np.concatenate([np.zeros((x.shape[0], shift), dtype=np.float32), x[:, :v - shift]], axis=1)
        x = (x + shifted).astype(np.float32)
        shift *= 2
    return x


def inverse_temperature(temperature: float) -> np.float32:
    """crates/dash-ops/src/sample.rs:89-91."""
    with np.errstate(divide="ignore", over="ignore"):
        return min(np.float32(1.0) / np.float32(temperature), F32_MAX)


def kept_mask(zm, m, masked_row, top_k: int, top_p: float, tau) -> np.ndarray | None:
    """reference.rs:141-196: the tokens top-k and top-p keep (``P``), or None when neither cuts."""
    b, v = zm.shape
    unmasked = v - int(masked_row.sum())
    k = top_k if 0 < top_k < unmasked else None
    p = np.float32(top_p) if top_p < 1.0 else None
    if k is None and p is None:
        return None
    order = np.argsort(-zm, axis=1, kind="stable")
    srt = np.take_along_axis(zm, order, axis=1)                       # descending, -inf last
    threshold = srt[:, k - 1:k] if k is not None else None
    if p is not None:
        with np.errstate(invalid="ignore"):
            weights = np.exp(((srt - m) * np.float32(tau)).astype(np.float32), dtype=np.float32)
        weights = np.where(np.isnan(weights), np.float32(0), weights)
        if threshold is not None:
            weights = np.where(srt < threshold, np.float32(0), weights)
        cumulative = tree_cumsum(weights)
        target = (cumulative[:, v - 1:v] * p).astype(np.float32)
        first = np.argmax(cumulative >= target, axis=1)
        threshold = np.take_along_axis(srt, first[:, None], axis=1)
    return (zm >= threshold) & ~masked_row[None, :]


def sample(logits, temperature=1.0, top_k=0, top_p=1.0, seed=0, offset=0, masked=()):
    """crates/dash-contract/src/sample.rs:1-96 as reference.rs:24-139 computes it.  ``logits
    [B, V]`` (values of the input dtype, widened to f32).  Returns ``(tokens int64 [B], logprob,
    tempered_logprob, sampling_logprob)``, the three f32 ``[B]``."""
    z = np.asarray(logits, dtype=np.float32)
    b, v = z.shape
    masked_row = np.zeros(v, dtype=bool)
    masked_row[list(masked)] = True
    ninf = np.float32(-np.inf)
    zm = np.where(masked_row[None, :], ninf, z)
    with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
        m = zm.max(axis=1, keepdims=True)
        s1 = tree_sum(np.nan_to_num(np.exp((zm - m).astype(np.float32), dtype=np.float32), nan=np.nan))
        lse = (m[:, 0] + np.log(s1, dtype=np.float32)).astype(np.float32)
        degenerate = m[:, 0] == ninf
        first_unmasked = np.argmax(~masked_row)
        if temperature == 0.0:
            tokens = np.argmax(zm, axis=1)
            tempered = np.zeros(b, dtype=np.float32)
            sampling = np.zeros(b, dtype=np.float32)
        else:
            tau = inverse_temperature(temperature)
            s = ((zm - m) * tau).astype(np.float32)
            kept = kept_mask(zm, m, masked_row, top_k, top_p, tau)
            noise = gumbel_of_inputs(np.stack([row_inputs(seed, offset, r, v) for r in range(b)]))
            leave_out = ~kept if kept is not None else (np.broadcast_to(masked_row[None, :], (b, v)) if masked_row.any() else None)
            score = (s + noise).astype(np.float32)
            if leave_out is not None:
                score = np.where(leave_out, ninf, score)
            score = np.where(np.isnan(score), ninf, score)
            tokens = np.argmax(score, axis=1)
            weights = np.exp(s, dtype=np.float32)
            s_t = np.take_along_axis(s, tokens[:, None], axis=1)[:, 0]
            tempered = None if tau == 1.0 else (s_t - np.log(tree_sum(weights), dtype=np.float32)).astype(np.float32)
            sampling = None
            if kept is not None:
                sampling = (s_t - np.log(tree_sum(np.where(leave_out, np.float32(0), weights)), dtype=np.float32)).astype(np.float32)
        tokens = np.where(degenerate, first_unmasked, tokens)
        z_t = np.take_along_axis(z, tokens[:, None], axis=1)[:, 0]
        logprob = (z_t - lse).astype(np.float32)
        tempered = logprob.copy() if tempered is None else tempered
        sampling = tempered.copy() if sampling is None else sampling
        nan = np.float32(np.nan)
        tempered = np.where(degenerate, nan, tempered).astype(np.float32)
        sampling = np.where(degenerate, nan, sampling).astype(np.float32)
    return tokens.astype(np.int64), logprob, tempered, sampling
