"""A seeded sweep over the decoding step's kernels (tensor-core split pass at D = 64 / 128 / 256 with its
warp pairs and its groups of more than sixteen heads, the FMA pass, the scalar pass), with and without
the appended row: shapes, lengths and windows nobody chose, every case against the f64 oracle within one
rounding of the output dtype, the appending form against write-then-decode to the bit."""
import numpy as np
import pytest
import torch

from dashmag_b200 import _lib
from dashmag_b200 import attention as A
from dashmag_b200.contract import AttentionOptions
from oracle import attention_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TORCH = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
ROUNDING = {"f32": 2e-6, "bf16": 2.0 ** -8, "f16": 2.0 ** -11}


def random_cases(count, seed):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(count):
        d = int(rng.choice([64, 128, 256, 40, 96]))
        hkv = int(rng.choice([1, 2, 3]))
        group = int(rng.choice([1, 2, 3, 4, 7, 8, 16, 17, 33]))
        b = int(rng.integers(1, 5))
        s = int(rng.choice([1, 17, 130, 700, 2100]))
        lengths = [int(x) for x in rng.integers(0, s + 1, size=b)]
        if rng.random() < 0.3:
            lengths[0] = s
        left = None if rng.random() < 0.5 else int(rng.integers(0, s + 10))
        dtype = str(rng.choice(["bf16", "f16", "f32"]))
        out.append((f"decode {i}: b{b} hq{hkv * group} hkv{hkv} s{s} d{d} {dtype} window {left}", [b, hkv * group, hkv, s, d], lengths, left, dtype, 7000 + 11 * i))
    return out


CASES = random_cases(48, 20261125)


@pytest.mark.parametrize("name,dims,lengths,left,dtype,seed", CASES, ids=[c[0] for c in CASES])
def test_random_decode(name, dims, lengths, left, dtype, seed):
    b, hq, hkv, s, d = dims
    q, k, v = oracle.seeded((b, hq, d), seed), oracle.seeded((b, s, hkv, d), seed + 1), oracle.seeded((b, s, hkv, d), seed + 2)
    kn, vn = oracle.seeded((b, hkv, d), seed + 3), oracle.seeded((b, hkv, d), seed + 4)
    to = lambda x: torch.from_numpy(x).to(DEV).to(TORCH[dtype])
    back = lambda t: t.float().cpu().numpy()
    tq, tk, tv, tkn, tvn = to(q), to(k), to(v), to(kn), to(vn)
    qh, kh, vh, knh, vnh = back(tq), back(tk), back(tv), back(tkn), back(tvn)
    options = AttentionOptions() if left is None else AttentionOptions().with_window(left, 0)
    lens = torch.tensor(lengths, dtype=torch.int32, device=DEV)

    got = back(A.attention_decode(tq, tk, tv, lens, options))
    want = oracle.decode(qh, kh, vh, lengths=lengths, window_left=left)
    slack = ROUNDING[dtype] * np.abs(want) * 1.02 + 2e-6 * max(np.abs(want).max(), 1e-30)
    assert np.all(np.abs(got - want) <= slack), f"{name}: {np.max(np.abs(got - want)):.3e}"

    # the appending step: the row written where the lengths say, the result that of write-then-decode, to the bit
    after = []
    for bi, n in enumerate(lengths):
        if n < s:
            kh[bi, n], vh[bi, n] = knh[bi], vnh[bi]
        after.append(min(n + 1, s))
    k2, v2 = tk.clone(), tv.clone()
    appended = A.attention_decode_append(tq, tkn, tvn, k2, v2, lens, options)
    torch.cuda.synchronize()
    assert _lib.lib().dash_attn_device_status(1) == 0
    assert np.array_equal(back(k2), kh) and np.array_equal(back(v2), vh)
    twin = A.attention_decode(tq, k2, v2, torch.tensor(after, dtype=torch.int32, device=DEV), options)
    assert torch.equal(appended, twin)
    want2 = oracle.decode(qh, kh, vh, lengths=after, window_left=left)
    slack2 = ROUNDING[dtype] * np.abs(want2) * 1.02 + 2e-6 * max(np.abs(want2).max(), 1e-30)
    assert np.all(np.abs(back(appended) - want2) <= slack2)
