"""The decoding step that appends the new key / value row on its way (dash_attn_decode_append):
the same result as writing the row first (crates/dash-mag/src/tensor.rs:732-744) and decoding
with the lengths plus one (crates/dash-ops/src/attention.rs:732-760), and the caches changed in
exactly that row."""
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

# b, hq, hkv, s, d, lengths before the step, window left
CASES = [
    ("tensor-core pass: group 4, D128", [5, 8, 2, 700, 128], [699, 0, 1, 511, 512], None),
    ("tensor-core pass, window", [3, 16, 2, 1300, 128], [1299, 600, 40], 100),
    ("full cache takes no row", [3, 8, 2, 300, 128], [300, 1000, 299], None),
    ("FMA pass: D64", [4, 4, 2, 333, 64], [0, 332, 100, 15], None),
    ("tensor-core pass: D64, group 8", [3, 16, 2, 700, 64], [699, 0, 350], None),
    ("tensor-core pass: D64, window", [2, 8, 2, 1300, 64], [1299, 40], 100),
    ("tensor-core pass: D256 over warp pairs", [3, 8, 2, 900, 256], [899, 0, 450], None),
    ("tensor-core pass: group of 32", [2, 32, 1, 800, 128], [799, 400], None),
    ("tensor-core pass: group of 3", [2, 6, 2, 500, 128], [499, 7], 64),
    ("FMA pass: group 2, D128", [2, 4, 2, 520, 128], [519, 77], 64),
    ("scalar pass: odd head dimension", [2, 4, 2, 90, 40], [89, 30], 10),
]


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("name,dims,lengths,left", CASES, ids=[c[0] for c in CASES])
def test_append_then_decode_equals_write_then_decode(name, dims, lengths, left, dtype):
    b, hq, hkv, s, d = dims
    q, k, v = oracle.seeded((b, hq, d), 700), oracle.seeded((b, s, hkv, d), 701), oracle.seeded((b, s, hkv, d), 702)
    kn, vn = oracle.seeded((b, hkv, d), 703), oracle.seeded((b, hkv, d), 704)
    dt = TORCH[dtype]
    to = lambda x: torch.from_numpy(x).to(DEV).to(dt)
    tq, tk, tv, tkn, tvn = to(q), to(k), to(v), to(kn), to(vn)
    back = lambda t: t.float().cpu().numpy()
    # what the oracle sees: the inputs as rounded to the dtype, the rows written, the lengths advanced
    qh, kh, vh, knh, vnh = back(tq), back(tk), back(tv), back(tkn), back(tvn)
    after = []
    for bi, n in enumerate(lengths):
        n = max(n, 0)
        if n < s:
            kh[bi, n], vh[bi, n] = knh[bi], vnh[bi]
        after.append(min(n + 1, s))
    options = AttentionOptions() if left is None else AttentionOptions().with_window(left, 0)
    k_before, v_before = tk.clone(), tv.clone()
    got = A.attention_decode_append(tq, tkn, tvn, tk, tv, torch.tensor(lengths, dtype=torch.int32, device=DEV), options)
    torch.cuda.synchronize()
    assert _lib.lib().dash_attn_device_status(1) == 0
    want = oracle.decode(qh, kh, vh, lengths=after, window_left=left)
    slack = ROUNDING[dtype] * np.abs(want) * 1.02 + 2e-6 * np.abs(want).max()
    assert np.all(np.abs(back(got) - want) <= slack), f"{name} {dtype}: {np.max(np.abs(back(got) - want)):.3e}"
    # the caches: the new rows where they belong, to the bit, and nothing else touched
    assert np.array_equal(back(tk), kh) and np.array_equal(back(tv), vh)
    changed = (tk != k_before).flatten(2).any(-1) | (tv != v_before).flatten(2).any(-1)   # [B, S]
    for bi, n in enumerate(lengths):
        rows = set(torch.nonzero(changed[bi]).flatten().tolist())
        assert rows <= ({max(n, 0)} if max(n, 0) < s else set()), f"{name}: sequence {bi} changed rows {sorted(rows)}"
    # the same step as two calls gives the same bits
    twin = A.attention_decode(tq, tk, tv, torch.tensor(after, dtype=torch.int32, device=DEV), options)
    assert torch.equal(twin, got)


def test_append_needs_lengths():
    q = torch.zeros((1, 4, 128), dtype=torch.bfloat16, device=DEV)
    k = torch.zeros((1, 8, 2, 128), dtype=torch.bfloat16, device=DEV)
    n = torch.zeros((1, 2, 128), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError, match="the lengths are needed"):
        A.attention_decode_append(q, n, n, k, k.clone(), None)
    with pytest.raises(ValueError, match="new_key must be"):
        A.attention_decode_append(q, n[:, :1], n, k, k.clone(), torch.tensor([3], dtype=torch.int32, device=DEV))
