"""The rotation kernel against the oracle, bit for bit (crates/dash-mag/src/rope.rs:94-165), and the
appending decoding step with the rotation in front against the same steps taken one by one."""
import numpy as np
import pytest
import torch

from dashmag_b200 import _lib
from dashmag_b200 import attention as A
from dashmag_b200.contract import AttentionOptions
from dashmag_b200.rope import Rope, attention_decode_append_rope
from oracle import attention_oracle as oracle
from oracle import rope_oracle as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TORCH = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
DTYPES = ["f32", "bf16", "f16"]
# features rotated, head dimension: whole head, half of it (the reference's model), shapes too narrow
# or too ragged for 16-byte vectors
SHAPES = [(128, 128), (64, 128), (32, 64), (8, 16), (4, 6), (2, 2), (6, 16)]


def to_dev(x, dtype):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(TORCH[dtype])


def back(t):
    return t.float().cpu().numpy()


def same_bits(got: torch.Tensor, want: np.ndarray):
    g = back(got)
    return np.array_equal(g.view(np.uint32), np.asarray(want, dtype=np.float32).view(np.uint32))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,d", SHAPES)
@pytest.mark.parametrize("inverse", [False, True])
def test_a_range_of_positions(dim, d, dtype, inverse):
    rope = Rope(dim, 10000.0, 64, TORCH[dtype], device=DEV)
    cos, sin = R.tables(dim, 10000.0, 64, dtype)
    x = R.round_to(oracle.seeded((3, 11, 5, d), 900 + d), dtype)
    got = rope.apply_range(to_dev(x, dtype), range(7, 18), inverse=inverse)
    assert same_bits(got, R.apply_range(x, 7, cos, sin, dim, dtype, inverse))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("index", [torch.int32, torch.int64])
def test_one_position_per_sequence(dtype, index):
    """crates/dash-mag/tests/rope.rs:31-43 and :93-108: a token at a time is the range's row, and
    the integers' width does not matter."""
    rope = Rope(64, 10000.0, 512, TORCH[dtype], device=DEV)
    cos, sin = R.tables(64, 10000.0, 512, dtype)
    x = R.round_to(oracle.seeded((6, 8, 128), 910), dtype)
    positions = [0, 511, 17, 17, 300, 1]
    got = rope.apply_at(to_dev(x, dtype), torch.tensor(positions, dtype=index, device=DEV))
    assert same_bits(got, R.apply_at(x, positions, cos, sin, 64, dtype))
    whole = rope.apply_range(to_dev(x[None, :1].repeat(4, axis=1), dtype), range(5, 9))   # [1, 4, 8, 128]
    for t in range(4):
        one = rope.apply_at(to_dev(x[:1], dtype), torch.tensor([5 + t], dtype=index, device=DEV))
        assert torch.equal(one[0], whole[0, t])


@pytest.mark.parametrize("dtype", DTYPES)
def test_query_and_key_in_one_launch(dtype):
    rope = Rope(64, 10000.0, 256, TORCH[dtype], device=DEV)
    cos, sin = R.tables(64, 10000.0, 256, dtype)
    q, k = R.round_to(oracle.seeded((2, 100, 8, 128), 920), dtype), R.round_to(oracle.seeded((2, 100, 2, 128), 921), dtype)
    before = _lib.probe("kernel_launches")
    gq, gk = rope.apply_range(to_dev(q, dtype), range(50, 150), other=to_dev(k, dtype))
    assert _lib.probe("kernel_launches") == before + 1
    assert same_bits(gq, R.apply_range(q, 50, cos, sin, 64, dtype)) and same_bits(gk, R.apply_range(k, 50, cos, sin, 64, dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("index", [torch.int32, torch.int64])
def test_packed_sequences(dtype, index):
    rope = Rope(128, 10000.0, 400, TORCH[dtype], device=DEV)
    cos, sin = R.tables(128, 10000.0, 400, dtype)
    cu = [0, 130, 130, 131, 500, 777]
    x = R.round_to(oracle.seeded((800, 4, 128), 930), dtype)
    k = R.round_to(oracle.seeded((800, 1, 128), 931), dtype)
    cu_dev = torch.tensor(cu, dtype=index, device=DEV)
    got, got_k = rope.apply_packed(to_dev(x, dtype), cu_dev, start=3, other=to_dev(k, dtype))
    assert same_bits(got, R.apply_packed(x, cu, 3, cos, sin, 128, dtype))
    assert same_bits(got_k, R.apply_packed(k, cu, 3, cos, sin, 128, dtype))
    grad = rope.apply_packed(to_dev(x, dtype), cu_dev, start=3, inverse=True)
    assert same_bits(grad, R.apply_packed(x, cu, 3, cos, sin, 128, dtype, inverse=True))


def test_a_position_outside_the_tables_shows():
    """The reference leaves it to the caller and may return garbage (rope.rs:137-140); here the
    rotated features are NaN, the rest passes, and nothing is read out of bounds."""
    rope = Rope(8, 10000.0, 16, torch.float32, device=DEV)
    x = torch.ones((3, 2, 12), device=DEV)
    y = rope.apply_at(x, torch.tensor([15, 16, -1], dtype=torch.int64, device=DEV))
    assert not torch.isnan(y[0]).any()
    assert torch.isnan(y[1:, :, :8]).all() and torch.equal(y[1:, :, 8:], x[1:, :, 8:])


def test_f64_is_not_taken_and_the_dtype_must_match():
    rope = Rope(4, 10000.0, 8, torch.float32, device=DEV)
    with pytest.raises(A.AttentionError, match="under a rotation of"):
        rope.apply_range(torch.zeros((1, 2, 1, 6), dtype=torch.bfloat16, device=DEV), range(3, 5))
    with pytest.raises(A.AttentionError, match="is not floating"):
        Rope(4, 10000.0, 8, torch.float64, device=DEV)


# b, hq, hkv, s, d, features rotated, lengths before the step, window left
STEPS = [
    ("tensor-core pass, half the head rotated", [5, 8, 2, 700, 128], 64, [699, 0, 1, 511, 512], None),
    ("tensor-core pass, window", [3, 16, 2, 1300, 128], 128, [1299, 600, 40], 100),
    ("full cache takes no row", [3, 8, 2, 300, 128], 64, [300, 299, 7], None),
    ("FMA pass: D64", [4, 4, 2, 333, 64], 32, [0, 332, 100, 15], None),
    ("scalar pass: odd head dimension", [2, 4, 2, 90, 40], 20, [89, 30], 10),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,dims,dim,lengths,left", STEPS, ids=[c[0] for c in STEPS])
def test_rotate_append_decode_in_one_call(name, dims, dim, lengths, left, dtype):
    b, hq, hkv, s, d = dims
    rope = Rope(dim, 10000.0, s + 1, TORCH[dtype], device=DEV)
    cos, sin = R.tables(dim, 10000.0, s + 1, dtype)
    q, kn, vn = (R.round_to(oracle.seeded(shape, seed), dtype) for shape, seed in
                 (((b, hq, d), 940), ((b, hkv, d), 941), ((b, hkv, d), 942)))
    k, v = R.round_to(oracle.seeded((b, s, hkv, d), 943), dtype), R.round_to(oracle.seeded((b, s, hkv, d), 944), dtype)
    tq, tkn, tvn, tk, tv = (to_dev(x, dtype) for x in (q, kn, vn, k, v))
    tk2, tv2 = tk.clone(), tv.clone()
    lens = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    options = AttentionOptions() if left is None else AttentionOptions().with_window(left, 0)

    got = attention_decode_append_rope(rope, tq, tkn, tvn, tk, tv, lens, options)
    torch.cuda.synchronize()
    assert _lib.lib().dash_attn_device_status(1) == 0

    # the same steps one by one, through the library: the same bits in the result and in the caches
    rq, rk = rope.apply_at(tq, lens, other=tkn)
    twin = A.attention_decode_append(rq, rk, tvn, tk2, tv2, lens, options)
    assert torch.equal(got, twin) and torch.equal(tk, tk2) and torch.equal(tv, tv2)

    # and against the oracle: rotation to the bit (the row in the cache), the step within the decode's bound
    qr, kr = R.apply_at(q, lengths, cos, sin, dim, dtype), R.apply_at(kn, lengths, cos, sin, dim, dtype)
    after = []
    for bi, n in enumerate(lengths):
        if n < s:
            k[bi, n], v[bi, n] = kr[bi], vn[bi]
        after.append(min(n + 1, s))
    assert same_bits(tk, k) and same_bits(tv, v)
    want = oracle.decode(qr, k, v, lengths=after, window_left=left)
    rounding = {"f32": 2e-6, "bf16": 2.0 ** -8, "f16": 2.0 ** -11}[dtype]
    slack = rounding * np.abs(want) * 1.02 + 2e-6 * np.abs(want).max()
    assert np.all(np.abs(back(got) - want) <= slack), f"{name} {dtype}: {np.max(np.abs(back(got) - want)):.3e}"


def test_other_positions_than_the_lengths():
    """A cache that slides keeps fewer rows than the sequence is long: the rotation then takes its
    positions from the caller, the row still goes where the lengths say."""
    dtype = "bf16"
    rope = Rope(64, 10000.0, 4096, TORCH[dtype], device=DEV)
    q, kn, vn = (to_dev(oracle.seeded(shape, seed), dtype) for shape, seed in (((2, 8, 128), 950), ((2, 2, 128), 951), ((2, 2, 128), 952)))
    k, v = to_dev(oracle.seeded((2, 256, 2, 128), 953), dtype), to_dev(oracle.seeded((2, 256, 2, 128), 954), dtype)
    k2, v2 = k.clone(), v.clone()
    lens = torch.tensor([100, 255], dtype=torch.int32, device=DEV)
    positions = torch.tensor([3000, 4095], dtype=torch.int64, device=DEV)
    got = attention_decode_append_rope(rope, q, kn, vn, k, v, lens, positions=positions)
    rq, rk = rope.apply_at(q, positions, other=kn)
    assert torch.equal(got, A.attention_decode_append(rq, rk, vn, k2, v2, lens)) and torch.equal(k, k2)
