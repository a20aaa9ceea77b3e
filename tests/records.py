"""The ten torch records of attention, loaded the way the reference's conformance crate loads
them (crates/dash-conformance/src/attention.rs:133-222): tensors swapped from torch's
``[B,H,T,D]`` into the contract's ``[B,T,H,D]``, the options rebuilt from the metadata (the scale
left to the default where it equals ``1/sqrt(D)``), the mask from ``kind``."""
import json
import math
import pathlib

import numpy as np

from dashmag_b200.contract import AttentionMask, AttentionOptions

GOLDEN = pathlib.Path(__file__).resolve().parent / "golden" / "attention"

#: crates/dash-conformance/src/attention.rs:40
CAUSAL = ["gqa8x2_d256_t40", "gqa6x2_d64_tq24_tk56"]
#: crates/dash-conformance/src/attention.rs:43-52
MASKS = [
    "none_b2_gqa2x1_d64_tq19_tk33",
    "causal_b2_gqa4x2_d64_tq17_tk41",
    "causal_window9_gqa3x1_d64_t40",
    "window6x4_b2_gqa2x1_d64_tq24_tk37",
    "padding_b3_gqa2x1_d64_t29",
    "padding_causal_b2_gqa2x1_d64_t26",
    "packed_causal_gqa2x1_d64",
    "packed_cross_causal_window5_gqa2x1_d64",
]
PARTS = ["o", "lse", "dq", "dk", "dv"]


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def swap_1_2(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(np.swapaxes(x, 1, 2))


class Record:
    def __init__(self, name: str):
        z = np.load(GOLDEN / f"{name}.npz")
        meta = json.loads(str(z["meta"]))
        self.name = name
        self.causal_set = name in CAUSAL
        read_in = lambda part: swap_1_2(bf16_bits_to_f32(z[part]))
        self.q, self.k, self.v, self.grad = read_in("q"), read_in("k"), read_in("v"), read_in("do")
        d = self.q.shape[3]
        scale = float(np.float32(float(meta["scale"])))
        # The causal records carry no `kind`: causal, no mask.
        causal = meta.get("causal", "true") == "true"
        options = AttentionOptions().with_causal(causal)
        if scale != float(np.float32(1.0 / math.sqrt(d))):
            options = options.with_scale(scale)
        left, right = int(meta.get("window_left", -1)), int(meta.get("window_right", -1))
        if left >= 0 or right >= 0:
            side = lambda r: None if r < 0 else r
            options = options.with_window(side(left), side(right))
        kind = meta.get("kind", "none")
        if kind == "none":
            self.mask = AttentionMask.none()
        elif kind == "padding":
            self.mask = AttentionMask.key_padding(z["key_padding"] != 0)
        elif kind == "packed":
            self.mask = AttentionMask.packed(z["cu_seqlens_q"].astype(np.int64), z["cu_seqlens_k"].astype(np.int64))
        else:
            raise ValueError(f"{name}: unknown mask kind {kind}")
        self.options = options
        self.expected = [swap_1_2(z[p].astype(np.float32)) for p in PARTS]

    def oracle_kwargs(self) -> dict:
        """The mask and options as the oracle's keyword arguments."""
        w = self.options.window
        return dict(
            key_padding=self.mask.key_padding_mask,
            cu_q=self.mask.cu_seqlens_q,
            cu_k=self.mask.cu_seqlens_k,
            causal=self.options.causal,
            window=(None, None) if w is None else (w.left, w.right),
            scale=self.options.scale,
        )


def records():
    return [Record(n) for n in CAUSAL + MASKS]


def errors(actual: np.ndarray, expected: np.ndarray):
    """crates/dash-conformance/src/attention.rs:231-249: the largest absolute difference and that
    over the largest reference magnitude, over the entries where the reference is finite; where the
    reference is -inf the result must be -inf, elsewhere finite."""
    assert actual.shape == expected.shape, f"shapes differ: {actual.shape} vs {expected.shape}"
    a = actual.astype(np.float32).ravel()
    e = expected.astype(np.float32).ravel()
    neg = np.isneginf(e)
    assert np.all(np.isneginf(a[neg])), "a value where -inf is expected"
    assert np.all(np.isfinite(a[~neg])), "non-finite value"
    if (~neg).sum() == 0:
        return 0.0, 0.0
    max_abs = float(np.max(np.abs(a[~neg] - e[~neg])))
    max_ref = float(np.max(np.abs(e[~neg])))
    return max_abs, max_abs / max(max_ref, float(np.finfo(np.float32).tiny))


def check_empty_rows(label, o, dq, expected_lse) -> int:
    """:253-279: queries whose reference log-sum-exp is -inf give exactly zero output and query
    gradient; returns how many there are."""
    rows = np.isneginf(expected_lse)
    assert np.all(o[rows] == 0.0), f"{label}: a query that sees no key has a non-zero output"
    if dq is not None:
        assert np.all(dq[rows] == 0.0), f"{label}: a query that sees no key has a non-zero gradient"
    return int(rows.sum())


def check(label, actual, expected, bounds):
    """:288-318: each of o, lse, dq, dk, dv within its bound; returns the relative errors."""
    empty = check_empty_rows(label, actual[0], actual[2], expected[1])
    worst = []
    for name, a, e, bound in zip(PARTS, actual, expected, bounds):
        abs_err, rel = errors(a, e)
        note = f", {empty} queries seeing no key" if name == "lse" and empty else ""
        print(f"{label} {name}: max abs {abs_err:.3e}, relative {rel:.3e} (tolerance {bound:.1e}){note}")
        assert rel <= bound, f"{label} {name}: relative error {rel:.3e} > {bound:.1e}"
        worst.append(rel)
    return worst
