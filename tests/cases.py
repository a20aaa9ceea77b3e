"""Seeded cases shared by the GPU tests: the shapes the reference tests its kernels on
(crates/dash-ops/tests/attention_masks.rs:418-527 ``tiled_cases``, :562-572 ``segment_cases``;
crates/dash-ops/tests/attention.rs:388-447, :528-628), with inputs from the same generator."""
import dataclasses

import numpy as np

from dashmag_b200.contract import AttentionMask, AttentionOptions
from oracle import attention_oracle as oracle


@dataclasses.dataclass
class Case:
    name: str
    q: np.ndarray
    k: np.ndarray
    v: np.ndarray
    grad: np.ndarray
    mask: AttentionMask
    options: AttentionOptions

    def oracle_kwargs(self):
        w = self.options.window
        return dict(key_padding=self.mask.key_padding_mask, cu_q=self.mask.cu_seqlens_q, cu_k=self.mask.cu_seqlens_k,
                    causal=self.options.causal, window=(None, None) if w is None else (w.left, w.right),
                    scale=self.options.scale)


def seeded(name, dims, mask, options, seed) -> Case:
    """dims = [B, Hq, Hkv, Tq, Tk, D] (attention_masks.rs:386-404)."""
    b, hq, hkv, tq, tk, d = dims
    return Case(name, oracle.seeded((b, tq, hq, d), seed), oracle.seeded((b, tk, hkv, d), seed + 1),
                oracle.seeded((b, tk, hkv, d), seed + 2), oracle.seeded((b, tq, hq, d), seed + 3), mask, options)


def offsets(lengths):
    return np.concatenate([[0], np.cumsum(lengths)]).astype(np.int64)


def tiled_cases():
    causal, full = AttentionOptions.causal_(), AttentionOptions()
    padding = oracle.coins(3 * 200, 0.3, 1)
    padding[400:] = True            # the third sequence is all padding
    left_padding = oracle.coins(2 * 170, 0.2, 2)
    left_padding[:37] = True
    left_padding[170:270] = True
    self_lengths = [130, 1, 0, 257, 64, 77]
    q_lengths, k_lengths = [50, 3, 140, 0, 31], [70, 99, 140, 9, 20]
    packed = lambda ql, kl: AttentionMask.packed(offsets(ql), offsets(kl))
    none = AttentionMask.none()
    return [
        seeded("none, Tq < Tk", [2, 8, 2, 200, 333, 128], none, full, 10),
        seeded("causal, window 100", [1, 8, 2, 300, 300, 256], none, causal.with_window(100, 0), 20),
        seeded("window 70 x 45, Tq < Tk", [1, 6, 2, 150, 260, 64], none, full.with_window(70, 45), 30),
        seeded("causal, Tq > Tk", [1, 4, 1, 230, 90, 64], none, causal, 40),
        seeded("causal, Tk - Tq = 30, D64", [1, 4, 2, 98, 128, 64], none, causal, 45),
        seeded("causal, Tk - Tq = 30, D256", [1, 8, 2, 66, 96, 256], none, causal, 46),
        seeded("causal, window 33", [1, 4, 2, 160, 160, 64], none, causal.with_window(33, 0), 47),
        seeded("window 20 x 1", [1, 4, 2, 160, 160, 64], none, full.with_window(20, 1), 48),
        seeded("key padding", [3, 4, 2, 200, 200, 128], AttentionMask.key_padding(padding.reshape(3, 200)), full, 50),
        seeded("key padding, causal, window 50", [2, 8, 2, 170, 170, 256],
               AttentionMask.key_padding(left_padding.reshape(2, 170)), causal.with_window(50, 0), 60),
        seeded("packed, causal", [1, 8, 2, 529, 529, 256], packed(self_lengths, self_lengths), causal, 70),
        seeded("packed, not causal", [1, 4, 4, 529, 529, 64], packed(self_lengths, self_lengths), full, 80),
        seeded("packed cross, causal, window 40", [1, 6, 2, 224, 338, 128], packed(q_lengths, k_lengths),
               causal.with_window(40, 0), 90),
    ]


def tensor_core_cases(d: int = 128):
    """Shapes of the tcgen05 path (bf16 / f16, D = 128; the forward also D = 64) with boundaries
    inside its 128-row tiles."""
    if d != 128:
        return [dataclasses.replace(c, name=c.name.replace("tc ", f"tc D{d} ")) for c in _tensor_core_cases(d)]
    return _tensor_core_cases(d)


def _tensor_core_cases(d: int):
    causal, full = AttentionOptions.causal_(), AttentionOptions()
    lens = [300, 1, 0, 515, 128, 77]
    q_lengths, k_lengths = [150, 3, 260, 0, 131], [170, 299, 260, 9, 120]
    packed = lambda ql, kl: AttentionMask.packed(offsets(ql), offsets(kl))
    pad = oracle.coins(2 * 400, 0.25, 7)
    pad[400 + 300:] = True
    none = AttentionMask.none()
    return [
        seeded("tc causal 1 tile", [1, 4, 2, 128, 128, d], none, causal, 101),
        seeded("tc causal ragged", [2, 4, 1, 333, 333, d], none, causal, 102),
        seeded("tc none, Tq < Tk", [2, 8, 2, 200, 461, d], none, full, 103),
        seeded("tc causal, Tq > Tk", [1, 4, 4, 400, 170, d], none, causal, 104),
        seeded("tc causal, window 100", [1, 8, 2, 700, 700, d], none, causal.with_window(100, 0), 105),
        seeded("tc window 70 x 45", [1, 4, 2, 300, 520, d], none, full.with_window(70, 45), 106),
        seeded("tc packed causal", [1, 8, 2, sum(lens), sum(lens), d], packed(lens, lens), causal, 107),
        seeded("tc packed cross, causal, window 140", [1, 4, 2, sum(q_lengths), sum(k_lengths), d],
               packed(q_lengths, k_lengths), causal.with_window(140, 0), 108),
        seeded("tc key padding, causal", [2, 4, 2, 400, 400, d], AttentionMask.key_padding(pad.reshape(2, 400)), causal, 109),
    ]
