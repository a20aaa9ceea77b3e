"""Regenerates tests/golden/attention/*.npz from the reference's recorded fixtures.

The reference pins attention at its boundary with ten records of torch's
``scaled_dot_product_attention`` (MATH backend, float64 or fp32, CPU, explicit boolean mask):
``crates/dash-ops/tests/fixtures/attention/*.safetensors``, read by
``crates/dash-conformance/src/fixtures.rs:36-89`` and listed in
``crates/dash-conformance/src/attention.rs:40-52``.  Those files are data, not source; this script
re-encodes them as ``.npz`` so that the tests need neither the reference checkout nor the
``safetensors`` package at run time.

Layout of each ``.npz`` (torch order ``[B, H, T, D]``, exactly as recorded):
  q, k, v, do      uint16   the bf16 bit patterns of the inputs and of the output's cotangent
  o, lse, dq, dk, dv  float32  torch's results
  cu_seqlens_q/k   int64    packed records only
  key_padding      uint8    padding records only (non-zero = key left out)
  meta             str      JSON of the record's metadata (scale, causal, window_left/right, kind)

Run from anywhere:  python tests/golden/make_golden.py <root of the reference checkout>
"""
import json
import pathlib
import sys

import numpy as np
import torch
from safetensors import safe_open

HERE = pathlib.Path(__file__).resolve().parent


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <root of the reference checkout>")
    root = pathlib.Path(sys.argv[1])
    src = root / "crates" / "dash-ops" / "tests" / "fixtures" / "attention"
    out = HERE / "attention"
    out.mkdir(parents=True, exist_ok=True)
    for path in sorted(src.glob("*.safetensors")):
        arrays = {}
        with safe_open(str(path), "pt") as f:
            meta = dict(f.metadata())
            for key in f.keys():
                t = f.get_tensor(key)
                if t.dtype == torch.bfloat16:
                    arrays[key] = t.view(torch.int16).numpy().view(np.uint16)
                else:
                    arrays[key] = t.numpy()
        arrays["meta"] = np.array(json.dumps(meta, sort_keys=True))
        np.savez_compressed(out / (path.stem + ".npz"), **arrays)
        print(path.stem, {k: v.shape for k, v in arrays.items() if k != "meta"})


if __name__ == "__main__":
    main()
