"""Regenerates tests/golden/oracle_small.npz: outputs of the pinned CPU oracle on small seeded cases.

The oracle itself is pinned to the reference by its known-answer hashes (tests/test_oracle_pins.py);
these vectors freeze its matmul results so that a later change of the oracle, of the synthetic
generators or of numpy's random streams is caught, and so that the GPU parity tests have fixed
references that travel without the reference tree.

Run from the repository root:  python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from oracle import oracle as O  # noqa: E402
from oxinfer_b200 import synth  # noqa: E402
from util import FORMATS, make_pair  # noqa: E402

CASES = {"mlx4": (40, 512, 9, 101), "q4_k": (40, 512, 9, 102), "q6_k": (24, 512, 9, 103), "q8_0": (24, 256, 9, 104), "f8_e4m3": (136, 384, 9, 105)}


def main():
    out = {}
    for fmt in FORMATS:
        n_out, n_in, t, seed = CASES[fmt]
        _, m = make_pair(fmt, n_out, n_in, seed)
        x = synth.activations(t, n_in, seed + 1)
        out[f"{fmt}_shape"] = np.array([n_out, n_in, t])
        out[f"{fmt}_seed"] = np.array(seed)
        out[f"{fmt}_deq_fnv"] = np.array(O.fnv_f32(m.dequantize_rows()), dtype=np.uint64)
        out[f"{fmt}_y_prefill"] = m.matmul_prefill(x)
        out[f"{fmt}_y_f64"] = m.matmul_f64(x)
    np.savez_compressed(Path(__file__).parent / "oracle_small.npz", **out)
    print("wrote", Path(__file__).parent / "oracle_small.npz")


if __name__ == "__main__":
    main()
