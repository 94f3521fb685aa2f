"""Test helpers: the same synthetic matrix as an oracle matrix (CPU) and as an uploaded device weight."""
import numpy as np

import oxinfer_b200 as ob
from oracle import oracle as O
from oxinfer_b200 import synth

FORMATS = ["mlx4", "q4_k", "q6_k", "q8_0", "f8_e4m3"]
KIND = {"q4_k": O.Q4_K, "q6_k": O.Q6_K, "q8_0": O.Q8_0, "f8_e4m3": O.F8E4M3}


def oracle_matrix(ref, n_out, n_in):
    if isinstance(ref, ob.MlxQ4):
        return O.Matrix.from_mlx_q4(ref.w.reshape(-1), ref.scales.reshape(-1), ref.biases.reshape(-1), n_out, n_in, ref.group)
    return O.Matrix.gguf(ref.kind, ref.data, n_out, n_in, ref.block_scales, ref.bs_rows, ref.bs_cols)


def make_pair(fmt, n_out, n_in, seed):
    """(weight ref, oracle matrix) for a seeded synthetic matrix."""
    ref = synth.make(fmt, n_out, n_in, seed)
    return ref, oracle_matrix(ref, n_out, n_in)


def row_err(y, r):
    return O.row_err(y, r)
