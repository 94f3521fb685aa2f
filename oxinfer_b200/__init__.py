"""oxinfer_b200: a B200 (sm_100a) quantized-matmul engine behind oxinfer's accelerator boundary.

The compute lives in ``libb200qmm.so`` (CUDA kernels + C ABI, sources in ``csrc``); this package is
the thin host-side mirror of the reference's ``Backend`` trait used by the tests and the benchmark.
"""
from ._lib import (BF16, DECLINED, F16, F32, FMT_F8E4M3, FMT_MLX4, FMT_Q4_K, FMT_Q6_K, FMT_Q8_0, LIB_PATH, MODE_ADD, MODE_ADD_GATED,
                   MODE_GELU_PAIR, MODE_SILU_PAIR, MODE_STORE, OK, OTHER_FORMATS, build, exported_names, lib)
from .backend import Backend, BackendError, DeviceWeight, Gguf, Job, MlxQ4, MoeWeights, Q4Matrix, RowsJob

__all__ = [
    "Backend", "BackendError", "DeviceWeight", "Gguf", "Job", "MlxQ4", "MoeWeights", "Q4Matrix", "RowsJob", "build", "lib", "exported_names", "LIB_PATH",
    "FMT_MLX4", "FMT_Q4_K", "FMT_Q6_K", "FMT_Q8_0", "FMT_F8E4M3", "OTHER_FORMATS", "F32", "BF16", "F16", "OK", "DECLINED",
    "MODE_STORE", "MODE_ADD", "MODE_SILU_PAIR", "MODE_GELU_PAIR", "MODE_ADD_GATED",
]
