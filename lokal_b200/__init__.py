"""lokal_b200 -- B200 (sm_100a) kernels for lokal's fused per-token layer ops.

The product is ``liblokal_cuda.so`` (sources in ``csrc/``, C ABI in
``include/lokal_cuda.h``). This package builds it, loads it through ctypes and
offers a thin handle named after the reference's ops. There is no CPU path.
"""
from . import capi
from ._build import build
from .capi import (BF16, F16, F32, IQ4_NL, IQ4_XS, Q2_K, Q3_K, Q4_0, Q4_K, Q5_0, Q5_K, Q6_K, Q8_0, QUANT_TYPES, KvLayout, LokalCudaError,
                   QkRopeParams)
from .gguf import GgufFile
from .ops import (Context, LayerPass, blk_bytes, blk_elems, dtype_id, row_bytes, shard_rows, window_cfg, window_slot_of,
                  window_write_spans)

__all__ = [
    "capi", "build", "Context", "LayerPass", "LokalCudaError", "QkRopeParams", "F32", "F16", "BF16", "Q8_0", "Q4_K",
    "Q4_0", "Q5_0", "Q2_K", "Q3_K", "Q5_K", "Q6_K", "IQ4_NL", "IQ4_XS", "QUANT_TYPES",
    "blk_elems", "blk_bytes", "row_bytes", "shard_rows", "dtype_id", "KvLayout", "window_cfg", "window_slot_of",
    "window_write_spans", "GgufFile",
]
