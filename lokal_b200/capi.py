"""ctypes binding of liblokal_cuda.so -- the same C ABI a Rust `-b cuda` backend binds.

The library is the product; this module only declares its symbols. There is no
CPU fallback: if the shared library is missing or a CUDA device cannot be
opened, the call raises.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

# lokal_type (GGUF tensor type ids)
F32, F16, Q8_0, Q4_K, BF16 = 0, 1, 8, 12, 30
Q4_0, Q5_0, Q2_K, Q3_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS = 2, 6, 10, 11, 13, 14, 20, 23
QUANT_TYPES = (Q4_0, Q5_0, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS)
# codebook types: decodable once their codebooks have been handed over (Context.set_iq_grids)
IQ2_XXS, IQ2_XS, IQ3_XXS, IQ1_S, IQ3_S, IQ2_S, IQ1_M = 16, 17, 18, 19, 21, 22, 29
GRID_TYPES = (IQ2_XXS, IQ2_XS, IQ3_XXS, IQ1_S, IQ3_S, IQ2_S, IQ1_M)
GRID_ORDER = ("iq2xxs", "iq2xs", "iq2s", "iq3xxs", "iq3s", "iq1s")  # index = lokal_iq_grid

# lokal_cuda_pass_set_schedule
PASS_SCHEDULE_AUTO, PASS_SCHEDULE_SEQUENTIAL, PASS_SCHEDULE_BRANCHES = 0, 1, 3

# lokal_status
OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_MISALIGNED, ERR_CUDA, ERR_ID_RANGE, ERR_TIMEOUT, ERR_NO_DEVICE = range(8)
ERR_IO, ERR_FORMAT, ERR_NOT_FOUND, ERR_POS_RANGE = 8, 9, 10, 11
KV_ROW_NONE = 0xFFFFFFFF
STATUS_NAMES = {
    OK: "LOKAL_OK", ERR_BAD_ARG: "LOKAL_ERR_BAD_ARG", ERR_UNSUPPORTED: "LOKAL_ERR_UNSUPPORTED",
    ERR_MISALIGNED: "LOKAL_ERR_MISALIGNED", ERR_CUDA: "LOKAL_ERR_CUDA", ERR_ID_RANGE: "LOKAL_ERR_ID_RANGE",
    ERR_TIMEOUT: "LOKAL_ERR_TIMEOUT", ERR_NO_DEVICE: "LOKAL_ERR_NO_DEVICE", ERR_IO: "LOKAL_ERR_IO",
    ERR_FORMAT: "LOKAL_ERR_FORMAT", ERR_NOT_FOUND: "LOKAL_ERR_NOT_FOUND", ERR_POS_RANGE: "LOKAL_ERR_POS_RANGE",
}


class QkRopeParams(C.Structure):
    """Mirror of lokal_qk_rope_params (include/lokal_cuda.h), field for field."""
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("q_out", C.c_void_p), ("k_out", C.c_void_p),
        ("q_bias", C.c_void_p), ("k_bias", C.c_void_p), ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p),
        ("cos_sin", C.c_void_p), ("k_out_rows", C.c_void_p),
        ("rows", C.c_uint64),
        ("n_q_heads", C.c_uint32), ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("rot_dim", C.c_uint32),
        ("q_row_stride", C.c_uint64), ("k_row_stride", C.c_uint64),
        ("q_out_row_stride", C.c_uint64), ("k_out_row_stride", C.c_uint64),
        ("eps", C.c_float),
        ("q_dtype", C.c_int32), ("k_dtype", C.c_int32), ("w_dtype", C.c_int32),
    ]


class KvLayout(C.Structure):
    """Mirror of lokal_kv_layout."""
    _fields_ = [("max_seq", C.c_uint64), ("sink", C.c_uint64), ("sink_pad", C.c_uint64), ("ring", C.c_uint64)]


class GgufTensor(C.Structure):
    """Mirror of lokal_gguf_tensor."""
    _fields_ = [
        ("name", C.c_char_p), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4), ("ggml_type", C.c_int32),
        ("file_offset", C.c_uint64), ("data_offset", C.c_uint64), ("nbytes", C.c_uint64), ("data", C.c_void_p),
    ]


class PassConfig(C.Structure):
    """Mirror of lokal_pass_config."""
    _fields_ = [
        ("max_rows", C.c_uint64),
        ("layers", C.c_uint32), ("hidden", C.c_uint32), ("inter", C.c_uint32), ("n_q_heads", C.c_uint32),
        ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("rot_dim", C.c_uint32),
        ("eps", C.c_float), ("theta", C.c_float),
        ("dtype", C.c_int32), ("w_dtype", C.c_int32), ("has_qk_bias", C.c_int32), ("has_qk_norm", C.c_int32),
        ("embed_type", C.c_int32), ("slots", C.c_uint32),
        ("vocab", C.c_uint64),
    ]


class PassWeights(C.Structure):
    """Mirror of lokal_pass_weights (host pointers)."""
    _fields_ = [
        ("embed_table", C.c_void_p), ("norm_w", C.c_void_p), ("final_w", C.c_void_p), ("q_bias", C.c_void_p),
        ("k_bias", C.c_void_p), ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p),
    ]


class PassInputs(C.Structure):
    """Mirror of lokal_pass_inputs."""
    _fields_ = [
        ("ids", C.c_void_p), ("positions", C.c_void_p), ("pos0", C.c_int64), ("rows", C.c_uint64),
        ("q", C.c_void_p), ("k", C.c_void_p), ("delta_att", C.c_void_p), ("delta_mlp", C.c_void_p),
        ("gate", C.c_void_p), ("up", C.c_void_p),
        ("q_layer_stride", C.c_uint64), ("k_layer_stride", C.c_uint64), ("delta_layer_stride", C.c_uint64),
        ("mlp_layer_stride", C.c_uint64),
    ]


_vp, _sz, _f, _i, _u32, _i64 = C.c_void_p, C.c_size_t, C.c_float, C.c_int, C.c_uint32, C.c_int64
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); every symbol include/lokal_cuda.h declares.
SIGNATURES = {
    "lokal_cuda_create": (_i, [_i, _pp]),
    "lokal_cuda_destroy": (None, [_vp]),
    "lokal_cuda_last_error": (C.c_char_p, [_vp]),
    "lokal_cuda_version": (C.c_char_p, []),
    "lokal_cuda_device_count": (_i, []),
    "lokal_cuda_malloc": (_i, [_vp, _sz, _pp]),
    "lokal_cuda_free": (_i, [_vp, _vp]),
    "lokal_cuda_host_alloc": (_i, [_vp, _sz, _pp]),
    "lokal_cuda_host_free": (_i, [_vp, _vp]),
    "lokal_cuda_memcpy_h2d": (_i, [_vp, _vp, _vp, _vp, _sz]),
    "lokal_cuda_memcpy_d2h": (_i, [_vp, _vp, _vp, _vp, _sz]),
    "lokal_cuda_stream_create": (_i, [_vp, _pp]),
    "lokal_cuda_stream_destroy": (_i, [_vp, _vp]),
    "lokal_cuda_stream_sync": (_i, [_vp, _vp]),
    "lokal_cuda_graph_begin": (_i, [_vp, _vp]),
    "lokal_cuda_graph_end": (_i, [_vp, _vp, _pp]),
    "lokal_cuda_graph_launch": (_i, [_vp, _vp, _vp]),
    "lokal_cuda_graph_destroy": (_i, [_vp, _vp]),
    "lokal_cuda_blk_elems": (_sz, [_i]),
    "lokal_cuda_blk_bytes": (_sz, [_i]),
    "lokal_cuda_row_bytes": (_sz, [_i, _sz]),
    "lokal_cuda_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _f, _i, _i, _i]),
    "lokal_cuda_add_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _f, _i, _i, _i]),
    "lokal_cuda_rope_table": (_i, [_vp, _vp, _f, _u32, _vp, _i64, _sz, _vp]),
    "lokal_cuda_qk_rope": (_i, [_vp, _vp, C.POINTER(QkRopeParams)]),
    "lokal_cuda_qk_rope_pos": (_i, [_vp, _vp, C.POINTER(QkRopeParams), _f, _vp, _i64]),
    "lokal_cuda_qk_rope_pos_noalloc": (_i, [_vp, _vp, C.POINTER(QkRopeParams), _f, _vp, _i64]),
    "lokal_cuda_swiglu": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i]),
    "lokal_cuda_embed_gather": (_i, [_vp, _vp, _vp, _i, _sz, _sz, _vp, _sz, _vp, _i]),
    "lokal_cuda_embed_gather_rmsnorm": (_i, [_vp, _vp, _vp, _i, _sz, _sz, _vp, _sz, _vp, _vp, _vp, _f, _i, _i]),
    "lokal_cuda_dequant_rows": (_i, [_vp, _vp, _i, _vp, _sz, _sz, _vp, _i]),
    "lokal_cuda_window_cfg": (_i, [C.c_uint64, C.c_uint64, C.c_uint64, C.POINTER(KvLayout)]),
    "lokal_cuda_window_slot_of": (C.c_uint64, [C.POINTER(KvLayout), C.c_uint64]),
    "lokal_cuda_window_write_spans": (_i, [C.POINTER(KvLayout), C.c_uint64, C.c_uint64, C.POINTER(C.c_uint64)]),
    "lokal_cuda_kv_rows": (_i, [_vp, _vp, C.POINTER(KvLayout), _vp, _i64, _vp, _u32, _sz, _vp]),
    "lokal_cuda_kv_stage": (_i, [_vp, _vp, _vp, _i, _sz, _vp, _i, _sz, _vp, _sz, _sz]),
    "lokal_cuda_l2norm_rows": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _f, _i]),
    "lokal_cuda_gated_output_norm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _f, _i, _i]),
    "lokal_cuda_attn_out_gate": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _i]),
    "lokal_cuda_split_q_gate": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _i]),
    "lokal_cuda_delta_gates": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz]),
    "lokal_cuda_ssm_conv": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _i, _i]),
    "lokal_cuda_bf16_to_f16_copy": (_i, [_vp, _vp, _vp, _vp, _sz, _vp]),
    "lokal_gguf_open": (_i, [C.c_char_p, C.POINTER(C.c_void_p), C.c_char_p, _sz]),
    "lokal_gguf_close": (None, [_vp]),
    "lokal_gguf_last_error": (C.c_char_p, [_vp]),
    "lokal_gguf_version": (_u32, [_vp]),
    "lokal_gguf_n_tensors": (_sz, [_vp]),
    "lokal_gguf_data_start": (C.c_uint64, [_vp]),
    "lokal_gguf_tensor_at": (_i, [_vp, _sz, C.POINTER(GgufTensor)]),
    "lokal_gguf_find_tensor": (_i, [_vp, C.c_char_p, C.POINTER(GgufTensor)]),
    "lokal_gguf_has_key": (_i, [_vp, C.c_char_p]),
    "lokal_gguf_get_u64": (_i, [_vp, C.c_char_p, C.POINTER(C.c_uint64)]),
    "lokal_gguf_get_f32": (_i, [_vp, C.c_char_p, C.POINTER(C.c_float)]),
    "lokal_gguf_get_str": (_i, [_vp, C.c_char_p, C.POINTER(C.c_char_p), C.POINTER(_sz)]),
    "lokal_gguf_get_arr_i64": (_i, [_vp, C.c_char_p, C.POINTER(C.POINTER(C.c_int64)), C.POINTER(_sz)]),
    "lokal_gguf_get_arr_str": (_i, [_vp, C.c_char_p, C.POINTER(C.POINTER(C.c_char_p)), C.POINTER(_sz)]),
    "lokal_cuda_gguf_upload": (_i, [_vp, _vp, _vp, C.c_char_p, C.POINTER(C.c_void_p), C.POINTER(GgufTensor)]),
    "lokal_cuda_set_iq_grid": (_i, [_vp, _i, _vp, _sz]),
    "lokal_cuda_shard_rows": (_i, [_sz, _i, _i, C.POINTER(_sz), C.POINTER(_sz)]),
    "lokal_cuda_pass_create": (_i, [_vp, C.POINTER(PassConfig), C.POINTER(PassWeights), _pp]),
    "lokal_cuda_pass_destroy": (_i, [_vp, _vp]),
    "lokal_cuda_pass_run_device": (_i, [_vp, _vp, _vp, C.POINTER(PassInputs), _vp]),
    "lokal_cuda_pass_run_host": (_i, [_vp, _vp, C.POINTER(PassInputs), _vp]),
    "lokal_cuda_pass_output": (_i, [_vp, _vp, _u32, _i, _pp]),
    "lokal_cuda_pass_launches": (C.c_uint64, [_vp]),
    "lokal_cuda_pass_set_schedule": (_i, [_vp, _vp, _i]),
    "lokal_cuda_host_rmsnorm": (_i, [_vp, _vp, _vp, _f, _sz, _sz, _vp]),
    "lokal_cuda_host_rope": (_i, [_vp, _vp, _sz, _sz, _sz, _f]),
    "lokal_cuda_host_swiglu": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "lokal_cuda_host_dequant_row": (_i, [_vp, _i, _vp, _sz, _vp, _sz]),
    "lokal_cuda_host_embed_gather": (_i, [_vp, _vp, _i, _sz, _sz, _vp, _sz, _vp]),
}

_lib = None


def library_path() -> str:
    return _build.SO


def load() -> C.CDLL:
    """dlopen liblokal_cuda.so (building it first if the sources are newer) and type every symbol."""
    global _lib
    if _lib is None:
        if _build.needs_build():
            _build.build()
        if not os.path.exists(_build.SO):
            raise RuntimeError("liblokal_cuda.so is missing and could not be built; there is no CPU fallback")
        lib = C.CDLL(_build.SO)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class LokalCudaError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.message = message
