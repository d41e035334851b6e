"""ctypes front end of the CPU oracle (``liblokal_oracle.so``).

Test infrastructure only: the test suite, the smoke check and the benchmark's
CPU-baseline leg import this module; the shipped package never does. Every
function here forwards to the C++ restatement in ``lokal_oracle.cpp``, whose
comments cite the reference lines each one follows.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liblokal_oracle.so")

F32, F16, Q8_0, Q4_K, BF16 = 0, 1, 8, 12, 30
Q4_0, Q5_0, Q2_K, Q3_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS = 2, 6, 10, 11, 13, 14, 20, 23
QUANT_TYPES = (Q4_0, Q5_0, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS)
IQ2_XXS, IQ2_XS, IQ3_XXS, IQ1_S, IQ3_S, IQ2_S, IQ1_M = 16, 17, 18, 19, 21, 22, 29
GRID_TYPES = (IQ2_XXS, IQ2_XS, IQ3_XXS, IQ1_S, IQ3_S, IQ2_S, IQ1_M)
GRID_ORDER = ("iq2xxs", "iq2xs", "iq2s", "iq3xxs", "iq3s", "iq1s")  # index = the `which` of lokal_ref_set_iq_grid


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (strict-IEEE flags)."""
    src = os.path.join(_HERE, "lokal_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liblokal_oracle.so"], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        vp, f32, sz, i32, i64, u32, u16 = C.c_void_p, C.c_float, C.c_size_t, C.c_int32, C.c_int64, C.c_uint32, C.c_uint16
        sigs = {
            "lokal_ref_f16_to_f32": (f32, [u16]),
            "lokal_ref_f32_to_f16": (u16, [f32]),
            "lokal_ref_bf16_to_f32": (f32, [u16]),
            "lokal_ref_f32_to_bf16": (u16, [f32]),
            "lokal_ref_f32_to_f16_array": (None, [vp, sz, vp]),
            "lokal_ref_f32_to_bf16_array": (None, [vp, sz, vp]),
            "lokal_ref_f16_to_f32_array": (None, [vp, sz, vp]),
            "lokal_ref_bf16_to_f32_array": (None, [vp, sz, vp]),
            "lokal_ref_dot": (f32, [vp, vp, sz]),
            "lokal_ref_rmsnorm": (None, [vp, vp, f32, sz, vp]),
            "lokal_ref_silu": (f32, [f32]),
            "lokal_ref_rope": (None, [vp, sz, sz, sz, f32]),
            "lokal_ref_rope_partial": (None, [vp, sz, sz, sz, sz, f32]),
            "lokal_ref_inv_freq": (None, [f32, sz, vp]),
            "lokal_ref_rope_table": (None, [f32, sz, vp, i64, sz, vp]),
            "lokal_ref_sincos_spellings_agree": (C.c_int, [f32]),
            "lokal_ref_add_rmsnorm_rows": (None, [vp, vp, vp, vp, sz, sz, f32, C.c_int]),
            "lokal_ref_qk_rope_rows": (None, [vp, vp, vp, vp, vp, vp, vp, i64, sz, sz, sz, sz, sz, f32, f32, C.c_int]),
            "lokal_ref_swiglu": (None, [vp, vp, sz, vp, C.c_int]),
            "lokal_ref_sigmoid": (f32, [f32]),
            "lokal_ref_l2norm_rows": (None, [vp, sz, sz, sz, sz, f32]),
            "lokal_ref_gated_output_norm": (None, [vp, vp, vp, sz, sz, f32]),
            "lokal_ref_attn_out_gate": (None, [vp, vp, sz]),
            "lokal_ref_split_q_gate": (None, [vp, vp, vp, sz, sz, sz]),
            "lokal_ref_softplus": (f32, [f32]),
            "lokal_ref_delta_gates": (None, [vp, vp, vp, vp, vp, vp, sz, sz]),
            "lokal_ref_ssm_conv": (None, [vp, vp, vp, vp, sz, sz, sz]),
            "lokal_ref_bf16_to_f16": (None, [vp, sz, vp, vp]),
            "lokal_ref_set_iq_grid": (C.c_int, [C.c_int, vp, sz]),
            "lokal_ref_blk_elems": (sz, [u32]),
            "lokal_ref_blk_bytes": (sz, [u32]),
            "lokal_ref_row_bytes": (sz, [u32, sz]),
            "lokal_ref_dequant_row": (C.c_int, [u32, vp, sz, vp, sz]),
            "lokal_ref_dequant_elem": (f32, [u32, vp, sz]),
            "lokal_ref_embed_gather": (i64, [vp, u32, sz, sz, vp, sz, vp, C.c_int]),
            "lokal_ref_adversarial_rows": (C.c_int, [u32, sz, sz, vp]),
            "lokal_ref_layer_pass": (None, [vp, C.c_int]),
            "lokal_ref_hardware_threads": (C.c_uint, []),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---- conversions -----------------------------------------------------------

def f32_to_f16_bits(x) -> np.ndarray:
    x = _f32c(x)
    out = np.empty(x.shape, np.uint16)
    lib().lokal_ref_f32_to_f16_array(_p(x), x.size, _p(out))
    return out


def f32_to_bf16_bits(x) -> np.ndarray:
    x = _f32c(x)
    out = np.empty(x.shape, np.uint16)
    lib().lokal_ref_f32_to_bf16_array(_p(x), x.size, _p(out))
    return out


def f16_bits_to_f32(b) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    out = np.empty(b.shape, np.float32)
    lib().lokal_ref_f16_to_f32_array(_p(b), b.size, _p(out))
    return out


def bf16_bits_to_f32(b) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    out = np.empty(b.shape, np.float32)
    lib().lokal_ref_bf16_to_f32_array(_p(b), b.size, _p(out))
    return out


# ---- math.rs / model.rs ops --------------------------------------------------

def dot(a, b) -> float:
    a, b = _f32c(a), _f32c(b)
    assert a.size == b.size
    return float(lib().lokal_ref_dot(_p(a), _p(b), a.size))


def rmsnorm(x, w, eps: float) -> np.ndarray:
    """math::rmsnorm(x, weight, eps) -> new vector (one row)."""
    x, w = _f32c(x), _f32c(w)
    assert x.ndim == 1 and x.size == w.size
    y = np.empty_like(x)
    lib().lokal_ref_rmsnorm(_p(x), _p(w), eps, x.size, _p(y))
    return y


def silu(x: float) -> float:
    return float(lib().lokal_ref_silu(x))


def rope(x, pos: int, head_dim: int, theta: float, rot_dim: int | None = None) -> np.ndarray:
    """model::rope on a copy of one row of whole heads; rot_dim < head_dim leaves each head's tail."""
    x = _f32c(x).copy()
    assert x.ndim == 1 and x.size % head_dim == 0
    if rot_dim is None or rot_dim == head_dim:
        lib().lokal_ref_rope(_p(x), x.size, pos, head_dim, theta)
    else:
        lib().lokal_ref_rope_partial(_p(x), x.size, pos, head_dim, rot_dim, theta)
    return x


def inv_freq(theta: float, rot_dim: int) -> np.ndarray:
    out = np.empty(rot_dim // 2, np.float32)
    lib().lokal_ref_inv_freq(theta, rot_dim, _p(out))
    return out


def rope_table(theta: float, rot_dim: int, rows: int, positions=None, pos0: int = 0) -> np.ndarray:
    out = np.empty((rows, rot_dim), np.float32)
    pos = None if positions is None else np.ascontiguousarray(positions, dtype=np.int32)
    lib().lokal_ref_rope_table(theta, rot_dim, _p(pos), pos0, rows, _p(out))
    return out


def add_rmsnorm_rows(x, delta, w, eps: float, threads: int = 1):
    """Returns (x + delta, rmsnorm(x + delta)); delta=None gives (x, rmsnorm(x))."""
    x = _f32c(x).copy()
    rows, dim = x.shape
    d = None if delta is None else _f32c(delta)
    w = _f32c(w)
    xn = np.empty_like(x)
    lib().lokal_ref_add_rmsnorm_rows(_p(x), _p(d), _p(w), _p(xn), rows, dim, eps, threads)
    return x, xn


def qk_rope_rows(q, k, *, n_q_heads, n_kv_heads, head_dim, theta, eps=0.0, rot_dim=None, q_bias=None,
                 k_bias=None, q_norm_w=None, k_norm_w=None, positions=None, pos0=0, threads=1):
    """bias add -> per-head rmsnorm -> rope for every row of q and k (copies returned)."""
    rot_dim = head_dim if rot_dim is None else rot_dim
    q = None if q is None else _f32c(q).copy()
    k = None if k is None else _f32c(k).copy()
    rows = (q if q is not None else k).shape[0]
    pos = None if positions is None else np.ascontiguousarray(positions, dtype=np.int32)
    opt = lambda a: None if a is None else _f32c(a)
    qb, kb, qn, kn = opt(q_bias), opt(k_bias), opt(q_norm_w), opt(k_norm_w)
    lib().lokal_ref_qk_rope_rows(_p(q), _p(k), _p(qb), _p(kb), _p(qn), _p(kn), _p(pos), pos0, rows, n_q_heads,
                                 n_kv_heads, head_dim, rot_dim, eps, theta, threads)
    return q, k


def swiglu(gate, up, threads: int = 1) -> np.ndarray:
    gate, up = _f32c(gate), _f32c(up)
    out = np.empty_like(gate)
    lib().lokal_ref_swiglu(_p(gate), _p(up), gate.size, _p(out), threads)
    return out


# ---- gated-deltanet (qwen35) per-row siblings ---------------------------------

def sigmoid(x: float) -> float:
    return float(lib().lokal_ref_sigmoid(x))


def l2norm_rows(x, dim: int, eps: float, rows_per_token: int | None = None, n_tokens: int = 1, tok_stride: int = 0) -> np.ndarray:
    """x / max(sqrt(sum x^2), eps) per row of `dim`; with n_tokens > 1, row r of token t starts at t*tok_stride + r*dim."""
    x = _f32c(x).copy()
    flat = x.reshape(-1)
    if rows_per_token is None:
        rows_per_token = flat.size // dim
    lib().lokal_ref_l2norm_rows(_p(flat), rows_per_token, n_tokens, tok_stride, dim, eps)
    return x


def gated_output_norm(o, w, z, eps: float) -> np.ndarray:
    """o: [heads, dim], w: [dim], z: [heads, dim] -> rmsnorm(o; w) * silu(z) per head."""
    o, w, z = _f32c(o).copy(), _f32c(w), _f32c(z)
    assert o.shape == z.shape and o.shape[-1] == w.size
    lib().lokal_ref_gated_output_norm(_p(o), _p(w), _p(z), o.size // w.size, w.size, eps)
    return o


def attn_out_gate(attn, gate) -> np.ndarray:
    attn, gate = _f32c(attn).copy(), _f32c(gate)
    assert attn.size == gate.size
    lib().lokal_ref_attn_out_gate(_p(attn), _p(gate), attn.size)
    return attn


def split_q_gate(src, rows: int, heads: int, head_dim: int):
    src = _f32c(src)
    assert src.size == rows * heads * 2 * head_dim
    q = np.empty((rows, heads * head_dim), np.float32)
    gate = np.empty_like(q)
    lib().lokal_ref_split_q_gate(_p(src), _p(q), _p(gate), rows, heads, head_dim)
    return q, gate


def softplus(x: float) -> float:
    return float(lib().lokal_ref_softplus(x))


def delta_gates(alpha, beta_in, a, dt_bias):
    """alpha, beta_in: [n, H_v]; a, dt_bias: [H_v] -> (g, beta), both [n, H_v]."""
    alpha, beta_in, a, dt_bias = _f32c(alpha), _f32c(beta_in), _f32c(a), _f32c(dt_bias)
    assert alpha.shape == beta_in.shape and alpha.shape[-1] == a.size == dt_bias.size
    g, beta = np.empty_like(alpha), np.empty_like(alpha)
    lib().lokal_ref_delta_gates(_p(alpha), _p(beta_in), _p(a), _p(dt_bias), _p(g), _p(beta), a.size, alpha.size // a.size)
    return g, beta


def ssm_conv(state, x, kernel, d_conv: int):
    """conv_step over the rows of x in turn. state: [C, d_conv-1]; x: [n, C]; kernel: [C, d_conv].
    Returns (out [n, C], state after the last token)."""
    state, x, kernel = _f32c(state).copy(), _f32c(x), _f32c(kernel)
    n, ch = x.shape
    assert state.size == ch * (d_conv - 1) and kernel.size == ch * d_conv
    out = np.empty_like(x)
    lib().lokal_ref_ssm_conv(_p(state), _p(x), _p(kernel), _p(out), ch, d_conv, n)
    return out, state


def bf16_to_f16(bits):
    """bf16 bit patterns -> (f16 bit patterns, clip flag)."""
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty_like(bits)
    clip = np.zeros(1, np.uint32)
    lib().lokal_ref_bf16_to_f16(_p(bits), bits.size, _p(out), _p(clip))
    return out, int(clip[0])


# ---- gguf dequant ------------------------------------------------------------

def blk_elems(ty: int) -> int:
    return lib().lokal_ref_blk_elems(ty)


def blk_bytes(ty: int) -> int:
    return lib().lokal_ref_blk_bytes(ty)


def row_bytes(ty: int, n: int) -> int:
    return lib().lokal_ref_row_bytes(ty, n)


def set_iq_grids(grids) -> None:
    """Hands the i-quant codebooks (a mapping with the keys of GRID_ORDER) to the oracle; they are data of the
    format, kept by the caller (src/lowmem/iq_grids.rs in the reference)."""
    for which, key in enumerate(GRID_ORDER):
        a = np.ascontiguousarray(grids[key])
        if lib().lokal_ref_set_iq_grid(which, _p(a), a.size) != 0:
            raise ValueError(f"codebook {key}: {a.size} entries of {a.dtype} is not what the format has")


def dequant_row_ref(ty: int, src, n: int) -> np.ndarray:
    """gguf::dequant_row_ref(ty, src, out[n]); raises where the reference panics."""
    src = np.ascontiguousarray(src, dtype=np.uint8)
    out = np.empty(n, np.float32)
    rc = lib().lokal_ref_dequant_row(ty, _p(src), src.size, _p(out), n)
    if rc == -1:
        raise ValueError(f"src/out size mismatch for ggml type {ty}")
    if rc == -3:
        raise ValueError(f"the codebook of ggml type {ty} has not been set (set_iq_grids)")
    if rc != 0:
        raise ValueError(f"ggml type {ty} is not on this path")
    return out


def dequant_elem(ty: int, row, col: int) -> float:
    row = np.ascontiguousarray(row, dtype=np.uint8)
    return lib().lokal_ref_dequant_elem(ty, _p(row), col)


def dequant_rows_elementwise(ty: int, table, rows: int, cols: int) -> np.ndarray:
    """Whole table through the independent per-element decoder (slow; small cases)."""
    table = np.ascontiguousarray(table, dtype=np.uint8)
    rb = row_bytes(ty, cols)
    out = np.empty((rows, cols), np.float32)
    fn = lib().lokal_ref_dequant_elem
    base = table.ctypes.data
    for r in range(rows):
        for c in range(cols):
            out[r, c] = fn(ty, base + r * rb, c)
    return out


def embed_gather(table, ty: int, vocab: int, dim: int, ids, threads: int = 1) -> np.ndarray:
    table = np.ascontiguousarray(table, dtype=np.uint8)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    assert table.size >= vocab * row_bytes(ty, dim)
    out = np.empty((ids.size, dim), np.float32)
    rc = lib().lokal_ref_embed_gather(_p(table), ty, vocab, dim, _p(ids), ids.size, _p(out), threads)
    if rc > 0:
        raise IndexError(f"token id at index {rc - 1} is out of range for {vocab} rows")
    if rc < 0:
        raise ValueError(f"ggml type {ty} is not on this path")
    return out


def adversarial_rows(ty: int, n_blocks: int, n_rows: int) -> np.ndarray:
    out = np.empty(n_rows * n_blocks * blk_bytes(ty), np.uint8)
    rc = lib().lokal_ref_adversarial_rows(ty, n_blocks, n_rows, _p(out))
    if rc != 0:
        raise ValueError(f"no adversarial generator for ggml type {ty}")
    return out


# ---- timed baseline ------------------------------------------------------------

class LayerPassArgs(C.Structure):
    _fields_ = [
        ("rows", C.c_uint64), ("layers", C.c_uint64), ("hidden", C.c_uint64), ("inter", C.c_uint64),
        ("n_q_heads", C.c_uint64), ("n_kv_heads", C.c_uint64), ("head_dim", C.c_uint64),
        ("eps", C.c_float), ("theta", C.c_float), ("has_bias", C.c_int32), ("has_qk_norm", C.c_int32),
        ("positions", C.c_void_p), ("pos0", C.c_int64),
        ("embed_table", C.c_void_p), ("embed_type", C.c_uint32), ("vocab", C.c_uint64), ("ids", C.c_void_p),
        ("norm_w", C.c_void_p), ("final_w", C.c_void_p), ("q_bias", C.c_void_p), ("k_bias", C.c_void_p),
        ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p),
        ("delta_att", C.c_void_p), ("delta_mlp", C.c_void_p), ("q", C.c_void_p), ("k", C.c_void_p),
        ("gate", C.c_void_p), ("up", C.c_void_p), ("layer_period", C.c_uint64),
        ("out", C.c_void_p), ("sink", C.c_void_p),
    ]


def layer_pass(args: LayerPassArgs, threads: int) -> None:
    lib().lokal_ref_layer_pass(C.byref(args), threads)


def hardware_threads() -> int:
    return int(lib().lokal_ref_hardware_threads()) or (os.cpu_count() or 1)
