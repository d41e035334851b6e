"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

No model checkpoint or dataset is involved: the configs name model SHAPES only,
and these generators stand in for the activations a real model would produce
(second distribution parameter read as a standard deviation). One generator
feeds both the oracle and the CUDA library, so there is one source of truth.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

F32, F16, Q8_0, Q4_K, BF16 = 0, 1, 8, 12, 30


@dataclass(frozen=True)
class LayerConfig:
    name: str
    dtype: int          # storage type of activations (lokal_type)
    rows: int           # token rows of one step
    hidden: int
    inter: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    vocab: int
    theta: float
    eps: float
    layers: int
    qk_bias: bool = False
    qk_norm: bool = False
    decode_positions: int = 0   # >0: per-row positions uniform in [0, decode_positions)
    seed: int = 0xB200

    @property
    def q_dim(self) -> int:
        return self.n_q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim


# The five configurations of the benchmark (shapes of SmolLM2-135M, Qwen2.5-0.5B,
# TinyLlama-1.1B, the Qwen2.5-0.5B embedding table, Qwen3-0.6B).
C1 = LayerConfig("smollm2-135m-f32-prefill512", F32, 512, 576, 1536, 9, 3, 64, 49152, 1e5, 1e-5, 30, seed=0xB201)
C2 = LayerConfig("qwen2.5-0.5b-f16-prefill2048", F16, 2048, 896, 4864, 14, 2, 64, 151936, 1e6, 1e-6, 24,
                 qk_bias=True, seed=0xB202)
C3 = LayerConfig("tinyllama-1.1b-f16-decode256", F16, 256, 2048, 5632, 32, 4, 64, 32000, 1e4, 1e-5, 22,
                 decode_positions=32768, seed=0xB203)
C5 = LayerConfig("qwen3-0.6b-bf16-prefill8192", BF16, 8192, 1024, 3072, 16, 8, 128, 151936, 1e6, 1e-6, 28,
                 qk_norm=True, seed=0xB205)
C4_VOCAB, C4_DIM_Q8, C4_DIM_Q4K, C4_IDS, C4_SEED = 151936, 896, 1024, 65536, 0xB204
CONFIGS = {"c1": C1, "c2": C2, "c3": C3, "c5": C5}


def round_to(x: np.ndarray, dtype: int) -> np.ndarray:
    """Round f32 values to what the storage type can hold (returned as f32)."""
    import torch
    if dtype == F32:
        return np.ascontiguousarray(x, np.float32)
    t = torch.from_numpy(np.ascontiguousarray(x, np.float32))
    t = t.to(torch.float16 if dtype == F16 else torch.bfloat16).to(torch.float32)
    return t.numpy()


def layer_inputs(cfg: LayerConfig, rows: int | None = None, layer: int = 0) -> dict:
    """Inputs of one layer's ops for `rows` token rows, as f32 arrays already rounded to cfg.dtype."""
    rows = cfg.rows if rows is None else rows
    rng = np.random.default_rng([cfg.seed, layer])
    n = lambda *shape, s=1.0: (rng.standard_normal(shape, dtype=np.float32) * np.float32(s))
    r = lambda a: round_to(a, cfg.dtype)
    d = {
        "x": r(n(rows, cfg.hidden)),
        "delta": r(n(rows, cfg.hidden)),
        "delta2": r(n(rows, cfg.hidden)),
        "w_norm": r(1.0 + n(cfg.hidden, s=0.1)),
        "w_norm2": r(1.0 + n(cfg.hidden, s=0.1)),
        "q": r(n(rows, cfg.q_dim)),
        "k": r(n(rows, cfg.kv_dim)),
        "gate": r(n(rows, cfg.inter, s=2.0)),
        "up": r(n(rows, cfg.inter, s=2.0)),
    }
    if cfg.qk_bias:
        d["q_bias"] = r(n(cfg.q_dim, s=0.1))
        d["k_bias"] = r(n(cfg.kv_dim, s=0.1))
    if cfg.qk_norm:
        d["q_norm_w"] = r(1.0 + n(cfg.head_dim, s=0.1))
        d["k_norm_w"] = r(1.0 + n(cfg.head_dim, s=0.1))
    if cfg.decode_positions:
        d["positions"] = rng.integers(0, cfg.decode_positions, rows, dtype=np.int32)
    return d


def token_ids_uniform(vocab: int, n: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, vocab, n, dtype=np.uint32)


def token_ids_zipf(vocab: int, n: int, seed: int, a: float = 1.1) -> np.ndarray:
    """n draws from Zipf(a) truncated to `vocab` ranks; rank -> id through a fixed permutation."""
    rng = np.random.default_rng(seed)
    p = np.arange(1, vocab + 1, dtype=np.float64) ** (-a)
    cdf = np.cumsum(p)
    cdf /= cdf[-1]
    ranks = np.searchsorted(cdf, rng.random(n), side="left").clip(0, vocab - 1)
    perm = np.random.default_rng(seed ^ 0x5EED).permutation(vocab).astype(np.uint32)
    return perm[ranks]


def _abs_normal_f16_bytes(rng, n: int, std: float) -> np.ndarray:
    v = np.abs(rng.standard_normal(n, dtype=np.float32) * np.float32(std)).astype(np.float16)
    return v.view(np.uint8).reshape(n, 2)


def q8_0_table(vocab: int, dim: int, seed: int) -> np.ndarray:
    """Q8_0 bytes: per 32-element block an f16 scale |N(0, 0.01)| and int8 quants uniform in [-127, 127]."""
    assert dim % 32 == 0
    rng = np.random.default_rng(seed)
    nb = vocab * dim // 32
    blocks = np.empty((nb, 34), np.uint8)
    blocks[:, :2] = _abs_normal_f16_bytes(rng, nb, 0.01)
    blocks[:, 2:] = rng.integers(-127, 128, (nb, 32), dtype=np.int8).view(np.uint8)
    return blocks.reshape(-1)


def q4_k_table(vocab: int, dim: int, seed: int) -> np.ndarray:
    """Q4_K bytes: per 256-element super-block f16 d and dmin |N(0, 0.01)|, 12 packed scale bytes and 128 nibble bytes uniform."""
    assert dim % 256 == 0
    rng = np.random.default_rng(seed)
    nb = vocab * dim // 256
    blocks = np.empty((nb, 144), np.uint8)
    blocks[:, 0:2] = _abs_normal_f16_bytes(rng, nb, 0.01)
    blocks[:, 2:4] = _abs_normal_f16_bytes(rng, nb, 0.01)
    blocks[:, 4:] = rng.integers(0, 256, (nb, 140), dtype=np.uint8)
    return blocks.reshape(-1)


# (block elements, block bytes, offsets of the f16 scale fields) per GGUF type id
QUANT_GEOMETRY = {2: (32, 18, (0,)), 6: (32, 22, (0,)), 8: (32, 34, (0,)), 10: (256, 84, (80, 82)), 11: (256, 110, (108,)),
                  12: (256, 144, (0, 2)), 13: (256, 176, (0, 2)), 14: (256, 210, (208,)), 20: (32, 18, (0,)), 23: (256, 136, (0,)),
                  # codebook types; IQ1_M (29) has no f16 field, its scale sits in four nibbles
                  16: (256, 66, (0,)), 17: (256, 74, (0,)), 18: (256, 98, (0,)), 19: (256, 50, (0,)), 21: (256, 110, (0,)),
                  22: (256, 82, (0,)), 29: (256, 56, ())}
QUANT_NAMES = {2: "q4_0", 6: "q5_0", 8: "q8_0", 10: "q2_k", 11: "q3_k", 12: "q4_k", 13: "q5_k", 14: "q6_k", 20: "iq4_nl", 23: "iq4_xs",
               16: "iq2_xxs", 17: "iq2_xs", 18: "iq3_xxs", 19: "iq1_s", 21: "iq3_s", 22: "iq2_s", 29: "iq1_m"}


def quant_table(ty: int, vocab: int, dim: int, seed: int) -> np.ndarray:
    """Bytes of a vocab x dim table of any covered block type: uniform random payload, f16 scales |N(0, 0.01)|."""
    be, bb, offs = QUANT_GEOMETRY[ty]
    assert dim % be == 0
    rng = np.random.default_rng(seed)
    nb = vocab * dim // be
    blocks = rng.integers(0, 256, (nb, bb), dtype=np.uint8)
    for off in offs:
        blocks[:, off:off + 2] = _abs_normal_f16_bytes(rng, nb, 0.01)
    if ty == 29:  # the f16 scale spread over the top nibbles of bytes 49, 51, 53, 55
        bits = _abs_normal_f16_bytes(rng, nb, 0.01).view(np.uint16).reshape(nb)
        for k in range(4):
            blocks[:, 49 + 2 * k] = (blocks[:, 49 + 2 * k] & 0x0F) | (((bits >> (4 * k)) & 0x0F) << 4).astype(np.uint8)
    return blocks.reshape(-1)


def f32_table(vocab: int, dim: int, seed: int, std: float = 0.02) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return rng.standard_normal((vocab, dim), dtype=np.float32) * np.float32(std)


# ---- tolerances the path is held to ----------------------------------------

F32_MAX_ABS = 1e-5        # norm / rope / swiglu on f32 rows
# 16-bit rows: |got - ref| <= rtol * |ref| + atol against the UNROUNDED f32 oracle.
# f16 keeps 11 significant bits, so a correctly rounded result is within 2^-11 = 4.9e-4 and the 2e-3 bar applies as
# stated. bf16 keeps 8 significant bits: rounding ALONE costs up to 2^-8 = 3.9e-3 relative, above the stated 2e-3,
# so no bf16-stored result can meet 2e-3 against an f32 reference. For bf16 the bar is therefore "the nearest-even
# bf16 rounding of a value that agrees with the oracle to f32 accuracy": half a bf16 ulp plus 1e-5 of slack for a
# rounding-direction flip caused by the last f32 bits.
HALF_RTOL = {F16: 2e-3, BF16: 2.0 ** -8 + 1e-5}


def check_f32(got: np.ndarray, ref: np.ndarray, what: str, atol: float = F32_MAX_ABS) -> float:
    got = np.asarray(got, np.float32)
    ref = np.asarray(ref, np.float32)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max()) if got.size else 0.0
    assert err <= atol, f"{what}: max abs error {err:.3e} > {atol:.1e}"
    return err


def check_half(got: np.ndarray, ref: np.ndarray, what: str, dtype: int, atol: float = 6e-8) -> float:
    """got: values read back from f16/bf16 storage (as f32); ref: the UNROUNDED f32 oracle on the same rounded inputs."""
    rtol = HALF_RTOL[dtype]
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    excess = np.abs(got - ref) - (rtol * np.abs(ref) + atol)
    worst = float(excess.max()) if got.size else 0.0
    if worst > 0:
        i = int(np.argmax(excess))
        raise AssertionError(f"{what}: element {i}: got {got.flat[i]!r} vs ref {ref.flat[i]!r} "
                             f"(beyond {rtol:.0e} relative + {atol:.0e})")
    rel = np.abs(got - ref) / np.maximum(np.abs(ref), 1e-30)
    return float(rel[np.abs(ref) > 1e-3].max()) if (np.abs(ref) > 1e-3).any() else 0.0


def assert_bits_equal(got: np.ndarray, ref: np.ndarray, what: str) -> None:
    g = np.ascontiguousarray(got)
    r = np.ascontiguousarray(ref)
    assert g.shape == r.shape and g.dtype.itemsize == r.dtype.itemsize, f"{what}: layout differs"
    view = {1: np.uint8, 2: np.uint16, 4: np.uint32}[g.dtype.itemsize]
    gb, rb = g.view(view), r.view(view)
    if not np.array_equal(gb, rb):
        bad = np.flatnonzero(gb.reshape(-1) != rb.reshape(-1))
        i = int(bad[0])
        raise AssertionError(f"{what}: {bad.size} of {gb.size} elements differ bitwise; first at {i}: "
                             f"{gb.reshape(-1)[i]:#x} vs {rb.reshape(-1)[i]:#x}")
