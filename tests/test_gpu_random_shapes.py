"""Seeded random sweep over shapes, types and flags of the four ops through the C ABI, against the CPU oracle.

The parametrised tests pin the shapes someone thought of; this file draws the rest: row counts on both sides of the
kernels' dispatch thresholds (multiples of the SM count), widths that are not multiples of the vector width, every
storage / weight type combination, bias and per-head norm on or off, partial rotation, in-place or not. Every case is
reproducible from its seed, which the assertion message carries. Same bars as the other parity tests."""
import numpy as np
import pytest

import gguf_np
import synth
from synth import BF16, F16, F32

pytestmark = pytest.mark.gpu

DTYPES = (F32, F16, BF16)
SM = 148
# row counts around the points where the launch shape changes (warp-per-row norm from 32 rows per SM, staged rope from
# 12 rows per SM), plus small and ragged ones
ROW_EDGES = (1, 2, 3, 7, 31, 33, 255, 257, SM * 12 - 1, SM * 12, SM * 12 + 5, SM * 32 - 1, SM * 32, SM * 32 + 9)


def pick_rows(rng, cap):
    r = int(rng.choice(ROW_EDGES)) if rng.random() < 0.6 else int(rng.integers(1, cap))
    return min(r, cap)


@pytest.mark.parametrize("seed", range(28))
def test_norm_random_case(ctx, dev, oracle, seed):
    rng = np.random.default_rng(0x4E4F524D + seed)
    dtype, w_dtype = int(rng.choice(DTYPES)), int(rng.choice(DTYPES))
    dim = int(rng.choice((8, 64, 128, 576, 896, 1024, 2048, 4096))) if rng.random() < 0.5 else int(rng.integers(1, 5000))
    rows = pick_rows(rng, max(1, min(5000, (24 << 20) // (dim * 4))))
    fused, in_place = bool(rng.random() < 0.6), bool(rng.random() < 0.3)
    eps = float(rng.choice((1e-5, 1e-6)))
    what = f"seed {seed}: rows {rows} dim {dim} dtype {dtype} w {w_dtype} fused {fused} in_place {in_place}"
    x = synth.round_to((rng.standard_normal((rows, dim)) * rng.uniform(0.1, 4)).astype(np.float32), dtype)
    dl = synth.round_to(rng.standard_normal((rows, dim)).astype(np.float32), dtype)
    w = synth.round_to((1 + 0.1 * rng.standard_normal(dim)).astype(np.float32), w_dtype)
    dx, dw = dev.put(x, dtype), dev.put(w, w_dtype)
    dy = dx if (in_place and not fused) else dev.empty((rows, dim), dtype, fill=7.0)
    if fused:
        ctx.add_rmsnorm(dx, dev.put(dl, dtype), dw, dy, rows=rows, dim=dim, eps=eps, dtype=dtype, w_dtype=w_dtype)
    else:
        ctx.rmsnorm(dx, dw, dy, rows=rows, dim=dim, eps=eps, dtype=dtype, w_dtype=w_dtype)
    ctx.stream_sync()
    ref_x, ref_y = oracle.add_rmsnorm_rows(x, dl if fused else None, w, eps)
    if fused:
        synth.assert_bits_equal(dev.get(dx), synth.round_to(ref_x, dtype), what + ": x + delta")
    if dtype == F32:
        synth.check_f32(dev.get(dy), ref_y, what)
    else:
        synth.check_half(dev.get(dy), ref_y, what, dtype, atol=1e-6)


@pytest.mark.parametrize("seed", range(32))
def test_qk_rope_random_case(ctx, dev, oracle, seed):
    rng = np.random.default_rng(0x524F5045 + seed)
    dtype, w_dtype = int(rng.choice(DTYPES)), int(rng.choice(DTYPES))
    hd, rot = ((64, 64), (128, 128), (256, 256), (256, 64), (128, 64))[int(rng.integers(0, 5))]
    if rng.random() < 0.35:  # geometries off the lane-mapped list
        hd = 2 * int(rng.integers(1, 129))
        rot = 2 * int(rng.integers(1, hd // 2 + 1))
    nq, nkv = int(rng.integers(1, 17)), int(rng.integers(1, 9))
    rows = pick_rows(rng, max(1, min(5000, (24 << 20) // ((nq + nkv) * hd * 4))))
    bias, norm = bool(rng.random() < 0.4), bool(rng.random() < 0.5)
    by_position = bool(rng.random() < 0.4)
    pos0 = int(rng.integers(0, 30000))
    theta = float(rng.choice((1e4, 1e5, 1e6, 1e7)))
    cfg = synth.LayerConfig("random", dtype, rows, 64, 64, nq, nkv, hd, 100, theta, 1e-6, 1, qk_bias=bias, qk_norm=norm,
                            decode_positions=32768 if by_position else 0, seed=9000 + seed)
    d = synth.layer_inputs(cfg, rows)
    what = f"seed {seed}: rows {rows} hd {hd} rot {rot} heads {nq}/{nkv} dtype {dtype} w {w_dtype} bias {bias} norm {norm} positions {by_position}"
    dq, dk = dev.put(d["q"], dtype), dev.put(d["k"], dtype)
    opt = lambda name: dev.put(synth.round_to(d[name], w_dtype), w_dtype) if name in d else None
    keep = [opt("q_bias"), opt("k_bias"), opt("q_norm_w"), opt("k_norm_w")]
    for name in ("q_bias", "k_bias", "q_norm_w", "k_norm_w"):
        if name in d:
            d[name] = synth.round_to(d[name], w_dtype)
    positions = d.get("positions")
    dpos = None if positions is None else dev.put(positions)
    p = ctx.qk_rope_params(q=dq, k=dk, q_bias=keep[0], k_bias=keep[1], q_norm_w=keep[2], k_norm_w=keep[3], rows=rows,
                           n_q_heads=nq, n_kv_heads=nkv, head_dim=hd, rot_dim=rot, eps=cfg.eps, q_dtype=dtype, k_dtype=dtype,
                           w_dtype=w_dtype)
    ctx.qk_rope_pos(p, theta=theta, positions=dpos, pos0=pos0)
    ctx.stream_sync()
    rq, rk = oracle.qk_rope_rows(d["q"], d["k"], n_q_heads=nq, n_kv_heads=nkv, head_dim=hd, theta=theta, eps=cfg.eps, rot_dim=rot,
                                 q_bias=d.get("q_bias"), k_bias=d.get("k_bias"), q_norm_w=d.get("q_norm_w"),
                                 k_norm_w=d.get("k_norm_w"), positions=positions, pos0=pos0)
    for got, ref, name in ((dev.get(dq), rq, "q"), (dev.get(dk), rk, "k")):
        if dtype == F32:
            synth.check_f32(got, ref, f"{what}: {name}", atol=2e-5 if (bias or norm) else synth.F32_MAX_ABS)
        else:
            synth.check_half(got, ref, f"{what}: {name}", dtype, atol=2e-3)


@pytest.mark.parametrize("seed", range(16))
def test_swiglu_random_case(ctx, dev, oracle, seed):
    rng = np.random.default_rng(0x5357494C + seed)
    dtype = int(rng.choice(DTYPES))
    n = int(rng.choice((1, 7, 8, 9, 255, 4097, SM * 2048 * 8, SM * 2048 * 8 + 3))) if rng.random() < 0.5 else int(rng.integers(1, 3_000_000))
    in_place = bool(rng.random() < 0.5)
    g = synth.round_to((rng.standard_normal(n) * 3).astype(np.float32), dtype)
    u = synth.round_to((rng.standard_normal(n) * 2).astype(np.float32), dtype)
    dg, du = dev.put(g, dtype), dev.put(u, dtype)
    out = dg if in_place else dev.empty((n,), dtype, fill=7.0)
    ctx.swiglu(dg, du, out, n=n, dtype=dtype)
    ctx.stream_sync()
    ref = oracle.swiglu(g, u)
    what = f"seed {seed}: n {n} dtype {dtype} in_place {in_place}"
    if dtype == F32:
        synth.check_f32(dev.get(out), ref, what)
    else:
        synth.check_half(dev.get(out), ref, what, dtype, atol=1e-6)


@pytest.mark.parametrize("seed", range(30))
def test_gather_random_case(ctx, dev, oracle, seed):
    rng = np.random.default_rng(0x47415448 + seed)
    ty = int(rng.choice(sorted(gguf_np.DECODERS)))
    be = oracle.blk_elems(ty)
    dim = be * int(rng.integers(1, max(2, 4096 // be + 1)))
    vocab = int(rng.integers(1, 3000))
    n = int(rng.choice((1, 2, 31, 1185, 9473))) if rng.random() < 0.5 else int(rng.integers(1, 6000))
    n = min(n, max(1, (48 << 20) // (dim * 4)))
    out_dtype = int(rng.choice(DTYPES))
    table = synth.quant_table(ty, vocab, dim, 7000 + seed)
    ids = rng.integers(0, vocab, n).astype(np.uint32)
    if rng.random() < 0.5:
        ids[rng.integers(0, n, max(1, n // 3))] = ids[0]  # a hot row
    out = dev.empty((n + 1, dim), out_dtype, fill=4.0)
    ctx.embed_gather(dev.put(table), dev.put(ids), out, ggml_type=ty, vocab=vocab, dim=dim, n=n, out_dtype=out_dtype)
    ctx.stream_sync()
    got = dev.get(out)
    what = f"seed {seed}: {gguf_np.NAMES[ty]} vocab {vocab} dim {dim} n {n} out {out_dtype}"
    assert (got[-1] == 4.0).all(), what + ": wrote past the last row"
    want = oracle.embed_gather(table, ty, vocab, dim, ids)
    with np.errstate(over="ignore"):
        synth.assert_bits_equal(got[:-1], synth.round_to(want, out_dtype), what)
