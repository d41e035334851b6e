"""RoPE table and the fused bias + per-head RMSNorm + rotation through the C ABI vs the CPU oracle.

Bar: max-abs 1e-5 on f32 rows, 2e-3 relative on f16/bf16 rows. The oracle
recomputes powf and sin/cos per head exactly as the reference does; the device
takes powf from the host C library and multiplies by the position in f32, so
the angles are bit-identical and only sin/cos implementations differ.
"""
import numpy as np
import pytest

import synth
from synth import BF16, F16, F32

pytestmark = pytest.mark.gpu

ROPE_HALF_ATOL = 1e-6  # absorbs the f32 sin/cos difference where a*cos - b*sin cancels


def device_table(ctx, dev, theta, rot, rows, positions=None, pos0=0):
    t = dev.empty((rows, rot), F32, fill=9.0)
    dp = None if positions is None else dev.put(np.asarray(positions, np.int32))
    ctx.rope_table(t, theta=theta, rot_dim=rot, rows=rows, positions=dp, pos0=pos0)
    ctx.stream_sync()
    return t


@pytest.mark.parametrize("theta,rot,rows,pos0", [(1e5, 64, 512, 0), (1e6, 64, 300, 1700), (1e6, 128, 257, 7935),
                                                  (1e4, 64, 64, 0), (1e7, 64, 3, 5), (1e4, 2, 5, 3)])
def test_table_matches_libm(ctx, dev, oracle, theta, rot, rows, pos0):
    got = dev.get(device_table(ctx, dev, theta, rot, rows, pos0=pos0))
    ref = oracle.rope_table(theta, rot, rows, pos0=pos0)
    # cos/sin are in [-1, 1]; the accurate device sincosf is within 2 ulp of libm's
    assert np.abs(got - ref).max() <= 5e-7
    assert np.abs(got).max() <= 1.0 + 1e-6 and np.abs(got).max() > 0.5


def test_table_decode_positions(ctx, dev, oracle):
    pos = np.random.default_rng(1).integers(0, 32768, 256, dtype=np.int32)
    got = dev.get(device_table(ctx, dev, 1e4, 64, 256, positions=pos))
    ref = oracle.rope_table(1e4, 64, 256, positions=pos)
    assert np.abs(got - ref).max() <= 5e-7


def run_qk(ctx, dev, cfg, d, rows, *, q_dtype=None, k_dtype=None, rot=None, pos0=0, use_pos_entry=False,
           w_dtype=None, out_of_place=False):
    q_dtype = cfg.dtype if q_dtype is None else q_dtype
    k_dtype = q_dtype if k_dtype is None else k_dtype
    w_dtype = cfg.dtype if w_dtype is None else w_dtype
    rot = cfg.head_dim if rot is None else rot
    dq, dk = dev.put(d["q"], q_dtype), dev.put(d["k"], k_dtype)
    oq = dev.empty(d["q"].shape, q_dtype, fill=0.0) if out_of_place else None
    ok = dev.empty(d["k"].shape, k_dtype, fill=0.0) if out_of_place else None
    opt = lambda name: dev.put(d[name], w_dtype) if name in d else None
    keep = [opt("q_bias"), opt("k_bias"), opt("q_norm_w"), opt("k_norm_w")]
    positions = d.get("positions")
    dpos = None if positions is None else dev.put(positions)
    p = ctx.qk_rope_params(q=dq, k=dk, q_out=oq, k_out=ok, q_bias=keep[0], k_bias=keep[1], q_norm_w=keep[2],
                           k_norm_w=keep[3], rows=rows, n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads,
                           head_dim=cfg.head_dim, rot_dim=rot, eps=cfg.eps, q_dtype=q_dtype, k_dtype=k_dtype,
                           w_dtype=w_dtype)
    if use_pos_entry:
        ctx.qk_rope_pos(p, theta=cfg.theta, positions=dpos, pos0=pos0)
    else:
        table = device_table(ctx, dev, cfg.theta, rot, rows, positions=positions, pos0=pos0)
        p.cos_sin = table.data_ptr()
        ctx.qk_rope(p)
    ctx.stream_sync()
    return dev.get(oq if out_of_place else dq), dev.get(ok if out_of_place else dk)


def oracle_qk(oracle, cfg, d, rot=None, pos0=0):
    return oracle.qk_rope_rows(d["q"], d["k"], n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads,
                               head_dim=cfg.head_dim, theta=cfg.theta, eps=cfg.eps, rot_dim=rot,
                               q_bias=d.get("q_bias"), k_bias=d.get("k_bias"), q_norm_w=d.get("q_norm_w"),
                               k_norm_w=d.get("k_norm_w"), positions=d.get("positions"), pos0=pos0)


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c5"])
@pytest.mark.parametrize("entry", ["table", "positions"])
def test_config_shapes(ctx, dev, oracle, name, entry):
    cfg = synth.CONFIGS[name]
    rows = min(cfg.rows, 301)
    d = synth.layer_inputs(cfg, rows)
    pos0 = 0 if name != "c5" else 7891  # long-context shard: absolute positions of a later block
    q, k = run_qk(ctx, dev, cfg, d, rows, pos0=pos0, use_pos_entry=(entry == "positions"))
    rq, rk = oracle_qk(oracle, cfg, d, pos0=pos0)
    assert np.abs(q - d["q"]).max() > 1e-2, "q did not change: the kernel did not run"
    if cfg.dtype == F32:
        synth.check_f32(q, rq, f"{name} q")
        synth.check_f32(k, rk, f"{name} k")
    else:
        synth.check_half(q, rq, f"{name} q", cfg.dtype, atol=ROPE_HALF_ATOL)
        synth.check_half(k, rk, f"{name} k", cfg.dtype, atol=ROPE_HALF_ATOL)


def test_full_size_decode_batch_positions(ctx, dev, oracle):
    cfg = synth.C3  # 256 sequences at positions up to 32767
    d = synth.layer_inputs(cfg)
    q, k = run_qk(ctx, dev, cfg, d, cfg.rows)
    rq, rk = oracle_qk(oracle, cfg, d)
    synth.check_half(q, rq, "c3 q", F16, atol=ROPE_HALF_ATOL)
    synth.check_half(k, rk, "c3 k", F16, atol=ROPE_HALF_ATOL)
    # same positions in f32: the absolute bar holds out to position 32767
    q32, k32 = run_qk(ctx, dev, cfg, d, cfg.rows, q_dtype=F32, w_dtype=F32)
    synth.check_f32(q32, rq, "c3 q f32")
    synth.check_f32(k32, rk, "c3 k f32")


def lcg_floats(seed, n):
    out = np.empty(n, np.float32)
    s = seed
    for i in range(n):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(s >> 8) / np.float32(1 << 24)) * np.float32(2.0) - np.float32(1.0)
    return out


def test_reference_partial_rope_structure(ctx, dev, oracle):
    # src/gpu/metal.rs:6523-6609: head_dim 256, rot 64, 2 heads, 3 rows, pos0 5, theta 1e7, LCG input.
    hd, rot, nh, rows = 256, 64, 2, 3
    x = lcg_floats(0x0A0B0C0D, rows * nh * hd).reshape(rows, nh * hd)
    dq = dev.put(x)
    table = device_table(ctx, dev, 1e7, rot, rows, pos0=5)
    p = ctx.qk_rope_params(q=dq, rows=rows, n_q_heads=nh, n_kv_heads=0, head_dim=hd, rot_dim=rot, cos_sin=table)
    ctx.qk_rope(p)
    ctx.stream_sync()
    got = dev.get(dq).reshape(rows, nh, hd)
    xin = x.reshape(rows, nh, hd)
    half = rot // 2
    for row in range(rows):
        want = oracle.rope(x[row], 5 + row, hd, 1e7, rot_dim=rot).reshape(nh, hd)
        for h in range(nh):
            a, b = got[row, h, :rot], want[h, :rot]
            rel = np.abs(a - b) / np.maximum(np.maximum(np.abs(a), np.abs(b)), 1e-30)
            assert rel.max() < 1e-5
            moved = (got[row, h, :half].view(np.uint32) != xin[row, h, :half].view(np.uint32)) | \
                    (got[row, h, half:rot].view(np.uint32) != xin[row, h, half:rot].view(np.uint32))
            assert moved.all(), "a pair did not rotate at all"
            # the tail must pass through untouched, bit for bit
            synth.assert_bits_equal(got[row, h, rot:], xin[row, h, rot:], "pass-through tail")
    # and the oracle's partial rope on the prefix equals a full-width rope of that size
    pre = oracle.rope(np.ascontiguousarray(xin[0, 0, :rot]), 5, rot, 1e7)
    synth.assert_bits_equal(pre, oracle.rope(x[0], 5, hd, 1e7, rot_dim=rot)[:rot], "prefix == full rope of rot dims")


@pytest.mark.parametrize("dtype", [F32, F16, BF16])
@pytest.mark.parametrize("hd,rot,nq,nkv", [(64, 64, 9, 3), (128, 128, 16, 8), (256, 256, 3, 1), (80, 80, 4, 2),
                                            (128, 64, 4, 2), (32, 32, 5, 5), (96, 32, 2, 1), (256, 64, 24, 4)])
def test_geometries_with_bias_and_norm(ctx, dev, oracle, dtype, hd, rot, nq, nkv):
    cfg = synth.LayerConfig("t", dtype, 37, 64, 64, nq, nkv, hd, 100, 1e6, 1e-6, 1, qk_bias=True, qk_norm=True,
                            seed=hd * 7 + rot)
    d = synth.layer_inputs(cfg, 37)
    q, k = run_qk(ctx, dev, cfg, d, 37, rot=rot, pos0=1000, w_dtype=F32)
    rq, rk = oracle_qk(oracle, cfg, d, rot=rot, pos0=1000)
    if dtype == F32:
        synth.check_f32(q, rq, "q")
        synth.check_f32(k, rk, "k")
    else:
        synth.check_half(q, rq, "q", dtype, atol=ROPE_HALF_ATOL)
        synth.check_half(k, rk, "k", dtype, atol=ROPE_HALF_ATOL)


def test_reference_gpu_layout_f32_q_with_f16_k(ctx, dev, oracle):
    # q in f32, k in f16 (rows of the KV cache): src/gpu/kernels.metal:2441-2476
    cfg = synth.C2
    d = synth.layer_inputs(cfg, 100)
    d["k"] = synth.round_to(d["k"], F16)
    q, k = run_qk(ctx, dev, cfg, d, 100, q_dtype=F32, k_dtype=F16, w_dtype=F32, pos0=3)
    rq, rk = oracle_qk(oracle, cfg, d, pos0=3)
    synth.check_f32(q, rq, "f32 q")
    synth.check_half(k, rk, "f16 k", F16, atol=ROPE_HALF_ATOL)


def test_out_of_place_and_cache_row_scatter(ctx, dev, oracle):
    cfg = synth.C5
    rows = 64
    d = synth.layer_inputs(cfg, rows)
    q, k = run_qk(ctx, dev, cfg, d, rows, out_of_place=True)
    rq, rk = oracle_qk(oracle, cfg, d)
    synth.check_half(q, rq, "q out of place", BF16, atol=ROPE_HALF_ATOL)
    synth.check_half(k, rk, "k out of place", BF16, atol=ROPE_HALF_ATOL)
    # k rows scattered to cache rows (slot*max_seq + pos), wider cache stride
    cache_rows, stride = 500, cfg.kv_dim + 64
    perm = np.random.default_rng(5).permutation(cache_rows)[:rows].astype(np.uint32)
    cache = dev.empty((cache_rows, stride), BF16, fill=3.0)
    dk = dev.put(d["k"], BF16)
    table = device_table(ctx, dev, cfg.theta, cfg.head_dim, rows)
    dperm, dknw = dev.put(perm), dev.put(d["k_norm_w"], BF16)  # named: the params hold raw addresses only
    p = ctx.qk_rope_params(k=dk, k_out=cache, k_out_rows=dperm, k_out_row_stride=stride, rows=rows,
                           n_q_heads=0, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, eps=cfg.eps,
                           k_norm_w=dknw, q_dtype=BF16, k_dtype=BF16, w_dtype=BF16, cos_sin=table)
    ctx.qk_rope(p)
    ctx.stream_sync()
    got = dev.get(cache)
    synth.check_half(got[perm, :cfg.kv_dim], rk, "scattered k", BF16, atol=ROPE_HALF_ATOL)
    untouched = np.ones(cache_rows, bool)
    untouched[perm] = False
    assert (got[untouched] == 3.0).all() and (got[:, cfg.kv_dim:] == 3.0).all()
    synth.assert_bits_equal(dev.get(dk), d["k"], "source rows stay as they were")


def test_negative_control_adjacent_pairs_fail(ctx, dev, oracle):
    # The classic mistake is rotating adjacent pairs (2i, 2i+1) instead of (i, i+half): the gate must fail on it.
    cfg = synth.C1
    d = synth.layer_inputs(cfg, 16)
    q, _ = run_qk(ctx, dev, cfg, d, 16)
    tab = oracle.rope_table(cfg.theta, 64, 16)
    x = d["q"].reshape(16, cfg.n_q_heads, 32, 2)
    c, s = tab[:, None, :32], tab[:, None, 32:]
    wrong = np.stack([x[..., 0] * c - x[..., 1] * s, x[..., 0] * s + x[..., 1] * c], axis=-1).reshape(16, -1)
    with pytest.raises(AssertionError):
        synth.check_f32(q, wrong.astype(np.float32), "planted bug")


def test_refusals(ctx, dev):
    import lokal_b200 as L
    q = dev.put(np.ones((2, 128), np.float32))
    t = dev.empty((2, 64), F32, fill=0.0)
    base = dict(q=q, rows=2, n_q_heads=2, n_kv_heads=0, head_dim=64, cos_sin=t)
    bad = [
        (dict(base, cos_sin=None), L.capi.ERR_BAD_ARG),
        (dict(base, q=None), L.capi.ERR_BAD_ARG),
        (dict(base, head_dim=63), L.capi.ERR_BAD_ARG),
        (dict(base, rot_dim=66), L.capi.ERR_BAD_ARG),
        (dict(base, q_row_stride=100), L.capi.ERR_BAD_ARG),
        (dict(base, q_dtype=L.Q4_K), L.capi.ERR_UNSUPPORTED),
        (dict(base, q=q.data_ptr() + 1), L.capi.ERR_MISALIGNED),
    ]
    for kw, status in bad:
        with pytest.raises(L.LokalCudaError) as e:
            ctx.qk_rope(ctx.qk_rope_params(**kw))
        assert e.value.status == status, kw
    with pytest.raises(L.LokalCudaError):
        ctx.rope_table(t, theta=1e4, rot_dim=63, rows=2)
    with pytest.raises(L.LokalCudaError):
        ctx.rope_table(t, theta=1e4, rot_dim=64, rows=2, pos0=-1)


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c5"])
def test_large_batches_staged_kernel_equals_register_kernel(ctx, dev, oracle, name, monkeypatch):
    # With enough rows one warp walks a whole row and the row is staged through shared memory by bulk copies;
    # LOKAL_CUDA_ROPE_STAGED=0 keeps the register kernel. Same arithmetic: the two must agree bit for bit,
    # and both must meet the bar against the oracle.
    import dataclasses
    cfg = dataclasses.replace(synth.CONFIGS[name], decode_positions=0)
    rows = 2600
    d = synth.layer_inputs(cfg, rows)
    d.pop("positions", None)
    q1, k1 = run_qk(ctx, dev, cfg, d, rows, pos0=123)
    monkeypatch.setenv("LOKAL_CUDA_ROPE_STAGED", "0")
    q0, k0 = run_qk(ctx, dev, cfg, d, rows, pos0=123)
    monkeypatch.delenv("LOKAL_CUDA_ROPE_STAGED")
    synth.assert_bits_equal(q1, q0, "staged vs register kernel, q")
    synth.assert_bits_equal(k1, k0, "staged vs register kernel, k")
    rq, rk = oracle.qk_rope_rows(d["q"], d["k"], n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                                 theta=cfg.theta, eps=cfg.eps, q_bias=d.get("q_bias"), k_bias=d.get("k_bias"),
                                 q_norm_w=d.get("q_norm_w"), k_norm_w=d.get("k_norm_w"), pos0=123, threads=8)
    if cfg.dtype == F32:
        synth.check_f32(q1, rq, f"{name} q")
        synth.check_f32(k1, rk, f"{name} k")
    else:
        synth.check_half(q1, rq, f"{name} q", cfg.dtype, atol=ROPE_HALF_ATOL)
        synth.check_half(k1, rk, f"{name} k", cfg.dtype, atol=ROPE_HALF_ATOL)


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c5"])
@pytest.mark.parametrize("rows", [1, 37, 700])
def test_small_batches_flat_kernel_equals_register_kernel(ctx, dev, oracle, name, rows, monkeypatch):
    # Few rows take the flat kernel (a warp per row and head group, nothing staged); LOKAL_CUDA_ROPE_FLAT=0 keeps the
    # register kernel with the row split over several warps. Same arithmetic: bit for bit the same, and within the bar.
    cfg = synth.CONFIGS[name]
    d = synth.layer_inputs(cfg, rows)
    q1, k1 = run_qk(ctx, dev, cfg, d, rows, pos0=4000)
    monkeypatch.setenv("LOKAL_CUDA_ROPE_FLAT", "0")
    q0, k0 = run_qk(ctx, dev, cfg, d, rows, pos0=4000)
    monkeypatch.delenv("LOKAL_CUDA_ROPE_FLAT")
    synth.assert_bits_equal(q1, q0, "flat vs register kernel, q")
    synth.assert_bits_equal(k1, k0, "flat vs register kernel, k")
    rq, rk = oracle.qk_rope_rows(d["q"], d["k"], n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                                 theta=cfg.theta, eps=cfg.eps, q_bias=d.get("q_bias"), k_bias=d.get("k_bias"),
                                 q_norm_w=d.get("q_norm_w"), k_norm_w=d.get("k_norm_w"), positions=d.get("positions"), pos0=4000)
    if cfg.dtype == F32:
        synth.check_f32(q1, rq, f"{name} q")
        synth.check_f32(k1, rk, f"{name} k")
    else:
        synth.check_half(q1, rq, f"{name} q", cfg.dtype, atol=ROPE_HALF_ATOL)
        synth.check_half(k1, rk, f"{name} k", cfg.dtype, atol=ROPE_HALF_ATOL)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_qwen35_partial_rope_large_batch(ctx, dev, oracle, dtype, monkeypatch):
    # head_dim 256 with 64 rotated dims, 24 q heads and 4 kv heads, per-head norm: the lane-mapped kernels
    # (staged and register) against the oracle and against each other; on f32 rows the tail of every head must be
    # exactly what the norm alone gives (the reference leaves it untouched, src/gpu/kernels.metal:2401-2425).
    cfg = synth.LayerConfig("q35", dtype, 1500, 64, 64, 24, 4, 256, 100, 1e7, 1e-6, 1, qk_bias=False, qk_norm=True, seed=35)
    rows = 1500
    d = synth.layer_inputs(cfg, rows)
    q1, k1 = run_qk(ctx, dev, cfg, d, rows, rot=64, pos0=77, w_dtype=F32)
    monkeypatch.setenv("LOKAL_CUDA_ROPE_STAGED", "0")
    q0, k0 = run_qk(ctx, dev, cfg, d, rows, rot=64, pos0=77, w_dtype=F32)
    monkeypatch.delenv("LOKAL_CUDA_ROPE_STAGED")
    synth.assert_bits_equal(q1, q0, "staged vs register kernel, q")
    synth.assert_bits_equal(k1, k0, "staged vs register kernel, k")
    rq, rk = oracle_qk(oracle, cfg, d, rot=64, pos0=77)
    if dtype == F32:
        synth.check_f32(q1, rq, "q")
        synth.check_f32(k1, rk, "k")
        # tails: norm only, never rotated. The parallel sum of squares may move the scale by an ulp against the
        # oracle's 8-lane order, so most, not all, tail values are bit-identical; none is further than the f32 bar.
        tail = q1.reshape(rows, 24, 256)[:, :, 64:]
        ref_tail = rq.reshape(rows, 24, 256)[:, :, 64:]
        rel = np.abs(tail - ref_tail) / np.maximum(np.abs(ref_tail), 1e-30)
        assert rel.max() < 4e-7 and (tail.view(np.uint32) == ref_tail.view(np.uint32)).mean() > 0.5
    else:
        synth.check_half(q1, rq, "q", dtype, atol=ROPE_HALF_ATOL)
        synth.check_half(k1, rk, "k", dtype, atol=ROPE_HALF_ATOL)


@pytest.mark.parametrize("dtype,nq,nkv,hd,norm", [(BF16, 40, 7, 128, True), (F32, 20, 3, 256, True), (BF16, 80, 12, 256, True),
                                                   (F32, 40, 7, 128, False)])
def test_rows_that_fill_the_staging_budget(ctx, dev, oracle, dtype, nq, nkv, hd, norm):
    # Rows whose staged size sits at the edge of the 48 KB a kernel gets without opting in (47 head slots of 128 in
    # bf16 with qk-norm: four rows per CTA fit the dynamic part alone, but not together with the staged norm weights):
    # the launcher must count the static part too and pick fewer rows per CTA, or another kernel, never a failed launch.
    cfg = synth.LayerConfig("edge", dtype, 1900, 64, 64, nq, nkv, hd, 100, 1e6, 1e-6, 1, qk_bias=False, qk_norm=norm, seed=47)
    rows = cfg.rows
    d = synth.layer_inputs(cfg, rows)
    q, k = run_qk(ctx, dev, cfg, d, rows, pos0=3)
    rq, rk = oracle.qk_rope_rows(d["q"], d["k"], n_q_heads=nq, n_kv_heads=nkv, head_dim=hd, theta=cfg.theta, eps=cfg.eps,
                                 q_norm_w=d.get("q_norm_w"), k_norm_w=d.get("k_norm_w"), pos0=3, threads=8)
    if dtype == F32:
        synth.check_f32(q, rq, "q")
        synth.check_f32(k, rk, "k")
    else:
        synth.check_half(q, rq, "q", dtype, atol=ROPE_HALF_ATOL)
        synth.check_half(k, rk, "k", dtype, atol=ROPE_HALF_ATOL)


@pytest.mark.parametrize("name", ["c2", "c5"])
@pytest.mark.parametrize("rows", [37, 3000])
def test_l2_priority_of_the_table_changes_no_bit(ctx, dev, name, rows, monkeypatch):
    # The cos/sin table is loaded with the high L2 eviction priority (tables of up to 32 MB);
    # LOKAL_CUDA_ROPE_TABLE_KEEP=0 turns it off. A cache hint may not change a result: flat, staged and register
    # kernels (37 rows take the flat one, 3000 the staged one), bit for bit.
    cfg = synth.CONFIGS[name]
    d = synth.layer_inputs(cfg, rows)
    q1, k1 = run_qk(ctx, dev, cfg, d, rows, pos0=123)
    monkeypatch.setenv("LOKAL_CUDA_ROPE_TABLE_KEEP", "0")
    q0, k0 = run_qk(ctx, dev, cfg, d, rows, pos0=123)
    monkeypatch.delenv("LOKAL_CUDA_ROPE_TABLE_KEEP")
    synth.assert_bits_equal(q1, q0, "q with and without the L2 priority of the table")
    synth.assert_bits_equal(k1, k0, "k with and without the L2 priority of the table")
