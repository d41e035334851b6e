"""K/V staging after RoPE: the windowed-store geometry (host, no GPU) and the device kernels that compute cache rows
and narrow + scatter fresh K/V rows into them."""
import numpy as np
import pytest

import lokal_b200 as L
import synth
from synth import BF16, F16, F32


# ---- the reference's geometry, restated in Python from src/lowmem/mod.rs:172-193 and src/lowmem/forward.rs:256-271 ----

def ref_window(w, sink, chunk=512):
    up = lambda v: (v + 127) // 128 * 128
    return dict(w=w, sink=sink, sink_pad=up(sink), ring=up(w + chunk))


def ref_slot_of(win, p):
    return p if p < win["sink"] else win["sink_pad"] + (p - win["sink"]) % win["ring"]


def ref_write_spans(win, pos0, n):
    end, spans = pos0 + n, []
    if pos0 < win["sink"]:
        spans.append((0, pos0, min(win["sink"], end) - pos0))
    p = max(pos0, win["sink"])
    while p < end:
        rel = (p - win["sink"]) % win["ring"]
        ln = min(win["ring"] - rel, end - p)
        spans.append((p - pos0, win["sink_pad"] + rel, ln))
        p += ln
    return spans


@pytest.mark.parametrize("w,sink", [(1024, 4), (4096, 0), (512, 128), (100, 100), (2000, 129)])
def test_window_geometry_matches_the_reference_formulas(w, sink):
    lay = L.window_cfg(w, sink)
    ref = ref_window(w, sink)
    assert (lay.sink, lay.sink_pad, lay.ring) == (ref["sink"], ref["sink_pad"], ref["ring"])
    assert lay.sink_pad % 128 == 0 and lay.ring % 128 == 0 and lay.ring >= w + 512
    for p in list(range(0, 300)) + [sink + lay.ring - 1, sink + lay.ring, sink + 3 * lay.ring + 17, 10 ** 7]:
        assert L.window_slot_of(lay, p) == ref_slot_of(ref, p)
    rng = np.random.default_rng(w + sink)
    for _ in range(200):
        pos0, n = int(rng.integers(0, 5 * lay.ring)), int(rng.integers(1, 513))
        spans = L.window_write_spans(lay, pos0, n)
        assert spans == ref_write_spans(ref, pos0, n) and len(spans) <= 3
        # every position of the chunk is written exactly once, to the row slot_of names
        rows = {}
        for first, slot, ln in spans:
            for i in range(ln):
                assert first + i not in rows
                rows[first + i] = slot + i
        assert sorted(rows) == list(range(n))
        assert all(rows[i] == ref_slot_of(ref, pos0 + i) for i in range(n))


def test_invalid_window_is_refused():
    for w, sink in ((0, 0), (10, 11)):
        with pytest.raises(L.LokalCudaError):
            L.window_cfg(w, sink)
    lin = L.KvLayout(max_seq=100, sink=0, sink_pad=0, ring=0)
    with pytest.raises(L.LokalCudaError):
        L.window_write_spans(lin, 0, 10)
    assert L.window_slot_of(lin, 37) == 37


# ---- device kernels ----

@pytest.mark.gpu
def test_cache_rows_linear_and_windowed(ctx, dev):
    rng = np.random.default_rng(2)
    rows = 777
    pos = rng.integers(0, 32768, rows, dtype=np.int32)
    slots = rng.integers(0, 8, rows).astype(np.uint32)
    out = dev.empty((rows,), F32).view(dev.torch.int32)
    lin = L.KvLayout(max_seq=32768, sink=0, sink_pad=0, ring=0)
    dpos, dslots = dev.put(pos), dev.put(slots.view(np.int32))
    ctx.kv_rows(out, layout=lin, rows=rows, positions=dpos, slots=dslots)
    ctx.stream_sync()
    got = out.cpu().numpy().view(np.uint32)
    assert np.array_equal(got, slots * 32768 + pos.astype(np.uint32))  # (slot*max_seq + pos), src/gpu/kernels.metal:3411
    win = L.window_cfg(1024, 4)
    ctx.kv_rows(out, layout=win, rows=rows, pos0=900, slot0=3)
    ctx.stream_sync()
    got = out.cpu().numpy().view(np.uint32)
    cap = win.sink_pad + win.ring
    want = np.array([3 * cap + L.window_slot_of(win, 900 + r) for r in range(rows)], np.uint32)
    assert np.array_equal(got, want)
    ctx.kv_rows(out, layout=win, rows=rows, positions=dpos, slots=dslots)
    ctx.stream_sync()
    got = out.cpu().numpy().view(np.uint32)
    want = np.array([int(s) * cap + L.window_slot_of(win, int(p)) for p, s in zip(pos, slots)], np.uint32)
    assert np.array_equal(got, want)
    with pytest.raises(L.LokalCudaError):
        ctx.kv_rows(out, layout=L.KvLayout(max_seq=0, sink=0, sink_pad=0, ring=0), rows=rows)


@pytest.mark.gpu
@pytest.mark.parametrize("src,dst", [(F32, F16), (F32, BF16), (F16, F16), (BF16, F32), (F16, F32), (F32, F32)])
@pytest.mark.parametrize("width", [256, 1024, 72, 5])
def test_stage_narrows_and_scatters(ctx, dev, oracle, src, dst, width):
    rng = np.random.default_rng(width + src + dst)
    rows, cache_rows, stride = 301, 2000, width + 8
    v = synth.round_to(rng.standard_normal((rows, width), dtype=np.float32) * 3, src)
    v[0, 0], v[1, 0] = 70000.0 if src == F32 else 100.0, 1e-9 if src == F32 else 0.0  # overflow to inf / underflow in f16
    v = synth.round_to(v, src)
    dest = rng.permutation(cache_rows)[:rows].astype(np.uint32)
    cache = dev.empty((cache_rows, stride), dst, fill=5.0)
    dsrc, drows = dev.put(v, src), dev.put(dest.view(np.int32))
    ctx.kv_stage(dsrc, cache, src_dtype=src, dst_dtype=dst, rows=rows, width=width, dst_row_stride=stride, dst_rows=drows)
    ctx.stream_sync()
    dev.torch.cuda.synchronize()
    got = cache.to(dev.torch.float32).cpu().numpy()
    with np.errstate(over="ignore"):
        want = synth.round_to(v, dst)  # one nearest-even rounding of the source value (f32_to_f16, kernels.metal:2118)
    if dst == F16:
        with np.errstate(over="ignore"):
            bits = oracle.f32_to_f16_bits(v)
        assert np.array_equal(oracle.f16_bits_to_f32(bits).view(np.uint32), want.view(np.uint32))
    synth.assert_bits_equal(got[dest, :width], want, "staged rows")
    untouched = np.ones(cache_rows, bool)
    untouched[dest] = False
    assert (got[untouched] == 5.0).all() and (got[:, width:] == 5.0).all()
    # without an index array the rows land in order
    plain = dev.empty((rows, width), dst, fill=0.0)
    ctx.kv_stage(dsrc, plain, src_dtype=src, dst_dtype=dst, rows=rows, width=width)
    ctx.stream_sync()
    synth.assert_bits_equal(plain.to(dev.torch.float32).cpu().numpy(), want, "in-order rows")


@pytest.mark.gpu
def test_rope_writes_k_into_windowed_cache_rows(ctx, dev, oracle):
    # the index array of kv_rows drives the rope kernel's k output: a chunk that wraps around the ring
    cfg = synth.C5
    rows = 96
    win = L.window_cfg(256, 4, prefill_chunk=128)  # ring = 384
    pos0 = 4 + 384 * 2 - 40                        # the chunk crosses the wrap
    d = synth.layer_inputs(cfg, rows)
    idx = dev.empty((rows,), F32).view(dev.torch.int32)
    ctx.kv_rows(idx, layout=win, rows=rows, pos0=pos0, slot0=1)
    cap = win.sink_pad + win.ring
    cache = dev.empty((2 * cap, cfg.kv_dim), BF16, fill=9.0)
    dk, knw = dev.put(d["k"], BF16), dev.put(d["k_norm_w"], BF16)
    p = ctx.qk_rope_params(k=dk, k_out=cache, k_out_rows=idx, rows=rows, n_q_heads=0, n_kv_heads=cfg.n_kv_heads,
                           head_dim=cfg.head_dim, eps=cfg.eps, k_norm_w=knw, q_dtype=BF16, k_dtype=BF16, w_dtype=BF16)
    ctx.qk_rope_pos(p, theta=cfg.theta, pos0=pos0)
    ctx.stream_sync()
    _, rk = oracle.qk_rope_rows(None, d["k"], n_q_heads=0, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, theta=cfg.theta,
                                eps=cfg.eps, k_norm_w=d["k_norm_w"], pos0=pos0)
    got = cache.to(dev.torch.float32).cpu().numpy()
    want_rows = np.array([cap + L.window_slot_of(win, pos0 + r) for r in range(rows)])
    assert len(L.window_write_spans(win, pos0, rows)) == 2  # the reference would need two spans here
    synth.check_half(got[want_rows], rk, "k rows in the ring", BF16, atol=1e-6)
    mask = np.ones(2 * cap, bool)
    mask[want_rows] = False
    assert (got[mask] == 9.0).all()


@pytest.mark.gpu
def test_stage_refusals(ctx, dev):
    a = dev.empty((4, 8), F32, fill=0.0)
    for kw, status in [(dict(src_dtype=L.Q8_0, dst_dtype=F16), L.capi.ERR_UNSUPPORTED),
                       (dict(src_dtype=F32, dst_dtype=F16, src_row_stride=4), L.capi.ERR_BAD_ARG)]:
        with pytest.raises(L.LokalCudaError) as e:
            ctx.kv_stage(a, a, rows=4, width=8, **kw)
        assert e.value.status == status
    with pytest.raises(L.LokalCudaError):
        ctx.kv_stage(None, a, src_dtype=F32, dst_dtype=F32, rows=4, width=8)
    ctx.kv_stage(a, a, src_dtype=F32, dst_dtype=F32, rows=0, width=8)


@pytest.mark.gpu
def test_bad_positions_are_refused_by_code_and_nothing_is_stored_for_them(ctx, dev, oracle):
    """A negative position, or one at or beyond max_seq in the linear layout (which would land in the next slot's rows or
    past the cache), gets LOKAL_KV_ROW_NONE from kv_rows; kv_stage and the rope's k output store nothing for such a row,
    every other row lands where it belongs, and the next synchronisation returns LOKAL_ERR_POS_RANGE."""
    import torch
    max_seq, slots, width, rows = 64, 3, 128, 10
    lay = L.KvLayout(max_seq=max_seq, sink=0, sink_pad=0, ring=0)
    pos = np.array([0, 5, -1, 63, 64, 10, 1 << 30, 7, -(1 << 31), 20], np.int32)
    slot = np.array([0, 1, 1, 2, 0, 2, 1, 0, 2, 1], np.uint32)
    good = (pos >= 0) & (pos < max_seq)
    idx = dev.empty((rows,), F32).view(torch.int32)
    dpos, dslot = dev.put(pos), dev.put(slot.view(np.int32))
    ctx.kv_rows(idx, layout=lay, rows=rows, positions=dpos, slots=dslot)
    with pytest.raises(L.LokalCudaError) as e:
        ctx.stream_sync()
    assert e.value.status == L.capi.ERR_POS_RANGE
    got = idx.cpu().numpy().view(np.uint32)
    want = np.where(good, slot.astype(np.int64) * max_seq + pos, L.capi.KV_ROW_NONE).astype(np.uint32)
    assert np.array_equal(got, want)
    # staging: rows with the sentinel are skipped, the cache holds its fill value everywhere else
    src = np.random.default_rng(1).standard_normal((rows, width), dtype=np.float32)
    cache = dev.empty((slots * max_seq, width), F16, fill=3.0)
    dsrc = dev.put(src)
    ctx.kv_stage(dsrc, cache, src_dtype=F32, dst_dtype=F16, rows=rows, width=width, dst_rows=idx)
    ctx.stream_sync()
    out = dev.get(cache)
    ref = np.full((slots * max_seq, width), 3.0, np.float32)
    ref[want[good]] = synth.round_to(src[good], F16)
    synth.assert_bits_equal(out, ref, "staged rows with refused positions")
    # the rope's k output through the same index array
    cfg = synth.LayerConfig("kvbad", F32, rows, 64, 64, 2, 2, 64, 100, 1e4, 1e-6, 1, seed=3)
    d = synth.layer_inputs(cfg, rows)
    table = dev.empty((rows, 64), F32, fill=0.0)
    dgood = dev.put(np.where(good, pos, 0).astype(np.int32))
    ctx.rope_table(table, theta=cfg.theta, rot_dim=64, rows=rows, positions=dgood)
    kcache = dev.empty((slots * max_seq, width), F32, fill=3.0)
    q, k = dev.put(d["q"]), dev.put(d["k"])
    p = ctx.qk_rope_params(q=q, k=k, k_out=kcache, k_out_rows=idx, k_out_row_stride=width, rows=rows, n_q_heads=2,
                           n_kv_heads=2, head_dim=64, eps=cfg.eps, cos_sin=table, q_dtype=F32, k_dtype=F32, w_dtype=F32)
    ctx.qk_rope(p)
    ctx.stream_sync()
    rq, rk = oracle.qk_rope_rows(d["q"], d["k"], n_q_heads=2, n_kv_heads=2, head_dim=64, theta=cfg.theta, eps=cfg.eps,
                                 positions=np.where(good, pos, 0).astype(np.int32))
    kout = dev.get(kcache)
    synth.check_f32(kout[want[good]], rk[good], "k rows with a valid position")
    mask = np.ones(slots * max_seq, bool)
    mask[want[good]] = False
    assert (kout[mask] == 3.0).all(), "a refused position must not be stored anywhere"
    synth.check_f32(dev.get(q), rq, "q is rotated for every row")
