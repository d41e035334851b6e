"""Pins the CPU oracle: the reference's own known-answer vectors, two independent decoders,
conversions against numpy, and the committed golden outputs. No GPU needed."""
import json
import os

import numpy as np
import pytest

import synth

HERE = os.path.dirname(os.path.abspath(__file__))
KATS = json.load(open(os.path.join(HERE, "golden", "reference_kats.json")))


def build_block(spec):
    blk = np.zeros(spec["block_bytes"], np.uint8)
    for f in spec["f16_fields"]:
        blk[f["offset"]:f["offset"] + 2] = np.array([f["value"]], np.float16).view(np.uint8)
    for b in spec["bytes"]:
        blk[b["offset"]] = b["value"]
    return blk


def test_block_size_table(oracle):
    for ty, n in KATS["block_sizes"]["blk_bytes"].items():
        assert oracle.blk_bytes(int(ty)) == n
    for ty, n in KATS["block_sizes"]["blk_elems"].items():
        assert oracle.blk_elems(int(ty)) == n
    for row in KATS["block_sizes"]["row_bytes"]:
        assert oracle.row_bytes(row["type"], row["n"]) == row["bytes"]
    assert oracle.row_bytes(oracle.Q8_0, 896) == 952
    assert oracle.blk_elems(3) == 0  # Q4_1: refused by the reference too (src/gguf/dequant.rs:58)


@pytest.mark.parametrize("key,ty", [("q8_0_hand_vector", 8), ("q4_k_hand_vector", 12)])
def test_reference_dequant_hand_vectors(oracle, key, ty):
    spec = KATS[key]
    y = oracle.dequant_row_ref(ty, build_block(spec), spec["n"])
    for e in spec["expect"]:
        assert y[e["index"]] == e["value"], (key, e)
    # and through the independent per-element decoder
    for e in spec["expect"]:
        assert oracle.dequant_elem(ty, build_block(spec), e["index"]) == e["value"]


def test_reference_q8_0_roundtrip_property(oracle):
    spec = KATS["q8_0_roundtrip"]
    d = np.float32(spec["d"])
    state = spec["lcg_seed"]
    xs = np.empty(32, np.float32)
    for i in range(32):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        xs[i] = (np.float32(state >> 8) / np.float32(1 << 24) * np.float32(2) - np.float32(1)) * np.float32(127) * d
    blk = np.zeros(34, np.uint8)
    blk[:2] = np.array([d], np.float16).view(np.uint8)
    q = np.clip(np.sign(xs / d) * np.floor(np.abs(xs / d) + 0.5), -127, 127).astype(np.int8)  # f32::round = half away from zero
    blk[2:] = q.view(np.uint8)
    y = oracle.dequant_row_ref(8, blk, 32)
    assert (np.abs(xs - y) <= d * 0.5 + 1e-7).all()


def test_size_mismatch_is_refused(oracle):
    with pytest.raises(ValueError):
        oracle.dequant_row_ref(8, np.zeros(33, np.uint8), 32)  # the reference panics (src/gguf/dequant.rs:192)
    with pytest.raises(ValueError):
        oracle.dequant_row_ref(3, np.zeros(20, np.uint8), 32)


def test_dot_and_rmsnorm_reference_vectors(oracle):
    a = np.array(KATS["dot_tail"]["a"], np.float32)
    assert oracle.dot(a, a) == KATS["dot_tail"]["expect"]
    s = KATS["rmsnorm_all_threes"]
    y = oracle.rmsnorm(np.array(s["x"], np.float32), np.array(s["w"], np.float32), s["eps"])
    assert np.abs(y - s["expect_each"]).max() < s["tol"]


def test_dot_keeps_the_eight_lane_order(oracle):
    # a vector on which lane order and sequential order round differently
    rng = np.random.default_rng(5)
    a = (rng.standard_normal(1000) * 10.0 ** rng.integers(-3, 4, 1000)).astype(np.float32)
    lanes = np.zeros(8, np.float32)
    for c in range(125):
        lanes = (lanes + a[c * 8:(c + 1) * 8] * a[c * 8:(c + 1) * 8]).astype(np.float32)
    s = np.float32(0)
    for v in lanes:
        s = np.float32(s + v)
    assert oracle.dot(a, a) == s
    seq = np.float32(0)
    for v in a:
        seq = np.float32(seq + np.float32(v * v))
    assert seq != s, "test vector does not distinguish the two orders"


def test_f16_bf16_conversions_match_numpy_and_torch(oracle):
    import torch
    bits = np.arange(65536, dtype=np.uint16)
    f = oracle.f16_bits_to_f32(bits)
    ref = bits.view(np.float16).astype(np.float32)
    ok = ~np.isnan(ref)
    assert np.array_equal(f[ok].view(np.uint32), ref[ok].view(np.uint32)) and np.isnan(f[~ok]).all()
    rng = np.random.default_rng(0)
    x = np.concatenate([
        (rng.standard_normal(200000) * 10.0 ** rng.integers(-9, 6, 200000)).astype(np.float32), f[ok],
        np.array([65504, 65519.9, 65520, 65536, 1e-8, 2.98e-8, 2.9802322e-8, 5.96e-8, 0.0, -0.0], np.float32)])
    with np.errstate(over="ignore"):
        assert np.array_equal(oracle.f32_to_f16_bits(x), x.astype(np.float16).view(np.uint16))
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.uint16).numpy()
    assert np.array_equal(oracle.f32_to_bf16_bits(x), want)
    b16 = oracle.bf16_bits_to_f32(bits)
    assert np.array_equal(b16.view(np.uint32), bits.astype(np.uint32) << 16)


@pytest.mark.parametrize("ty", [8, 12])
def test_adversarial_rows_two_decoders_agree(oracle, ty):
    spec = KATS["adversarial_rows"]
    nb, rows = spec["n_blocks"], spec["n_rows"]
    adv = oracle.adversarial_rows(ty, nb, rows)
    bb = oracle.blk_bytes(ty)
    blocks = adv.reshape(rows * nb, bb)
    # recipe structure: variant (row*nb+blk)%4 -> zero block / scale bytes of the table
    for i, blk in enumerate(blocks):
        v = i % 4
        if v == 0:
            assert not blk.any()
        else:
            assert list(blk[:2]) == spec["scale_bytes"][v]
            if ty == 12:
                assert list(blk[2:4]) == spec["scale_bytes"][3 - v + 1]
    payload = 2 if ty == 8 else 4  # first byte after the f16 field(s)
    assert (blocks[3, payload:] == (0x80 if ty == 8 else 0xFF)).all()
    # LCG bytes are drawn for the whole block before the scale bytes overwrite the head:
    # the first payload byte of the first non-zero block is draw number payload+1 from the seed
    s = spec["lcg_seed"]
    for _ in range(payload + 1):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
    assert blocks[1, payload] == (s >> 16) & 0xFF
    cols = nb * oracle.blk_elems(ty)
    rb = oracle.row_bytes(ty, cols)
    seq = np.stack([oracle.dequant_row_ref(ty, adv[r * rb:(r + 1) * rb], cols) for r in range(rows)])
    ele = oracle.dequant_rows_elementwise(ty, adv, rows, cols)
    synth.assert_bits_equal(seq, ele, "sequential vs per-element decode")


@pytest.mark.parametrize("ty,dim", [(8, 896), (12, 1024)])
def test_random_table_two_decoders_agree_and_gather(oracle, ty, dim):
    vocab = 40
    table = (synth.q8_0_table if ty == 8 else synth.q4_k_table)(vocab, dim, seed=2)
    full = oracle.dequant_rows_elementwise(ty, table, 6, dim)
    ids = np.array([5, 0, 3, 5], np.uint32)
    g = oracle.embed_gather(table, ty, vocab, dim, ids)
    synth.assert_bits_equal(g, full[ids], "gather == per-element decode of the same rows")
    synth.assert_bits_equal(oracle.embed_gather(table, ty, vocab, dim, ids, threads=3), g, "threaded gather")
    with pytest.raises(IndexError):
        oracle.embed_gather(table, ty, vocab, dim, np.array([1, vocab], np.uint32))


def test_q4k_arithmetic_is_not_fused(oracle):
    # d1*q - m1 with separately rounded product: pick values where an FMA would differ
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.array([0.0999755859375], np.float16).view(np.uint8)  # d
    blk[2:4] = np.array([0.0333251953125], np.float16).view(np.uint8)  # dmin
    blk[4], blk[8] = 61, 59
    blk[16:48] = 0x0F
    y = oracle.dequant_row_ref(12, blk, 256)
    d, dmin = np.float32(np.float16(0.0999755859375)), np.float32(np.float16(0.0333251953125))
    d1, m1 = np.float32(d * np.float32(61)), np.float32(dmin * np.float32(59))
    assert y[0] == np.float32(np.float32(d1 * np.float32(15)) - m1)


def test_rope_matches_float64_envelope_and_structure(oracle):
    rng = np.random.default_rng(8)
    hd, nh = 64, 3
    x = rng.standard_normal(nh * hd).astype(np.float32)
    for pos, theta in [(0, 1e4), (1, 1e5), (511, 1e5), (32767, 1e4), (8191, 1e6)]:
        y = oracle.rope(x, pos, hd, theta).reshape(nh, hd)
        if pos == 0:
            synth.assert_bits_equal(y.reshape(-1), x, "position 0 is the identity")
            continue
        inv = oracle.inv_freq(theta, hd).astype(np.float64)
        ang = (np.float32(pos) * oracle.inv_freq(theta, hd)).astype(np.float64)  # the f32 angle the reference forms
        a, b = x.reshape(nh, hd)[:, :32].astype(np.float64), x.reshape(nh, hd)[:, 32:].astype(np.float64)
        want = np.concatenate([a * np.cos(ang) - b * np.sin(ang), a * np.sin(ang) + b * np.cos(ang)], axis=1)
        assert np.abs(y - want).max() < 2e-6
        assert np.all(np.diff(inv) < 0) and inv[0] == 1.0
    # half-split pairing, not adjacent pairs: rotating only element 0 and element hd/2 interact
    e = np.zeros(hd, np.float32)
    e[0] = 1
    y = oracle.rope(e, 1, hd, 1e4)
    assert y[0] == np.float32(np.cos(1.0)) and y[32] == np.float32(np.sin(1.0)) and y[1] == 0  # libm is correctly rounded here
    # partial rope: tail untouched, prefix equals a full rope of rot dims
    spec = json.load(open(os.path.join(HERE, "golden", "reference_kats.json")))["partial_rope"]
    xx = rng.standard_normal(2 * 256).astype(np.float32)
    yy = oracle.rope(xx, spec["pos0"], 256, spec["theta"], rot_dim=64).reshape(2, 256)
    synth.assert_bits_equal(yy[:, 64:], xx.reshape(2, 256)[:, 64:], "tail")
    synth.assert_bits_equal(yy[0, :64], oracle.rope(np.ascontiguousarray(xx[:64]), spec["pos0"], 64, spec["theta"]), "prefix")


def test_rope_table_and_libm_spellings(oracle):
    t = oracle.rope_table(1e6, 128, 50, pos0=8000)
    inv = oracle.inv_freq(1e6, 128)
    ang = (np.float32(8010) * inv)
    assert np.abs(t[10, :64] - np.cos(ang.astype(np.float64))).max() < 1e-6
    pos = np.array([5, 32767], np.int32)
    synth.assert_bits_equal(oracle.rope_table(1e4, 64, 2, positions=pos)[1], oracle.rope_table(1e4, 64, 1, pos0=32767)[0], "positions")
    # sincosf and sinf/cosf of glibc agree bit for bit over the angles the configs produce
    for cfg in (synth.C1, synth.C3, synth.C5):
        inv = oracle.inv_freq(cfg.theta, cfg.head_dim)
        for p in (1, 511, 8191, 32767):
            for f in inv:
                assert oracle.lib().lokal_ref_sincos_spellings_agree(float(np.float32(p) * f))


def test_swiglu_and_composites_against_float64(oracle):
    rng = np.random.default_rng(4)
    g = (2 * rng.standard_normal(5000)).astype(np.float32)
    u = (2 * rng.standard_normal(5000)).astype(np.float32)
    y = oracle.swiglu(g, u)
    g64, u64 = g.astype(np.float64), u.astype(np.float64)
    want = g64 / (1 + np.exp(-g64)) * u64
    # four rounded f32 operations (exp, 1+e, divide, multiply): a sanity envelope, not the parity target
    assert (np.abs(y - want) <= 4 * np.spacing(np.abs(want).astype(np.float32)) + 1e-12).all()
    assert oracle.silu(0.0) == 0.0 and abs(oracle.silu(1.0) - 0.7310585786) < 1e-7
    synth.assert_bits_equal(oracle.swiglu(g, u, threads=4), y, "threaded swiglu")
    # add_rmsnorm = residual add then rmsnorm; qk_rope = bias -> per-head norm -> rope
    cfg = synth.C5
    d = synth.layer_inputs(cfg, 5)
    xs, xn = oracle.add_rmsnorm_rows(d["x"], d["delta"], d["w_norm"], cfg.eps)
    synth.assert_bits_equal(xs, d["x"] + d["delta"], "residual")
    synth.assert_bits_equal(xn[2], oracle.rmsnorm(xs[2], d["w_norm"], cfg.eps), "row norm")
    q, k = oracle.qk_rope_rows(d["q"], d["k"], n_q_heads=16, n_kv_heads=8, head_dim=128, theta=cfg.theta, eps=cfg.eps,
                               q_norm_w=d["q_norm_w"], k_norm_w=d["k_norm_w"], pos0=100)
    head = oracle.rmsnorm(d["q"][3, 128:256], d["q_norm_w"], cfg.eps)
    synth.assert_bits_equal(q[3, 128:256], oracle.rope(head, 103, 128, cfg.theta), "qk-norm then rope")
    q2, _ = oracle.qk_rope_rows(d["q"], d["k"], n_q_heads=16, n_kv_heads=8, head_dim=128, theta=cfg.theta, eps=cfg.eps,
                                q_norm_w=d["q_norm_w"], k_norm_w=d["k_norm_w"], pos0=100, threads=3)
    synth.assert_bits_equal(q2, q, "threaded rows")


def test_committed_golden_outputs_still_reproduce(oracle):
    z = np.load(os.path.join(HERE, "golden", "oracle_small.npz"))
    xs, xn = oracle.add_rmsnorm_rows(z["norm_x"], z["norm_delta"], z["norm_w"], float(z["norm_eps"]))
    synth.assert_bits_equal(xs, z["norm_sum"], "golden residual")
    synth.assert_bits_equal(xn, z["norm_out"], "golden norm")
    q, k = oracle.qk_rope_rows(z["rope_q"], z["rope_k"], n_q_heads=4, n_kv_heads=2, head_dim=64, theta=float(z["rope_theta"]),
                               q_bias=z["rope_qb"], k_bias=z["rope_kb"], positions=z["rope_pos"])
    synth.assert_bits_equal(q, z["rope_q_out"], "golden rope q")
    synth.assert_bits_equal(k, z["rope_k_out"], "golden rope k")
    synth.assert_bits_equal(oracle.swiglu(z["sw_gate"], z["sw_up"]), z["sw_out"], "golden swiglu")
    for name, ty, dim in (("q8", 8, 96), ("q4k", 12, 512)):
        synth.assert_bits_equal(oracle.embed_gather(z[f"{name}_table"], ty, 9, dim, z[f"{name}_ids"]), z[f"{name}_out"], name)
        synth.assert_bits_equal(oracle.adversarial_rows(ty, 8, 3), z[f"{name}_adv"], name + " adversarial bytes")


def test_layer_pass_equals_op_by_op(oracle):
    """The timed CPU baseline walks tokens through all layers; it must equal the ops applied one by one."""
    import ctypes as C
    cfg = synth.LayerConfig("t", 0, 6, 64, 96, 4, 2, 16, 50, 1e4, 1e-5, 3, qk_bias=True, qk_norm=True, seed=1)
    L, R, H, I = cfg.layers, cfg.rows, cfg.hidden, cfg.inter
    rng = np.random.default_rng(12)
    f = lambda *s: rng.standard_normal(s, dtype=np.float32)
    table = synth.q8_0_table(cfg.vocab, H, 3)
    ids = synth.token_ids_uniform(cfg.vocab, R, 4)
    a = dict(norm_w=1 + 0.1 * f(L, 2, H), final_w=1 + 0.1 * f(H), q_bias=0.1 * f(L, cfg.q_dim), k_bias=0.1 * f(L, cfg.kv_dim),
             q_norm_w=1 + 0.1 * f(L, 16), k_norm_w=1 + 0.1 * f(L, 16), delta_att=f(L, R, H), delta_mlp=f(L, R, H),
             q=f(L, R, cfg.q_dim), k=f(L, R, cfg.kv_dim), gate=2 * f(L, R, I), up=2 * f(L, R, I))
    a = {k: np.ascontiguousarray(v, np.float32) for k, v in a.items()}
    out = np.zeros((R, H), np.float32)
    sink = np.zeros(1, np.float32)
    args = oracle.LayerPassArgs(rows=R, layers=L, hidden=H, inter=I, n_q_heads=4, n_kv_heads=2, head_dim=16, eps=cfg.eps,
                                theta=cfg.theta, has_bias=1, has_qk_norm=1, positions=None, pos0=10,
                                embed_table=table.ctypes.data, embed_type=8, vocab=cfg.vocab, ids=ids.ctypes.data,
                                layer_period=L, out=out.ctypes.data, sink=sink.ctypes.data,
                                **{k: v.ctypes.data for k, v in a.items()})
    oracle.layer_pass(args, 1)
    x = oracle.embed_gather(table, 8, cfg.vocab, H, ids)
    for l in range(L):
        x, _ = oracle.add_rmsnorm_rows(x, a["delta_att"][l], a["norm_w"][l, 1], cfg.eps)
        x = x + a["delta_mlp"][l]
    want = np.stack([oracle.rmsnorm(x[r], a["final_w"], cfg.eps) for r in range(R)])
    synth.assert_bits_equal(out, want, "layer pass residual stream")
    out2 = np.zeros_like(out)
    args.out = out2.ctypes.data
    oracle.layer_pass(args, 3)
    synth.assert_bits_equal(out2, out, "threaded layer pass")
