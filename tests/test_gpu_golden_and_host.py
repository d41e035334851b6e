"""CUDA path vs the committed golden fixtures, and the host-slice mirrors of the reference's CPU signatures."""
import os

import numpy as np
import pytest

import synth
from synth import F32, Q4_K, Q8_0

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(HERE, "golden", "oracle_small.npz"))


def test_golden_norm(ctx, dev, gold):
    dx, dd, dw = dev.put(gold["norm_x"]), dev.put(gold["norm_delta"]), dev.put(gold["norm_w"])
    xn = dev.empty((4, 576), F32, fill=0.0)
    ctx.add_rmsnorm(dx, dd, dw, xn, rows=4, dim=576, eps=float(gold["norm_eps"]), dtype=F32)
    ctx.stream_sync()
    synth.assert_bits_equal(dev.get(dx), gold["norm_sum"], "golden residual")
    synth.check_f32(dev.get(xn), gold["norm_out"], "golden norm")


def test_golden_rope(ctx, dev, gold):
    dq, dk = dev.put(gold["rope_q"]), dev.put(gold["rope_k"])
    qb, kb, pos = dev.put(gold["rope_qb"]), dev.put(gold["rope_kb"]), dev.put(gold["rope_pos"])  # params hold raw addresses
    p = ctx.qk_rope_params(q=dq, k=dk, q_bias=qb, k_bias=kb, rows=3, n_q_heads=4, n_kv_heads=2, head_dim=64)
    ctx.qk_rope_pos(p, theta=float(gold["rope_theta"]), positions=pos)
    ctx.stream_sync()
    synth.check_f32(dev.get(dq), gold["rope_q_out"], "golden rope q")
    synth.check_f32(dev.get(dk), gold["rope_k_out"], "golden rope k")
    dq, dk = dev.put(gold["qn_q"]), dev.put(gold["qn_k"])
    qw, kw = dev.put(gold["qn_qw"]), dev.put(gold["qn_kw"])
    p = ctx.qk_rope_params(q=dq, k=dk, q_norm_w=qw, k_norm_w=kw, rows=2, n_q_heads=2, n_kv_heads=1, head_dim=128, eps=1e-6)
    ctx.qk_rope_pos(p, theta=1e6, pos0=8000)
    ctx.stream_sync()
    synth.check_f32(dev.get(dq), gold["qn_q_out"], "golden qk-norm rope q")
    synth.check_f32(dev.get(dk), gold["qn_k_out"], "golden qk-norm rope k")


def test_golden_swiglu_and_gather(ctx, dev, gold):
    out = dev.empty((512,), F32, fill=0.0)
    ctx.swiglu(dev.put(gold["sw_gate"]), dev.put(gold["sw_up"]), out, n=512, dtype=F32)
    ctx.stream_sync()
    synth.check_f32(dev.get(out), gold["sw_out"], "golden swiglu")
    for name, ty, dim in (("q8", Q8_0, 96), ("q4k", Q4_K, 512)):
        ids = gold[f"{name}_ids"]
        o = dev.empty((len(ids), dim), F32, fill=0.0)
        ctx.embed_gather(dev.put(gold[f"{name}_table"]), dev.put(ids), o, ggml_type=ty, vocab=9, dim=dim, n=len(ids))
        ctx.stream_sync()
        synth.assert_bits_equal(dev.get(o), gold[f"{name}_out"], f"golden {name} gather")
        cols = 8 * (32 if ty == Q8_0 else 256)
        o = dev.empty((3, cols), F32, fill=0.0)
        ctx.dequant_rows(dev.put(gold[f"{name}_adv"]), o, ggml_type=ty, rows=3, cols=cols)
        ctx.stream_sync()
        synth.assert_bits_equal(dev.get(o), gold[f"{name}_adv_out"], f"golden {name} adversarial rows")


def test_host_rmsnorm_mirror(ctx, oracle):
    # math::rmsnorm(x, weight, eps) -> Vec (src/math.rs:45)
    d = synth.layer_inputs(synth.C1, 9)
    y = ctx.host_rmsnorm(d["x"][0], d["w_norm"], 1e-5)
    synth.check_f32(y, oracle.rmsnorm(d["x"][0], d["w_norm"], 1e-5), "one row")
    y = ctx.host_rmsnorm(d["x"], d["w_norm"], 1e-5)
    synth.check_f32(y, oracle.add_rmsnorm_rows(d["x"], None, d["w_norm"], 1e-5)[1], "rows")
    assert np.abs(ctx.host_rmsnorm(np.full(4, 3, np.float32), np.ones(4, np.float32), 1e-6) - 1).max() < 1e-3


def test_host_rope_mirror(ctx, oracle):
    # model::rope(x, pos, head_dim, theta) (src/model.rs:268)
    rng = np.random.default_rng(1)
    for hd, nh, pos, theta in [(64, 9, 511, 1e5), (128, 16, 8191, 1e6), (64, 4, 32767, 1e4), (10, 3, 7, 1e4)]:
        x = rng.standard_normal(nh * hd).astype(np.float32)
        synth.check_f32(ctx.host_rope(x, pos, hd, theta), oracle.rope(x, pos, hd, theta), f"hd {hd} pos {pos}")
    import lokal_b200 as L
    with pytest.raises(L.LokalCudaError):
        ctx.host_rope(np.zeros(10, np.float32), 0, 4, 1e4)  # not whole heads


def test_host_swiglu_and_dequant_mirrors(ctx, oracle):
    import lokal_b200 as L
    d = synth.layer_inputs(synth.C1, 5)
    synth.check_f32(ctx.host_swiglu(d["gate"], d["up"]), oracle.swiglu(d["gate"], d["up"]), "host swiglu")
    for ty, dim in ((Q8_0, 896), (Q4_K, 1024)):
        table = (synth.q8_0_table if ty == Q8_0 else synth.q4_k_table)(3, dim, 9)
        rb = oracle.row_bytes(ty, dim)
        row = table[rb:2 * rb]
        synth.assert_bits_equal(ctx.host_dequant_row(ty, row, dim), oracle.dequant_row_ref(ty, row, dim), "host dequant_row")
        with pytest.raises(L.LokalCudaError) as e:  # the reference panics on a size mismatch (src/gguf/dequant.rs:192)
            ctx.host_dequant_row(ty, row[:-1], dim)
        assert e.value.status == L.capi.ERR_BAD_ARG


def test_host_embed_gather_mirror(ctx, dev, oracle):
    import lokal_b200 as L
    vocab, dim = 300, 896
    table = synth.q8_0_table(vocab, dim, 2)
    ids = synth.token_ids_zipf(vocab, 1000, 3)
    dt = dev.put(table)
    synth.assert_bits_equal(ctx.host_embed_gather(dt, Q8_0, vocab, dim, ids), oracle.embed_gather(table, Q8_0, vocab, dim, ids),
                            "host embed_gather")
    with pytest.raises(L.LokalCudaError) as e:
        ctx.host_embed_gather(dt, Q8_0, vocab, dim, np.array([1, vocab], np.uint32))
    assert e.value.status == L.capi.ERR_ID_RANGE


def test_host_embed_gather_large_result_pageable_and_pinned(ctx, dev, oracle):
    """A result of tens of MB: ordinary memory is filled by several worker threads pulling 4 MB chunks through pinned
    staging, page-locked caller buffers are written by DMA. Both must be the oracle's rows bit for bit, tail included."""
    import lokal_b200 as L
    torch = dev.torch
    vocab, dim, n = 2000, 896, 20011  # 71.7 MB of f32 rows, not a whole number of chunks
    table = synth.q8_0_table(vocab, dim, 21)
    ids = synth.token_ids_zipf(vocab, n, 22)
    dt = dev.put(table)
    want = oracle.embed_gather(table, Q8_0, vocab, dim, ids, threads=8)
    synth.assert_bits_equal(ctx.host_embed_gather(dt, Q8_0, vocab, dim, ids), want, "pageable result")
    pin_ids = torch.from_numpy(ids.view(np.int32)).pin_memory()
    pin_out = torch.full((n + 1, dim), 7.0, dtype=torch.float32).pin_memory()
    got = ctx.host_embed_gather(dt, Q8_0, vocab, dim, pin_ids.numpy().view(np.uint32), out=pin_out.numpy()[:n])
    synth.assert_bits_equal(got, want, "pinned result")
    assert (pin_out.numpy()[n] == 7.0).all(), "wrote past the caller's buffer"
    # a small call afterwards still works (the staging block was regrown and is reused)
    synth.assert_bits_equal(ctx.host_embed_gather(dt, Q8_0, vocab, dim, ids[:5]), want[:5], "small call after a large one")
    with pytest.raises(L.LokalCudaError) as e:
        bad = ids.copy()
        bad[-1] = vocab
        ctx.host_embed_gather(dt, Q8_0, vocab, dim, bad)
    assert e.value.status == L.capi.ERR_ID_RANGE
