"""One context shared by several host threads, each with its own stream: the reference's engine is `Send + Sync` and
shared across request threads while every session owns its submission queue (src/engine.rs:13-27, 49; src/server.rs:24).
The threads launch the ops concurrently on separate buffers; every result must match the oracle."""
import threading

import numpy as np
import pytest

import lokal_b200 as L
import synth
from synth import BF16, F32

pytestmark = pytest.mark.gpu


def test_four_threads_four_streams_one_context(ctx, dev, oracle):
    cfg = synth.C2  # f16 rows, q/k bias
    rows, n_threads, reps = 160, 4, 12
    inputs = [synth.layer_inputs(cfg, rows, layer=10 + i) for i in range(n_threads)]
    for d in inputs:
        d.pop("positions", None)
    table = synth.q8_0_table(512, cfg.hidden, 77)
    dtab = dev.put(table)
    errors, results = [], [None] * n_threads

    def work(i):
        try:
            d = inputs[i]
            stream = ctx.stream_create()
            for rep in range(reps):
                x, delta, w = dev.put(d["x"], cfg.dtype), dev.put(d["delta"], cfg.dtype), dev.put(d["w_norm"], cfg.dtype)
                xn = dev.empty((rows, cfg.hidden), cfg.dtype, fill=0.0)
                g, u = dev.put(d["gate"], cfg.dtype), dev.put(d["up"], cfg.dtype)
                inner = dev.empty((rows, cfg.inter), cfg.dtype, fill=0.0)
                q, k = dev.put(d["q"], cfg.dtype), dev.put(d["k"], cfg.dtype)
                qb, kb = dev.put(d["q_bias"], cfg.dtype), dev.put(d["k_bias"], cfg.dtype)
                ids = synth.token_ids_uniform(512, rows, seed=i * 100 + rep)
                dids = dev.put(ids)
                gout = dev.empty((rows, cfg.hidden), F32, fill=0.0)
                dev.torch.cuda.synchronize()  # the uploads above ran on torch's stream
                ctx.add_rmsnorm(x, delta, w, xn, rows=rows, dim=cfg.hidden, eps=cfg.eps, dtype=cfg.dtype, w_dtype=cfg.dtype, stream=stream)
                ctx.swiglu(g, u, inner, n=rows * cfg.inter, dtype=cfg.dtype, stream=stream)
                p = ctx.qk_rope_params(q=q, k=k, q_bias=qb, k_bias=kb, rows=rows, n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads,
                                       head_dim=cfg.head_dim, eps=cfg.eps, q_dtype=cfg.dtype, w_dtype=cfg.dtype)
                ctx.qk_rope_pos(p, theta=cfg.theta, pos0=1000 * i, stream=stream)
                ctx.embed_gather(dtab, dids, gout, ggml_type=L.Q8_0, vocab=512, dim=cfg.hidden, n=rows, stream=stream)
                ctx.stream_sync(stream)
                results[i] = (dev.get(xn), dev.get(inner), dev.get(q), dev.get(k), dev.get(gout), ids)
            ctx.stream_destroy(stream)
        except Exception as e:  # surfaced in the main thread
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=work, args=(i,)) for i in range(n_threads)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for i, d in enumerate(inputs):
        xn, inner, q, k, gout, ids = results[i]
        _, rxn = oracle.add_rmsnorm_rows(d["x"], d["delta"], d["w_norm"], cfg.eps)
        synth.check_half(xn, rxn, f"thread {i} add_rmsnorm", cfg.dtype, atol=1e-6)
        synth.check_half(inner, oracle.swiglu(d["gate"], d["up"]), f"thread {i} swiglu", cfg.dtype, atol=1e-6)
        rq, rk = oracle.qk_rope_rows(d["q"], d["k"], n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                                     theta=cfg.theta, eps=cfg.eps, q_bias=d["q_bias"], k_bias=d["k_bias"], pos0=1000 * i)
        synth.check_half(q, rq, f"thread {i} q", cfg.dtype, atol=2e-3)
        synth.check_half(k, rk, f"thread {i} k", cfg.dtype, atol=2e-3)
        synth.assert_bits_equal(gout, oracle.embed_gather(table, L.Q8_0, 512, cfg.hidden, ids), f"thread {i} gather")


def test_rope_pos_on_a_user_stream_interleaved_with_host_mirrors(ctx, dev, oracle):
    """lokal_cuda_qk_rope_pos leaves its table and rope kernels queued on the caller's stream; the host-slice mirrors
    called right after it on the same context run on the context's own stream and stage through a device block of
    their own, so neither disturbs the other: both results match the oracle, call after call."""
    import torch
    cfg = synth.C5
    rows = 3000
    d = synth.layer_inputs(cfg, rows)
    rng = np.random.default_rng(5)
    hx = rng.standard_normal((64, 1024), dtype=np.float32)
    hw = (1 + 0.1 * rng.standard_normal(1024, dtype=np.float32)).astype(np.float32)
    _, want_norm = oracle.add_rmsnorm_rows(hx, None, hw, 1e-6)
    rq, rk = oracle.qk_rope_rows(d["q"], d["k"], n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                                 theta=cfg.theta, eps=cfg.eps, q_norm_w=d["q_norm_w"], k_norm_w=d["k_norm_w"], pos0=100, threads=8)
    s = ctx.stream_create()
    qn, kn = dev.put(d["q_norm_w"], cfg.dtype), dev.put(d["k_norm_w"], cfg.dtype)
    # a long kernel queue on the user stream first, so that the rope's table is still waiting to be read when the
    # host mirrors run
    filler_g, filler_u = dev.put(np.zeros((1 << 24,), np.float32)), dev.put(np.zeros((1 << 24,), np.float32))
    filler_o = dev.empty((1 << 24,), 0)
    torch.cuda.synchronize()
    for rep in range(3):
        q, k = dev.put(d["q"], cfg.dtype), dev.put(d["k"], cfg.dtype)
        torch.cuda.synchronize()
        for _ in range(20):
            ctx.swiglu(filler_g, filler_u, filler_o, n=1 << 24, dtype=0, stream=s)
        p = ctx.qk_rope_params(q=q, k=k, q_norm_w=qn, k_norm_w=kn, rows=rows, n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads,
                               head_dim=cfg.head_dim, eps=cfg.eps, q_dtype=cfg.dtype, w_dtype=cfg.dtype)
        ctx.qk_rope_pos(p, theta=cfg.theta, pos0=100, stream=s)
        got_norm = ctx.host_rmsnorm(hx, hw, 1e-6)          # 256 KB through the mirrors' own block
        got_sw = ctx.host_swiglu(hx.reshape(-1), hx.reshape(-1)[::-1].copy())
        ctx.stream_sync(s)
        synth.check_f32(got_norm, want_norm, "host rmsnorm beside a queued rope")
        synth.check_f32(got_sw, oracle.swiglu(hx.reshape(-1), hx.reshape(-1)[::-1].copy()), "host swiglu beside a queued rope")
        synth.check_half(dev.get(q), rq, "q", cfg.dtype, atol=1e-6)
        synth.check_half(dev.get(k), rk, "k", cfg.dtype, atol=1e-6)
    ctx.stream_destroy(s)


def test_rope_pos_under_capture_cannot_grow_and_keeps_its_block(ctx, dev, oracle):
    import lokal_b200 as L
    cfg = synth.C1
    rows = 64
    d = synth.layer_inputs(cfg, rows)
    s = ctx.stream_create()
    q, k = dev.put(d["q"]), dev.put(d["k"])
    p = ctx.qk_rope_params(q=q, k=k, rows=rows, n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                           eps=cfg.eps, q_dtype=cfg.dtype, w_dtype=cfg.dtype)
    ctx.qk_rope_pos(p, theta=cfg.theta, pos0=0, stream=s)  # sizes the block
    ctx.stream_sync(s)
    q2, k2 = dev.put(d["q"]), dev.put(d["k"])
    p2 = ctx.qk_rope_params(q=q2, k=k2, rows=rows, n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                            eps=cfg.eps, q_dtype=cfg.dtype, w_dtype=cfg.dtype)
    ctx.graph_begin(s)
    ctx.qk_rope_pos(p2, theta=cfg.theta, pos0=0, stream=s)
    # a captured call that would need a larger block is refused by name, and the capture goes on
    big = ctx.qk_rope_params(q=q2, k=k2, rows=1 << 22, n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                             eps=cfg.eps, q_dtype=cfg.dtype, w_dtype=cfg.dtype)
    with pytest.raises(L.LokalCudaError) as e:
        ctx.qk_rope_pos(big, theta=cfg.theta, pos0=0, stream=s)
    assert e.value.status == L.capi.ERR_BAD_ARG and "captured" in e.value.message
    g = ctx.graph_end(s)
    # an uncaptured, larger call replaces the block; the graph still holds the old one and must replay correctly
    rows_big = 40000
    qb, kb = dev.empty((rows_big, cfg.q_dim), 0, fill=1.0), dev.empty((rows_big, cfg.kv_dim), 0, fill=1.0)
    pb = ctx.qk_rope_params(q=qb, k=kb, rows=rows_big, n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                            eps=cfg.eps, q_dtype=cfg.dtype, w_dtype=cfg.dtype)
    ctx.qk_rope_pos(pb, theta=cfg.theta, pos0=0, stream=s)
    ctx.stream_sync(s)
    ctx.graph_launch(g, s)
    ctx.stream_sync(s)
    synth.assert_bits_equal(dev.get(q2), dev.get(q), "graph replay after the block was replaced, q")
    synth.assert_bits_equal(dev.get(k2), dev.get(k), "graph replay after the block was replaced, k")
    ctx.graph_destroy(g)
    ctx.stream_destroy(s)
