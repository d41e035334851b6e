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
