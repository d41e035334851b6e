"""A bounded device-side wait that runs out comes back as LOKAL_ERR_TIMEOUT, and the context stays usable.

Every kernel that waits on a staged copy polls its mbarrier a bounded number of times; when the polls are used up it
sets a bit in the context's error word and returns. Here the wait is made to run out on the host's say-so: the staged
copy announces 16 bytes more than it delivers (LOKAL_CUDA_TEST_EXTRA_TX), so the barrier's phase never completes, and the
poll limit is lowered (LOKAL_CUDA_WAIT_LIMIT) so that the kernel gives up after a few milliseconds. Nothing faults and
nothing spins without limit: the copies themselves land, the kernel leaves, and the next synchronisation reports the
status (the reference asserts a run's status before it compares results, src/lowmem/pool.rs:1291-1320).
"""
import numpy as np
import pytest

import synth
from synth import F16, F32, Q8_0

pytestmark = pytest.mark.gpu


def starve(monkeypatch):
    monkeypatch.setenv("LOKAL_CUDA_TEST_EXTRA_TX", "16")
    monkeypatch.setenv("LOKAL_CUDA_WAIT_LIMIT", "2000")


def feed(monkeypatch):
    monkeypatch.delenv("LOKAL_CUDA_TEST_EXTRA_TX")
    monkeypatch.delenv("LOKAL_CUDA_WAIT_LIMIT")


@pytest.mark.parametrize("out_dtype", [F32, F16])  # one row per warp (f32 rows) and two rows per warp (16-bit rows)
def test_gather_wait_runs_out_and_reports(ctx, dev, oracle, monkeypatch, out_dtype):
    import lokal_b200 as L
    vocab, dim, n = 64, 256, 41
    table = synth.q8_0_table(vocab, dim, 3)
    ids = synth.token_ids_uniform(vocab, n, 4)
    dt, di = dev.put(table), dev.put(ids.view(np.int32))
    out = dev.empty((n, dim), out_dtype, fill=7.0)
    starve(monkeypatch)
    ctx.embed_gather(dt, di, out, ggml_type=Q8_0, vocab=vocab, dim=dim, n=n, out_dtype=out_dtype)
    with pytest.raises(L.LokalCudaError) as e:
        ctx.stream_sync()
    assert e.value.status == L.capi.ERR_TIMEOUT
    assert "wait" in e.value.message
    # the error word was cleared with the report; the same call without the starved barrier is bit-exact
    feed(monkeypatch)
    ctx.stream_sync()
    ctx.embed_gather(dt, di, out, ggml_type=Q8_0, vocab=vocab, dim=dim, n=n, out_dtype=out_dtype)
    ctx.stream_sync()
    want = synth.round_to(oracle.embed_gather(table, Q8_0, vocab, dim, ids), out_dtype)
    synth.assert_bits_equal(dev.get(out), want, "gather after a timed-out launch")


def test_staged_rope_wait_runs_out_and_reports(ctx, dev, oracle, monkeypatch):
    import lokal_b200 as L
    # enough rows for the staged kernel (one warp per row, rows brought in by bulk copy)
    cfg = synth.LayerConfig("timeout", F32, 2400, 64, 64, 2, 1, 64, 100, 1e4, 1e-6, 1, seed=11)
    d = synth.layer_inputs(cfg, cfg.rows)
    table = dev.empty((cfg.rows, 64), F32, fill=0.0)
    ctx.rope_table(table, theta=cfg.theta, rot_dim=64, rows=cfg.rows, pos0=0)
    ctx.stream_sync()

    def run():
        q, k = dev.put(d["q"]), dev.put(d["k"])
        p = ctx.qk_rope_params(q=q, k=k, rows=cfg.rows, n_q_heads=2, n_kv_heads=1, head_dim=64, eps=cfg.eps, cos_sin=table,
                               q_dtype=F32, k_dtype=F32, w_dtype=F32)
        ctx.qk_rope(p)
        return q, k

    starve(monkeypatch)
    run()
    with pytest.raises(L.LokalCudaError) as e:
        ctx.stream_sync()
    assert e.value.status == L.capi.ERR_TIMEOUT
    feed(monkeypatch)
    ctx.stream_sync()
    q, k = run()
    ctx.stream_sync()
    rq, rk = oracle.qk_rope_rows(d["q"], d["k"], n_q_heads=2, n_kv_heads=1, head_dim=64, theta=cfg.theta, eps=cfg.eps, pos0=0)
    synth.check_f32(dev.get(q), rq, "q after a timed-out launch")
    synth.check_f32(dev.get(k), rk, "k after a timed-out launch")
