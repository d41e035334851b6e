"""lokal_cuda_qk_rope_pos_noalloc: the qk_rope entry point for callers that must not allocate.

Some users of this library cannot call cudaMalloc where they call these ops: a serving loop that must not stall
(an allocation synchronises the whole device), or an engine that gave every remaining byte of HBM to its KV-cache
pool when it started. For them the cos/sin table of the rotation lives in a fixed 1 MiB array inside the library
instead of a scratch block that grows on demand. This file checks, through the C ABI, that the variant gives what
lokal_cuda_qk_rope_pos gives -- on two calls in a row, because every call shares that array and finds the previous
call's table in it -- and that a request larger than the array is refused with a message that names the limit.

Collected last on purpose (the file name sorts after every other test file), so a run that stops at the first
failure has already run everything else.
"""
import numpy as np
import pytest

import synth
from synth import BF16, F32

pytestmark = pytest.mark.gpu

TABLE_BYTES = 1 << 20  # LOKAL_NOALLOC_TABLE_BYTES in include/lokal_cuda.h


def run_both(ctx, dev, cfg, d, rows, dtype, pos0=0, positions=None):
    """Same inputs through the existing entry point and through the no-alloc one; returns both results."""
    results = []
    dpos = None if positions is None else dev.put(np.asarray(positions, np.int32))
    for entry in (ctx.qk_rope_pos, ctx.qk_rope_pos_noalloc):
        dq, dk = dev.put(d["q"], dtype), dev.put(d["k"], dtype)
        qn, kn = dev.put(d["q_norm_w"], dtype), dev.put(d["k_norm_w"], dtype)  # named: the params hold raw addresses
        p = ctx.qk_rope_params(q=dq, k=dk, q_norm_w=qn, k_norm_w=kn, rows=rows, n_q_heads=cfg.n_q_heads,
                               n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, eps=cfg.eps, q_dtype=dtype, w_dtype=dtype)
        entry(p, theta=cfg.theta, positions=dpos, pos0=pos0)
        ctx.stream_sync()
        results.append((dev.get(dq), dev.get(dk)))
    return results


def compare(a, b, dtype, what):
    # the tolerance the other tests hold this op to (the two paths run the same kernels, so they agree far inside it)
    if dtype == F32:
        synth.check_f32(a, b, what)
    else:
        synth.check_half(a, b, what, dtype, atol=1e-6)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_matches_the_allocating_entry_point_twice_in_a_row(ctx, dev, oracle, dtype):
    cfg = synth.C5  # 16 q heads / 8 kv heads of 128, per-head qk-norm
    rows = 2048     # 2048 rows x rot_dim 128 x 4 bytes = exactly the 1 MiB the built-in table holds
    assert rows * cfg.head_dim * 4 == TABLE_BYTES
    d = synth.layer_inputs(cfg, rows)
    d = {k: synth.round_to(v, dtype) if v.dtype == np.float32 else v for k, v in d.items()}
    # first call: prefill positions of a late block
    (q_ref, k_ref), (q_new, k_new) = run_both(ctx, dev, cfg, d, rows, dtype, pos0=6144)
    assert np.abs(q_new - d["q"]).max() > 1e-2, "q did not change: the kernel did not run"
    compare(q_new, q_ref, dtype, "first call, q")
    compare(k_new, k_ref, dtype, "first call, k")
    # second call straight after: other positions, fewer rows; the table still holds the first call's rows
    pos = np.random.default_rng(1).integers(0, 32768, 700, dtype=np.int32)
    d2 = {k: (v[:700] if v.ndim == 2 else v) for k, v in d.items()}
    (q_ref, k_ref), (q_new, k_new) = run_both(ctx, dev, cfg, d2, 700, dtype, positions=pos)
    compare(q_new, q_ref, dtype, "second call, q")
    compare(k_new, k_ref, dtype, "second call, k")
    # and both agree with the CPU oracle
    rq, rk = oracle.qk_rope_rows(d2["q"], d2["k"], n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                                 theta=cfg.theta, eps=cfg.eps, q_norm_w=d2["q_norm_w"], k_norm_w=d2["k_norm_w"], positions=pos)
    compare(q_new, rq, dtype, "second call vs oracle, q")
    compare(k_new, rk, dtype, "second call vs oracle, k")


def test_requests_beyond_the_built_in_table_are_refused(ctx, dev):
    import lokal_b200 as L
    cfg = synth.C5
    rows = 2049  # one row more than fits
    q = dev.empty((rows, cfg.q_dim), F32, fill=1.0)
    p = ctx.qk_rope_params(q=q, rows=rows, n_q_heads=cfg.n_q_heads, n_kv_heads=0, head_dim=cfg.head_dim)
    with pytest.raises(L.LokalCudaError) as e:
        ctx.qk_rope_pos_noalloc(p, theta=cfg.theta)
    assert e.value.status == L.capi.ERR_BAD_ARG
    assert str(TABLE_BYTES) in e.value.message and "rows" in e.value.message
    ctx.stream_sync()
    assert (dev.get(q) == 1.0).all(), "a refused call must not touch its buffers"
    ctx.qk_rope_pos(p, theta=cfg.theta)  # the allocating entry point takes the same request
    ctx.stream_sync()
