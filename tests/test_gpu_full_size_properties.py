"""The ops at the benchmark's full sizes (C5: 8192 token rows of the Qwen3-0.6B shapes, bf16; C4: 65,536 ids),
checked through properties that need no CPU pass over the whole batch: exact identities of the arithmetic
(rotation by angle zero, scaling by powers of two, equal ids give equal rows), conservation laws (a rotation keeps
the length of each pair), and a plain torch fp32 statement of the floating-point ops evaluated on the device."""
import numpy as np
import pytest

import lokal_b200 as L
import synth
from synth import BF16, F32

pytestmark = pytest.mark.gpu

CFG = synth.C5
ROWS = CFG.rows  # 8192


def rnd(dev, *shape, scale=1.0, seed=0, dtype=None):
    t = dev.torch
    g = t.Generator(device="cuda")
    g.manual_seed(seed)
    x = t.randn(*shape, generator=g, device="cuda", dtype=t.float32) * scale
    return x.to(dev.tdt[dtype]) if dtype else x


def test_add_rmsnorm_full_size_against_torch_fp32(ctx, dev):
    t = dev.torch
    H = CFG.hidden
    x, delta = rnd(dev, ROWS, H, seed=1, dtype=BF16), rnd(dev, ROWS, H, seed=2, dtype=BF16)
    w = (1 + 0.1 * rnd(dev, H, seed=3)).to(t.bfloat16)
    x0 = x.clone()
    xn = t.empty_like(x)
    ctx.add_rmsnorm(x, delta, w, xn, rows=ROWS, dim=H, eps=CFG.eps, dtype=BF16, w_dtype=BF16)
    ctx.stream_sync()
    s = x0.float() + delta.float()
    assert t.equal(x, s.to(t.bfloat16)), "the stored residual is not the rounded f32 sum"
    ref = (s * t.rsqrt((s * s).mean(dim=1, keepdim=True) + CFG.eps)) * w.float()
    err = (xn.float() - ref).abs()
    assert bool((err <= synth.HALF_RTOL[BF16] * ref.abs() + 1e-6).all()), float((err / ref.abs().clamp_min(1e-30)).max())
    # scale invariance: rmsnorm(4 x) == rmsnorm(x) up to eps (a power of two moves no mantissa bit)
    x4, xn4 = (x0.float() * 4).to(t.bfloat16), t.empty_like(x)
    ctx.rmsnorm(x4, w, xn4, rows=ROWS, dim=H, eps=CFG.eps, dtype=BF16, w_dtype=BF16)
    xn1 = t.empty_like(x)
    ctx.rmsnorm(x0, w, xn1, rows=ROWS, dim=H, eps=CFG.eps, dtype=BF16, w_dtype=BF16)
    ctx.stream_sync()
    assert float((xn4.float() - xn1.float()).abs().max()) <= 2.0 ** -7 * float(xn1.float().abs().max())
    assert float((xn4 == xn1).float().mean()) > 0.99


def test_rope_full_size_identities(ctx, dev):
    t = dev.torch
    nq, nkv, hd = CFG.n_q_heads, CFG.n_kv_heads, CFG.head_dim
    for dtype in (BF16, F32):
        q, k = rnd(dev, ROWS, nq * hd, seed=4, dtype=dtype), rnd(dev, ROWS, nkv * hd, seed=5, dtype=dtype)
        q0, k0 = q.clone(), k.clone()
        # every row at position 0: cos = 1, sin = 0, the rotation must return its input bit for bit
        zeros = t.zeros(ROWS, dtype=t.int32, device="cuda")
        p = ctx.qk_rope_params(q=q, k=k, rows=ROWS, n_q_heads=nq, n_kv_heads=nkv, head_dim=hd, q_dtype=dtype, w_dtype=dtype)
        ctx.qk_rope_pos(p, theta=CFG.theta, positions=zeros)
        ctx.stream_sync()
        assert t.equal(q, q0) and t.equal(k, k0), "rotation by angle zero changed a value"
        # real positions: each (i, i + hd/2) pair keeps its length
        ctx.qk_rope_pos(p, theta=CFG.theta, pos0=12345)
        ctx.stream_sync()
        assert not t.equal(q, q0)

        def pair_len2(v, heads):
            v = v.float().view(ROWS, heads, 2, hd // 2)
            return v[:, :, 0] ** 2 + v[:, :, 1] ** 2
        for got, ref, heads in ((q, q0, nq), (k, k0, nkv)):
            a, b = pair_len2(got, heads), pair_len2(ref, heads)
            tol = 2.0 ** -6 if dtype == BF16 else 1e-5
            assert bool(((a - b).abs() <= tol * b + 1e-6).all())
        # and against torch fp32 on the device (same table the library builds)
        table = t.empty(ROWS, hd, dtype=t.float32, device="cuda")
        ctx.rope_table(table, theta=CFG.theta, rot_dim=hd, rows=ROWS, pos0=12345)
        ctx.stream_sync()
        cos, sin = table[:, None, :hd // 2], table[:, None, hd // 2:]
        v = q0.float().view(ROWS, nq, 2, hd // 2)
        ref = t.stack([v[:, :, 0] * cos - v[:, :, 1] * sin, v[:, :, 0] * sin + v[:, :, 1] * cos], dim=2).view(ROWS, nq * hd)
        err = (q.float() - ref).abs()
        if dtype == F32:
            assert float(err.max()) <= synth.F32_MAX_ABS
        else:
            assert bool((err <= synth.HALF_RTOL[BF16] * ref.abs() + 2e-3).all())


def test_swiglu_full_size_linearity_and_torch(ctx, dev):
    t = dev.torch
    n = ROWS * CFG.inter
    g, u = rnd(dev, n, scale=2.0, seed=6, dtype=BF16), rnd(dev, n, scale=2.0, seed=7, dtype=BF16)
    out, out2 = t.empty_like(g), t.empty_like(g)
    ctx.swiglu(g, u, out, n=n, dtype=BF16)
    ctx.swiglu(g, (u.float() * 2).to(t.bfloat16), out2, n=n, dtype=BF16)  # doubling is exact in bf16
    ctx.stream_sync()
    assert t.equal(out2.float(), out.float() * 2), "swiglu is not linear in `up` under an exact scaling"
    ref = g.float() / (1 + t.exp(-g.float())) * u.float()
    err = (out.float() - ref).abs()
    assert bool((err <= synth.HALF_RTOL[BF16] * ref.abs() + 1e-6).all())
    zero = t.zeros_like(g)
    ctx.swiglu(zero, u, out, n=n, dtype=BF16)
    ctx.stream_sync()
    assert float(out.float().abs().max()) == 0.0


def test_gather_full_size_equal_ids_equal_rows_and_full_table(ctx, dev):
    t = dev.torch
    vocab, dim, n = synth.C4_VOCAB, synth.C4_DIM_Q8, synth.C4_IDS
    table = t.from_numpy(synth.q8_0_table(vocab, dim, synth.C4_SEED)).cuda()
    ids_np = synth.token_ids_zipf(vocab, n, synth.C4_SEED)
    ids = t.from_numpy(ids_np.view(np.int32)).cuda()
    out = t.empty(n, dim, dtype=t.float32, device="cuda")
    ctx.embed_gather(table, ids, out, ggml_type=L.Q8_0, vocab=vocab, dim=dim, n=n)
    full = t.empty(vocab, dim, dtype=t.float32, device="cuda")
    ctx.dequant_rows(table, full, ggml_type=L.Q8_0, rows=vocab, cols=dim)
    ctx.stream_sync()
    # gather(ids) is the full dequantised table indexed by ids, bit for bit
    assert t.equal(out.view(t.int32), full[ids.long()].view(t.int32))
    # the full table against a torch statement of Q8_0 on the raw bytes: q * d, one multiply
    blocks = table.view(vocab * dim // 32, 34)
    d = blocks[:, :2].contiguous().view(t.float16).float()
    qv = blocks[:, 2:].contiguous().view(t.int8).float()
    assert t.equal(full.view(-1, 32), qv * d)
