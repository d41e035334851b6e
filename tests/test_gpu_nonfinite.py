"""Rows with infinities, NaNs, zeros, subnormals and values whose squares overflow, through the f32 ops on the GPU.

The reference's CPU code is plain IEEE arithmetic, so such rows have defined results there (a NaN anywhere in a row
makes the whole normalised row NaN; an overflowing sum of squares gives scale 0, hence zeros, and NaN where the element
itself is infinite; subnormal inputs are kept, not flushed). The kernels must agree with the oracle on WHERE the
non-finite results are, and within the usual bar where they are finite (cf. src/deltanet_ref.rs:322-341: adversarial
values must behave)."""
import numpy as np
import pytest

import synth
from synth import F32

pytestmark = pytest.mark.gpu


def same_nonfinite_pattern(got, ref, what):
    assert np.array_equal(np.isnan(got), np.isnan(ref)), f"{what}: NaNs in different places"
    inf = np.isinf(ref)
    assert np.array_equal(np.isinf(got), inf) and np.array_equal(np.sign(got[inf]), np.sign(ref[inf])), f"{what}: infinities differ"
    fin = np.isfinite(ref)
    err = np.abs(got[fin].astype(np.float64) - ref[fin].astype(np.float64))
    tol = 1e-5 + 1e-6 * np.abs(ref[fin].astype(np.float64))
    assert (err <= tol).all(), f"{what}: finite values off by {float(err.max()):.3e}"


def special_rows(dim, seed):
    rng = np.random.default_rng(seed)
    base = rng.standard_normal((10, dim)).astype(np.float32)
    base[1, 3] = np.nan                      # one NaN poisons its row
    base[2, 5] = np.inf                      # an infinity: sum of squares is inf, scale 0, inf * 0 = NaN there
    base[3, :] = 0.0                         # all zeros: scale = 1/sqrt(eps), result zeros
    base[4, :] = 1e-41                       # subnormals survive the load
    base[5, :] *= np.float32(1e25)           # squares overflow f32
    base[6, 7] = -np.inf
    base[7, :] = np.float32(3.0e38)
    base[8, ::2] = -0.0
    return base


@pytest.mark.parametrize("dim", [64, 1024, 1000, 4096])
def test_rmsnorm_and_add_rmsnorm_on_special_rows(ctx, dev, oracle, dim):
    x = special_rows(dim, dim)
    w = (1 + 0.1 * np.random.default_rng(1).standard_normal(dim)).astype(np.float32)
    rows = x.shape[0]
    with np.errstate(all="ignore"):
        _, ref = oracle.add_rmsnorm_rows(x, None, w, 1e-6)
        delta = np.zeros_like(x)
        delta[9, :] = np.float32(3.0e38)
        x9 = x.copy()
        x9[9, :] = np.float32(3.0e38)        # the residual sum itself overflows to +inf
        ref_x, ref_fused = oracle.add_rmsnorm_rows(x9, delta, w, 1e-6)
    dx, dy = dev.put(x), dev.empty((rows, dim), F32, fill=7.0)
    ctx.rmsnorm(dx, dev.put(w), dy, rows=rows, dim=dim, eps=1e-6, dtype=F32, w_dtype=F32)
    ctx.stream_sync()
    same_nonfinite_pattern(dev.get(dy), ref, f"rmsnorm dim {dim}")
    dx9 = dev.put(x9)
    ctx.add_rmsnorm(dx9, dev.put(delta), dev.put(w), dy, rows=rows, dim=dim, eps=1e-6, dtype=F32, w_dtype=F32)
    ctx.stream_sync()
    same_nonfinite_pattern(dev.get(dx9), ref_x, f"residual sum dim {dim}")
    same_nonfinite_pattern(dev.get(dy), ref_fused, f"add_rmsnorm dim {dim}")


def test_swiglu_on_special_values(ctx, dev, oracle):
    g = np.array([np.inf, -np.inf, np.nan, 0.0, -0.0, 1e-41, -1e-41, 3e38, -3e38, 89.0, -89.0, 104.0, -104.0, 1.0], np.float32)
    for u_val in (1.5, 0.0, np.inf, -2.0):
        u = np.full_like(g, u_val)
        with np.errstate(all="ignore"):
            ref = oracle.swiglu(g, u)
        out = dev.empty((g.size,), F32, fill=7.0)
        ctx.swiglu(dev.put(g), dev.put(u), out, n=g.size, dtype=F32)
        ctx.stream_sync()
        same_nonfinite_pattern(dev.get(out), ref, f"swiglu with up = {u_val}")


def test_rope_on_special_values(ctx, dev, oracle):
    nq, nkv, hd, rows = 2, 1, 64, 6
    rng = np.random.default_rng(3)
    q = rng.standard_normal((rows, nq * hd)).astype(np.float32)
    k = rng.standard_normal((rows, nkv * hd)).astype(np.float32)
    q[1, 0], q[2, 40], k[3, 5], q[4, :] = np.inf, np.nan, -np.inf, 1e-41
    q[5, :] = np.float32(3e38)               # a rotation can overflow: a*cos - b*sin with both near the f32 limit
    with np.errstate(all="ignore"):
        rq, rk = oracle.qk_rope_rows(q, k, n_q_heads=nq, n_kv_heads=nkv, head_dim=hd, theta=1e4, pos0=7)
    dq, dk = dev.put(q), dev.put(k)
    p = ctx.qk_rope_params(q=dq, k=dk, rows=rows, n_q_heads=nq, n_kv_heads=nkv, head_dim=hd, q_dtype=F32, w_dtype=F32)
    ctx.qk_rope_pos(p, theta=1e4, pos0=7)
    ctx.stream_sync()
    for got, ref, name in ((dev.get(dq), rq, "q"), (dev.get(dk), rk, "k")):
        assert np.array_equal(np.isnan(got), np.isnan(ref)) and np.array_equal(np.isinf(got), np.isinf(ref)), f"rope {name}: non-finite pattern"
        fin = np.isfinite(ref)
        assert (np.abs(got[fin].astype(np.float64) - ref[fin]) <= 1e-5 + 2e-6 * np.abs(ref[fin].astype(np.float64))).all(), f"rope {name}"
