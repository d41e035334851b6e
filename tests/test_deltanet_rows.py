"""The gated-deltanet (qwen35) per-row siblings: l2norm_rows, gated_output_norm, attn_out_gate, split_q_gate.

The reference tests each of them in two halves (src/gpu/metal.rs:5668-5950, 6611-6752): an EXACT half on inputs whose
sums are exactly representable (bit-for-bit), and a BOUNDED half on random inputs, where the device may differ from
the CPU code by at most 4x a measured one-rounding yardstick; plus a negative control per op. Same here, with the
reference's seeds and input recipes."""
import numpy as np
import pytest

import lokal_b200 as L
import synth
from synth import BF16, F16, F32


def lcg_stream(seed, n):
    """The reference's test LCG (src/gpu/metal.rs:5088-5091): uniform f32 in [-1, 1)."""
    out = np.empty(n, np.float32)
    for i in range(n):
        seed = (seed * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(seed >> 8) / np.float32(1 << 24)) * np.float32(2.0) - np.float32(1.0)
    return out, seed


def rel_err(a, b):
    scale = np.maximum(np.abs(a), np.abs(b))
    with np.errstate(invalid="ignore", divide="ignore"):
        return float(np.max(np.where(scale == 0, 0.0, np.abs(a - b) / scale)))


# ---- the oracle against the reference's CPU known answers (no GPU) ----

def test_oracle_l2_norm_known_answers(oracle):
    # src/deltanet_ref.rs:229-235, 327-329
    v = oracle.l2norm_rows(np.array([3.0, 4.0], np.float32), 2, 1e-6)
    assert abs(v[0] - 0.6) < 1e-7 and abs(v[1] - 0.8) < 1e-7
    assert (oracle.l2norm_rows(np.zeros(2, np.float32), 2, 1e-6) == 0).all()  # scale = 1/eps, stays a finite zero
    assert np.isfinite(oracle.l2norm_rows(np.array([1e-40, 1e-41], np.float32), 2, 1e-6)).all()


def test_oracle_gated_norm_and_attn_gate_known_answers(oracle):
    # src/deltanet_ref.rs:306-320: d_state 2, two heads
    o = oracle.gated_output_norm(np.array([[1, 2], [3, 4]], np.float32), np.ones(2, np.float32),
                                 np.array([[0, 1], [-1, 10]], np.float32), 1e-6)
    rms = np.sqrt(np.float32(2.5) + np.float32(1e-6))
    silu = lambda x: np.float32(x) * np.float32(oracle.sigmoid(x))
    assert abs(o[0, 0] - 1.0 / rms * silu(0.0)) < 1e-6 and abs(o[0, 1] - 2.0 / rms * silu(1.0)) < 1e-6
    a = oracle.attn_out_gate(np.array([2, 2], np.float32), np.array([0, 100], np.float32))
    assert abs(a[0] - 1.0) < 1e-7 and abs(a[1] - 2.0) < 1e-6
    assert oracle.sigmoid(0.0) == 0.5 and oracle.sigmoid(100.0) == 1.0 and oracle.sigmoid(-100.0) < 1e-40


def test_oracle_f64_sum_differs_from_f32_sum_on_random_rows(oracle):
    # the gap the reference's bounded halves measure must exist, or those halves prove nothing
    x, _ = lcg_stream(0x1234ABCD, 6 * 128)
    want = oracle.l2norm_rows(x.reshape(6, 128), 128, 1e-6)
    rows = x.reshape(6, 128)
    s32 = np.array([np.sum((r * r).astype(np.float32), dtype=np.float32) for r in rows], np.float32)
    narrowed = rows * (np.float32(1.0) / np.maximum(np.sqrt(s32), np.float32(1e-6)))[:, None]
    assert 0 < rel_err(want, narrowed) < 1e-6


def test_oracle_split_q_gate(oracle):
    src = np.arange(2 * 3 * 2 * 4, dtype=np.float32)
    q, g = oracle.split_q_gate(src, 2, 3, 4)
    v = src.reshape(2, 3, 2, 4)
    assert np.array_equal(q, v[:, :, 0].reshape(2, 12)) and np.array_equal(g, v[:, :, 1].reshape(2, 12))


# ---- l2norm_rows on the device ----

def gpu_l2norm(ctx, dev, rows, eps, dtype=F32, **kw):
    t = dev.put(np.ascontiguousarray(rows, np.float32), dtype)
    ctx.l2norm_rows(t, dim=rows.shape[-1], eps=eps, rows_per_token=rows.size // rows.shape[-1], dtype=dtype, **kw)
    ctx.stream_sync()
    return dev.get(t)


@pytest.mark.gpu
def test_l2norm_matches_reference_where_the_sums_agree(ctx, dev, oracle):
    # src/gpu/metal.rs:6648-6669: small integers, every partial sum exact in f32 and f64, in any order
    x, _ = lcg_stream(0xC0FFEE11, 6 * 128)
    rows = np.round(x * 8.0).reshape(6, 128)
    synth.assert_bits_equal(gpu_l2norm(ctx, dev, rows, 1e-6), oracle.l2norm_rows(rows, 128, 1e-6), "l2norm, exact half")


@pytest.mark.gpu
def test_l2norm_zero_row_is_zero_not_nan(ctx, dev, oracle):
    # src/gpu/metal.rs:6671-6693: dropping the clamp gives 0 * inf = NaN
    rows = np.stack([np.zeros(128, np.float32), np.ones(128, np.float32)])
    got = gpu_l2norm(ctx, dev, rows, 1e-6)
    assert not np.isnan(got).any()
    synth.assert_bits_equal(got, oracle.l2norm_rows(rows, 128, 1e-6), "zero row and ones row")
    assert (got[0] == 0).all() and abs(got[1, 0] - 1.0 / np.sqrt(128.0)) < 1e-7


@pytest.mark.gpu
def test_l2norm_bounded_by_the_measured_accumulation_gap(ctx, dev, oracle):
    # src/gpu/metal.rs:6695-6745. The device sums in f64 like the CPU code, so it must also sit far inside the bound.
    x, _ = lcg_stream(0x1234ABCD, 6 * 128)
    rows = x.reshape(6, 128)
    want = oracle.l2norm_rows(rows, 128, 1e-6)
    s32 = np.array([np.sum((r * r).astype(np.float32), dtype=np.float32) for r in rows], np.float32)
    narrowed = rows * (np.float32(1.0) / np.maximum(np.sqrt(s32), np.float32(1e-6)))[:, None]
    yardstick = rel_err(want, narrowed)
    got = gpu_l2norm(ctx, dev, rows, 1e-6)
    assert yardstick > 0, "narrowing the sum to f32 changed nothing: probe is broken"
    assert rel_err(want, got) <= 4.0 * yardstick
    assert np.mean(got.view(np.uint32) == want.view(np.uint32)) > 0.99, "an f64 sum should reproduce the CPU bits"


@pytest.mark.gpu
def test_l2norm_batched_addressing_and_other_widths(ctx, dev, oracle):
    # rows of token t start at t*tok_stride (src/gpu/kernels.metal:3708-3720); the gap between tokens is not touched
    rng = np.random.default_rng(5)
    rpt, ntok, dim, stride = 4, 3, 128, 4 * 128 + 64
    buf = rng.standard_normal(ntok * stride).astype(np.float32)
    want = oracle.l2norm_rows(buf, dim, 1e-6, rows_per_token=rpt, n_tokens=ntok, tok_stride=stride)
    t = dev.put(buf)
    ctx.l2norm_rows(t, dim=dim, eps=1e-6, rows_per_token=rpt, n_tokens=ntok, tok_stride=stride)
    ctx.stream_sync()
    got = dev.get(t)
    assert np.mean(got.view(np.uint32) == want.view(np.uint32)) > 0.99 and rel_err(want, got) < 2e-7
    gap = np.concatenate([np.arange(tk * stride + rpt * dim, (tk + 1) * stride) for tk in range(ntok)])
    assert np.array_equal(got[gap], buf[gap])
    # widths that take two and four vectors per lane, one that is not vectorisable and one beyond a warp's registers
    for dim in (256, 512, 100, 5000):
        rows = rng.standard_normal((37, dim)).astype(np.float32)
        got = gpu_l2norm(ctx, dev, rows, 1e-6)
        want = oracle.l2norm_rows(rows, dim, 1e-6)
        assert rel_err(want, got) < 2e-7, dim
        y = dev.empty((37, dim), F32, fill=0.0)  # out of place
        xin = dev.put(rows)
        ctx.l2norm_rows(xin, y, dim=dim, eps=1e-6, rows_per_token=37)
        ctx.stream_sync()
        synth.assert_bits_equal(dev.get(y), got, "out of place == in place")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F16, BF16])
def test_l2norm_16_bit_rows(ctx, dev, oracle, dtype):
    rng = np.random.default_rng(dtype)
    rows = synth.round_to(rng.standard_normal((300, 128)).astype(np.float32), dtype)
    got = gpu_l2norm(ctx, dev, rows, 1e-6, dtype=dtype)
    synth.check_half(got, oracle.l2norm_rows(rows, 128, 1e-6), "l2norm 16-bit", dtype, atol=1e-6)


# ---- gated_output_norm ----

def gpu_gated(ctx, dev, o, w, z, eps, dtype=F32, w_dtype=F32):
    t = dev.put(np.ascontiguousarray(o, np.float32), dtype)
    ctx.gated_output_norm(t, dev.put(np.ascontiguousarray(w, np.float32), w_dtype), dev.put(np.ascontiguousarray(z, np.float32), dtype),
                          rows=o.shape[0], dim=o.shape[1], eps=eps, dtype=dtype, w_dtype=w_dtype)
    ctx.stream_sync()
    return dev.get(t)


@pytest.mark.gpu
def test_gated_output_norm_matches_reference_where_the_sums_agree(ctx, dev, oracle):
    # src/gpu/metal.rs:5837-5852: integer o and w, z = 100 so silu(z) = 100 exactly (d_state 128, 4 V heads)
    s, h = 128, 4
    x, seed = lcg_stream(0xBEEF0001, s * h)
    o = np.round(x * 8.0).reshape(h, s)
    w = np.round(lcg_stream(seed, s)[0] * 4.0)
    z = np.full((h, s), 100.0, np.float32)
    synth.assert_bits_equal(gpu_gated(ctx, dev, o, w, z, 1e-5), oracle.gated_output_norm(o, w, z, 1e-5), "gated norm, exact half")


def gated_inputs(seed, s=128, h=4):
    x, seed = lcg_stream(seed, s * h)
    w, seed = lcg_stream(seed, s)
    z, seed = lcg_stream(seed, s * h)
    return x.reshape(h, s), w, (z * np.float32(4.0)).reshape(h, s)


@pytest.mark.gpu
def test_gated_output_norm_bounded_by_its_two_measured_floors(ctx, dev, oracle):
    # src/gpu/metal.rs:5854-5895: yardstick = max(f64-vs-f32 mean gap, 2^-24)
    o, w, z = gated_inputs(0xBEEF0002)
    want = oracle.gated_output_norm(o, w, z, 1e-5)
    silu = np.array([np.float32(v) * np.float32(oracle.sigmoid(float(v))) for v in z.reshape(-1)], np.float32).reshape(z.shape)
    mean32 = np.array([np.sum((r * r).astype(np.float32), dtype=np.float32) / np.float32(128) for r in o], np.float32)
    scale = np.float32(1.0) / np.sqrt(mean32 + np.float32(1e-5))
    narrowed = ((o * scale[:, None]) * w[None, :]) * silu
    accum_gap = rel_err(want, narrowed)
    yardstick = max(accum_gap, 2.0 ** -24)
    got = gpu_gated(ctx, dev, o, w, z, 1e-5)
    assert accum_gap > 0, "narrowing the mean changed nothing: probe is broken"
    assert rel_err(want, got) <= 4.0 * yardstick


@pytest.mark.gpu
def test_gated_output_norm_oracle_sees_a_misaligned_weight(ctx, dev, oracle):
    # src/gpu/metal.rs:5897-5915
    o, w, z = gated_inputs(0xBEEF0003)
    got = gpu_gated(ctx, dev, o, w, z, 1e-5)
    wrong = oracle.gated_output_norm(o, np.roll(w, -1), z, 1e-5)
    assert (got.view(np.uint32) != wrong.view(np.uint32)).any()
    assert rel_err(oracle.gated_output_norm(o, w, z, 1e-5), got) < 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,w_dtype", [(F16, F16), (BF16, BF16), (BF16, F32), (F32, BF16)])
@pytest.mark.parametrize("dim", [128, 256, 72])
def test_gated_output_norm_storage_types_and_widths(ctx, dev, oracle, dtype, w_dtype, dim):
    rng = np.random.default_rng(dim + dtype)
    o = synth.round_to(rng.standard_normal((211, dim)).astype(np.float32), dtype)
    z = synth.round_to(rng.standard_normal((211, dim)).astype(np.float32) * 3, dtype)
    w = synth.round_to(1 + 0.1 * rng.standard_normal(dim).astype(np.float32), w_dtype)
    got = gpu_gated(ctx, dev, o, w, z, 1e-6, dtype, w_dtype)
    want = oracle.gated_output_norm(o, w, z, 1e-6)
    if dtype == F32:
        assert rel_err(want, got) < 1e-6
    else:
        synth.check_half(got, want, "gated norm 16-bit", dtype, atol=1e-6)


# ---- attn_out_gate ----

def gpu_gate(ctx, dev, attn, gate, dtype=F32):
    t = dev.put(np.ascontiguousarray(attn, np.float32), dtype)
    ctx.attn_out_gate(t, dev.put(np.ascontiguousarray(gate, np.float32), dtype), n=attn.size, dtype=dtype)
    ctx.stream_sync()
    return dev.get(t)


@pytest.mark.gpu
def test_attn_out_gate_is_exact_at_saturation_and_zero(ctx, dev, oracle):
    # src/gpu/metal.rs:5708-5722: sigma(0) = 0.5, sigma(100) = 1, sigma(-100) = 0 in any implementation
    attn, _ = lcg_stream(0x7A110000, 256)
    gate = np.array([(0.0, 100.0, -100.0)[i % 3] for i in range(256)], np.float32)
    got = gpu_gate(ctx, dev, attn, gate)
    want = oracle.attn_out_gate(attn, gate)
    synth.assert_bits_equal(got[1::3], attn[1::3], "an open gate must leave values alone")
    assert (got[2::3] == 0).all()  # exp(100) overflows to inf, 1 / inf = 0: a zero, not NaN
    synth.assert_bits_equal(got, want, "attn_out_gate, exact half")


@pytest.mark.gpu
def test_attn_out_gate_bounded_by_sigmoids_measured_floor(ctx, dev, oracle):
    # src/gpu/metal.rs:5724-5771: exp nudged by one f32 rounding inside the reference's own sigmoid is the yardstick
    attn, seed = lcg_stream(0x7A110001, 1024)
    gate, _ = lcg_stream(seed, 1024)
    # the reference interleaves nothing here: attn is drawn first, then gate, both from one stream
    attn, gate = attn * np.float32(4.0), gate * np.float32(8.0)
    want = oracle.attn_out_gate(attn, gate)
    e = np.exp(-gate.astype(np.float64)).astype(np.float32) * (np.float32(1.0) + np.float32(np.finfo(np.float32).eps))
    nudged = attn * (np.float32(1.0) / (np.float32(1.0) + e))
    yardstick = rel_err(want, nudged)
    got = gpu_gate(ctx, dev, attn, gate)
    assert yardstick > 0
    assert rel_err(want, got) <= 4.0 * yardstick


@pytest.mark.gpu
def test_attn_out_gate_oracle_sees_a_misaligned_gate(ctx, dev, oracle):
    # src/gpu/metal.rs:5773-5792
    attn, seed = lcg_stream(0x7A110002, 256)
    gate = lcg_stream(seed, 256)[0] * np.float32(4.0)
    got = gpu_gate(ctx, dev, attn, gate)
    assert (got.view(np.uint32) != oracle.attn_out_gate(attn, np.roll(gate, -1)).view(np.uint32)).any()
    assert rel_err(oracle.attn_out_gate(attn, gate), got) < 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, F16, BF16])
@pytest.mark.parametrize("n", [1, 7, 4096 + 3, 1 << 20])
def test_attn_out_gate_sizes_and_types(ctx, dev, oracle, dtype, n):
    rng = np.random.default_rng(n)
    attn = synth.round_to(rng.standard_normal(n).astype(np.float32) * 2, dtype)
    gate = synth.round_to(rng.standard_normal(n).astype(np.float32) * 4, dtype)
    got = gpu_gate(ctx, dev, attn, gate, dtype)
    want = oracle.attn_out_gate(attn, gate)
    if dtype == F32:
        assert rel_err(want, got) < 1e-6
    else:
        synth.check_half(got, want, "attn_out_gate 16-bit", dtype, atol=1e-7)


# ---- split_q_gate ----

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, F16, BF16])
@pytest.mark.parametrize("rows,heads,hd", [(5, 16, 256), (33, 3, 64), (4, 2, 6), (1, 1, 1)])
def test_split_q_gate_is_a_pure_copy(ctx, dev, oracle, dtype, rows, heads, hd):
    rng = np.random.default_rng(rows * hd)
    src = synth.round_to(rng.standard_normal(rows * heads * 2 * hd).astype(np.float32), dtype)
    q = dev.empty((rows + 1, heads * hd), dtype, fill=7.0)
    g = dev.empty((rows + 1, heads * hd), dtype, fill=7.0)
    ctx.split_q_gate(dev.put(src, dtype), q, g, rows=rows, n_heads=heads, head_dim=hd, dtype=dtype)
    ctx.stream_sync()
    wq, wg = oracle.split_q_gate(src, rows, heads, hd)
    gq, gg = dev.get(q), dev.get(g)
    synth.assert_bits_equal(gq[:-1], wq, "q")
    synth.assert_bits_equal(gg[:-1], wg, "gate")
    assert (gq[-1] == 7.0).all() and (gg[-1] == 7.0).all()


@pytest.mark.gpu
def test_sibling_refusals(ctx, dev):
    a = dev.empty((4, 128), F32, fill=1.0)
    E = L.capi
    cases = [
        (lambda: ctx.l2norm_rows(a, dim=128, eps=1e-6, rows_per_token=4, dtype=L.Q8_0), E.ERR_UNSUPPORTED),
        (lambda: ctx.l2norm_rows(a, dim=0, eps=1e-6, rows_per_token=4), E.ERR_BAD_ARG),
        (lambda: ctx.l2norm_rows(a, dim=128, eps=1e-6, rows_per_token=2, n_tokens=2, tok_stride=128), E.ERR_BAD_ARG),
        (lambda: ctx.l2norm_rows(None, dim=128, eps=1e-6, rows_per_token=4), E.ERR_BAD_ARG),
        (lambda: ctx.gated_output_norm(a, None, a, rows=4, dim=128, eps=1e-6), E.ERR_BAD_ARG),
        (lambda: ctx.gated_output_norm(a, a, a, rows=4, dim=128, eps=1e-6, w_dtype=L.Q4_K), E.ERR_UNSUPPORTED),
        (lambda: ctx.attn_out_gate(a, None, n=8), E.ERR_BAD_ARG),
        (lambda: ctx.split_q_gate(a, a, a, rows=1, n_heads=1, head_dim=4), E.ERR_BAD_ARG),
        (lambda: ctx.split_q_gate(a, a[1:], a[2:], rows=1, n_heads=0, head_dim=4), E.ERR_BAD_ARG),
    ]
    for call, status in cases:
        with pytest.raises(L.LokalCudaError) as e:
            call()
        assert e.value.status == status
    ctx.l2norm_rows(a, dim=128, eps=1e-6, rows_per_token=0)
    ctx.attn_out_gate(a, a, n=0)
    ctx.stream_sync()
    assert (dev.get(a) == 1.0).all()
