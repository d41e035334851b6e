"""Per-token ops of the gated-deltanet (qwen35) blocks: the gate scalars, the depthwise causal conv with its rolling
window, and the bf16 -> f16 page conversion of the weight stage-in.

CPU part: the oracle against the known answers of the reference's own tests (src/deltanet_ref.rs:225-236, 289-303)
and against a second, windowed reading of the conv (the whole-chunk form of src/gpu/kernels.metal:4039-4068).
GPU part: the kernels through the C ABI against the oracle. Softplus above its threshold, the rolled window and the
page conversion are bit-exact; the rest is bounded by the f32 bar of the other ops."""
import numpy as np
import pytest

import lokal_b200 as L
import synth
from synth import BF16, F16, F32


def windowed_conv(state, x, w, k):
    """The whole-chunk form: token t's window is x[t-(k-1) .. t-1], or state entries for negative indices."""
    n, ch = x.shape
    out = np.empty_like(x)
    for t in range(n):
        acc = np.zeros(ch, np.float32)
        for j in range(k - 1):
            u = t - (k - 1) + j
            wv = state[:, k - 1 + u] if u < 0 else x[u]
            acc = (acc + (wv * w[:, j]).astype(np.float32)).astype(np.float32)
        acc = (acc + (x[t] * w[:, k - 1]).astype(np.float32)).astype(np.float32)
        out[t] = acc
    new_state = np.empty_like(state)
    for m in range(k - 1):
        u = n - (k - 1) + m
        new_state[:, m] = state[:, k - 1 + u] if u < 0 else x[u]
    return out, new_state


# ---- the oracle against the reference's known answers (no GPU) ----

def test_oracle_scalar_forms_known_answers(oracle):
    # src/deltanet_ref.rs:225-236
    assert oracle.softplus(25.0) == 25.0  # the > 20 shortcut, exact
    assert abs(oracle.softplus(0.0) - np.float32(np.log(2.0))) < 1e-7
    assert 0.0 <= oracle.softplus(-100.0) < 1e-6
    g, beta = oracle.delta_gates(np.array([[25.0, 0.0]], np.float32), np.array([[0.0, 100.0]], np.float32),
                                 np.array([-2.0, -0.5], np.float32), np.array([0.0, 0.0], np.float32))
    assert g[0, 0] == -50.0 and abs(g[0, 1] + 0.5 * np.log(2.0)) < 1e-7
    assert beta[0, 0] == 0.5 and beta[0, 1] == 1.0


def test_oracle_conv_step_hand_vector_and_roll(oracle):
    # src/deltanet_ref.rs:289-303: three channels, two taps
    out, state = oracle.ssm_conv(np.array([[10.0], [20.0], [30.0]], np.float32), np.array([[1.0, 2.0, 3.0]], np.float32),
                                 np.array([[1.0, 2.0], [0.5, 0.5], [-1.0, 1.0]], np.float32), 2)
    assert abs(out[0, 0] - 12.0 * oracle.sigmoid(12.0)) < 1e-4
    assert abs(out[0, 1] - 11.0 * oracle.sigmoid(11.0)) < 1e-4
    assert abs(out[0, 2]) < 1e-6
    assert (state.ravel() == [1.0, 2.0, 3.0]).all()


@pytest.mark.parametrize("k,n", [(4, 1), (4, 2), (4, 3), (4, 50), (2, 7), (3, 2), (8, 5), (1, 4)])
def test_oracle_sequential_steps_equal_the_windowed_form(oracle, k, n):
    # the reference's claim (src/gpu/kernels.metal:4046-4052): the whole-chunk form is bit-identical to n decode steps
    rng = np.random.default_rng(k * 100 + n)
    ch = 12
    state = rng.standard_normal((ch, k - 1)).astype(np.float32)
    x = rng.standard_normal((n, ch)).astype(np.float32)
    w = rng.standard_normal((ch, k)).astype(np.float32)
    out, new_state = oracle.ssm_conv(state, x, w, k)
    acc, want_state = windowed_conv(state, x, w, k)
    sig = np.array([oracle.sigmoid(float(v)) for v in acc.ravel()], np.float32).reshape(acc.shape)
    synth.assert_bits_equal(out, (acc * sig).astype(np.float32), "conv outputs")
    synth.assert_bits_equal(new_state.reshape(ch, k - 1), want_state, "rolled window")


def test_oracle_bf16_to_f16_all_patterns(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    got, clip = oracle.bf16_to_f16(bits)
    f32 = (bits.astype(np.uint32) << 16).view(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        want = f32.astype(np.float16).view(np.uint16)
    nan = np.isnan(f32)
    assert (got[~nan] == want[~nan]).all() and (np.isnan(got[nan].view(np.float16))).all()
    assert clip == 1
    small, clip = oracle.bf16_to_f16(np.array([0x3F80, 0x477F, 0x7F80, 0xFF80], np.uint16))  # 1, 65280, +inf, -inf
    assert clip == 0 and small[1] == np.float16(65280.0).view(np.uint16)
    _, clip = oracle.bf16_to_f16(np.array([0x4780], np.uint16))  # 65536 is finite in bf16, not in f16
    assert clip == 1


# ---- the kernels through the C ABI ----

@pytest.mark.gpu
@pytest.mark.parametrize("n_tokens,heads", [(1, 48), (300, 48), (4096, 32), (7, 5)])
def test_gpu_delta_gates(ctx, dev, oracle, n_tokens, heads):
    rng = np.random.default_rng(n_tokens * 7 + heads)
    alpha = (rng.standard_normal((n_tokens, heads)) * 8).astype(np.float32)
    alpha.ravel()[::5] += 30.0  # above the softplus threshold: no transcendental runs, so these must be bit-exact
    beta_in = (rng.standard_normal((n_tokens, heads)) * 4).astype(np.float32)
    a = -np.exp(rng.standard_normal(heads)).astype(np.float32)
    dt_bias = rng.standard_normal(heads).astype(np.float32)
    g, beta = dev.empty((n_tokens, heads), F32, fill=7.0), dev.empty((n_tokens, heads), F32, fill=7.0)
    ctx.delta_gates(dev.put(alpha), dev.put(beta_in), dev.put(a), dev.put(dt_bias), g, beta, n_v_heads=heads, n_tokens=n_tokens)
    ctx.stream_sync()
    rg, rb = oracle.delta_gates(alpha, beta_in, a, dt_bias)
    got_g, got_b = dev.get(g), dev.get(beta)
    above = (alpha + dt_bias[None, :]).astype(np.float32) > 20.0
    assert above.any()
    synth.assert_bits_equal(got_g[above], rg[above], "g above the softplus threshold")
    # 1 + exp(x) may round to the neighbouring float when exp differs in its last bit: 1.2e-7 of softplus, times |a|
    assert np.all(np.abs(got_g - rg) <= 1e-6 * np.abs(rg) + 2.5e-7 * np.abs(a)[None, :]), float(np.abs(got_g - rg).max())
    assert np.all(np.abs(got_b - rb) <= 2e-7), float(np.abs(got_b - rb).max())
    # in place, as a caller that keeps no copy of the projections would run it
    da, db = dev.put(alpha), dev.put(beta_in)
    ctx.delta_gates(da, db, dev.put(a), dev.put(dt_bias), da, db, n_v_heads=heads, n_tokens=n_tokens)
    ctx.stream_sync()
    synth.assert_bits_equal(dev.get(da), got_g, "in-place g")
    synth.assert_bits_equal(dev.get(db), got_b, "in-place beta")


def run_conv(ctx, dev, state, x, w, k, dtype, roll=True):
    n, ch = x.shape
    dstate = dev.put(state) if k > 1 else None
    out = dev.empty((n + 1, ch), dtype, fill=7.0)
    ctx.ssm_conv(dstate, dev.put(x, dtype), dev.put(w), out, channels=ch, d_conv=k, n_tokens=n, dtype=dtype, roll=roll)
    ctx.stream_sync()
    got = dev.get(out)
    assert (got[-1] == 7.0).all(), "wrote past the last token"
    return got[:-1], (dev.get(dstate) if k > 1 else state)


@pytest.mark.gpu
def test_gpu_conv_reference_hand_vector(ctx, dev, oracle):
    state = np.array([[10.0], [20.0], [30.0]], np.float32)
    x = np.array([[1.0, 2.0, 3.0]], np.float32)
    w = np.array([[1.0, 2.0], [0.5, 0.5], [-1.0, 1.0]], np.float32)
    out, new_state = run_conv(ctx, dev, state, x, w, 2, F32)
    assert abs(out[0, 0] - 12.0 * oracle.sigmoid(12.0)) < 1e-4 and abs(out[0, 1] - 11.0 * oracle.sigmoid(11.0)) < 1e-4
    assert abs(out[0, 2]) < 1e-6 and (new_state.ravel() == [1.0, 2.0, 3.0]).all()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, F16, BF16])
@pytest.mark.parametrize("k,n,ch", [(4, 1, 10240), (4, 2, 1024), (4, 3, 1024), (4, 37, 1024), (4, 300, 10240), (4, 2500, 512),
                                     (2, 9, 64), (3, 2, 40), (8, 5, 128), (1, 6, 64), (4, 33, 10), (4, 70, 1028), (5, 1, 7)])
def test_gpu_conv_shapes(ctx, dev, oracle, dtype, k, n, ch):
    rng = np.random.default_rng(k * 1000 + n * 7 + ch)
    state = synth.round_to(rng.standard_normal((ch, max(k - 1, 0))).astype(np.float32), dtype)
    x = synth.round_to(rng.standard_normal((n, ch)).astype(np.float32), dtype)
    w = (rng.standard_normal((ch, k)) * 0.5).astype(np.float32)
    out, new_state = run_conv(ctx, dev, state, x, w, k, dtype)
    ref, ref_state = oracle.ssm_conv(state, x, w, k)
    if dtype == F32:
        synth.check_f32(out, ref, f"conv k={k} n={n} C={ch}")
    else:
        synth.check_half(out, ref, f"conv k={k} n={n} C={ch}", dtype, atol=1e-6)
    if k > 1:
        synth.assert_bits_equal(new_state, ref_state.reshape(ch, k - 1), "rolled window")


@pytest.mark.gpu
def test_gpu_conv_chunk_equals_decode_steps_bit_for_bit(ctx, dev):
    # the property the reference builds its prefill kernel on (src/gpu/kernels.metal:4046-4052)
    rng = np.random.default_rng(77)
    k, n, ch = 4, 45, 2048
    state = rng.standard_normal((ch, k - 1)).astype(np.float32)
    x = rng.standard_normal((n, ch)).astype(np.float32)
    w = (rng.standard_normal((ch, k)) * 0.5).astype(np.float32)
    whole, whole_state = run_conv(ctx, dev, state, x, w, k, F32)
    dstate, dw = dev.put(state), dev.put(w)
    steps = np.empty_like(whole)
    for t in range(n):
        o = dev.empty((1, ch), F32)
        ctx.ssm_conv(dstate, dev.put(x[t:t + 1]), dw, o, channels=ch, d_conv=k, n_tokens=1, dtype=F32, roll=True)
        ctx.stream_sync()
        steps[t] = dev.get(o)[0]
    synth.assert_bits_equal(whole, steps, "chunk vs decode steps")
    synth.assert_bits_equal(whole_state, dev.get(dstate), "window after the chunk vs after the steps")


@pytest.mark.gpu
def test_gpu_conv_without_roll_leaves_the_window_and_refusals(ctx, dev, oracle):
    rng = np.random.default_rng(5)
    k, n, ch = 4, 100, 256
    state = rng.standard_normal((ch, k - 1)).astype(np.float32)
    x = rng.standard_normal((n, ch)).astype(np.float32)
    w = rng.standard_normal((ch, k)).astype(np.float32)
    out, kept = run_conv(ctx, dev, state, x, w, k, F32, roll=False)
    synth.assert_bits_equal(kept, state, "window must stay when roll is off")
    synth.check_f32(out, oracle.ssm_conv(state, x, w, k)[0], "conv without roll")
    # negative control: feeding the window newest-first must be caught by the same comparison
    flipped, _ = run_conv(ctx, dev, state[:, ::-1].copy(), x, w, k, F32, roll=False)
    assert np.abs(flipped[:3] - out[:3]).max() > 1e-3
    dx = dev.put(x)
    for kwargs, status in ((dict(d_conv=9), L.capi.ERR_UNSUPPORTED), (dict(d_conv=0), L.capi.ERR_UNSUPPORTED), (dict(dtype=L.Q8_0), L.capi.ERR_UNSUPPORTED),
                           (dict(channels=0), L.capi.ERR_BAD_ARG)):
        args = dict(channels=ch, d_conv=k, n_tokens=n, dtype=F32)
        args.update(kwargs)
        with pytest.raises(L.LokalCudaError) as e:
            ctx.ssm_conv(dev.put(state), dx, dev.put(w), dev.empty((n, ch), F32), **args)
        assert e.value.status == status
    with pytest.raises(L.LokalCudaError) as e:  # in place would let later tokens read outputs
        ctx.ssm_conv(dev.put(state), dx, dev.put(w), dx, channels=ch, d_conv=k, n_tokens=n, dtype=F32)
    assert e.value.status == L.capi.ERR_BAD_ARG
    with pytest.raises(L.LokalCudaError) as e:
        ctx.ssm_conv(None, dx, dev.put(w), dev.empty((n, ch), F32), channels=ch, d_conv=k, n_tokens=n, dtype=F32)
    assert e.value.status == L.capi.ERR_BAD_ARG


@pytest.mark.gpu
def test_gpu_bf16_to_f16_all_patterns_and_clip_flag(ctx, dev, oracle):
    t = dev.torch
    bits = np.tile(np.arange(65536, dtype=np.uint16), 3)[: 3 * 65536 - 5]  # a ragged tail for the scalar path
    want, _ = oracle.bf16_to_f16(bits)
    src = t.from_numpy(bits.view(np.int16)).cuda()
    dst = t.zeros(bits.size + 8, dtype=t.int16, device="cuda")
    flag = t.zeros(1, dtype=t.int32, device="cuda")
    ctx.bf16_to_f16_copy(src, dst, n=bits.size, clip_flag=flag)
    ctx.stream_sync()
    got = dst.cpu().numpy().view(np.uint16)
    assert (got[bits.size:] == 0).all(), "wrote past the end"
    nan = np.isnan((bits.astype(np.uint32) << 16).view(np.float32))
    assert (got[:bits.size][~nan] == want[~nan]).all() and np.isnan(got[:bits.size][nan].view(np.float16)).all()
    assert int(flag.item()) == 1
    # in-range page: the flag stays clear; source two bytes off a 16-byte boundary takes the per-element path
    rng = np.random.default_rng(3)
    vals = (rng.standard_normal(100_003) * 100).astype(np.float32)
    page = (vals.view(np.uint32) >> 16).astype(np.uint16)
    page[:2] = (0x7F80, 0xFF80)  # infinities are not clipping
    want, clip = oracle.bf16_to_f16(page)
    assert clip == 0
    for shift in (0, 1):
        buf = t.zeros(page.size + 9, dtype=t.int16, device="cuda")
        buf[shift:shift + page.size] = t.from_numpy(page.view(np.int16)).cuda()
        out = t.zeros(page.size, dtype=t.int16, device="cuda")
        flag.zero_()
        ctx.bf16_to_f16_copy(buf[shift:], out, n=page.size, clip_flag=flag)
        ctx.stream_sync()
        assert (out.cpu().numpy().view(np.uint16) == want).all() and int(flag.item()) == 0
    ctx.bf16_to_f16_copy(src, dst, n=bits.size)  # no flag wanted
    ctx.stream_sync()
