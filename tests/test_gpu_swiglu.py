"""SiLU(gate) * up through the C ABI vs the CPU oracle.

Bar: max-abs 1e-5 on f32 (gate, up ~ N(0, 2): |out| reaches ~60, where one f32 ulp is 3.8e-6),
2e-3 relative on f16/bf16.
"""
import numpy as np
import pytest

import synth
from synth import BF16, F16, F32

pytestmark = pytest.mark.gpu


def run(ctx, dev, g, u, dtype, in_place=False, want_h=None):
    dg, du = dev.put(g, dtype), dev.put(u, dtype)
    n = g.size
    out = dg if in_place else dev.empty((n + 16,), dtype, fill=5.0)
    dh = dev.empty((n,), want_h, fill=0.0) if want_h else None
    ctx.swiglu(dg, du, out, n=n, dtype=dtype, out_h=dh, h_dtype=want_h or F16)
    ctx.stream_sync()
    res = dev.get(out).reshape(-1)
    if not in_place:
        assert (res[n:] == 5.0).all(), "wrote past the end"
    return res[:n].reshape(g.shape), (None if dh is None else dev.get(dh).reshape(g.shape))


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c5"])
def test_config_shapes(ctx, dev, oracle, name):
    cfg = synth.CONFIGS[name]
    rows = min(cfg.rows, 200)
    d = synth.layer_inputs(cfg, rows)
    got, _ = run(ctx, dev, d["gate"], d["up"], cfg.dtype)
    ref = oracle.swiglu(d["gate"], d["up"])
    assert np.abs(got).max() > 1.0
    if cfg.dtype == F32:
        synth.check_f32(got, ref, name)
    else:
        synth.check_half(got, ref, name, cfg.dtype)


def test_f32_error_by_magnitude(ctx, dev, oracle):
    # The absolute bar is tightest where |out| is largest: check the 1000 largest outputs on their own.
    rng = np.random.default_rng(11)
    g = rng.standard_normal(1 << 22, dtype=np.float32) * 2
    u = rng.standard_normal(1 << 22, dtype=np.float32) * 2
    got, _ = run(ctx, dev, g, u, F32)
    ref = oracle.swiglu(g, u)
    synth.check_f32(got, ref, "4M elements")
    top = np.argsort(-np.abs(ref))[:1000]
    assert np.abs(ref[top]).min() > 20
    ulp = np.spacing(np.abs(ref[top]))
    # a last-bit difference between the device's expf and libm's can move the quotient by one ulp, which the
    # multiply by u can turn into two ulps of the product; more than that would mean a different expression
    assert (np.abs(got[top] - ref[top]) <= 2 * ulp).all(), "a large output is more than two ulps off"
    assert (np.abs(got[top] - ref[top]) <= ulp).mean() > 0.9


@pytest.mark.parametrize("dtype", [F32, F16, BF16])
@pytest.mark.parametrize("n", [1, 3, 8, 31, 1000, 4097, 1 << 16])
def test_tails_and_alignment(ctx, dev, oracle, dtype, n):
    rng = np.random.default_rng(n)
    g = synth.round_to(rng.standard_normal(n, dtype=np.float32) * 2, dtype)
    u = synth.round_to(rng.standard_normal(n, dtype=np.float32) * 2, dtype)
    got, _ = run(ctx, dev, g, u, dtype)
    ref = oracle.swiglu(g, u)
    synth.check_f32(got, ref, f"n={n}") if dtype == F32 else synth.check_half(got, ref, f"n={n}", dtype)


def test_special_values(ctx, dev, oracle):
    g = np.array([0.0, -0.0, 1.0, -1.0, 20.0, -20.0, 88.0, -88.0, 100.0, -100.0, 1e-30, -1e-30], np.float32)
    u = np.full_like(g, 1.5)
    got, _ = run(ctx, dev, g, u, F32)
    synth.check_f32(got, oracle.swiglu(g, u), "special values")
    for dt in (F16, BF16):
        gg, uu = synth.round_to(g, dt), synth.round_to(u, dt)
        got, _ = run(ctx, dev, gg, uu, dt)
        synth.check_half(got, oracle.swiglu(gg, uu), "special values 16-bit", dt)


def test_in_place_and_half_copy(ctx, dev, oracle):
    d = synth.layer_inputs(synth.C1, 33)
    ref = oracle.swiglu(d["gate"], d["up"])
    got, _ = run(ctx, dev, d["gate"], d["up"], F32, in_place=True)  # the reference writes into gate
    synth.check_f32(got, ref, "in place")
    for h in (F16, BF16):
        got, gh = run(ctx, dev, d["gate"], d["up"], F32, want_h=h)
        synth.assert_bits_equal(gh, synth.round_to(got, h), "half copy")


def test_negative_control_sigmoid_form_is_distinguishable(ctx, dev, oracle):
    # g * sigmoid(g) is the same function but rounds differently; bitwise it must not equal the reference form
    # everywhere, which shows the comparison is sharp enough to see an expression-shape change.
    rng = np.random.default_rng(2)
    g = rng.standard_normal(100000, dtype=np.float32) * 2
    u = rng.standard_normal(100000, dtype=np.float32) * 2
    ref = oracle.swiglu(g, u)
    other = (g * (np.float32(1) / (np.float32(1) + np.exp(-g)))) * u
    assert (other.view(np.uint32) != ref.view(np.uint32)).any()
    got, _ = run(ctx, dev, g, u, F32)
    synth.check_f32(got, ref, "reference expression shape")
    # and a genuinely wrong activation (gelu-like tanh form) is far outside the bar
    wrong = (0.5 * g * (1 + np.tanh(0.79788456 * (g + 0.044715 * g ** 3)))) * u
    with pytest.raises(AssertionError):
        synth.check_f32(got, wrong.astype(np.float32), "planted bug")


def test_refusals(ctx, dev):
    import lokal_b200 as L
    g = dev.put(np.ones(8, np.float32))
    with pytest.raises(L.LokalCudaError) as e:
        ctx.swiglu(g, None, g, n=8, dtype=F32)
    assert e.value.status == L.capi.ERR_BAD_ARG
    with pytest.raises(L.LokalCudaError) as e:
        ctx.swiglu(g, g, g, n=8, dtype=L.Q8_0)
    assert e.value.status == L.capi.ERR_UNSUPPORTED
    with pytest.raises(L.LokalCudaError) as e:
        ctx.swiglu(g, g, g, n=4, dtype=F16, out_h=g)
    assert e.value.status == L.capi.ERR_UNSUPPORTED
    with pytest.raises(L.LokalCudaError) as e:
        ctx.swiglu(g.data_ptr() + 2, g, g, n=4, dtype=F32)
    assert e.value.status == L.capi.ERR_MISALIGNED
    ctx.swiglu(g, g, g, n=0, dtype=F32)
