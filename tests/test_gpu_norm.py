"""RMSNorm and fused residual-add + RMSNorm through the C ABI vs the CPU oracle.

Bar: max-abs 1e-5 on f32 rows; 2e-3 relative on f16/bf16 rows (against the
unrounded f32 oracle evaluated on the same rounded inputs); the residual sum
itself is a single IEEE add and must be bit-exact.
"""
import numpy as np
import pytest

import synth
from synth import BF16, F16, F32

pytestmark = pytest.mark.gpu


def run_norm(ctx, dev, x, delta, w, eps, dtype, w_dtype=F32, want_h=None):
    rows, dim = x.shape
    dx = dev.put(x, dtype)
    dw = dev.put(w, w_dtype)
    dxn = dev.empty((rows + 2, dim), dtype, fill=7.0)  # two canary rows behind the output
    dh = dev.empty((rows, dim), want_h, fill=0.0) if want_h else None
    if delta is None:
        ctx.rmsnorm(dx, dw, dxn, rows=rows, dim=dim, eps=eps, dtype=dtype, w_dtype=w_dtype, y_h=dh,
                    h_dtype=want_h or F16)
    else:
        dd = dev.put(delta, dtype)
        ctx.add_rmsnorm(dx, dd, dw, dxn, rows=rows, dim=dim, eps=eps, dtype=dtype, w_dtype=w_dtype, xn_h=dh,
                        h_dtype=want_h or F16)
    ctx.stream_sync()
    out = dev.get(dxn)
    assert (out[rows:] == 7.0).all(), "wrote past the last row"
    return dev.get(dx), out[:rows], (dh if dh is None else dev.get(dh)), dxn


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c5"])
@pytest.mark.parametrize("fused", [False, True])
def test_config_shapes(ctx, dev, oracle, name, fused):
    cfg = synth.CONFIGS[name]
    rows = min(cfg.rows, 333)
    d = synth.layer_inputs(cfg, rows)
    x_new, xn, _, _ = run_norm(ctx, dev, d["x"], d["delta"] if fused else None, d["w_norm"], cfg.eps, cfg.dtype,
                               w_dtype=cfg.dtype)
    ref_x, ref_xn = oracle.add_rmsnorm_rows(d["x"], d["delta"] if fused else None, d["w_norm"], cfg.eps)
    assert np.abs(xn).max() > 0.1, "output is all zeros: the kernel did not run"
    if cfg.dtype == F32:
        synth.assert_bits_equal(x_new, ref_x, "x + delta")
        synth.check_f32(xn, ref_xn, f"{name} rmsnorm")
    else:
        # the stored residual is the f32 sum rounded once to the storage type
        synth.assert_bits_equal(x_new, synth.round_to(ref_x, cfg.dtype), "x + delta")
        synth.check_half(xn, ref_xn, f"{name} rmsnorm", cfg.dtype)


@pytest.mark.parametrize("dtype", [F32, F16, BF16])
@pytest.mark.parametrize("rows,dim", [(1, 8), (3, 37), (5, 100), (2, 576), (7, 4096), (3, 8192), (2, 16384),
                                       (1, 33000), (4100, 64), (300, 1024)])
def test_shapes_and_tails(ctx, dev, oracle, dtype, rows, dim):
    rng = np.random.default_rng(dim * 31 + rows)
    x = synth.round_to(rng.standard_normal((rows, dim), dtype=np.float32), dtype)
    dl = synth.round_to(rng.standard_normal((rows, dim), dtype=np.float32), dtype)
    w = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    x_new, xn, _, _ = run_norm(ctx, dev, x, dl, w, 1e-5, dtype)
    ref_x, ref_xn = oracle.add_rmsnorm_rows(x, dl, w, 1e-5)
    if dtype == F32:
        synth.assert_bits_equal(x_new, ref_x, "x + delta")
        synth.check_f32(xn, ref_xn, f"rmsnorm {rows}x{dim}")
    else:
        synth.assert_bits_equal(x_new, synth.round_to(ref_x, dtype), "x + delta")
        synth.check_half(xn, ref_xn, f"rmsnorm {rows}x{dim}", dtype)


def test_reference_all_threes_vector(ctx, dev):
    # src/math.rs:100-108: every element 3 with unit weights -> every element ~1 (tol 1e-3)
    _, xn, _, _ = run_norm(ctx, dev, np.full((1, 4), 3, np.float32), None, np.ones(4, np.float32), 1e-6, F32)
    assert np.abs(xn - 1.0).max() < 1e-3


def test_exact_half_is_bit_identical(ctx, dev, oracle):
    # Small integers and a power-of-two row: the sum of squares and the mean are exact in f32 in any
    # summation order, so scale and output must match the oracle bit for bit.
    rng = np.random.default_rng(3)
    x = rng.integers(-3, 4, (64, 512)).astype(np.float32)
    x[:, 0] = 1  # no all-zero row
    w = rng.integers(1, 5, 512).astype(np.float32) * 0.25
    _, xn, _, _ = run_norm(ctx, dev, x, None, w, 0.0, F32)
    _, ref = oracle.add_rmsnorm_rows(x, None, w, 0.0)
    synth.assert_bits_equal(xn, ref, "exactly representable rows")


def test_negative_control_catches_wrong_association(ctx, dev, oracle):
    # x * (scale * w) instead of (x * scale) * w differs in the last bit often enough to be seen bitwise,
    # and eps outside the root is far outside the tolerance: the gates must be able to fail.
    cfg = synth.C1
    d = synth.layer_inputs(cfg, 64)
    _, xn, _, _ = run_norm(ctx, dev, d["x"], None, d["w_norm"], cfg.eps, F32)
    x = d["x"]
    ms = (x.astype(np.float64) ** 2).mean(axis=1, keepdims=True)
    wrong = (x / (np.sqrt(ms) + 0.05) * d["w_norm"]).astype(np.float32)
    with pytest.raises(AssertionError):
        synth.check_f32(xn, wrong, "planted bug")


@pytest.mark.parametrize("h", [F16, BF16])
def test_half_copy_is_the_rounded_f32_row(ctx, dev, oracle, h):
    d = synth.layer_inputs(synth.C1, 50)
    _, xn, xh, _ = run_norm(ctx, dev, d["x"], d["delta"], d["w_norm"], 1e-5, F32, want_h=h)
    synth.assert_bits_equal(xh, synth.round_to(xn, h), "half copy")


@pytest.mark.parametrize("w_dtype", [F32, F16, BF16])
def test_weight_types(ctx, dev, oracle, w_dtype):
    d = synth.layer_inputs(synth.C5, 40)
    w = synth.round_to(d["w_norm"], w_dtype)
    _, xn, _, _ = run_norm(ctx, dev, d["x"], d["delta"], w, 1e-6, BF16, w_dtype=w_dtype)
    _, ref = oracle.add_rmsnorm_rows(d["x"], d["delta"], w, 1e-6)
    synth.check_half(xn, ref, "bf16 rows", BF16)


def test_in_place_output(ctx, dev, oracle):
    d = synth.layer_inputs(synth.C1, 20)
    dx = dev.put(d["x"])
    dw = dev.put(d["w_norm"])
    ctx.rmsnorm(dx, dw, dx, rows=20, dim=576, eps=1e-5, dtype=F32)
    ctx.stream_sync()
    _, ref = oracle.add_rmsnorm_rows(d["x"], None, d["w_norm"], 1e-5)
    synth.check_f32(dev.get(dx), ref, "in place")


def test_misaligned_rows_take_the_scalar_path(ctx, dev, oracle):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((6, 64), dtype=np.float32)
    w = np.ones(64, np.float32)
    buf = dev.put(np.concatenate([np.zeros(1, np.float32), x.reshape(-1)]))
    out = dev.empty((6 * 64 + 1,), F32, fill=0.0)
    ctx.rmsnorm(buf.data_ptr() + 4, dev.put(w), out.data_ptr() + 4, rows=6, dim=64, eps=1e-5, dtype=F32)
    ctx.stream_sync()
    _, ref = oracle.add_rmsnorm_rows(x, None, w, 1e-5)
    synth.check_f32(dev.get(out)[1:].reshape(6, 64), ref, "4-byte aligned rows")


def test_refusals(ctx, dev):
    import lokal_b200 as L
    x = dev.put(np.ones((2, 8), np.float32))
    w = dev.put(np.ones(8, np.float32))
    cases = [
        (dict(x=None, w=w, y=x, dtype=F32), L.capi.ERR_BAD_ARG),
        (dict(x=x, w=w, y=x, dtype=L.Q8_0), L.capi.ERR_UNSUPPORTED),
        (dict(x=x.data_ptr() + 2, w=w, y=x, dtype=F32), L.capi.ERR_MISALIGNED),
    ]
    for kw, status in cases:
        with pytest.raises(L.LokalCudaError) as e:
            ctx.rmsnorm(kw["x"], kw["w"], kw["y"], rows=2, dim=8, eps=1e-5, dtype=kw["dtype"])
        assert e.value.status == status and e.value.message
    with pytest.raises(L.LokalCudaError) as e:
        ctx.rmsnorm(x, w, x, rows=2, dim=8, eps=1e-5, dtype=F16, y_h=x)
    assert e.value.status == L.capi.ERR_UNSUPPORTED
    with pytest.raises(L.LokalCudaError) as e:
        ctx.add_rmsnorm(x, None, w, x, rows=2, dim=8, eps=1e-5, dtype=F32)
    assert e.value.status == L.capi.ERR_BAD_ARG
    ctx.rmsnorm(x, w, x, rows=0, dim=8, eps=1e-5, dtype=F32)  # empty batch is fine
    ctx.stream_sync()


@pytest.mark.parametrize("name", ["c1", "c2", "c5"])
@pytest.mark.parametrize("fused", [False, True])
def test_large_batches(ctx, dev, oracle, name, fused):
    cfg = synth.CONFIGS[name]
    rows = 2600
    d = synth.layer_inputs(cfg, rows)
    delta = d["delta"] if fused else None
    x1, n1, _, _ = run_norm(ctx, dev, d["x"], delta, d["w_norm"], cfg.eps, cfg.dtype, w_dtype=cfg.dtype)
    ref_x, ref_xn = oracle.add_rmsnorm_rows(d["x"], delta, d["w_norm"], cfg.eps, threads=8)
    if cfg.dtype == F32:
        synth.check_f32(n1, ref_xn, f"{name} rmsnorm")
    else:
        synth.check_half(n1, ref_xn, f"{name} rmsnorm", cfg.dtype)
    synth.assert_bits_equal(x1, synth.round_to(ref_x, cfg.dtype), "x + delta")


@pytest.mark.parametrize("dtype", [F32, F16, BF16])
def test_l2_priority_of_the_residual_stream_changes_no_bit(ctx, dev, dtype, monkeypatch):
    """add_rmsnorm loads and stores x with the high L2 eviction priority (a residual stream of up to 32 MB);
    LOKAL_CUDA_NORM_L2_KEEP=0 turns the priority off. A cache hint may not change a result: both forms, a chain of
    three calls over one x each, bit for bit."""
    rows, dim = 4099, 1024
    rng = np.random.default_rng(5)
    x = synth.round_to(rng.standard_normal((rows, dim), dtype=np.float32), dtype)
    deltas = [synth.round_to(0.1 * rng.standard_normal((rows, dim), dtype=np.float32), dtype) for _ in range(3)]
    w = synth.round_to(1 + 0.1 * rng.standard_normal(dim, dtype=np.float32), dtype)
    outs = []
    for keep in ("1", "0"):
        monkeypatch.setenv("LOKAL_CUDA_NORM_L2_KEEP", keep)
        dx, dw = dev.put(x, dtype), dev.put(w, dtype)
        dxn = dev.empty((3, rows, dim), dtype, fill=0.0)
        for l in range(3):
            ctx.add_rmsnorm(dx, dev.put(deltas[l], dtype), dw, dxn[l], rows=rows, dim=dim, eps=1e-6, dtype=dtype, w_dtype=dtype)
        ctx.stream_sync()
        outs.append((dev.get(dx), dev.get(dxn)))
    synth.assert_bits_equal(outs[0][0], outs[1][0], "x after three add-norms, with and without the L2 priority")
    synth.assert_bits_equal(outs[0][1], outs[1][1], "xn of three add-norms, with and without the L2 priority")
