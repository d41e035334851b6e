"""The layer pass (lokal_cuda_pass_*): a whole step of the per-token ops vs the oracle applied op by op,
the host-input path vs the device-input path, and replay from a captured graph."""
import numpy as np
import pytest

import synth
from synth import BF16, F16, F32, Q8_0

pytestmark = pytest.mark.gpu


def make_case(dtype, rows=70, layers=3, qk_bias=False, qk_norm=False, decode=False, hd=64):
    cfg = synth.LayerConfig("t", dtype, rows, 192, 320, 4, 2, hd, 211, 1e6, 1e-6, layers, qk_bias=qk_bias,
                            qk_norm=qk_norm, decode_positions=5000 if decode else 0, seed=77)
    rng = np.random.default_rng(5)
    r = lambda a: synth.round_to(a.astype(np.float32), dtype)
    f = lambda *s, sc=1.0: rng.standard_normal(s, dtype=np.float32) * np.float32(sc)
    L, R, H, I = layers, rows, cfg.hidden, cfg.inter
    a = dict(norm_w=r(1 + f(L, 2, H, sc=0.1)), final_w=r(1 + f(H, sc=0.1)),
             q=r(f(L, R, cfg.q_dim)), k=r(f(L, R, cfg.kv_dim)), delta_att=r(f(L, R, H)), delta_mlp=r(f(L, R, H)),
             gate=r(f(L, R, I, sc=2.0)), up=r(f(L, R, I, sc=2.0)))
    if qk_bias:
        a.update(q_bias=r(f(L, cfg.q_dim, sc=0.1)), k_bias=r(f(L, cfg.kv_dim, sc=0.1)))
    if qk_norm:
        a.update(q_norm_w=r(1 + f(L, hd, sc=0.1)), k_norm_w=r(1 + f(L, hd, sc=0.1)))
    a["table"] = synth.q8_0_table(cfg.vocab, H, 9)
    a["ids"] = synth.token_ids_zipf(cfg.vocab, R, 3)
    a["positions"] = rng.integers(0, 5000, R, dtype=np.int32) if decode else None
    return cfg, a


def oracle_step(oracle, cfg, a, pos0):
    """Op by op with the storage rounding between ops that the device buffers impose."""
    rd = lambda v: synth.round_to(v, cfg.dtype)
    x = rd(oracle.embed_gather(a["table"], Q8_0, cfg.vocab, cfg.hidden, a["ids"]))
    res = {"xn_att": [], "xn_mlp": [], "inner": [], "q": [], "k": []}
    _, xn0 = oracle.add_rmsnorm_rows(x, None, a["norm_w"][0, 0], cfg.eps)
    res["xn0"] = xn0
    for l in range(cfg.layers):
        q, k = oracle.qk_rope_rows(a["q"][l], a["k"][l], n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads,
                                   head_dim=cfg.head_dim, theta=cfg.theta, eps=cfg.eps,
                                   q_bias=a["q_bias"][l] if cfg.qk_bias else None, k_bias=a["k_bias"][l] if cfg.qk_bias else None,
                                   q_norm_w=a["q_norm_w"][l] if cfg.qk_norm else None,
                                   k_norm_w=a["k_norm_w"][l] if cfg.qk_norm else None, positions=a["positions"], pos0=pos0)
        res["q"].append(q)
        res["k"].append(k)
        x, xn = oracle.add_rmsnorm_rows(x, a["delta_att"][l], a["norm_w"][l, 1], cfg.eps)
        x = rd(x)
        res["xn_att"].append(xn)
        res["inner"].append(oracle.swiglu(a["gate"][l], a["up"][l]))
        w = a["norm_w"][l + 1, 0] if l + 1 < cfg.layers else a["final_w"]
        x, xn = oracle.add_rmsnorm_rows(x, a["delta_mlp"][l], w, cfg.eps)
        x = rd(x)
        res["xn_mlp"].append(xn)
    res["x"] = x
    return res


def build_pass(ctx, dev, cfg, a, slots=None):
    import lokal_b200 as L
    import torch
    tdt = dev.tdt[cfg.dtype]
    host = lambda v: None if v is None else torch.from_numpy(np.ascontiguousarray(v)).to(tdt)
    keep = {n: host(a.get(n)) for n in ("norm_w", "final_w", "q_bias", "k_bias", "q_norm_w", "k_norm_w")}
    p = L.LayerPass(ctx, max_rows=cfg.rows, layers=cfg.layers, hidden=cfg.hidden, inter=cfg.inter, n_q_heads=cfg.n_q_heads,
                    n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, eps=cfg.eps, theta=cfg.theta, dtype=cfg.dtype,
                    w_dtype=cfg.dtype, embed_type=Q8_0, vocab=cfg.vocab, embed_table=a["table"], slots=slots, **keep)
    return p


def inputs_on(where, dev, cfg, a):
    """Per-layer inputs as torch tensors on the device ('dev') or in pinned host memory ('host')."""
    import torch
    tdt = dev.tdt[cfg.dtype]
    mk = (lambda v: dev.put(v, cfg.dtype)) if where == "dev" else (lambda v: torch.from_numpy(np.ascontiguousarray(v)).to(tdt).pin_memory())
    t = {n: mk(a[n]) for n in ("q", "k", "delta_att", "delta_mlp", "gate", "up")}
    raw = (lambda v: torch.from_numpy(v).cuda()) if where == "dev" else (lambda v: torch.from_numpy(v).pin_memory())
    t["ids"] = raw(a["ids"].view(np.int32))
    t["positions"] = None if a["positions"] is None else raw(a["positions"])
    return t


def pass_inputs(cfg, t, pos0):
    import lokal_b200 as L
    R = cfg.rows
    return L.LayerPass.inputs(ids=t["ids"], rows=R, q=t["q"], k=t["k"], delta_att=t["delta_att"], delta_mlp=t["delta_mlp"],
                              gate=t["gate"], up=t["up"], positions=t["positions"], pos0=pos0, q_layer_stride=R * cfg.q_dim,
                              k_layer_stride=R * cfg.kv_dim, delta_layer_stride=R * cfg.hidden, mlp_layer_stride=R * cfg.inter)


@pytest.mark.parametrize("dtype,qk_bias,qk_norm,decode,hd", [(F32, False, False, False, 64), (F16, True, False, False, 64),
                                                              (F16, False, False, True, 64), (BF16, False, True, False, 128)])
def test_device_step_matches_op_by_op_oracle(ctx, dev, oracle, dtype, qk_bias, qk_norm, decode, hd):
    import torch
    cfg, a = make_case(dtype, qk_bias=qk_bias, qk_norm=qk_norm, decode=decode, hd=hd)
    p = build_pass(ctx, dev, cfg, a)
    t = inputs_on("dev", dev, cfg, a)
    out = dev.empty((cfg.rows, cfg.hidden), dtype, fill=0.0)
    p.run_device(pass_inputs(cfg, t, 40), out)
    ctx.stream_sync()
    assert p.launches == 2 + 4 * cfg.layers  # gather + first norm in one launch (quantised table), rope table, 4 per layer
    ref = oracle_step(oracle, cfg, a, 40)
    chk = (lambda g, r, w: synth.check_f32(g, r, w)) if dtype == F32 else (lambda g, r, w: synth.check_half(g, r, w, dtype, atol=1e-6))
    chk(dev.get(out), ref["xn_mlp"][-1], "final normed hidden")
    esz = 4 if dtype == F32 else 2
    for l in range(cfg.layers):
        chk(dev.get(t["q"][l]), ref["q"][l], f"layer {l} q")
        chk(dev.get(t["k"][l]), ref["k"][l], f"layer {l} k")
        for which, name, width in ((0, "xn_att", cfg.hidden), (1, "xn_mlp", cfg.hidden), (2, "inner", cfg.inter)):
            raw = np.empty(cfg.rows * width, np.float32 if dtype == F32 else np.uint16)
            ctx.memcpy_d2h(raw, p.output(l, which), raw.nbytes)
            ctx.stream_sync()
            vals = raw if dtype == F32 else (raw.view(np.float16).astype(np.float32) if dtype == F16 else oracle.bf16_bits_to_f32(raw))
            chk(vals.reshape(cfg.rows, width), ref[name][l], f"layer {l} {name}")
    if dtype == F32:
        # f32 end to end equals the reference's token-by-token walk through all layers
        sink = np.zeros(1, np.float32)
        o = np.zeros((cfg.rows, cfg.hidden), np.float32)
        zq = np.zeros((cfg.layers, cfg.q_dim), np.float32)
        args = oracle.LayerPassArgs(rows=cfg.rows, layers=cfg.layers, hidden=cfg.hidden, inter=cfg.inter, n_q_heads=cfg.n_q_heads,
                                    n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, eps=cfg.eps, theta=cfg.theta, has_bias=0,
                                    has_qk_norm=0, positions=None, pos0=40, embed_table=a["table"].ctypes.data, embed_type=8,
                                    vocab=cfg.vocab, ids=a["ids"].ctypes.data, norm_w=a["norm_w"].ctypes.data,
                                    final_w=a["final_w"].ctypes.data, q_bias=zq.ctypes.data, k_bias=zq.ctypes.data,
                                    q_norm_w=zq.ctypes.data, k_norm_w=zq.ctypes.data, delta_att=a["delta_att"].ctypes.data,
                                    delta_mlp=a["delta_mlp"].ctypes.data, q=a["q"].ctypes.data, k=a["k"].ctypes.data,
                                    gate=a["gate"].ctypes.data, up=a["up"].ctypes.data, layer_period=cfg.layers,
                                    out=o.ctypes.data, sink=sink.ctypes.data)
        oracle.layer_pass(args, 2)
        synth.check_f32(dev.get(out), o, "token-by-token CPU walk")
    p.close()


@pytest.mark.parametrize("dtype,slots", [(BF16, 2), (F32, 3), (F16, 1)])
def test_host_step_equals_device_step_bitwise(ctx, dev, oracle, dtype, slots):
    import torch
    cfg, a = make_case(dtype, layers=5, qk_norm=True, hd=128)
    pd = build_pass(ctx, dev, cfg, a)
    td = inputs_on("dev", dev, cfg, a)
    out_d = dev.empty((cfg.rows, cfg.hidden), dtype, fill=0.0)
    pd.run_device(pass_inputs(cfg, td, 7), out_d)
    ctx.stream_sync()
    ph = build_pass(ctx, dev, cfg, a, slots=slots)
    th = inputs_on("host", dev, cfg, a)
    out_h = torch.zeros(cfg.rows, cfg.hidden, dtype=dev.tdt[dtype]).pin_memory()
    for _ in range(2):  # twice: the ring and its events are reused
        ph.run_host(pass_inputs(cfg, th, 7), out_h)
        synth.assert_bits_equal(out_h.to(torch.float32).numpy(), dev.get(out_d), "host-input step vs device-input step")
    assert ph.launches == 2 + 4 * cfg.layers
    # host inputs are left as they were (rotation happens in the staged device copies)
    synth.assert_bits_equal(th["q"].to(torch.float32).numpy(), a["q"], "host q untouched")
    pd.close()
    ph.close()


def test_graph_replay_equals_direct_run(ctx, dev, oracle):
    cfg, a = make_case(BF16, layers=4, qk_norm=True, hd=128)
    p = build_pass(ctx, dev, cfg, a)
    t = inputs_on("dev", dev, cfg, a)
    out = dev.empty((cfg.rows, cfg.hidden), BF16, fill=0.0)
    p.run_device(pass_inputs(cfg, t, 0), out)
    ctx.stream_sync()
    want = dev.get(out)
    t2 = inputs_on("dev", dev, cfg, a)
    out2 = dev.empty((cfg.rows, cfg.hidden), BF16, fill=0.0)
    s = ctx.stream_create()
    ctx.graph_begin(s)
    p.run_device(pass_inputs(cfg, t2, 0), out2, stream=s)
    g = ctx.graph_end(s)
    assert (dev.get(out2) == 0).all(), "capture must not execute"
    ctx.graph_launch(g, s)
    ctx.stream_sync(s)
    synth.assert_bits_equal(dev.get(out2), want, "graph replay")
    ctx.graph_destroy(g)
    ctx.stream_destroy(s)
    p.close()


@pytest.mark.parametrize("captured", [False, True])
def test_branch_schedule_equals_sequential_bitwise(ctx, dev, captured):
    """The three op families on parallel branches (forked from and joined into the caller's stream) give the bits of
    the one-stream order, run directly or replayed from a captured graph, for every per-layer output."""
    import lokal_b200 as L
    cfg, a = make_case(BF16, rows=333, layers=6, qk_norm=True, hd=128)
    outs = {}
    for sched in (L.capi.PASS_SCHEDULE_SEQUENTIAL, L.capi.PASS_SCHEDULE_BRANCHES):
        p = build_pass(ctx, dev, cfg, a)
        p.set_schedule(sched)
        t = inputs_on("dev", dev, cfg, a)
        out = dev.empty((cfg.rows, cfg.hidden), BF16, fill=0.0)
        s = ctx.stream_create()
        if captured:
            ctx.graph_begin(s)
            p.run_device(pass_inputs(cfg, t, 11), out, stream=s)
            g = ctx.graph_end(s)
            for _ in range(2):  # q/k are rotated in place: the second replay rotates again, identically in both schedules
                ctx.graph_launch(g, s)
            ctx.stream_sync(s)
            ctx.graph_destroy(g)
        else:
            p.run_device(pass_inputs(cfg, t, 11), out, stream=s)
            ctx.stream_sync(s)
        got = {"out": dev.get(out), "q": dev.get(t["q"]), "k": dev.get(t["k"])}
        for l in range(cfg.layers):
            for which in (0, 1, 2):
                width = cfg.inter if which == 2 else cfg.hidden
                raw = np.empty(cfg.rows * width, np.uint16)
                ctx.memcpy_d2h(raw, p.output(l, which), raw.nbytes)
                ctx.stream_sync()
                got[(l, which)] = raw
        outs[sched] = got
        ctx.stream_destroy(s)
        p.close()
    a_, b_ = outs[L.capi.PASS_SCHEDULE_SEQUENTIAL], outs[L.capi.PASS_SCHEDULE_BRANCHES]
    for key in a_:
        assert np.array_equal(a_[key].view(np.uint8), b_[key].view(np.uint8)), f"schedules differ in {key}"
    with pytest.raises(L.LokalCudaError):
        p2 = build_pass(ctx, dev, cfg, a)
        try:
            p2.set_schedule(7)
        finally:
            p2.close()


def test_refusals(ctx, dev):
    import lokal_b200 as L
    cfg, a = make_case(F32, layers=2)
    with pytest.raises(L.LokalCudaError) as e:
        build_pass(ctx, dev, cfg, a, slots=9)
    assert e.value.status == L.capi.ERR_BAD_ARG
    p = build_pass(ctx, dev, cfg, a)
    t = inputs_on("dev", dev, cfg, a)
    out = dev.empty((cfg.rows, cfg.hidden), F32)
    inp = pass_inputs(cfg, t, 0)
    inp.rows = cfg.rows + 1
    with pytest.raises(L.LokalCudaError):
        p.run_device(inp, out)
    inp = pass_inputs(cfg, t, 0)
    inp.gate = None
    with pytest.raises(L.LokalCudaError):
        p.run_device(inp, out)
    # an out-of-range id surfaces from the host step as an error code, not a fault
    bad = dict(a)
    bad["ids"] = a["ids"].copy()
    bad["ids"][3] = cfg.vocab + 5
    th = inputs_on("host", dev, cfg, bad)
    import torch
    oh = torch.zeros(cfg.rows, cfg.hidden).pin_memory()
    with pytest.raises(L.LokalCudaError) as e:
        p.run_host(pass_inputs(cfg, th, 0), oh)
    assert e.value.status == L.capi.ERR_ID_RANGE
    p.close()
