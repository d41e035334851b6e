#!/usr/bin/env python
"""Benchmark of the fused per-token layer ops on B200 (one process per GPU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5|c2|c1|c3] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

A step is one pass of the hot path over one batch of token rows: embedding gather (Q8_0 table), the rope table, and
for each layer qk-norm/bias + RoPE, two residual-add + RMSNorm, and SwiGLU (lokal_cuda_pass_*). The projections and
attention between them are out of scope, so their outputs are synthetic tensors, distinct per layer, resident in HBM
(several GB per step, far larger than L2). `value` times the step with inputs resident on the device (one CUDA graph
per step); `e2e` times the same step through lokal_cuda_pass_run_host with all inputs in pinned host memory and the
result copied back. The token rows of the batch are PARTITIONED over the GPUs with no collective on the path (strong
scaling: at N GPUs every rank runs its contiguous share of the 8192 rows, as the configuration is stated);
`--scaling weak` gives every GPU a full batch instead, and at N > 1 the weak figure is printed beside the strong one
(`weak_tokens_per_s`). The timed region is `--blocks` blocks of K steps, each block bracketed by a barrier and timed
with CUDA events on the launching stream, maximum over ranks per block; `value` is the median block. Rank 0 prints
ONE JSON line. `roofline.kernels` carries each kernel timed alone and, beside it, the driver's device-to-device copy
of the same number of bytes launched the same way (`d2d_copy_same_bytes_us`). At N = 1 the line also carries
`configs`: the other benchmark configurations (C1-C3 steps, C4 gathers) measured briefly in the same run.

Other workloads: `--workload c4` (65,536 Zipf ids through every GGUF block type; `--only q8_0_f16,q4_k_f32` picks
variants) and `--workload rows` (the neighbouring per-row ops and K/V staging).

--impl reference times the reference's own CPU algorithm for the same step (the C++ restatement in oracle/, all host
threads, f32 as the reference computes) on a bounded sample of the rows.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import synth  # noqa: E402  (workload shapes and seeded generators)

METRIC = "fused per-token layer ops (embed gather + per layer: qk-norm/bias+RoPE, 2x residual-add+RMSNorm, SwiGLU), tokens/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def ncu_traffic(workload: str, kernel: str):
    """(DRAM bytes per launch of `kernel`, where and when they were captured) from the committed ncu capture of this
    workload (profiles/ncu_traffic.json), or (None, None)."""
    p = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        t = json.load(open(p))
        if t.get("workload") == workload:
            stamp = {"source": t.get("source"), "commit": t.get("captured_at_commit"),
                     "kernel": (t.get("kernel_names") or {}).get(kernel)}
            return t["dram_bytes_per_launch"].get(kernel), stamp
    except Exception:
        pass
    return None, None


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def embed_dim_ok(cfg):
    return cfg.hidden % 32 == 0


def bind_to_gpu_cpus(cuda_index: int) -> int:
    """Restricts this process to the host CPUs NVML reports as local to the GPU (process-local affinity, read-only NVML
    query), so that the pinned staging buffers it then allocates land on the GPU's NUMA node. Returns how many CPUs it
    was bound to, 0 if nothing was changed."""
    try:
        import pynvml
        import torch
        pynvml.nvmlInit()
        props = torch.cuda.get_device_properties(cuda_index)
        bus = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        local = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        cpus = local & allowed
        if cpus and cpus != allowed:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
        # NVML named every CPU: ask sysfs for the GPU's NUMA node instead (read-only), where the box exposes it
        node = int(open(f"/sys/bus/pci/devices/{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0/numa_node").read())
        if node >= 0:
            cpus = set()
            for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            cpus &= allowed
            if cpus and cpus != allowed:
                os.sched_setaffinity(0, cpus)
                return len(cpus)
    except Exception:
        pass
    return 0


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs (read-only)."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, cuda_index: int):
        super().__init__(daemon=True)
        self.samples, self.reasons, self.max_mhz, self.ok = [], set(), None, False
        self._halt = threading.Event()
        self._active = threading.Event()  # samples are taken only inside timed regions (see timed())
        self._active.set()
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            props = torch.cuda.get_device_properties(cuda_index)
            h = None
            try:
                bus = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
                h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(cuda_index)
            self.h = h
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        while not self._halt.is_set():
            if not self._active.is_set():
                self._active.wait(0.05)
                continue
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                try:
                    bits = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    bits = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for b, name in self.REASONS.items():
                    if bits & b:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(0.001)  # the timed regions are tens of milliseconds: sample every millisecond or so

    def pause(self):
        self._active.clear()

    def resume(self):
        self._active.set()

    def finish(self):
        self._halt.set()
        self._active.set()
        if self.is_alive():
            self.join(2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# reference arm: the reference's CPU algorithm (oracle port) on the host cores
# ------------------------------------------------------------------------------------------------

def cpu_inputs(cfg, rows, period, seed):
    """f32 host inputs for `rows` token rows and `period` layers of distinct data (the reference computes in f32)."""
    rng = np.random.default_rng(seed)
    f = lambda *s, sc=1.0: rng.standard_normal(s, dtype=np.float32) * np.float32(sc)
    L = cfg.layers
    return dict(
        norm_w=1 + f(L, 2, cfg.hidden, sc=0.1), final_w=1 + f(cfg.hidden, sc=0.1),
        q_bias=f(L, cfg.q_dim, sc=0.1), k_bias=f(L, cfg.kv_dim, sc=0.1),
        q_norm_w=1 + f(L, cfg.head_dim, sc=0.1), k_norm_w=1 + f(L, cfg.head_dim, sc=0.1),
        delta_att=f(period, rows, cfg.hidden), delta_mlp=f(period, rows, cfg.hidden),
        q=f(period, rows, cfg.q_dim), k=f(period, rows, cfg.kv_dim),
        gate=f(period, rows, cfg.inter, sc=2.0), up=f(period, rows, cfg.inter, sc=2.0))


def cpu_step_fn(cfg, rows, table, vocab, seed=1):
    """Returns (run(threads) -> seconds, description) for one CPU step over `rows` rows."""
    from oracle import lokal_oracle as O
    period = 2
    a = cpu_inputs(cfg, rows, period, seed)
    ids = synth.token_ids_zipf(vocab, rows, seed)
    pos = (np.random.default_rng(seed).integers(0, cfg.decode_positions, rows, dtype=np.int32)
           if cfg.decode_positions else None)
    out = np.zeros((rows, cfg.hidden), np.float32)
    sink = np.zeros(1, np.float32)
    args = O.LayerPassArgs(rows=rows, layers=cfg.layers, hidden=cfg.hidden, inter=cfg.inter, n_q_heads=cfg.n_q_heads,
                           n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, eps=cfg.eps, theta=cfg.theta,
                           has_bias=int(cfg.qk_bias), has_qk_norm=int(cfg.qk_norm),
                           positions=None if pos is None else pos.ctypes.data, pos0=0,
                           embed_table=table.ctypes.data, embed_type=O.Q8_0, vocab=vocab, ids=ids.ctypes.data,
                           layer_period=period, out=out.ctypes.data, sink=sink.ctypes.data,
                           **{k: v.ctypes.data for k, v in a.items()})
    keep = (a, ids, pos, out, sink, table)

    def run(threads):
        t0 = time.perf_counter()
        O.layer_pass(args, threads)
        _ = keep
        return time.perf_counter() - t0
    return run


def shard_of(cfg, args, rank, world):
    """(first row, rows) of this rank's share: a contiguous block of the batch (strong), or a whole batch (weak)."""
    if args.scaling == "strong":
        per = (cfg.rows + world - 1) // world  # the same split as lokal_cuda_shard_rows
        r0 = min(cfg.rows, per * rank)
        return r0, min(cfg.rows, r0 + per) - r0
    return rank * cfg.rows, cfg.rows


def reference_arm(args, cfg, rank, world):
    if rank != 0:
        return
    from oracle import lokal_oracle as O
    O.build()
    threads = O.hardware_threads()
    vocab = cfg.vocab  # the full table, as the GPU arm
    table = synth.q8_0_table(vocab, cfg.hidden, cfg.seed)
    # calibrate on a small probe, then size the per-step sample for about 2 s of wall time
    probe_rows = min(cfg.rows, 4 * threads)
    probe = cpu_step_fn(cfg, probe_rows, table, vocab)
    probe(threads)
    dt = probe(threads)
    rows = int(min(cfg.rows, max(threads, probe_rows * 2.0 / max(dt, 1e-6))))
    rows = max(threads, rows // threads * threads)
    step = cpu_step_fn(cfg, rows, table, vocab)
    for _ in range(args.warmup):
        step(threads)
    times = [step(threads) for _ in range(args.steps)]
    total = float(sum(times))
    value = rows * args.steps / total
    sample = (f"{rows} of {cfg.rows} token rows per step, all {cfg.layers} layers, f32, {threads} threads (token-parallel), "
              f"Q8_0 table {vocab}x{cfg.hidden}; layer_period 2: the per-layer inputs cycle over 2 distinct layers of data "
              f"({2 * rows * (cfg.q_dim + cfg.kv_dim + 2 * cfg.hidden + 2 * cfg.inter) * 4 / 1e6:.0f} MB, beyond the host caches)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, shard_of(cfg, args, 0, max(1, args.gpus))[1], args),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg, rows_per_gpu, args):
    """The same dictionary in both arms (the CPU arm's sampling is described in its cpu_baseline.sample)."""
    return {"workload": cfg.name, "rows": cfg.rows, "rows_per_gpu": rows_per_gpu, "layers": cfg.layers, "hidden": cfg.hidden,
            "intermediate": cfg.inter, "q_heads": cfg.n_q_heads, "kv_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
            "qk_norm": cfg.qk_norm, "qk_bias": cfg.qk_bias, "embed_table": f"Q8_0 {cfg.vocab}x{cfg.hidden}",
            "sharding": f"token rows over {args.gpus} GPU(s) ({args.scaling} scaling), no collective on the path",
            "l2": "inputs larger than L2: per-layer inputs and outputs are distinct buffers, never reused inside a step "
                  "(GPU arm: every layer has its own, several GB per full batch; CPU arm: see cpu_baseline.sample)"}


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------

class StepBench:
    """One GPU's share of a layer-pass workload: weights, device-resident synthetic inputs (distinct per layer), the
    pass object and one CUDA graph per schedule ("encode everything, submit once")."""

    def __init__(self, L, ctx, cfg, T, r0, rank, dev, stream):
        import torch
        self.L, self.ctx, self.cfg, self.T, self.r0, self.dev, self.stream = L, ctx, cfg, T, r0, dev, stream
        self.tdt = {L.F32: torch.float32, L.F16: torch.float16, L.BF16: torch.bfloat16}[cfg.dtype]
        self.es = 2 if cfg.dtype != L.F32 else 4
        H, I, QD, KD, NL = cfg.hidden, cfg.inter, cfg.q_dim, cfg.kv_dim, cfg.layers
        gen = torch.Generator(device=dev)
        gen.manual_seed(cfg.seed + rank)
        self.rn = lambda *shape, s=1.0: (torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32) * s).to(self.tdt)
        rn = self.rn
        wrng = np.random.default_rng(cfg.seed)
        wnp = lambda *shape, s=0.1, one=True: synth.round_to((1.0 if one else 0.0) + wrng.standard_normal(shape, dtype=np.float32) * np.float32(s), cfg.dtype)
        as_bits = lambda a: (torch.from_numpy(a).to(self.tdt).contiguous())
        self.table = synth.q8_0_table(cfg.vocab, H, cfg.seed)
        self.weights = dict(norm_w=as_bits(wnp(NL, 2, H)), final_w=as_bits(wnp(H)))
        if cfg.qk_bias:
            self.weights.update(q_bias=as_bits(wnp(NL, QD, one=False)), k_bias=as_bits(wnp(NL, KD, one=False)))
        if cfg.qk_norm:
            self.weights.update(q_norm_w=as_bits(wnp(NL, cfg.head_dim)), k_norm_w=as_bits(wnp(NL, cfg.head_dim)))
        self.common = dict(max_rows=T, layers=NL, hidden=H, inter=I, n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads,
                           head_dim=cfg.head_dim, eps=cfg.eps, theta=cfg.theta, dtype=cfg.dtype, w_dtype=cfg.dtype,
                           embed_type=L.Q8_0, vocab=cfg.vocab, embed_table=self.table, **self.weights)
        self.pass_dev = L.LayerPass(ctx, slots=NL, **self.common)  # every layer's outputs go to their own buffers
        self.q, self.k = rn(NL, T, QD), rn(NL, T, KD)
        self.da, self.dm = rn(NL, T, H), rn(NL, T, H)
        self.g, self.u = rn(NL, T, I, s=2.0), rn(NL, T, I, s=2.0)
        self.ids_np = synth.token_ids_zipf(cfg.vocab, T, cfg.seed + rank)
        self.ids = torch.from_numpy(self.ids_np.astype(np.int64)).to(dev).to(torch.int32)  # same bits as u32 for ids < 2^31
        self.pos = None
        if cfg.decode_positions:
            self.pos = torch.randint(0, cfg.decode_positions, (T,), generator=gen, device=dev, dtype=torch.int32)
        self.out = torch.empty(T, H, dtype=self.tdt, device=dev)
        self.inp = L.LayerPass.inputs(ids=self.ids, rows=T, q=self.q, k=self.k, delta_att=self.da, delta_mlp=self.dm, gate=self.g,
                                      up=self.u, positions=self.pos, pos0=r0, q_layer_stride=T * QD, k_layer_stride=T * KD,
                                      delta_layer_stride=T * H, mlp_layer_stride=T * I)
        torch.cuda.synchronize()
        self.graphs = {}

    def graph(self, schedule):
        if schedule not in self.graphs:
            self.pass_dev.set_schedule(schedule)
            self.ctx.graph_begin(self.stream)
            self.pass_dev.run_device(self.inp, self.out, stream=self.stream)
            self.graphs[schedule] = self.ctx.graph_end(self.stream)
            self.launches_per_step = self.pass_dev.launches
        return self.graphs[schedule]

    def step_bytes(self):
        cfg, T, es = self.cfg, self.T, self.es
        rb = self.L.row_bytes(self.L.Q8_0, cfg.hidden)
        uniq = int(np.unique(self.ids_np).size)
        gather = T * (4 + cfg.hidden * es) + uniq * rb
        per_token_layer = 2 * 4 * cfg.hidden * es + (2 * (cfg.q_dim + cfg.kv_dim) * es + cfg.head_dim * 4) + 3 * cfg.inter * es
        return cfg.layers * per_token_layer * T + gather + 2 * cfg.hidden * es * T + cfg.head_dim * 4 * T, gather

    def l2_resident_bytes(self):
        """Algorithmic bytes of a step that do not cross HBM: the residual stream x, which every add-norm reads and
        rewrites with the high L2 eviction priority (all but its first read and last write), and the cos/sin table,
        read again by every layer's rope launch (all but the first read). Both priorities apply up to 32 MB, as in the
        library; ncu's per-launch DRAM bytes (profiles/c5_dram_traffic_per_kernel.md) are the measured counterpart."""
        cfg, T, es = self.cfg, self.T, self.es
        x_bytes, table_bytes = T * cfg.hidden * es, T * cfg.head_dim * 4
        keep = 0
        if x_bytes <= (32 << 20):
            keep += (2 * cfg.layers * 2 - 2) * x_bytes
        if table_bytes <= (32 << 20):
            keep += (cfg.layers - 1) * table_bytes
        return keep

    def time_blocks(self, schedule, steps, blocks, warmup, barrier, sampler=None):
        """`blocks` timed blocks of `steps` graph launches, each between a barrier and a stream sync, timed with CUDA
        events on the launching stream. Returns the per-block milliseconds of this rank."""
        import torch
        g = self.graph(schedule)
        ts = torch.cuda.ExternalStream(self.stream, device=self.dev)
        for _ in range(max(warmup, 3)):
            self.ctx.graph_launch(g, self.stream)
        self.ctx.stream_sync(self.stream)
        out = []
        for _ in range(blocks):
            barrier()
            if sampler:
                sampler.resume()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(ts)
            for _ in range(steps):
                self.ctx.graph_launch(g, self.stream)
            e1.record(ts)
            self.ctx.stream_sync(self.stream)
            if sampler:
                sampler.pause()
            out.append(e0.elapsed_time(e1))
        barrier()
        return out

    def close(self):
        for g in self.graphs.values():
            self.ctx.graph_destroy(g)
        self.graphs = {}
        self.pass_dev.close()


def max_over_ranks(values, world, dev):
    if world == 1:
        return [float(v) for v in values]
    import torch
    import torch.distributed as dist
    t = torch.tensor(values, device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def quick_configs(L, ctx, dev, stream, sampler, peak):
    """The other benchmark configurations, briefly, for the default line: a C1 / C2 / C3 step (device-resident
    inputs, one graph, median of 5 blocks of 20 steps) and the four C4 gathers the configuration names."""
    import torch
    out = {}
    nobar = lambda: torch.cuda.synchronize()
    for key in ("c1", "c2", "c3"):
        cfg = synth.CONFIGS[key]
        sb = StepBench(L, ctx, cfg, cfg.rows, 0, 0, dev, stream)
        ms = float(np.median(sb.time_blocks(L.capi.PASS_SCHEDULE_AUTO, 20, 5, 3, nobar, sampler))) / 20
        nbytes, _ = sb.step_bytes()
        out[key] = {"workload": cfg.name, "rows": cfg.rows, "ms_per_step": ms, "tokens_per_s": cfg.rows / (ms * 1e-3),
                    "launches_per_step": int(sb.launches_per_step), "step_algorithmic_gbs": nbytes / (ms * 1e-3) / 1e9,
                    "step_frac": nbytes / (ms * 1e-3) / 1e9 / peak}
        sb.close()
        del sb
        torch.cuda.empty_cache()
    out["c4"] = gather_variants(L, ctx, dev, stream, sampler, peak, ["q8_0_f32", "q8_0_f16", "q4_k_f32", "q4_k_f16"], warmup=3, reps=5)[0]
    return out


def ours(args, cfg, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    import lokal_b200 as L

    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    bound_cpus = bind_to_gpu_cpus(local_rank)  # before any pinned allocation: host buffers on the GPU's NUMA node
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = L.Context(local_rank)
    r0, T = shard_of(cfg, args, rank, world)
    assert T > 0, "more GPUs than token rows"
    H, I, QD, KD, NL = cfg.hidden, cfg.inter, cfg.q_dim, cfg.kv_dim, cfg.layers
    stream = ctx.stream_create()
    tstream = torch.cuda.ExternalStream(stream, device=dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sb = StepBench(L, ctx, cfg, T, r0, rank, dev, stream)
    tdt, es = sb.tdt, sb.es
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.pause()
        sampler.start()
    step_bytes, gather_bytes = sb.step_bytes()
    l2_bytes = sb.l2_resident_bytes()

    # ---- per-kernel timing on this GPU (rank 0 reports): L launches over distinct per-layer buffers ----
    rn, q, k, da, dm, g, u, ids, pos = sb.rn, sb.q, sb.k, sb.da, sb.dm, sb.g, sb.u, sb.ids, sb.pos
    weights, table, vocab = sb.weights, sb.table, cfg.vocab
    alg = {
        "add_rmsnorm": 4 * H * es * T,
        "qk_rope": (2 * (QD + KD) * es + cfg.head_dim * 4) * T,
        "swiglu": 3 * I * es * T,
        "embed_gather": gather_bytes,
    }
    kern = {}
    ksampler = ClockSampler(local_rank) if rank == 0 else None  # clocks while the kernels are timed alone
    if ksampler:
        ksampler.pause()
        ksampler.start()
    if rank == 0 and not args.no_kernel_timing:
        xs = rn(NL, T, H)
        xn = torch.empty(NL, T, H, dtype=tdt, device=dev)
        inner = torch.empty(NL, T, I, dtype=tdt, device=dev)
        table_dev = torch.from_numpy(table).to(dev)
        tab = torch.empty(T, cfg.head_dim, dtype=torch.float32, device=dev)
        ctx.rope_table(tab, theta=cfg.theta, rot_dim=cfg.head_dim, rows=T, positions=pos, pos0=r0, stream=stream)
        wn = weights["norm_w"].to(dev)
        qb = weights["q_bias"].to(dev) if cfg.qk_bias else None
        kb = weights["k_bias"].to(dev) if cfg.qk_bias else None
        qn = weights["q_norm_w"].to(dev) if cfg.qk_norm else None
        kn = weights["k_norm_w"].to(dev) if cfg.qk_norm else None
        gout = torch.empty(NL if NL < 8 else 8, T, H, dtype=tdt, device=dev)

        def k_norm(l):
            ctx.add_rmsnorm(xs[l], da[l], wn[l, 1], xn[l], rows=T, dim=H, eps=cfg.eps, dtype=cfg.dtype, w_dtype=cfg.dtype, stream=stream)

        def k_rope(l):
            p = ctx.qk_rope_params(q=q[l], k=k[l], q_bias=None if qb is None else qb[l], k_bias=None if kb is None else kb[l],
                                   q_norm_w=None if qn is None else qn[l], k_norm_w=None if kn is None else kn[l], cos_sin=tab,
                                   rows=T, n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                                   eps=cfg.eps, q_dtype=cfg.dtype, w_dtype=cfg.dtype)
            ctx.qk_rope(p, stream=stream)

        def k_swiglu(l):
            ctx.swiglu(g[l], u[l], inner[l], n=T * I, dtype=cfg.dtype, stream=stream)

        def k_gather(l):
            ctx.embed_gather(table_dev, ids, gout[l % gout.shape[0]], ggml_type=L.Q8_0, vocab=vocab, dim=H, n=T, out_dtype=cfg.dtype, stream=stream)

        for name, fn in (("add_rmsnorm", k_norm), ("qk_rope", k_rope), ("swiglu", k_swiglu), ("embed_gather", k_gather)):
            # the NL launches go into one graph so host launch overhead stays out of the device time
            ctx.graph_begin(stream)
            for l in range(NL):
                fn(l)
            kg = ctx.graph_end(stream)
            times = []
            for rep in range(6):
                if rep == 1:
                    ksampler.resume()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record(tstream)
                ctx.graph_launch(kg, stream)
                a1.record(tstream)
                ctx.stream_sync(stream)
                if rep:  # first repetition is warm-up
                    times.append(a0.elapsed_time(a1) / NL)
            ksampler.pause()
            ctx.graph_destroy(kg)
            avg = float(np.mean(times))
            # warm single launches, one at a time on layer 0's buffers (what survives of them in L2 is reused): not a
            # bandwidth figure, the latency a decode-size caller sees per call
            singles = []
            for rep in range(24):
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record(tstream)
                fn(0)
                a1.record(tstream)
                ctx.stream_sync(stream)
                if rep >= 4:
                    singles.append(a0.elapsed_time(a1))
            kern[name] = {"us_per_launch": 1e3 * avg, "us_best": 1e3 * min(times), "launches_timed": NL * len(times),
                          "bytes_per_launch": int(alg[name]), "gbs": alg[name] / (avg * 1e-3) / 1e9,
                          "warm_single_launch_us": 1e3 * float(np.median(singles))}
        # The add-norm as a step uses it: NL launches that read and rewrite ONE residual stream, each with its own delta
        # and output. x is loaded and stored with the high L2 eviction priority and stays on chip between launches, so
        # half of the launch's algorithmic bytes do not cross HBM; the figure above (a fresh x per launch) has all of
        # them crossing it.
        ctx.graph_begin(stream)
        for l in range(NL):
            ctx.add_rmsnorm(xs[0], da[l], wn[l, 1], xn[l], rows=T, dim=H, eps=cfg.eps, dtype=cfg.dtype, w_dtype=cfg.dtype, stream=stream)
        kg = ctx.graph_end(stream)
        times = []
        for rep in range(6):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(tstream)
            ctx.graph_launch(kg, stream)
            a1.record(tstream)
            ctx.stream_sync(stream)
            if rep:
                times.append(a0.elapsed_time(a1) / NL)
        ctx.graph_destroy(kg)
        chain = float(np.mean(times))
        kern["add_rmsnorm"]["one_residual_stream_us"] = 1e3 * chain
        kern["add_rmsnorm"]["one_residual_stream_algorithmic_gbs"] = alg["add_rmsnorm"] / (chain * 1e-3) / 1e9
        kern["add_rmsnorm"]["one_residual_stream_hbm_bytes"] = int(alg["add_rmsnorm"] // 2)
        # Calibration beside each figure: the driver's own device-to-device copy moving the same number of bytes
        # (half read, half written), launched the same way (one graph of back-to-back copies over distinct memory).
        # A kernel this short cannot be held to the bandwidth of a seconds-long copy; this is the size-matched bar.
        src_flat, dst_flat = u.view(-1).view(torch.uint8), inner.view(-1).view(torch.uint8)
        cs = torch.cuda.Stream(device=dev)
        for name in ("add_rmsnorm", "qk_rope", "swiglu"):
            chunk = (int(alg[name]) // 2) & ~255
            n_copies = min(NL, src_flat.numel() // chunk)
            if n_copies < 1:
                continue
            with torch.cuda.stream(cs):
                def copies():
                    for i in range(n_copies):
                        dst_flat[i * chunk:(i + 1) * chunk].copy_(src_flat[i * chunk:(i + 1) * chunk], non_blocking=True)
                copies()
                cs.synchronize()
                cg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(cg, stream=cs):
                    copies()
                ct = []
                for rep in range(6):
                    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a0.record(cs)
                    cg.replay()
                    a1.record(cs)
                    cs.synchronize()
                    if rep:
                        ct.append(a0.elapsed_time(a1) / n_copies)
                del cg
            copy_us = 1e3 * float(np.mean(ct))
            kern[name]["d2d_copy_same_bytes_us"] = copy_us
            kern[name]["d2d_copy_same_bytes_gbs"] = 2 * chunk / (copy_us * 1e-6) / 1e9
            kern[name]["speed_vs_d2d_copy"] = copy_us / kern[name]["us_per_launch"]
        del xs, xn, inner, gout, src_flat, dst_flat, table_dev
    torch.cuda.synchronize()
    kernel_clocks = ksampler.finish() if ksampler else None

    SEQ, BR, AUTO = L.capi.PASS_SCHEDULE_SEQUENTIAL, L.capi.PASS_SCHEDULE_BRANCHES, L.capi.PASS_SCHEDULE_AUTO
    sched = {"auto": AUTO, "sequential": SEQ, "branches": BR}[args.schedule]
    # the headline: `blocks` blocks of K steps, maximum over ranks per block, median block
    blocks_ms = max_over_ranks(sb.time_blocks(sched, args.steps, args.blocks, args.warmup, barrier, sampler), world, dev)
    launches_per_step = sb.launches_per_step
    clocks = sampler.finish() if sampler else None  # sampled inside the timed blocks only
    ms_total = float(np.median(blocks_ms))
    ms_step = ms_total / args.steps
    total_rows = cfg.rows if args.scaling == "strong" else T * world
    value = total_rows / (ms_step * 1e-3)
    # the same step under each schedule (same kernels, same results; see lokal_cuda_pass_set_schedule)
    by_schedule = {}
    for name, sc in (() if args.no_extras else (("sequential", SEQ), ("branches", BR))):
        ms = float(np.median(max_over_ranks(sb.time_blocks(sc, args.steps, 3, args.warmup, barrier), world, dev))) / args.steps
        by_schedule[name] = {"ms_per_step": ms, "tokens_per_s": total_rows / (ms * 1e-3)}

    # ---- end to end: host inputs in pinned memory, result back on the host ----
    e2e = None
    if not args.no_e2e:
        common = sb.common
        sb.close()
        pass_host = L.LayerPass(ctx, slots=min(3, NL), **common)
        pin = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)
        hq, hk, hda, hdm, hg, hu = (pin(t) for t in (q, k, da, dm, g, u))
        hids = pin(ids)
        hpos = pin(pos) if pos is not None else None
        hout = torch.empty(T, H, dtype=tdt, pin_memory=True)
        hin = L.LayerPass.inputs(ids=hids, rows=T, q=hq, k=hk, delta_att=hda, delta_mlp=hdm, gate=hg, up=hu, positions=hpos,
                                 pos0=r0, q_layer_stride=T * QD, k_layer_stride=T * KD, delta_layer_stride=T * H,
                                 mlp_layer_stride=T * I)
        # the device arm rotated q/k in place on the device; the host copies above were taken after it, so both
        # arms have seen the same kind of data. One untimed run first.
        pass_host.run_host(hin, hout)
        e2e_steps = max(2, min(args.steps, args.e2e_steps))
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            pass_host.run_host(hin, hout)
        torch.cuda.synchronize()
        dt_own = time.perf_counter() - t0
        dt = max_over_ranks([dt_own], world, dev)[0]
        h2d = T * 4 + (T * 4 if pos is not None else 0) + NL * T * (QD + KD + 2 * H + 2 * I) * es
        # What bounds it: every rank ships its inputs over its own PCIe link, but the ranks of one box share the host's
        # memory and PCIe root bandwidth; the per-GPU rate shows which of the two a run sat on.
        e2e = {"value": total_rows * e2e_steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(T * H * es), "steps": e2e_steps, "ms_per_step": 1e3 * dt / e2e_steps,
               "h2d_gbs_per_gpu": h2d * e2e_steps / dt / 1e9, "h2d_gbs_all_gpus": world * h2d * e2e_steps / dt / 1e9,
               "bound": "host-to-device copies (PCIe link per GPU; host memory / PCIe root shared by the ranks of a box)",
               "api": "lokal_cuda_pass_run_host (pinned host inputs, 3-slot layer ring, copies overlap kernels)"}
        del pass_host, hq, hk, hda, hdm, hg, hu
    else:
        sb.close()
    del q, k, da, dm, g, u
    sb = None
    torch.cuda.empty_cache()

    # ---- at N > 1: the weak figure beside the strong one (every GPU runs a full batch of its own) ----
    weak = None
    if world > 1 and args.scaling == "strong" and not args.no_extras:
        wb = StepBench(L, ctx, cfg, cfg.rows, rank * cfg.rows, rank, dev, stream)
        wms = float(np.median(max_over_ranks(wb.time_blocks(AUTO, args.steps, 3, args.warmup, barrier), world, dev))) / args.steps
        weak = {"tokens_per_s": cfg.rows * world / (wms * 1e-3), "ms_per_step": wms, "rows_per_gpu": cfg.rows}
        wb.close()
        del wb
        torch.cuda.empty_cache()

    if rank == 0:
        peak, peak_kind = measured_peak()
        configs = None
        if world == 1 and not args.no_extras and args.workload == "c5" and not (args.layers or args.rows):
            s2 = ClockSampler(local_rank)
            s2.pause()
            s2.start()
            configs = quick_configs(L, ctx, dev, stream, s2, peak)
            configs["clocks"] = s2.finish()
        roof = None
        if kern:
            dom = max(kern, key=lambda n: kern[n]["us_per_launch"] * (2 * NL if n == "add_rmsnorm" else (1 if n == "embed_gather" else NL)))
            traffic, stamp = ncu_traffic(cfg.name.split("[")[0], dom)
            scale_t = T / synth.CONFIGS[args.workload].rows  # the capture is of full-batch launches; traffic grows in proportion to the rows
            roof = {"bound": "hbm", "kernel": dom, "achieved": kern[dom]["gbs"], "peak": peak, "peak_kind": f"of {peak_kind}",
                    "unit": "GB/s", "frac": kern[dom]["gbs"] / peak, "frac_of_nominal_8000": kern[dom]["gbs"] / NOMINAL_HBM_GBS,
                    "traffic": None if traffic is None else int(traffic * scale_t), "traffic_captured_at": stamp,
                    "clocks_while_kernels_timed_alone": kernel_clocks,
                    "kernels": {n: dict(v, frac=v["gbs"] / peak, frac_of_nominal_8000=v["gbs"] / NOMINAL_HBM_GBS) for n, v in kern.items()}}
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": {L.F32: "f32", L.F16: "f16", L.BF16: "bf16"}[cfg.dtype] + " storage, f32 arithmetic", "data": "synthetic",
            "config": workload_config(cfg, T, args),
            "blocks_ms_per_step": [b / args.steps for b in blocks_ms], "value_is": "median block of K steps, maximum over ranks per block",
            "schedule": args.schedule, "by_schedule": by_schedule,
            "host_cpus_bound_to_gpu": bound_cpus,
            "step_algorithmic_bytes": int(step_bytes), "step_algorithmic_gbs": step_bytes / (ms_step * 1e-3) / 1e9,
            "step_l2_resident_bytes": int(l2_bytes), "step_hbm_gbs": (step_bytes - l2_bytes) / (ms_step * 1e-3) / 1e9,
            "gpu_launches": int(launches_per_step * args.steps), "launches_per_step": int(launches_per_step),
            "roofline": roof, "clocks": clocks, "e2e": e2e,
        }
        if weak:
            line["weak_tokens_per_s"] = weak["tokens_per_s"]
            line["weak"] = weak
        if configs:
            line["configs"] = configs
        if not args.no_cpu_baseline and world >= 1:
            line["cpu_baseline"] = cpu_baseline(cfg)
            line["parity"] = parity_gate(ctx, cfg, dev, stream, r0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def parity_gate(ctx, cfg, dev, stream, pos0, rows=192):
    """Runs with every measurement (part of the CPU leg): the four ops on a fresh sample of rows of this workload's
    shapes through the C ABI, checked against the CPU restatement. Gather must be bit-exact; the others must meet
    the bar of their storage type. The errors are also binned by the magnitude of the reference value."""
    import torch

    import lokal_b200 as L
    from oracle import lokal_oracle as O
    O.build()
    tdt = {L.F32: torch.float32, L.F16: torch.float16, L.BF16: torch.bfloat16}[cfg.dtype]
    d = synth.layer_inputs(cfg, rows, layer=1)
    d.pop("positions", None)  # the gate rotates by pos0 + row
    put = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(dev).to(tdt)
    get = lambda t: t.to(torch.float32).cpu().numpy()
    result = {"rows": rows, "bar": "f32: max abs 1e-5; f16: 2e-3 relative; bf16: one bf16 rounding (2^-8) of an f32-accurate value"}

    def grade(name, got, ref, atol):
        got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
        err = np.abs(got - ref)
        if cfg.dtype == L.F32:
            ok = bool(err.max() <= synth.F32_MAX_ABS)
        else:
            ok = bool((err <= synth.HALF_RTOL[cfg.dtype] * np.abs(ref) + atol).all())
        bins = {}
        for lo, hi, label in ((0, 1e-2, "|ref|<1e-2"), (1e-2, 1.0, "1e-2<=|ref|<1"), (1.0, np.inf, "|ref|>=1")):
            m = (np.abs(ref) >= lo) & (np.abs(ref) < hi)
            if m.any():
                bins[label] = {"n": int(m.sum()), "max_abs": float(err[m].max()), "max_rel": float((err[m] / np.maximum(np.abs(ref[m]), 1e-30)).max()) if lo > 0 else None}
        result[name] = {"ok": ok, "max_abs": float(err.max()), "by_magnitude": bins}

    # add_rmsnorm
    x, xn = put(d["x"]), torch.empty(rows, cfg.hidden, dtype=tdt, device=dev)
    ctx.add_rmsnorm(x, put(d["delta"]), put(d["w_norm"]), xn, rows=rows, dim=cfg.hidden, eps=cfg.eps, dtype=cfg.dtype, w_dtype=cfg.dtype, stream=stream)
    # qk_rope
    q, k = put(d["q"]), put(d["k"])
    opt = lambda name: put(d[name]) if name in d else None
    keep = [opt("q_bias"), opt("k_bias"), opt("q_norm_w"), opt("k_norm_w")]
    p = ctx.qk_rope_params(q=q, k=k, q_bias=keep[0], k_bias=keep[1], q_norm_w=keep[2], k_norm_w=keep[3], rows=rows,
                           n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, eps=cfg.eps,
                           q_dtype=cfg.dtype, w_dtype=cfg.dtype)
    ctx.qk_rope_pos(p, theta=cfg.theta, pos0=pos0, stream=stream)
    # swiglu
    g, u = put(d["gate"]), put(d["up"])
    inner = torch.empty(rows, cfg.inter, dtype=tdt, device=dev)
    ctx.swiglu(g, u, inner, n=rows * cfg.inter, dtype=cfg.dtype, stream=stream)
    # gather
    vocab = 4096
    table = synth.q8_0_table(vocab, cfg.hidden, cfg.seed + 9)
    ids = synth.token_ids_zipf(vocab, rows, cfg.seed + 9)
    gout = torch.empty(rows, cfg.hidden, dtype=tdt, device=dev)
    tdev, idev = torch.from_numpy(table).to(dev), torch.from_numpy(ids.view(np.int32)).to(dev)
    ctx.embed_gather(tdev, idev, gout, ggml_type=L.Q8_0, vocab=vocab, dim=cfg.hidden, n=rows, out_dtype=cfg.dtype, stream=stream)
    ctx.stream_sync(stream)

    rx, rxn = O.add_rmsnorm_rows(d["x"], d["delta"], d["w_norm"], cfg.eps)
    grade("add_rmsnorm", get(xn), rxn, 1e-6)
    rq, rk = O.qk_rope_rows(d["q"], d["k"], n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, theta=cfg.theta,
                            eps=cfg.eps, q_bias=d.get("q_bias"), k_bias=d.get("k_bias"), q_norm_w=d.get("q_norm_w"),
                            k_norm_w=d.get("k_norm_w"), pos0=pos0)
    grade("qk_rope", np.concatenate([get(q), get(k)], axis=1), np.concatenate([rq, rk], axis=1), 2e-6)
    grade("swiglu", get(inner), O.swiglu(d["gate"], d["up"]), 1e-6)
    want = synth.round_to(O.embed_gather(table, L.Q8_0, vocab, cfg.hidden, ids), cfg.dtype)
    gg = get(gout)
    result["embed_gather"] = {"ok": bool(np.array_equal(gg.view(np.uint32), want.view(np.uint32))), "bit_exact": True}
    result["ok"] = all(v["ok"] for v in result.values() if isinstance(v, dict))
    return result


def cpu_baseline(cfg):
    """The reference's CPU algorithm (oracle port) on a bounded sample, timed on this box's host cores."""
    from oracle import lokal_oracle as O
    O.build()
    threads = O.hardware_threads()
    vocab = cfg.vocab
    table = synth.q8_0_table(vocab, cfg.hidden, cfg.seed)
    probe_rows = min(cfg.rows, 4 * threads)
    probe = cpu_step_fn(cfg, probe_rows, table, vocab)
    probe(threads)
    dt = probe(threads)
    rows = int(min(cfg.rows, max(threads, probe_rows * 4.0 / max(dt, 1e-6))))  # about 4 s per step
    rows = max(threads, rows // threads * threads)
    step = cpu_step_fn(cfg, rows, table, vocab)
    step(threads)
    times = [step(threads) for _ in range(3)]
    one = cpu_step_fn(cfg, max(1, rows // threads), table, vocab)
    one(1)
    t1 = one(1)
    return {"value": rows / float(np.median(times)), "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{rows} of {cfg.rows} token rows, all {cfg.layers} layers, f32, median of 3 steps, {threads} token-parallel threads, "
                      f"Q8_0 table {vocab}x{cfg.hidden}, layer_period 2 (per-layer inputs cycle over 2 distinct layers of data)",
            "single_thread_value": max(1, rows // threads) / t1, "ops": cpu_ops(cfg, threads)}


def cpu_ops(cfg, threads, rows=None):
    """Each op of the path on its own, one layer, f32: token rows per second with 1 thread and with all threads."""
    from oracle import lokal_oracle as O
    rows = min(cfg.rows, 2048) if rows is None else rows
    d = synth.layer_inputs(cfg, rows)

    def best(fn, reps=3):
        fn()
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return rows / min(ts)

    kw = dict(n_q_heads=cfg.n_q_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, theta=cfg.theta, eps=cfg.eps,
              q_bias=d.get("q_bias"), k_bias=d.get("k_bias"), q_norm_w=d.get("q_norm_w"), k_norm_w=d.get("k_norm_w"),
              positions=d.get("positions"))
    out = {}
    for name, fn in (("add_rmsnorm", lambda t: O.add_rmsnorm_rows(d["x"], d["delta"], d["w_norm"], cfg.eps, threads=t)),
                     ("qk_rope", lambda t: O.qk_rope_rows(d["q"], d["k"], threads=t, **kw)),
                     ("swiglu", lambda t: O.swiglu(d["gate"], d["up"], threads=t))):
        out[name] = {"rows_per_s_1_thread": best(lambda: fn(1)), f"rows_per_s_{threads}_threads": best(lambda: fn(threads))}
    return out


# ------------------------------------------------------------------------------------------------
# C4: embedding gather + GGUF row dequant on its own (65536 Zipf(1.1) ids over a 151936-row table)
# ------------------------------------------------------------------------------------------------

def gather_variant_list(L):
    variants = [("q8_0_f32", L.Q8_0, synth.C4_DIM_Q8, L.F32), ("q8_0_f16", L.Q8_0, synth.C4_DIM_Q8, L.F16),
                ("q4_k_f32", L.Q4_K, synth.C4_DIM_Q4K, L.F32), ("q4_k_f16", L.Q4_K, synth.C4_DIM_Q4K, L.F16)]
    # the other block types of the gather, f32 out: 32-element blocks at the Q8_0 width, 256-element ones at the Q4_K width
    for ty in L.QUANT_TYPES + L.capi.GRID_TYPES:
        if ty not in (L.Q8_0, L.Q4_K):
            dim = synth.C4_DIM_Q8 if synth.QUANT_GEOMETRY[ty][0] == 32 else synth.C4_DIM_Q4K
            variants.append((synth.QUANT_NAMES[ty] + "_f32", ty, dim, L.F32))
    # dense tables: the reference's own `embed` kernel reads an f16 table into f32 rows (src/gpu/kernels.metal:30)
    variants += [("f16_table_f32", L.F16, synth.C4_DIM_Q8, L.F32), ("bf16_table_bf16", L.BF16, synth.C4_DIM_Q4K, L.BF16)]
    return variants


def gather_variants(L, ctx, dev, stream, sampler, peak, names, warmup, reps):
    """Times the named C4 variants (65,536 Zipf ids, 151,936-row table), each as a graph of 16 launches over rotating
    outputs, and checks the first 2048 rows of each bit for bit against the oracle. Returns (results, tables, ids)."""
    import torch
    from oracle import lokal_oracle as O
    O.build()
    threads = O.hardware_threads()
    vocab, n = synth.C4_VOCAB, synth.C4_IDS
    ids_np = synth.token_ids_zipf(vocab, n, synth.C4_SEED)
    uniq = int(np.unique(ids_np).size)
    ids = torch.from_numpy(ids_np.view(np.int32)).to(dev)
    tstream = torch.cuda.ExternalStream(stream, device=dev)
    tdt = {L.F32: torch.float32, L.F16: torch.float16, L.BF16: torch.bfloat16}
    variants = [v for v in gather_variant_list(L) if v[0] in names]
    if any(v[1] in L.capi.GRID_TYPES for v in variants):
        # the codebook types read the i-quant codebooks the caller hands over (the test fixture's copy of the format's tables)
        grids = np.load(os.path.join(ROOT, "tests", "golden", "iq_grids.npz"))
        ctx.set_iq_grids(grids)
        O.set_iq_grids(grids)
    tables, kern = {}, {}
    for name, ty, dim, odt in variants:
        if (ty, dim) not in tables:
            gen = {L.Q8_0: synth.q8_0_table, L.Q4_K: synth.q4_k_table}.get(ty)
            if ty in (L.F16, L.BF16):
                dense = synth.f32_table(vocab, dim, synth.C4_SEED + ty)
                host = dense.astype(np.float16).view(np.uint8).reshape(-1) if ty == L.F16 else \
                    (synth.round_to(dense, L.BF16).view(np.uint32) >> 16).astype(np.uint16).view(np.uint8).reshape(-1)
            else:
                host = gen(vocab, dim, synth.C4_SEED + ty) if gen else synth.quant_table(ty, vocab, dim, synth.C4_SEED + ty)
            tables[(ty, dim)] = (host, torch.from_numpy(host).to(dev))
        host, table = tables[(ty, dim)]
        es = 4 if odt == L.F32 else 2
        nbuf = 8  # rotating outputs: 8 x (up to 268 MB) between reuses, far beyond L2
        outs = torch.empty(nbuf, n, dim, dtype=tdt[odt], device=dev)
        reps_per_graph = 16
        ctx.graph_begin(stream)
        for r in range(reps_per_graph):
            ctx.embed_gather(table, ids, outs[r % nbuf], ggml_type=ty, vocab=vocab, dim=dim, n=n, out_dtype=odt, stream=stream)
        g = ctx.graph_end(stream)
        times = []
        for rep in range(warmup + reps):
            if sampler and rep == warmup:
                sampler.resume()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(tstream)
            ctx.graph_launch(g, stream)
            a1.record(tstream)
            ctx.stream_sync(stream)
            if rep >= warmup:
                times.append(a0.elapsed_time(a1) / reps_per_graph)
        if sampler:
            sampler.pause()
        ctx.graph_destroy(g)
        rb = L.row_bytes(ty, dim)
        alg = n * (4 + dim * es) + uniq * rb
        ms = float(np.mean(times))
        kern[name] = {"us_per_launch": 1e3 * ms, "tokens_per_s": n / (ms * 1e-3), "bytes_per_launch": int(alg),
                      "bytes_not_deduplicated": int(n * (rb + 4 + dim * es)), "gbs": alg / (ms * 1e-3) / 1e9,
                      "frac": alg / (ms * 1e-3) / 1e9 / peak, "frac_of_nominal_8000": alg / (ms * 1e-3) / 1e9 / NOMINAL_HBM_GBS,
                      "launches_timed": len(times) * reps_per_graph}
        # bit-exact spot check against the oracle on the first 2048 ids, every run
        want = O.embed_gather(host, ty, vocab, dim, ids_np[:2048], threads=threads)
        got = outs[0][:2048].to(torch.float32).cpu().numpy()
        ref = want if odt == L.F32 else synth.round_to(want, odt)
        kern[name]["bit_exact_vs_oracle_first_2048_rows"] = bool(np.array_equal(got.view(np.uint32), ref.view(np.uint32)))
        del outs
    return kern, tables, ids_np


def gather_workload(args, rank, world, local_rank):
    import torch

    import lokal_b200 as L
    from oracle import lokal_oracle as O

    if rank != 0:
        return
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ctx = L.Context(local_rank)
    vocab, n = synth.C4_VOCAB, synth.C4_IDS
    stream = ctx.stream_create()
    peak, peak_kind = measured_peak()
    names = [v[0] for v in gather_variant_list(L)]
    if args.only:  # a subset of the variants, e.g. for a profiler capture of one kernel
        names = [v for v in names if v in args.only.split(",")] or names[:1]
    sampler = ClockSampler(local_rank)
    sampler.pause()
    sampler.start()
    warmup, reps = max(args.warmup, 3), max(3, min(args.steps, 10))
    kern, tables, ids_np = gather_variants(L, ctx, dev, stream, sampler, peak, names, warmup, reps)
    clocks = sampler.finish()
    uniq = int(np.unique(ids_np).size)
    threads = O.hardware_threads()
    times, reps_per_graph = [0] * reps, 16
    # end to end: host ids in, host f32 rows out (Q8_0 -> f32, the configuration's first variant)
    if (L.Q8_0, synth.C4_DIM_Q8) not in tables:
        h8 = synth.q8_0_table(vocab, synth.C4_DIM_Q8, synth.C4_SEED + L.Q8_0)
        tables[(L.Q8_0, synth.C4_DIM_Q8)] = (h8, torch.from_numpy(h8).to(dev))
    host, table = tables[(L.Q8_0, synth.C4_DIM_Q8)]
    # ids and rows in page-locked host memory (reached by DMA), and the same call with ordinary arrays, the result in a
    # fresh allocation every time as the reference's Vec-returning gather has it (staged, pulled by worker threads)
    pin_ids = torch.from_numpy(ids_np.view(np.int32)).pin_memory()
    pin_out = torch.empty(n, synth.C4_DIM_Q8, dtype=torch.float32, pin_memory=True)
    e2e_reps = 5
    timings = {}
    for kind in ("pinned", "pageable"):
        call = (lambda: ctx.host_embed_gather(table, L.Q8_0, vocab, synth.C4_DIM_Q8, pin_ids.numpy().view(np.uint32), out=pin_out.numpy())) \
            if kind == "pinned" else (lambda: ctx.host_embed_gather(table, L.Q8_0, vocab, synth.C4_DIM_Q8, ids_np))
        got = call()
        t0 = time.perf_counter()
        for _ in range(e2e_reps):
            got = call()
        timings[kind] = (time.perf_counter() - t0) / e2e_reps
        assert np.array_equal(got[:64].view(np.uint32), O.embed_gather(host, L.Q8_0, vocab, synth.C4_DIM_Q8, ids_np[:64]).view(np.uint32))
    dt = timings["pinned"]
    e2e = {"value": n / dt, "unit": "tokens/s", "h2d_bytes_per_step": n * 4, "d2h_bytes_per_step": n * synth.C4_DIM_Q8 * 4,
           "ms_per_step": 1e3 * dt, "d2h_gbs": n * synth.C4_DIM_Q8 * 4 / dt / 1e9,
           "pageable_fresh_output_tokens_per_s": n / timings["pageable"], "pageable_ms_per_step": 1e3 * timings["pageable"],
           "api": "lokal_cuda_host_embed_gather (host ids in, host f32 rows out, table resident; pinned caller buffers)"}
    # CPU: the reference's gather loop (one row at a time, dequant_row_ref), 1 thread and all threads
    cpu = {}
    for t in (1, threads):
        O.embed_gather(host, L.Q8_0, vocab, synth.C4_DIM_Q8, ids_np, threads=t)
        t0 = time.perf_counter()
        O.embed_gather(host, L.Q8_0, vocab, synth.C4_DIM_Q8, ids_np, threads=t)
        cpu[t] = n / (time.perf_counter() - t0)
    first = kern.get("q8_0_f32") or next(iter(kern.values()))
    line = {
        "metric": "embedding gather + GGUF row dequant, tokens/s", "value": first["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
        "steps": len(times) * reps_per_graph, "warmup": max(args.warmup, 3), "ms_per_step": first["us_per_launch"] * 1e-3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8 blocks -> f32", "data": "synthetic",
        "config": {"workload": "gguf-gather-zipf65536", "vocab": vocab, "ids": n, "unique_ids": uniq,
                   "tables": "Q8_0 151936x896; Q4_K 151936x1024 (a 896-wide Q4_K row cannot exist: 256-element super-blocks)",
                   "l2": "outputs rotate over 8 buffers (up to 2.1 GB) between reuses"},
        "gpu_launches": sum(v["launches_timed"] for v in kern.values()),
        "roofline": {"bound": "hbm", "kernel": "gather_quant_staged_kernel<Q8_0,f32>", "achieved": first["gbs"], "peak": peak,
                     "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": first["frac"], "traffic": None, "kernels": kern},
        "clocks": clocks, "e2e": e2e,
        "cpu_baseline": {"value": cpu[threads], "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"all {n} ids, Q8_0 896-wide rows to f32", "single_thread_value": cpu[1]},
    }
    print(json.dumps(line), flush=True)


def row_ops_workload(args, rank, world, local_rank):
    """The ops either side of the layer path, each timed alone as a graph of launches over rotating buffers:
    K/V staging after RoPE and the gated-deltanet per-row siblings, at 8192 token rows of the qwen35-27B geometry
    (d_state 128, 48 V heads, 16 K heads, 24 attention heads of 256)."""
    import torch

    import lokal_b200 as L
    from oracle import lokal_oracle as O

    if rank != 0:
        return
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ctx = L.Context(local_rank)
    stream = ctx.stream_create()
    tstream = torch.cuda.ExternalStream(stream, device=dev)
    peak, peak_kind = measured_peak()
    T, S, HV, HK, HA, HD = args.rows or 8192, 128, 48, 16, 24, 256
    nbuf, reps = 6, 12
    rnd = lambda *shape: torch.randn(*shape, device=dev, dtype=torch.float32)
    kern = {}
    sampler = ClockSampler(local_rank)  # samples inside the timed loops only
    sampler.pause()
    sampler.start()

    def timed(name, alg_bytes, launch):
        ctx.graph_begin(stream)
        for r in range(reps):
            launch(r % nbuf)
        g = ctx.graph_end(stream)
        times = []
        for rep in range(max(args.warmup, 3) + max(3, min(args.steps, 10))):
            if rep == max(args.warmup, 3):
                sampler.resume()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(tstream)
            ctx.graph_launch(g, stream)
            a1.record(tstream)
            ctx.stream_sync(stream)
            if rep >= max(args.warmup, 3):
                times.append(a0.elapsed_time(a1) / reps)
        sampler.pause()
        ctx.graph_destroy(g)
        ms = float(np.mean(times))
        kern[name] = {"us_per_launch": 1e3 * ms, "bytes_per_launch": int(alg_bytes), "gbs": alg_bytes / (ms * 1e-3) / 1e9,
                      "frac": alg_bytes / (ms * 1e-3) / 1e9 / peak, "launches_timed": len(times) * reps}

    # l2norm over the q and k heads of every token: read + write
    x = rnd(nbuf, T, 2 * HK * S)
    timed("l2norm_rows_f32", 2 * T * 2 * HK * S * 4, lambda b: ctx.l2norm_rows(x[b], dim=S, eps=1e-6, rows_per_token=T * 2 * HK, stream=stream))
    # one row against the oracle, every run
    probe = rnd(4, S)
    want = O.l2norm_rows(probe.cpu().numpy(), S, 1e-6)
    ctx.l2norm_rows(probe, dim=S, eps=1e-6, rows_per_token=4, stream=stream)
    ctx.stream_sync(stream)
    kern["l2norm_rows_f32"]["max_rel_err_vs_oracle"] = float(np.max(np.abs(probe.cpu().numpy() - want) / np.maximum(np.abs(want), 1e-30)))
    del x
    # gated output norm: o and z read, y written
    o, z, w = rnd(nbuf, T * HV, S), rnd(nbuf, T * HV, S), rnd(S)
    timed("gated_output_norm_f32", 3 * T * HV * S * 4, lambda b: ctx.gated_output_norm(o[b], w, z[b], rows=T * HV, dim=S, eps=1e-6, stream=stream))
    del o, z
    # attention out-gate and the q/gate split it depends on
    a, gt = rnd(nbuf, T, HA * HD), rnd(nbuf, T, HA * HD)
    timed("attn_out_gate_f32", 3 * T * HA * HD * 4, lambda b: ctx.attn_out_gate(a[b], gt[b], n=T * HA * HD, stream=stream))
    src = rnd(2, T, HA * 2 * HD)
    timed("split_q_gate_f32", 2 * T * HA * 2 * HD * 4,
          lambda b: ctx.split_q_gate(src[b % 2], a[b], gt[b], rows=T, n_heads=HA, head_dim=HD, stream=stream))
    del a, gt, src
    # partial RoPE with per-head norm at the qwen35 attention geometry: 24 q heads + 4 kv heads of 256, 64 rotated dims
    HKV, ROT = 4, 64
    q, k = rnd(nbuf, T, HA * HD), rnd(nbuf, T, HKV * HD)
    qw, kw = 1 + 0.1 * rnd(HD), 1 + 0.1 * rnd(HD)
    table = torch.empty(T, ROT, device=dev, dtype=torch.float32)
    ctx.rope_table(table, theta=1e7, rot_dim=ROT, rows=T, pos0=0, stream=stream)
    params = [ctx.qk_rope_params(q=q[b], k=k[b], rows=T, n_q_heads=HA, n_kv_heads=HKV, head_dim=HD, rot_dim=ROT, eps=1e-6, q_norm_w=qw,
                                 k_norm_w=kw, cos_sin=table, q_dtype=L.F32, k_dtype=L.F32, w_dtype=L.F32) for b in range(nbuf)]
    timed("qk_rope_partial_64_of_256_f32", T * (2 * (HA + HKV) * HD * 4 + ROT * 4), lambda b: ctx.qk_rope(params[b], stream=stream))
    del q, k
    # K/V staging: f32 rows of 8 KV heads x 128 narrowed to f16 and scattered into a windowed cache (sink 4, ring 8704)
    kvd = 1024
    lay = L.window_cfg(8192, 4)
    cap = lay.sink_pad + lay.ring
    fresh = rnd(nbuf, T, kvd)
    cache = torch.zeros(nbuf, cap, kvd, device=dev, dtype=torch.float16)
    idx = torch.empty(T, device=dev, dtype=torch.int32)
    timed("kv_rows_windowed", T * 4, lambda b: ctx.kv_rows(idx, layout=lay, rows=T, pos0=20000, slot0=0, stream=stream))
    timed("kv_stage_f32_to_f16", T * (kvd * 6 + 4), lambda b: ctx.kv_stage(fresh[b], cache[b], src_dtype=L.F32, dst_dtype=L.F16, rows=T, width=kvd,
                                                                            dst_rows=idx, stream=stream))
    del fresh, cache
    # the deltanet conv over the whole chunk (10240 channels, 4 taps, window rolled at the end) and its gate scalars
    CH, KC = 2 * HK * S + HV * S, 4
    cx, cout = rnd(nbuf, T, CH), torch.empty(nbuf, T, CH, device=dev, dtype=torch.float32)
    cstate, cw = rnd(CH, KC - 1), 0.5 * rnd(CH, KC)
    timed("ssm_conv_chunk_f32", 2 * T * CH * 4, lambda b: ctx.ssm_conv(cstate, cx[b], cw, cout[b], channels=CH, d_conv=KC, n_tokens=T, stream=stream))
    ref_out, _ = O.ssm_conv(np.ones((256, KC - 1), np.float32), cx[0, :8, :256].cpu().numpy(), cw[:256].cpu().numpy(), KC)
    small = torch.empty(8, 256, device=dev, dtype=torch.float32)
    ctx.ssm_conv(torch.ones(256, KC - 1, device=dev), cx[0, :8, :256].contiguous(), cw[:256].contiguous(), small, channels=256, d_conv=KC, n_tokens=8,
                 roll=False, stream=stream)
    ctx.stream_sync(stream)
    kern["ssm_conv_chunk_f32"]["max_abs_err_vs_oracle"] = float(np.abs(small.cpu().numpy() - ref_out).max())
    del cx, cout
    hx = torch.randn(nbuf, T, CH, device=dev, dtype=torch.float32).to(torch.bfloat16)
    hout = torch.empty_like(hx)
    timed("ssm_conv_chunk_bf16", 2 * T * CH * 2, lambda b: ctx.ssm_conv(cstate, hx[b], cw, hout[b], channels=CH, d_conv=KC, n_tokens=T, dtype=L.BF16, stream=stream))
    del hx, hout
    al, bi = rnd(nbuf, T, HV), rnd(nbuf, T, HV)
    ga, gb, aw, dtb = torch.empty(nbuf, T, HV, device=dev), torch.empty(nbuf, T, HV, device=dev), -torch.exp(rnd(HV)), rnd(HV)
    timed("delta_gates_f32", 4 * T * HV * 4, lambda b: ctx.delta_gates(al[b], bi[b], aw, dtb, ga[b], gb[b], n_v_heads=HV, n_tokens=T, stream=stream))
    # the weight-page conversion of the low-memory stage-in: 64 Mi bf16 values to f16
    PN = 64 << 20
    page = torch.randn(2, PN, device=dev, dtype=torch.float32).to(torch.bfloat16)
    pout = torch.empty(2, PN, device=dev, dtype=torch.float16)
    clip = torch.zeros(1, device=dev, dtype=torch.int32)
    timed("bf16_to_f16_page", 4 * PN, lambda b: ctx.bf16_to_f16_copy(page[b % 2], pout[b % 2], n=PN, clip_flag=clip, stream=stream))
    kern["bf16_to_f16_page"]["equals_torch_conversion"] = bool(torch.equal(pout[0], page[0].to(torch.float16)))
    first = kern["gated_output_norm_f32"]
    line = {
        "metric": "gated output norm rows/s", "value": T * HV / (first["us_per_launch"] * 1e-6), "unit": "rows/s", "n_gpus": 1,
        "steps": first["launches_timed"], "warmup": max(args.warmup, 3), "ms_per_step": first["us_per_launch"] * 1e-3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "row-ops-next-to-the-layer-path", "token_rows": T, "d_state": S, "v_heads": HV, "k_heads": HK,
                   "attn_heads": HA, "head_dim": HD, "l2": f"each op rotates over {nbuf} buffer sets far larger than L2"},
        "gpu_launches": sum(k["launches_timed"] for k in kern.values()),
        "roofline": {"bound": "hbm", "kernel": "deltanet_rows_kernel<f32,1,gated>", "achieved": first["gbs"], "peak": peak,
                     "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": first["frac"], "traffic": None, "kernels": kern},
        "clocks": sampler.finish(),
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(synth.CONFIGS) + ["c4", "rows"], default="c5")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="strong",
                    help="strong: the batch's token rows are partitioned over the GPUs (the configuration as stated); weak: a full batch per GPU")
    ap.add_argument("--blocks", type=int, default=5, help="timed blocks of --steps steps; value is the median block")
    ap.add_argument("--schedule", choices=["auto", "sequential", "branches"], default="auto",
                    help="how the pass orders the kernels of a step (lokal_cuda_pass_set_schedule)")
    ap.add_argument("--no-extras", action="store_true", help="skip the weak figure (N > 1) and the other configs (N = 1)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (small captures under a profiler)")
    ap.add_argument("--rows", type=int, default=0, help="override the token rows per GPU")
    ap.add_argument("--only", default="", help="c4: comma-separated variant names to run (e.g. q8_0_f16)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-kernel-timing", action="store_true", help="skip the per-kernel section (launch lists under a profiler)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank, world, local_rank = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    if world == 1 and args.gpus > 1:
        sys.exit("bench.py --gpus N > 1 must be launched with torch.distributed.run (one process per GPU)")
    if args.workload == "c4":
        if args.impl == "reference":
            sys.exit("--impl reference is defined for the layer workloads; the c4 line carries its own cpu_baseline")
        return gather_workload(args, rank, world, local_rank)
    if args.workload == "rows":
        if args.impl == "reference":
            sys.exit("--impl reference is defined for the layer workloads")
        return row_ops_workload(args, rank, world, local_rank)
    cfg = synth.CONFIGS[args.workload]
    if args.layers or args.rows:  # reduced sizes for profiler captures; the default is the full workload
        import dataclasses
        cfg = dataclasses.replace(cfg, layers=args.layers or cfg.layers, rows=args.rows or cfg.rows,
                                  name=cfg.name + f"[layers={args.layers or cfg.layers},rows={args.rows or cfg.rows}]")
    if args.impl == "reference":
        reference_arm(args, cfg, rank, world)
    else:
        ours(args, cfg, rank, world, local_rank)


if __name__ == "__main__":
    main()
