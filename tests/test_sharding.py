"""Token-row sharding over ranks (world_size 2, gloo, CPU): each rank takes its contiguous block with its
own absolute positions and ids, nothing is exchanged on the path, and the concatenation of the shards
equals the single-rank result. The per-row work is done by the CPU oracle here; on GPUs the same
partition feeds the CUDA ops."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_rows, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, HERE)
    import lokal_b200
    import synth
    from oracle import lokal_oracle as O
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    cfg = synth.LayerConfig("t", 0, n_rows, 64, 96, 4, 2, 16, 97, 1e6, 1e-6, 1, qk_norm=True, seed=21)
    d = synth.layer_inputs(cfg)               # every rank can generate the whole batch deterministically
    table = synth.q8_0_table(cfg.vocab, cfg.hidden, 5)
    ids = synth.token_ids_uniform(cfg.vocab, n_rows, 6)
    r0, cnt = lokal_b200.shard_rows(n_rows, world, rank)
    sl = slice(r0, r0 + cnt)
    x = O.embed_gather(table, 8, cfg.vocab, cfg.hidden, ids[sl])
    x, xn = O.add_rmsnorm_rows(x, d["delta"][sl], d["w_norm"], cfg.eps)
    q, k = O.qk_rope_rows(d["q"][sl], d["k"][sl], n_q_heads=4, n_kv_heads=2, head_dim=16, theta=cfg.theta,
                          eps=cfg.eps, q_norm_w=d["q_norm_w"], k_norm_w=d["k_norm_w"], pos0=1000 + r0)
    inner = O.swiglu(d["gate"][sl], d["up"][sl])
    local = np.concatenate([xn, q, k, inner], axis=1)
    # optional final gather, off the op path: pad to the largest shard so all_gather sees equal shapes
    per = -(-n_rows // world)
    pad = np.zeros((per, local.shape[1]), np.float32)
    pad[:cnt] = local
    bufs = [torch.empty(per, local.shape[1]) for _ in range(world)]
    dist.all_gather(bufs, torch.from_numpy(pad))
    counts = [lokal_b200.shard_rows(n_rows, world, r)[1] for r in range(world)]
    whole = np.concatenate([b.numpy()[:c] for b, c in zip(bufs, counts)])
    if rank == 0:
        x1 = O.embed_gather(table, 8, cfg.vocab, cfg.hidden, ids)
        x1, xn1 = O.add_rmsnorm_rows(x1, d["delta"], d["w_norm"], cfg.eps)
        q1, k1 = O.qk_rope_rows(d["q"], d["k"], n_q_heads=4, n_kv_heads=2, head_dim=16, theta=cfg.theta, eps=cfg.eps,
                                q_norm_w=d["q_norm_w"], k_norm_w=d["k_norm_w"], pos0=1000)
        ref = np.concatenate([xn1, q1, k1, O.swiglu(d["gate"], d["up"])], axis=1)
        ret["equal"] = bool(np.array_equal(whole.view(np.uint32), ref.view(np.uint32)))
        ret["rows"] = int(whole.shape[0])
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("n_rows", [64, 37])
def test_two_rank_shards_concatenate_to_the_single_rank_result(n_rows):
    from oracle import lokal_oracle
    lokal_oracle.build()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as m:
        ret = m.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, n_rows, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
            assert p.exitcode == 0
        assert ret["rows"] == n_rows and ret["equal"]


def test_bench_partition_is_the_librarys_and_both_arms_print_the_same_config():
    """bench.py splits the batch's rows over the ranks exactly as lokal_cuda_shard_rows does (strong scaling: the
    configuration's 8192 rows are partitioned, never replicated), and the `config` object it prints is the same
    dictionary in the GPU arm and in the CPU arm for every world size."""
    import argparse
    import importlib.util
    import lokal_b200
    sys.path.insert(0, HERE)
    import synth
    spec = importlib.util.spec_from_file_location("bench_for_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    cfg = synth.C5
    for world in (1, 2, 3, 4, 8):
        args = argparse.Namespace(scaling="strong", gpus=world)
        spans = [bench.shard_of(cfg, args, r, world) for r in range(world)]
        assert spans == [lokal_b200.shard_rows(cfg.rows, world, r) for r in range(world)]
        assert sum(c for _, c in spans) == cfg.rows
        # what rank 0 of the GPU arm prints, and what the CPU arm (rank 0 only) prints
        ours = bench.workload_config(cfg, spans[0][1], args)
        ref = bench.workload_config(cfg, bench.shard_of(cfg, args, 0, max(1, args.gpus))[1], args)
        assert ours == ref and ours["rows"] == 8192 and ours["rows_per_gpu"] == -(-8192 // world)
        weak = argparse.Namespace(scaling="weak", gpus=world)
        assert [bench.shard_of(cfg, weak, r, world) for r in range(world)] == [(r * cfg.rows, cfg.rows) for r in range(world)]
