"""Regenerates tests/golden/oracle_small.npz: small seeded inputs with the oracle's outputs.

The reference is Rust and cannot be run in this environment (no Rust toolchain), so these vectors
come from the C++ restatement in oracle/ after it has been pinned against the reference's own
known-answer vectors (reference_kats.json). They serve two purposes: a regression guard on the
oracle itself (a changed compiler flag or an accidental FMA shows up as changed bits), and a set
of committed input/output pairs the CUDA path is compared with on the GPU.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

import synth  # noqa: E402
from oracle import lokal_oracle as O  # noqa: E402


def main():
    O.build()
    out = {}
    rng = np.random.default_rng(0x601D)
    # rmsnorm / add_rmsnorm, f32, SmolLM2 width
    x = rng.standard_normal((4, 576), dtype=np.float32)
    dl = rng.standard_normal((4, 576), dtype=np.float32)
    w = (1 + 0.1 * rng.standard_normal(576)).astype(np.float32)
    xs, xn = O.add_rmsnorm_rows(x, dl, w, 1e-5)
    out.update(norm_x=x, norm_delta=dl, norm_w=w, norm_eps=np.float32(1e-5), norm_sum=xs, norm_out=xn)
    # qk_rope: Qwen2-style bias (head_dim 64) and Qwen3-style per-head norm (head_dim 128)
    q = rng.standard_normal((3, 4 * 64), dtype=np.float32)
    k = rng.standard_normal((3, 2 * 64), dtype=np.float32)
    qb = (0.1 * rng.standard_normal(4 * 64)).astype(np.float32)
    kb = (0.1 * rng.standard_normal(2 * 64)).astype(np.float32)
    pos = np.array([0, 17, 32767], np.int32)
    rq, rk = O.qk_rope_rows(q, k, n_q_heads=4, n_kv_heads=2, head_dim=64, theta=1e6, q_bias=qb, k_bias=kb, positions=pos)
    out.update(rope_q=q, rope_k=k, rope_qb=qb, rope_kb=kb, rope_pos=pos, rope_theta=np.float32(1e6), rope_q_out=rq, rope_k_out=rk)
    q3 = rng.standard_normal((2, 2 * 128), dtype=np.float32)
    k3 = rng.standard_normal((2, 1 * 128), dtype=np.float32)
    qn = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    kn = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    r3q, r3k = O.qk_rope_rows(q3, k3, n_q_heads=2, n_kv_heads=1, head_dim=128, theta=1e6, eps=1e-6, q_norm_w=qn, k_norm_w=kn, pos0=8000)
    out.update(qn_q=q3, qn_k=k3, qn_qw=qn, qn_kw=kn, qn_q_out=r3q, qn_k_out=r3k)
    # swiglu
    g = (2 * rng.standard_normal(512)).astype(np.float32)
    u = (2 * rng.standard_normal(512)).astype(np.float32)
    out.update(sw_gate=g, sw_up=u, sw_out=O.swiglu(g, u))
    # gather: small random tables + the adversarial rows
    for name, ty, dim in (("q8", O.Q8_0, 96), ("q4k", O.Q4_K, 512)):
        table = (synth.q8_0_table if ty == O.Q8_0 else synth.q4_k_table)(9, dim, seed=77)
        ids = np.array([8, 0, 3, 3, 7, 1], np.uint32)
        out[f"{name}_table"] = table
        out[f"{name}_ids"] = ids
        out[f"{name}_out"] = O.embed_gather(table, ty, 9, dim, ids)
        adv = O.adversarial_rows(ty, 8, 3)
        cols = 8 * O.blk_elems(ty)
        rb = O.row_bytes(ty, cols)
        out[f"{name}_adv"] = adv
        out[f"{name}_adv_out"] = np.stack([O.dequant_row_ref(ty, adv[r * rb:(r + 1) * rb], cols) for r in range(3)])
    np.savez_compressed(os.path.join(HERE, "oracle_small.npz"), **out)
    print("wrote", os.path.join(HERE, "oracle_small.npz"), sum(v.nbytes for v in out.values()), "bytes raw")


if __name__ == "__main__":
    main()
