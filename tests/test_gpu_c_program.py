"""The C ABI driven from a plain C program, no Python and no torch between the caller and the library: what a
backend written in a compiled language sees. The program reads one layer's inputs from a file, runs embed gather,
residual-add + RMSNorm, bias + qk-norm + RoPE and SwiGLU on the device through `lokal_cuda.h`, writes the results back,
and this test compares them with the CPU oracle (same bars as the other parity tests)."""
import os
import shutil
import subprocess

import numpy as np
import pytest

import synth
from lokal_b200 import capi
from synth import F32

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r'''
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "lokal_cuda.h"

#define CHECK(call) do { int rc_ = (call); if (rc_ != LOKAL_OK) { \
    fprintf(stderr, "%s failed: %d %s\n", #call, rc_, ctx ? lokal_cuda_last_error(ctx) : ""); return 10; } } while (0)

static void* slurp(FILE* f, size_t bytes) {
    void* p = malloc(bytes);
    if (!p || fread(p, 1, bytes, f) != bytes) { fprintf(stderr, "short read\n"); exit(11); }
    return p;
}

int main(int argc, char** argv) {
    lokal_cuda_ctx* ctx = NULL;
    lokal_cuda_stream s = NULL;
    unsigned hdr[8]; /* rows, hidden, inter, n_q, n_kv, head_dim, vocab, table_bytes */
    FILE* in = fopen(argv[1], "rb");
    FILE* out = fopen(argv[2], "wb");
    if (argc != 3 || !in || !out || fread(hdr, 4, 8, in) != 8) return 12;
    const size_t rows = hdr[0], H = hdr[1], I = hdr[2], nq = hdr[3], nkv = hdr[4], hd = hdr[5], vocab = hdr[6], tb = hdr[7];
    const size_t qd = nq * hd, kd = nkv * hd;
    void* table = slurp(in, tb);
    unsigned* ids = slurp(in, rows * 4);
    float* delta = slurp(in, rows * H * 4);
    float* w = slurp(in, H * 4);
    float* q = slurp(in, rows * qd * 4);
    float* k = slurp(in, rows * kd * 4);
    float* qw = slurp(in, hd * 4);
    float* kw = slurp(in, hd * 4);
    float* gate = slurp(in, rows * I * 4);
    float* up = slurp(in, rows * I * 4);

    CHECK(lokal_cuda_create(0, &ctx));
    CHECK(lokal_cuda_stream_create(ctx, &s));
    void *d_table, *d_ids, *d_x, *d_delta, *d_w, *d_xn, *d_q, *d_k, *d_qw, *d_kw, *d_gate, *d_up, *d_tab;
    CHECK(lokal_cuda_malloc(ctx, tb, &d_table));
    CHECK(lokal_cuda_malloc(ctx, rows * 4, &d_ids));
    CHECK(lokal_cuda_malloc(ctx, rows * H * 4, &d_x));
    CHECK(lokal_cuda_malloc(ctx, rows * H * 4, &d_delta));
    CHECK(lokal_cuda_malloc(ctx, H * 4, &d_w));
    CHECK(lokal_cuda_malloc(ctx, rows * H * 4, &d_xn));
    CHECK(lokal_cuda_malloc(ctx, rows * qd * 4, &d_q));
    CHECK(lokal_cuda_malloc(ctx, rows * kd * 4, &d_k));
    CHECK(lokal_cuda_malloc(ctx, hd * 4, &d_qw));
    CHECK(lokal_cuda_malloc(ctx, hd * 4, &d_kw));
    CHECK(lokal_cuda_malloc(ctx, rows * I * 4, &d_gate));
    CHECK(lokal_cuda_malloc(ctx, rows * I * 4, &d_up));
    CHECK(lokal_cuda_malloc(ctx, rows * hd * 4, &d_tab));
    CHECK(lokal_cuda_memcpy_h2d(ctx, s, d_table, table, tb));
    CHECK(lokal_cuda_memcpy_h2d(ctx, s, d_ids, ids, rows * 4));
    CHECK(lokal_cuda_memcpy_h2d(ctx, s, d_delta, delta, rows * H * 4));
    CHECK(lokal_cuda_memcpy_h2d(ctx, s, d_w, w, H * 4));
    CHECK(lokal_cuda_memcpy_h2d(ctx, s, d_q, q, rows * qd * 4));
    CHECK(lokal_cuda_memcpy_h2d(ctx, s, d_k, k, rows * kd * 4));
    CHECK(lokal_cuda_memcpy_h2d(ctx, s, d_qw, qw, hd * 4));
    CHECK(lokal_cuda_memcpy_h2d(ctx, s, d_kw, kw, hd * 4));
    CHECK(lokal_cuda_memcpy_h2d(ctx, s, d_gate, gate, rows * I * 4));
    CHECK(lokal_cuda_memcpy_h2d(ctx, s, d_up, up, rows * I * 4));

    /* the step: x = embed(ids); x += delta, xn = rmsnorm(x); q,k = rope(qk-norm(q,k)); inner = silu(gate) * up */
    CHECK(lokal_cuda_embed_gather(ctx, s, d_table, LOKAL_Q8_0, vocab, H, d_ids, rows, d_x, LOKAL_F32));
    CHECK(lokal_cuda_add_rmsnorm(ctx, s, d_x, d_delta, d_w, d_xn, NULL, rows, H, 1e-6f, LOKAL_F32, LOKAL_F32, LOKAL_F16));
    CHECK(lokal_cuda_rope_table(ctx, s, 1e6f, (unsigned)hd, NULL, 100, rows, d_tab));
    {
        lokal_qk_rope_params p;
        memset(&p, 0, sizeof p);
        p.q = d_q; p.k = d_k; p.q_norm_w = d_qw; p.k_norm_w = d_kw; p.cos_sin = d_tab;
        p.rows = rows; p.n_q_heads = (unsigned)nq; p.n_kv_heads = (unsigned)nkv; p.head_dim = (unsigned)hd; p.rot_dim = (unsigned)hd;
        p.q_row_stride = qd; p.k_row_stride = kd; p.eps = 1e-6f;
        p.q_dtype = LOKAL_F32; p.k_dtype = LOKAL_F32; p.w_dtype = LOKAL_F32;
        CHECK(lokal_cuda_qk_rope(ctx, s, &p));
    }
    CHECK(lokal_cuda_swiglu(ctx, s, d_gate, d_up, d_gate, NULL, rows * I, LOKAL_F32, LOKAL_F16));

    CHECK(lokal_cuda_memcpy_d2h(ctx, s, delta, d_x, rows * H * 4));    /* reuse the host buffers for the results */
    CHECK(lokal_cuda_memcpy_d2h(ctx, s, gate, d_gate, rows * I * 4));
    CHECK(lokal_cuda_memcpy_d2h(ctx, s, q, d_q, rows * qd * 4));
    CHECK(lokal_cuda_memcpy_d2h(ctx, s, k, d_k, rows * kd * 4));
    float* xn = malloc(rows * H * 4);
    CHECK(lokal_cuda_memcpy_d2h(ctx, s, xn, d_xn, rows * H * 4));
    CHECK(lokal_cuda_stream_sync(ctx, s));
    fwrite(delta, 4, rows * H, out);
    fwrite(xn, 4, rows * H, out);
    fwrite(q, 4, rows * qd, out);
    fwrite(k, 4, rows * kd, out);
    fwrite(gate, 4, rows * I, out);
    fclose(out);

    /* an id outside the table is reported at the next sync, by code and by message */
    ids[0] = (unsigned)vocab;
    CHECK(lokal_cuda_memcpy_h2d(ctx, s, d_ids, ids, rows * 4));
    CHECK(lokal_cuda_embed_gather(ctx, s, d_table, LOKAL_Q8_0, vocab, H, d_ids, rows, d_x, LOKAL_F32));
    if (lokal_cuda_stream_sync(ctx, s) != LOKAL_ERR_ID_RANGE || !strstr(lokal_cuda_last_error(ctx), "out of range")) return 13;
    if (lokal_cuda_stream_sync(ctx, s) != LOKAL_OK) return 14; /* the error word was cleared */
    CHECK(lokal_cuda_free(ctx, d_table));
    CHECK(lokal_cuda_stream_destroy(ctx, s));
    lokal_cuda_destroy(ctx);
    printf("ok %s\n", lokal_cuda_version());
    return 0;
}
'''


def test_a_c_program_runs_a_layer_step_through_the_abi(tmp_path, oracle):
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    capi.load()
    libdir = os.path.dirname(capi.library_path()) if hasattr(capi, "library_path") else os.path.join(ROOT, "lokal_b200")
    src, exe = tmp_path / "layer_step.c", tmp_path / "layer_step"
    src.write_text(PROGRAM)
    subprocess.run([cc, "-std=c99", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", libdir, "-llokal_cuda", f"-Wl,-rpath,{libdir}"], check=True, capture_output=True, text=True)

    rows, H, I, nq, nkv, hd, vocab = 77, 256, 640, 4, 2, 64, 500
    cfg = synth.LayerConfig("c-program", F32, rows, H, I, nq, nkv, hd, vocab, 1e6, 1e-6, 1, qk_norm=True, seed=4242)
    d = synth.layer_inputs(cfg, rows)
    table = synth.q8_0_table(vocab, H, 4243)
    ids = synth.token_ids_uniform(vocab, rows, 4244)
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(fin, "wb") as f:
        f.write(np.array([rows, H, I, nq, nkv, hd, vocab, table.size], np.uint32).tobytes())
        for a in (table, ids, d["delta"], d["w_norm"], d["q"], d["k"], d["q_norm_w"], d["k_norm_w"], d["gate"], d["up"]):
            f.write(np.ascontiguousarray(a).tobytes())
    res = subprocess.run([str(exe), str(fin), str(fout)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and res.stdout.startswith("ok "), (res.returncode, res.stdout, res.stderr)

    got = np.fromfile(fout, np.float32)
    sizes = [rows * H, rows * H, rows * nq * hd, rows * nkv * hd, rows * I]
    assert got.size == sum(sizes)
    x_new, xn, q, k, inner = [part.reshape(rows, -1) for part in np.split(got, np.cumsum(sizes)[:-1])]
    emb = oracle.embed_gather(table, 8, vocab, H, ids)
    ref_x, ref_xn = oracle.add_rmsnorm_rows(emb, d["delta"], d["w_norm"], 1e-6)
    synth.assert_bits_equal(x_new, ref_x, "embed + delta")  # gather is exact and the residual is one IEEE add
    synth.check_f32(xn, ref_xn, "rmsnorm")
    rq, rk = oracle.qk_rope_rows(d["q"], d["k"], n_q_heads=nq, n_kv_heads=nkv, head_dim=hd, theta=1e6, eps=1e-6,
                                 q_norm_w=d["q_norm_w"], k_norm_w=d["k_norm_w"], pos0=100)
    synth.check_f32(q, rq, "q", atol=2e-5)
    synth.check_f32(k, rk, "k", atol=2e-5)
    synth.check_f32(inner, oracle.swiglu(d["gate"], d["up"]), "swiglu")
