"""Embedding gather + GGUF row dequant through the C ABI: bit-exact against the CPU oracle."""
import numpy as np
import pytest

import synth
from synth import BF16, F16, F32, Q4_K, Q8_0

pytestmark = pytest.mark.gpu


def f16b(v):
    return np.array([v], np.float16).view(np.uint8)


def gather(ctx, dev, table, ty, vocab, dim, ids, out_dtype=F32):
    dt = dev.put(table)
    di = dev.put(np.asarray(ids, np.uint32))
    out = dev.empty((len(ids) + 1, dim), out_dtype, fill=4.0)
    ctx.embed_gather(dt, di, out, ggml_type=ty, vocab=vocab, dim=dim, n=len(ids), out_dtype=out_dtype)
    ctx.stream_sync()
    res = dev.get(out)
    assert (res[-1] == 4.0).all(), "wrote past the last row"
    return res[:-1]


def dequant(ctx, dev, src, ty, rows, cols, out_dtype=F32):
    out = dev.empty((rows, cols), out_dtype, fill=4.0)
    ctx.dequant_rows(dev.put(src), out, ggml_type=ty, rows=rows, cols=cols, out_dtype=out_dtype)
    ctx.stream_sync()
    return dev.get(out)


def test_reference_hand_vectors(ctx, dev):
    # src/gguf/dequant.rs:683-692
    blk = np.zeros(34, np.uint8)
    blk[:2] = f16b(0.5)
    blk[2] = np.uint8(256 - 7)
    blk[33] = 100
    y = dequant(ctx, dev, blk, Q8_0, 1, 32)[0]
    assert y[0] == -3.5 and y[31] == 50.0 and (y[1:31] == 0).all()
    # src/gguf/dequant.rs:714-730
    blk = np.zeros(144, np.uint8)
    blk[:2] = f16b(1.0)
    blk[2:4] = f16b(0.5)
    blk[4], blk[8], blk[16] = 3, 2, 0x51
    y = dequant(ctx, dev, blk, Q4_K, 1, 256)[0]
    assert y[0] == 2.0 and y[1] == -1.0 and y[32] == 0.0


@pytest.mark.parametrize("ty", [Q8_0, Q4_K])
@pytest.mark.parametrize("out_dtype", [F32, F16, BF16])
def test_adversarial_blocks_bit_for_bit(ctx, dev, oracle, ty, out_dtype):
    # src/lowmem/pool.rs:1079-1195: zero blocks, subnormal scales of both signs, max f16 scale with
    # max-magnitude quants, dense LCG bytes; 8 blocks x 3 rows as in the reference's gate.
    nb, rows = 8, 3
    cols = nb * oracle.blk_elems(ty)
    src = oracle.adversarial_rows(ty, nb, rows)
    rb = oracle.row_bytes(ty, cols)
    want = np.stack([oracle.dequant_row_ref(ty, src[r * rb:(r + 1) * rb], cols) for r in range(rows)])
    assert np.abs(want).max() > 1e6 and (want == 0).mean() > 0.2  # the recipe's extremes are present
    got = dequant(ctx, dev, src, ty, rows, cols, out_dtype)
    assert np.abs(got[np.isfinite(got)]).max() > 0, "all zeros: the kernel did not run"
    if out_dtype == F32:
        synth.assert_bits_equal(got, want, "adversarial rows")
    else:
        # the exact f32 value rounded once (overflow to inf included)
        with np.errstate(over="ignore"):
            synth.assert_bits_equal(got, synth.round_to(want, out_dtype), "adversarial rows, 16-bit out")
    # the same rows gathered in scrambled order with repeats
    ids = np.array([2, 0, 1, 1, 2, 0, 0], np.uint32)
    g = gather(ctx, dev, src, ty, rows, cols, ids, F32)
    synth.assert_bits_equal(g, want[ids], "gather of adversarial rows")


def test_negative_control_scale_unpack_bug_is_seen(ctx, dev, oracle):
    # The reference plants q[j+4] for q[j] in the Q4_K min unpack and requires its gate to fail
    # (src/lowmem/pool.rs:597-599). Same here, with the bug planted in a copy of the expected values.
    nb, rows = 8, 3
    src = oracle.adversarial_rows(Q4_K, nb, rows)
    got = dequant(ctx, dev, src, Q4_K, rows, nb * 256)

    def buggy_row(row):
        out = np.empty(nb * 256, np.float32)
        for b in range(nb):
            blk = row[b * 144:(b + 1) * 144]
            d = np.float32(blk[0:2].view(np.float16)[0])
            dmin = np.float32(blk[2:4].view(np.float16)[0])
            s = blk[4:16].astype(np.uint32)
            for j in range(8):
                if j < 4:
                    sc, mn = s[j] & 63, s[j + 4] & 63
                else:
                    sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4)
                    mn = (s[j + 4] >> 4) | ((s[j + 4] >> 6) << 4)  # bug: q[j+4] where q[j] belongs
                q = blk[16 + (j // 2) * 32:16 + (j // 2) * 32 + 32]
                q = (q >> 4) if j & 1 else (q & 0xF)
                with np.errstate(over="ignore", invalid="ignore"):
                    out[b * 256 + j * 32:b * 256 + j * 32 + 32] = (d * np.float32(sc)) * q.astype(np.float32) - dmin * np.float32(mn)
        return out
    rb = nb * 144
    wrong = np.stack([buggy_row(src[r * rb:(r + 1) * rb]) for r in range(rows)])
    with pytest.raises(AssertionError):
        synth.assert_bits_equal(got, wrong, "planted bug")


@pytest.mark.parametrize("ty,dim", [(Q8_0, 896), (Q8_0, 32), (Q8_0, 2048), (Q4_K, 1024), (Q4_K, 768), (Q4_K, 256)])
@pytest.mark.parametrize("out_dtype", [F32, F16])
def test_random_tables(ctx, dev, oracle, ty, dim, out_dtype):
    vocab = 1531
    table = (synth.q8_0_table if ty == Q8_0 else synth.q4_k_table)(vocab, dim, seed=dim + ty)
    ids = np.concatenate([synth.token_ids_zipf(vocab, 3000, seed=7), [vocab - 1, 0, vocab - 1, 1, vocab - 2]]).astype(np.uint32)
    want = oracle.embed_gather(table, ty, vocab, dim, ids)
    got = gather(ctx, dev, table, ty, vocab, dim, ids, out_dtype)
    if out_dtype == F32:
        synth.assert_bits_equal(got, want, "gather")
    else:
        synth.assert_bits_equal(got, synth.round_to(want, out_dtype), "gather, f16 out")


@pytest.mark.parametrize("ty", [F32, F16, BF16])
@pytest.mark.parametrize("out_dtype", [F32, F16, BF16])
@pytest.mark.parametrize("dim", [576, 50])
def test_float_tables(ctx, dev, oracle, ty, out_dtype, dim):
    vocab = 700
    t32 = synth.round_to(synth.f32_table(vocab, dim, seed=3, std=0.02), ty)
    raw = t32 if ty == F32 else dev.bits16(dev.put(t32, ty))
    ids = synth.token_ids_uniform(vocab, 500, seed=4)
    want = oracle.embed_gather(np.ascontiguousarray(raw).view(np.uint8).reshape(-1), ty, vocab, dim, ids)
    synth.assert_bits_equal(want, t32[ids], "oracle widening is exact")
    dt = dev.put(t32, ty)
    out = dev.empty((500, dim), out_dtype, fill=0.0)
    ctx.embed_gather(dt, dev.put(ids), out, ggml_type=ty, vocab=vocab, dim=dim, n=500, out_dtype=out_dtype)
    ctx.stream_sync()
    synth.assert_bits_equal(dev.get(out), synth.round_to(want, out_dtype), "float table gather")
    if dim % 8 == 0:  # rows that start 16 bytes past a 32-byte boundary: the 16-byte stores instead of the 32-byte ones
        es = 4 if out_dtype == F32 else 2
        flat = dev.empty((500 * dim + 2 * (16 // es),), out_dtype, fill=4.0)
        shifted = flat[16 // es:16 // es + 500 * dim]
        assert shifted.data_ptr() % 32 == 16
        ctx.embed_gather(dt, dev.put(ids), shifted, ggml_type=ty, vocab=vocab, dim=dim, n=500, out_dtype=out_dtype)
        ctx.stream_sync()
        got = dev.get(flat)
        synth.assert_bits_equal(got[16 // es:-(16 // es)].reshape(500, dim), synth.round_to(want, out_dtype), "float table gather, 16-byte-aligned rows")
        assert (got[:16 // es] == 4.0).all() and (got[-(16 // es):] == 4.0).all()


def test_out_of_range_id_is_reported_and_zero_filled(ctx, dev, oracle):
    import lokal_b200 as L
    vocab, dim = 64, 128
    table = synth.q8_0_table(vocab, dim, seed=1)
    ids = np.array([3, 64, 5, 4000000000], np.uint32)
    with pytest.raises(IndexError):
        oracle.embed_gather(table, Q8_0, vocab, dim, ids)  # the reference returns Err (src/lowmem/mod.rs:662-664)
    dt, di = dev.put(table), dev.put(ids)
    out = dev.empty((4, dim), F32, fill=9.0)
    ctx.embed_gather(dt, di, out, ggml_type=Q8_0, vocab=vocab, dim=dim, n=4)
    with pytest.raises(L.LokalCudaError) as e:
        ctx.stream_sync()
    assert e.value.status == L.capi.ERR_ID_RANGE
    got = dev.get(out)
    want = oracle.embed_gather(table, Q8_0, vocab, dim, ids[[0, 2]])
    synth.assert_bits_equal(got[[0, 2]], want, "valid rows")
    assert (got[[1, 3]] == 0).all()
    ctx.stream_sync()  # the error word was cleared; the context stays usable
    for ty, tab in ((F32, np.zeros((vocab, dim), np.float32)),):
        ctx.embed_gather(dev.put(tab), di, out, ggml_type=ty, vocab=vocab, dim=dim, n=4)
        with pytest.raises(L.LokalCudaError):
            ctx.stream_sync()


def test_refusals(ctx, dev):
    import lokal_b200 as L
    t = dev.put(np.zeros(34 * 4, np.uint8))
    ids = dev.put(np.zeros(2, np.uint32))
    out = dev.empty((2, 64), F32)
    for kw, status in [
        (dict(ggml_type=3, dim=256), L.capi.ERR_UNSUPPORTED),    # Q4_1: refused by name, as the reference refuses it
        (dict(ggml_type=Q8_0, dim=48), L.capi.ERR_BAD_ARG),      # not whole blocks (src/gguf/container.rs:220-226)
        (dict(ggml_type=Q4_K, dim=896), L.capi.ERR_BAD_ARG),     # 3.5 super-blocks cannot exist
        (dict(ggml_type=Q8_0, dim=64, out_dtype=Q8_0), L.capi.ERR_UNSUPPORTED),
    ]:
        with pytest.raises(L.LokalCudaError) as e:
            ctx.embed_gather(t, ids, out, vocab=2, n=2, **kw)
        assert e.value.status == status, kw
    with pytest.raises(L.LokalCudaError):
        ctx.embed_gather(t, None, out, ggml_type=Q8_0, vocab=2, dim=64, n=2)
    ctx.embed_gather(t, ids, out, ggml_type=Q8_0, vocab=2, dim=64, n=0)


def test_full_size_zipf_gather_q8_0(ctx, dev, oracle):
    # 151936 x 896 Q8_0 table, 65536 ids from Zipf(1.1): bit-exact in f32 and f16
    vocab, dim, n = synth.C4_VOCAB, synth.C4_DIM_Q8, synth.C4_IDS
    table = synth.q8_0_table(vocab, dim, synth.C4_SEED)
    ids = synth.token_ids_zipf(vocab, n, synth.C4_SEED)
    want = oracle.embed_gather(table, Q8_0, vocab, dim, ids, threads=8)
    dt, di = dev.put(table), dev.put(ids)
    out = dev.empty((n, dim), F32, fill=1.0)
    ctx.embed_gather(dt, di, out, ggml_type=Q8_0, vocab=vocab, dim=dim, n=n)
    ctx.stream_sync()
    synth.assert_bits_equal(dev.get(out), want, "full-size Q8_0 gather")
    out16 = dev.empty((n, dim), F16, fill=1.0)
    ctx.embed_gather(dt, di, out16, ggml_type=Q8_0, vocab=vocab, dim=dim, n=n, out_dtype=F16)
    ctx.stream_sync()
    synth.assert_bits_equal(dev.get(out16), synth.round_to(want, F16), "full-size Q8_0 gather, f16 out")


def test_full_size_zipf_gather_q4_k(ctx, dev, oracle):
    # Q4_K super-blocks hold 256 elements, so the 896-wide table of the benchmark cannot exist
    # (the reference refuses it at open); the table is 151936 x 1024 instead.
    vocab, dim, n = synth.C4_VOCAB, synth.C4_DIM_Q4K, synth.C4_IDS
    table = synth.q4_k_table(vocab, dim, synth.C4_SEED + 1)
    ids = synth.token_ids_zipf(vocab, n, synth.C4_SEED + 1)
    want = oracle.embed_gather(table, Q4_K, vocab, dim, ids, threads=8)
    dt, di = dev.put(table), dev.put(ids)
    out = dev.empty((n, dim), F32, fill=1.0)
    ctx.embed_gather(dt, di, out, ggml_type=Q4_K, vocab=vocab, dim=dim, n=n)
    ctx.stream_sync()
    synth.assert_bits_equal(dev.get(out), want, "full-size Q4_K gather")


@pytest.mark.parametrize("ty", [Q8_0, 2, 6])  # Q8_0, Q4_0, Q5_0: value = (integer) * (f16 scale), one exact product
def test_f16_rows_of_single_product_types_over_every_scale_and_quant(ctx, dev, oracle, ty):
    """f16 rows of Q8_0 / Q4_0 / Q5_0 tables are computed in half precision on the device, on the strength of an
    exactness argument: integer (at most 8 bits) times f16 scale is exact in f32, so rounding it to f16 and multiplying
    in f16 give the same bits. Checked here over EVERY f16 scale pattern (all 65,536, infinities and NaNs included) times
    every quant value the block type can hold, against the f32 formula rounded once (numpy), and against the oracle."""
    be, bb, _ = synth.QUANT_GEOMETRY[ty]
    nq = 256 if ty == Q8_0 else (16 if ty == 2 else 32)
    n_scales, per_row = 65536, 256 // 32  # 8 blocks per row: 256 elements
    scales = np.arange(n_scales, dtype=np.uint16)
    blocks = np.zeros((n_scales, per_row, bb), np.uint8)
    blocks[:, :, 0:2] = scales.view(np.uint8).reshape(n_scales, 1, 2)
    elem = np.arange(256).reshape(per_row, 32)  # element index -> which quant value it carries
    if ty == Q8_0:
        blocks[:, :, 2:] = elem.astype(np.uint8)[None]                     # all 256 int8 patterns
        qv = elem.astype(np.uint8).view(np.int8).astype(np.float32)
    else:
        vals = (elem % nq).astype(np.uint8)                                 # 0..15 or 0..31, every value many times
        qs = 2 if ty == 2 else 6
        lo, hi = vals[:, :16], vals[:, 16:]
        blocks[:, :, qs:qs + 16] = ((lo & 15) | ((hi & 15) << 4))[None]
        if ty == 6:
            bits = ((vals >> 4) & 1).astype(np.uint32)
            qh = (bits << np.arange(32, dtype=np.uint32)[None, :]).sum(axis=1).astype(np.uint32)
            blocks[:, :, 2:6] = qh.view(np.uint8).reshape(per_row, 4)[None]
        qv = vals.astype(np.float32) - (8 if ty == 2 else 16)
    table = blocks.reshape(-1)
    got = dequant(ctx, dev, table, ty, n_scales, 256, F16)          # f32 view of the f16 rows
    d = scales.view(np.float16).astype(np.float32)
    with np.errstate(all="ignore"):
        want = (qv.reshape(1, 256) * d.reshape(-1, 1)).astype(np.float16)   # exact f32 product, one rounding
    got16 = got.astype(np.float16)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got16), nan)
    assert np.array_equal(got16.view(np.uint16)[~nan], want.view(np.uint16)[~nan])
    assert nan.sum() > 0 and np.isinf(want).sum() > 0 and (want.view(np.uint16)[~nan] & 0x7C00 == 0).sum() > 1000  # NaN, inf, subnormals all occur
    # and the oracle agrees on a slice (finite scales)
    rows = slice(0x3000, 0x3040)
    ref = synth.round_to(oracle.embed_gather(table[rows.start * per_row * bb:rows.stop * per_row * bb], ty, 64, 256, np.arange(64, dtype=np.uint32)), F16)
    synth.assert_bits_equal(got[rows], ref, "oracle slice")


@pytest.mark.parametrize("ty,dim", [(Q8_0, 896), (Q8_0, 2048), (Q4_K, 1024), (Q4_K, 2304), (14, 512), (21, 768), (20, 64)])
@pytest.mark.parametrize("out_dtype", [F32, F16, BF16])
def test_gather_fused_with_the_first_norm(ctx, dev, oracle, ty, dim, out_dtype, monkeypatch):
    """lokal_cuda_embed_gather_rmsnorm: x is bit for bit the gather's, xn is the RMSNorm of x as stored (rounded to the row
    type), within the norm's bar against the oracle, and equal to what gather + rmsnorm give as two launches to the last
    bits of the scale; an out-of-range id gives zero rows in both outputs and the error code."""
    import lokal_b200 as L
    if ty in L.capi.GRID_TYPES:
        from test_oracle_iq_grids import GRIDS
        ctx.set_iq_grids(GRIDS)
        oracle.set_iq_grids(GRIDS)
    vocab, n, eps = 300, 700, 1e-6
    table = synth.quant_table(ty, vocab, dim, 31) if ty not in (Q8_0, Q4_K) else (synth.q8_0_table if ty == Q8_0 else synth.q4_k_table)(vocab, dim, 31)
    ids = synth.token_ids_uniform(vocab, n, 32)
    ids[5] = vocab + 7  # out of range
    w = synth.round_to(1 + 0.1 * np.random.default_rng(33).standard_normal(dim, dtype=np.float32), out_dtype)
    dt, di, dw = dev.put(table), dev.put(ids.view(np.int32)), dev.put(w, out_dtype)
    x, xn = dev.empty((n, dim), out_dtype, fill=5.0), dev.empty((n, dim), out_dtype, fill=5.0)
    ctx.embed_gather_rmsnorm(dt, di, x, xn, dw, ggml_type=ty, vocab=vocab, dim=dim, n=n, eps=eps, out_dtype=out_dtype, w_dtype=out_dtype)
    with pytest.raises(L.LokalCudaError) as e:
        ctx.stream_sync()
    assert e.value.status == L.capi.ERR_ID_RANGE
    good = np.ones(n, bool)
    good[5] = False
    want_x = synth.round_to(oracle.embed_gather(table, ty, vocab, dim, np.where(good, ids, 0).astype(np.uint32)), out_dtype)
    want_x[5] = 0.0
    got_x, got_xn = dev.get(x), dev.get(xn)
    synth.assert_bits_equal(got_x, want_x, "x of the fused call")
    assert (got_xn[5] == 0.0).all()
    _, ref_xn = oracle.add_rmsnorm_rows(want_x, None, w, eps)  # norm of the rows AS STORED
    if out_dtype == F32:
        # quantised rows can be large (scales |N(0, 0.01)| times quants up to 127): compare relative to the row's magnitude
        tol = 1e-5 * np.maximum(1.0, np.abs(ref_xn).max())
        assert np.abs(got_xn - ref_xn).max() <= tol
    else:
        synth.check_half(got_xn[good], ref_xn[good], "xn of the fused call", out_dtype, atol=1e-6)
    # the two-launch form (LOKAL_CUDA_GATHER_FUSE_NORM=0 keeps the norm in its own launch)
    x2, xn2 = dev.empty((n, dim), out_dtype, fill=5.0), dev.empty((n, dim), out_dtype, fill=5.0)
    monkeypatch.setenv("LOKAL_CUDA_GATHER_FUSE_NORM", "0")
    ctx.embed_gather_rmsnorm(dt, di, x2, xn2, dw, ggml_type=ty, vocab=vocab, dim=dim, n=n, eps=eps, out_dtype=out_dtype, w_dtype=out_dtype)
    monkeypatch.delenv("LOKAL_CUDA_GATHER_FUSE_NORM")
    with pytest.raises(L.LokalCudaError):
        ctx.stream_sync()
    synth.assert_bits_equal(dev.get(x2), got_x, "x, two launches")
    two = dev.get(xn2)
    rel = np.abs(two - got_xn) / np.maximum(np.abs(two), 1e-20)
    assert rel.max() <= (2e-6 if out_dtype == F32 else 2.0 ** -7), "fused and two-launch norms differ by more than the last bits of the scale"


def test_gather_rmsnorm_on_float_tables_and_refusals(ctx, dev, oracle):
    import lokal_b200 as L
    vocab, dim, n = 50, 96, 33
    table = synth.f32_table(vocab, dim, 3)
    ids = synth.token_ids_uniform(vocab, n, 4)
    w = (1 + 0.1 * np.random.default_rng(5).standard_normal(dim, dtype=np.float32)).astype(np.float32)
    dt, di, dw = dev.put(table), dev.put(ids.view(np.int32)), dev.put(w)
    x, xn = dev.empty((n, dim), F32, fill=5.0), dev.empty((n, dim), F32, fill=5.0)
    ctx.embed_gather_rmsnorm(dt, di, x, xn, dw, ggml_type=F32, vocab=vocab, dim=dim, n=n, eps=1e-5)
    ctx.stream_sync()
    synth.assert_bits_equal(dev.get(x), table[ids], "dense rows")
    _, ref = oracle.add_rmsnorm_rows(table[ids], None, w, 1e-5)
    synth.check_f32(dev.get(xn), ref, "norm of dense rows")
    for kw in (dict(w=None), dict(xn=None)):
        args = dict(table=dt, ids=di, x=x, xn=xn, w=dw)
        args.update(kw)
        with pytest.raises(L.LokalCudaError) as e:
            ctx.embed_gather_rmsnorm(args["table"], args["ids"], args["x"], args["xn"], args["w"], ggml_type=F32, vocab=vocab, dim=dim, n=n, eps=1e-5)
        assert e.value.status == L.capi.ERR_BAD_ARG


@pytest.mark.parametrize("ty,dim", [(Q8_0, 896), (Q4_K, 1024)])
@pytest.mark.parametrize("chunk", [1000, 1001])
def test_a_call_split_into_several_launches(ctx, dev, oracle, ty, dim, chunk, monkeypatch):
    """The staged kernel counts rows in 32 bits, so a call of more than 2^30 rows goes out as several launches over
    consecutive slices. The test lowers the slice to 1000 / 1001 rows (1001 moves the table pointer of the id-less form
    off the 16-byte grid, which sends those slices through the plain-load staging) and compares with one launch."""
    vocab = 2300
    table = (synth.q8_0_table if ty == Q8_0 else synth.q4_k_table)(vocab, dim, seed=11)
    ids = np.concatenate([synth.token_ids_zipf(vocab, 3300, seed=5), [vocab - 1, 0, vocab - 1]]).astype(np.uint32)
    want = oracle.embed_gather(table, ty, vocab, dim, ids)
    whole = oracle.embed_gather(table, ty, vocab, dim, np.arange(vocab, dtype=np.uint32))
    monkeypatch.setenv("LOKAL_CUDA_GATHER_CHUNK_ROWS", str(chunk))
    for out_dtype in (F32, F16):
        synth.assert_bits_equal(gather(ctx, dev, table, ty, vocab, dim, ids, out_dtype), synth.round_to(want, out_dtype), "sliced gather")
        synth.assert_bits_equal(dequant(ctx, dev, table, ty, vocab, dim, out_dtype), synth.round_to(whole, out_dtype), "sliced dequant of the whole table")


@pytest.mark.parametrize("ty,dim", [(Q8_0, 896), (Q8_0, 32), (Q4_K, 1024), (Q4_K, 512), (Q4_K, 1280), (13, 768), (14, 256), (20, 64), (21, 512), (19, 256),
                                    (2, 64), (6, 96), (10, 256), (11, 512), (16, 256), (17, 256), (18, 512), (22, 256), (23, 512), (29, 256)])
@pytest.mark.parametrize("out_dtype", [F16, BF16])
def test_two_rows_per_warp_against_one(ctx, dev, oracle, ty, dim, out_dtype, monkeypatch):
    """16-bit rows are decoded two to a warp. Odd and tiny row counts, the table's last row (whose window may need the
    plain-load staging) in either half, ids out of range in either half: bit for bit the oracle's rows, and the same
    bytes as the one-row-per-warp kernel."""
    import lokal_b200 as L
    if ty in L.capi.GRID_TYPES:
        from test_oracle_iq_grids import GRIDS
        ctx.set_iq_grids(GRIDS)
        oracle.set_iq_grids(GRIDS)
    vocab = 301
    table = synth.quant_table(ty, vocab, dim, seed=ty + dim)
    for n in (1, 2, 3, 777):
        ids = synth.token_ids_uniform(vocab, n, seed=n).astype(np.uint32)
        ids[-1] = vocab - 1
        if n > 2:
            ids[0] = vocab - 1
            ids[n // 2] = vocab - 1
        want = synth.round_to(oracle.embed_gather(table, ty, vocab, dim, ids), out_dtype)
        got = gather(ctx, dev, table, ty, vocab, dim, ids, out_dtype)
        synth.assert_bits_equal(got, want, f"two rows per warp, n={n}")
        monkeypatch.setenv("LOKAL_CUDA_GATHER_PAIR", "0")
        synth.assert_bits_equal(gather(ctx, dev, table, ty, vocab, dim, ids, out_dtype), got, f"one row per warp, n={n}")
        monkeypatch.delenv("LOKAL_CUDA_GATHER_PAIR")
    # out-of-range ids in the low half, the high half and both halves of a pair
    ids = synth.token_ids_uniform(vocab, 41, seed=9).astype(np.uint32)
    bad = [4, 9, 20, 21, 40]
    ids[bad] = [vocab, 4000000000, vocab + 5, vocab, vocab]
    good = [i for i in range(41) if i not in bad]
    dt, di = dev.put(table), dev.put(ids)
    out = dev.empty((42, dim), out_dtype, fill=4.0)
    ctx.embed_gather(dt, di, out, ggml_type=ty, vocab=vocab, dim=dim, n=41, out_dtype=out_dtype)
    with pytest.raises(L.LokalCudaError) as e:
        ctx.stream_sync()
    assert e.value.status == L.capi.ERR_ID_RANGE
    got = dev.get(out)
    synth.assert_bits_equal(got[good], synth.round_to(oracle.embed_gather(table, ty, vocab, dim, ids[good]), out_dtype), "valid rows")
    assert (got[bad] == 0).all() and (got[41] == 4.0).all()


@pytest.mark.parametrize("ty,dim", [(Q8_0, 896), (Q4_K, 1024), (21, 512)])
def test_l2_priority_of_table_rows_changes_no_bit(ctx, dev, oracle, ty, dim, monkeypatch):
    """Table rows are fetched with the high L2 eviction priority; LOKAL_CUDA_GATHER_TABLE_KEEP=0 turns it off. A cache
    hint may not change a result."""
    import lokal_b200 as L
    if ty in L.capi.GRID_TYPES:
        from test_oracle_iq_grids import GRIDS
        ctx.set_iq_grids(GRIDS)
    vocab = 1777
    table = synth.quant_table(ty, vocab, dim, seed=3)
    ids = synth.token_ids_zipf(vocab, 5001, seed=4).astype(np.uint32)
    for out_dtype in (F32, F16):
        on = gather(ctx, dev, table, ty, vocab, dim, ids, out_dtype)
        monkeypatch.setenv("LOKAL_CUDA_GATHER_TABLE_KEEP", "0")
        off = gather(ctx, dev, table, ty, vocab, dim, ids, out_dtype)
        monkeypatch.delenv("LOKAL_CUDA_GATHER_TABLE_KEEP")
        synth.assert_bits_equal(on, off, "gather with and without the L2 priority of the table rows")
