"""Every GGUF block type of the gather / row-dequant path on the GPU, bit for bit against the CPU oracle:
the reference's hand vectors, its adversarial block recipe, random tables through both kernels (staged rows and
the per-element kernel that takes any alignment), f32 and 16-bit outputs."""
import numpy as np
import pytest

import gguf_np
import synth
from synth import BF16, F16, F32

pytestmark = pytest.mark.gpu

TYPES = sorted(gguf_np.DECODERS)


def f16b(v):
    return np.array([v], np.float16).view(np.uint8)


def dequant(ctx, dev, src, ty, rows, cols, out_dtype=F32):
    out = dev.empty((rows + 1, cols), out_dtype, fill=4.0)
    ctx.dequant_rows(dev.put(src), out, ggml_type=ty, rows=rows, cols=cols, out_dtype=out_dtype)
    ctx.stream_sync()
    res = dev.get(out)
    assert (res[-1] == 4.0).all(), "wrote past the last row"
    return res[:-1]


def test_reference_hand_vectors_on_the_gpu(ctx, dev):
    # the six vectors of src/gguf/dequant.rs:579-766
    blk = np.full(18, 0x88, np.uint8)
    blk[:2], blk[2] = f16b(2.0), 0xA3
    y = dequant(ctx, dev, blk, 2, 1, 32)[0]
    assert y[0] == -10.0 and y[16] == 4.0 and (np.delete(y, [0, 16]) == 0).all()
    blk = np.zeros(84, np.uint8)
    blk[0], blk[16] = 0x21, 3
    blk[80:82], blk[82:84] = f16b(0.5), f16b(0.25)
    y = dequant(ctx, dev, blk, 10, 1, 256)[0]
    assert y[0] == 1.0 and y[1] == -0.5 and y[16] == 0.0
    blk = np.zeros(110, np.uint8)
    blk[0], blk[32] = 1, 1
    blk[108:110] = f16b(0.5)
    y = dequant(ctx, dev, blk, 11, 1, 256)[0]
    assert y[0] == -16.0 and y[1] == 64.0 and y[128] == 64.0
    blk = np.zeros(22, np.uint8)
    blk[:2] = f16b(0.5)
    blk[2], blk[4], blk[6] = 0x01, 0x01, 0x21
    y = dequant(ctx, dev, blk, 6, 1, 32)[0]
    assert y[0] == 0.5 and y[16] == 1.0 and y[1] == -8.0 and y[31] == -8.0
    blk = np.zeros(176, np.uint8)
    blk[:2], blk[2:4] = f16b(1.0), f16b(0.5)
    blk[4], blk[8], blk[16], blk[48] = 3, 2, 0x01, 0x01
    y = dequant(ctx, dev, blk, 13, 1, 256)[0]
    assert y[0] == 50.0 and y[1] == -1.0
    blk = np.zeros(210, np.uint8)
    blk[0], blk[192], blk[196] = 0x21, 2, 1
    blk[208:210] = f16b(0.25)
    y = dequant(ctx, dev, blk, 14, 1, 256)[0]
    assert y[0] == -15.5 and y[64] == -7.5 and y[32] == 0.0


@pytest.mark.parametrize("ty", TYPES)
@pytest.mark.parametrize("out_dtype", [F32, F16, BF16])
def test_adversarial_rows_every_type(ctx, dev, oracle, ty, out_dtype):
    # src/lowmem/pool.rs:1079-1195, generalised to each block layout's scale fields
    nb, rows = 8, 3
    cols = nb * oracle.blk_elems(ty)
    src = oracle.adversarial_rows(ty, nb, rows)
    rb = oracle.row_bytes(ty, cols)
    want = np.stack([oracle.dequant_row_ref(ty, src[r * rb:(r + 1) * rb], cols) for r in range(rows)])
    got = dequant(ctx, dev, src, ty, rows, cols, out_dtype)
    assert np.abs(got[np.isfinite(got)]).max() > 0, "all zeros: the kernel did not run"
    with np.errstate(over="ignore"):
        synth.assert_bits_equal(got, synth.round_to(want, out_dtype), f"{gguf_np.NAMES[ty]} adversarial rows")


@pytest.mark.parametrize("ty", TYPES)
@pytest.mark.parametrize("blocks_per_row", [1, 3, 8])
def test_random_tables_every_type(ctx, dev, oracle, ty, blocks_per_row):
    be, bb = oracle.blk_elems(ty), oracle.blk_bytes(ty)
    if be == 32:
        blocks_per_row *= 7  # 224 / 672 / 1792 columns
    vocab, dim = 517, be * blocks_per_row
    table = gguf_np.random_blocks(ty, vocab * blocks_per_row, seed=ty + dim, blk_bytes=bb, scale_offsets=gguf_np.SCALE_OFFSETS[ty])
    ids = np.concatenate([synth.token_ids_zipf(vocab, 1500, seed=9), [vocab - 1, 0, vocab - 1, 1, vocab - 2]]).astype(np.uint32)
    want = oracle.embed_gather(table, ty, vocab, dim, ids)
    assert len(np.unique(want)) > 100
    dt, di = dev.put(table), dev.put(ids)
    for out_dtype in (F32, F16):
        out = dev.empty((len(ids) + 1, dim), out_dtype, fill=4.0)
        ctx.embed_gather(dt, di, out, ggml_type=ty, vocab=vocab, dim=dim, n=len(ids), out_dtype=out_dtype)
        ctx.stream_sync()
        res = dev.get(out)
        assert (res[-1] == 4.0).all()
        synth.assert_bits_equal(res[:-1], synth.round_to(want, out_dtype), f"{gguf_np.NAMES[ty]} gather")


@pytest.mark.parametrize("ty", TYPES)
def test_table_at_an_odd_address_takes_the_per_element_kernel(ctx, dev, oracle, ty):
    # a table that starts 2 bytes past a 16-byte boundary (a tensor inside a file image) cannot be bulk-copied
    be, bb = oracle.blk_elems(ty), oracle.blk_bytes(ty)
    vocab, dim = 64, be * 2
    table = gguf_np.random_blocks(ty, vocab * 2, seed=100 + ty, blk_bytes=bb, scale_offsets=gguf_np.SCALE_OFFSETS[ty])
    ids = synth.token_ids_uniform(vocab, 200, seed=ty)
    want = oracle.embed_gather(table, ty, vocab, dim, ids)
    shifted = dev.put(np.concatenate([np.zeros(2, np.uint8), table]))[2:]
    assert shifted.data_ptr() % 16 == 2
    out = dev.empty((200, dim), F32, fill=4.0)
    ctx.embed_gather(shifted, dev.put(ids), out, ggml_type=ty, vocab=vocab, dim=dim, n=200)
    ctx.stream_sync()
    synth.assert_bits_equal(dev.get(out), want, f"{gguf_np.NAMES[ty]} per-element kernel")


def test_host_mirror_decodes_every_type(ctx, oracle):
    # dequant_row_ref's calling convention (src/gguf/dequant.rs:191): host bytes in, host f32 out
    for ty in TYPES:
        be, bb = oracle.blk_elems(ty), oracle.blk_bytes(ty)
        raw = gguf_np.random_blocks(ty, 4, seed=ty, blk_bytes=bb, scale_offsets=gguf_np.SCALE_OFFSETS[ty])
        got = ctx.host_dequant_row(ty, raw, 4 * be)
        synth.assert_bits_equal(got, oracle.dequant_row_ref(ty, raw, 4 * be), gguf_np.NAMES[ty])
