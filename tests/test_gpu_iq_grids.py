"""The codebook block types (IQ1_S, IQ1_M, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S) on the GPU, bit for bit against the
CPU oracle: refused until the caller has handed the codebooks over, then the reference's adversarial recipe
(src/lowmem/pool.rs:1079-1195; its gate is GPU == CPU bit for bit) and random tables through both kernels."""
import numpy as np
import pytest

import gguf_np
import lokal_b200 as L
import synth
from synth import BF16, F16, F32
from test_oracle_iq_grids import GRIDS, iq_random_blocks

pytestmark = pytest.mark.gpu
TYPES = sorted(gguf_np.GRID_DECODERS)


@pytest.fixture(scope="module")
def grid_ctx(oracle):
    """A context of its own: the session-wide one must stay without codebooks for the refusal test."""
    oracle.set_iq_grids(GRIDS)
    c = L.Context(0)
    c.set_iq_grids(GRIDS)
    yield c
    c.close()


def test_refused_until_the_codebook_is_handed_over(dev):
    fresh = L.Context(0)
    t = dev.put(np.zeros(66 * 4, np.uint8))
    out = dev.empty((1, 1024), F32)
    with pytest.raises(L.LokalCudaError) as e:
        fresh.dequant_rows(t, out, ggml_type=L.capi.IQ2_XXS, rows=1, cols=1024)
    assert e.value.status == L.capi.ERR_UNSUPPORTED and "iq2xxs codebook" in e.value.message and "lokal_cuda_set_iq_grid" in e.value.message
    with pytest.raises(L.LokalCudaError) as e:
        fresh.set_iq_grids({"iq2xxs": GRIDS["iq2xs"]})  # 512 entries where 256 belong
    assert e.value.status == L.capi.ERR_BAD_ARG
    fresh.set_iq_grids({"iq2xxs": GRIDS["iq2xxs"]})
    fresh.dequant_rows(t, out, ggml_type=L.capi.IQ2_XXS, rows=1, cols=1024)
    fresh.stream_sync()
    assert (dev.get(out) == 0).all()
    with pytest.raises(L.LokalCudaError):  # the other codebooks are still missing
        fresh.dequant_rows(t, out, ggml_type=L.capi.IQ3_S, rows=1, cols=256)


@pytest.mark.parametrize("ty", TYPES)
@pytest.mark.parametrize("out_dtype", [F32, F16, BF16])
def test_adversarial_rows(grid_ctx, dev, oracle, ty, out_dtype):
    nb, rows = 8, 3
    cols = nb * 256
    src = oracle.adversarial_rows(ty, nb, rows)
    rb = oracle.row_bytes(ty, cols)
    want = np.stack([oracle.dequant_row_ref(ty, src[r * rb:(r + 1) * rb], cols) for r in range(rows)])
    out = dev.empty((rows + 1, cols), out_dtype, fill=4.0)
    grid_ctx.dequant_rows(dev.put(src), out, ggml_type=ty, rows=rows, cols=cols, out_dtype=out_dtype)
    grid_ctx.stream_sync()
    got = dev.get(out)
    assert (got[-1] == 4.0).all() and np.abs(got[:-1][np.isfinite(got[:-1])]).max() > 0
    with np.errstate(over="ignore"):
        synth.assert_bits_equal(got[:-1], synth.round_to(want, out_dtype), f"{gguf_np.GRID_NAMES[ty]} adversarial rows")


@pytest.mark.parametrize("ty", TYPES)
def test_random_tables_both_kernels(grid_ctx, dev, oracle, ty):
    vocab, dim = 211, 768
    bb = gguf_np.GRID_BLOCK_BYTES[ty]
    table = iq_random_blocks(ty, vocab * dim // 256, seed=50 + ty)
    ids = np.concatenate([synth.token_ids_zipf(vocab, 900, seed=3), [vocab - 1, 0, vocab - 1]]).astype(np.uint32)
    want = oracle.embed_gather(table, ty, vocab, dim, ids)
    assert len(np.unique(want)) > 100
    synth.assert_bits_equal(want, gguf_np.GRID_DECODERS[ty](table, GRIDS).reshape(vocab, dim)[ids], "oracle vs numpy")
    di = dev.put(ids)
    for out_dtype in (F32, F16):
        out = dev.empty((len(ids) + 1, dim), out_dtype, fill=4.0)
        grid_ctx.embed_gather(dev.put(table), di, out, ggml_type=ty, vocab=vocab, dim=dim, n=len(ids), out_dtype=out_dtype)
        grid_ctx.stream_sync()
        res = dev.get(out)
        assert (res[-1] == 4.0).all()
        synth.assert_bits_equal(res[:-1], synth.round_to(want, out_dtype), f"{gguf_np.GRID_NAMES[ty]} staged gather")
    # a table 2 bytes past a 16-byte boundary takes the per-element kernel
    shifted = dev.put(np.concatenate([np.zeros(2, np.uint8), table]))[2:]
    out = dev.empty((len(ids), dim), F32, fill=4.0)
    grid_ctx.embed_gather(shifted, di, out, ggml_type=ty, vocab=vocab, dim=dim, n=len(ids))
    grid_ctx.stream_sync()
    synth.assert_bits_equal(dev.get(out), want, f"{gguf_np.GRID_NAMES[ty]} per-element gather")
    # f32 rows that start 16 bytes past a 32-byte boundary: two 16-byte stores per lane instead of one of 32 bytes
    flat = dev.empty((len(ids) * dim + 8,), F32, fill=4.0)
    out16 = flat[4:4 + len(ids) * dim]
    assert out16.data_ptr() % 32 == 16
    grid_ctx.embed_gather(dev.put(table), di, out16, ggml_type=ty, vocab=vocab, dim=dim, n=len(ids))
    grid_ctx.stream_sync()
    got = dev.get(flat)
    synth.assert_bits_equal(got[4:-4].reshape(len(ids), dim), want, f"{gguf_np.GRID_NAMES[ty]} staged gather, 16-byte-aligned rows")
    assert (got[:4] == 4.0).all() and (got[-4:] == 4.0).all()
    assert bb * (dim // 256) == oracle.row_bytes(ty, dim)
