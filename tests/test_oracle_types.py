"""The wider set of GGUF block types (Q4_0, Q5_0, Q2_K, Q3_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS next to Q8_0 and Q4_K):
the C++ oracle against the reference's hand vectors and against an independent numpy reading of the layouts. No GPU."""
import numpy as np
import pytest

import gguf_np
import synth

TYPES = sorted(gguf_np.DECODERS)


def f16b(v):
    return np.array([v], np.float16).view(np.uint8)


def test_block_sizes_match_ggml_structs(oracle):
    # src/gguf/dequant.rs:567-577 (static_asserts of ggml-common.h) and :94-114
    want = {2: (32, 18), 6: (32, 22), 8: (32, 34), 10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176),
            14: (256, 210), 20: (32, 18), 23: (256, 136)}
    for ty, (elems, size) in want.items():
        assert (oracle.blk_elems(ty), oracle.blk_bytes(ty)) == (elems, size), gguf_np.NAMES[ty]
    assert oracle.row_bytes(14, 1024) == 840 and oracle.row_bytes(6, 896) == 616


def test_reference_hand_vectors(oracle):
    # Q4_0, src/gguf/dequant.rs:579-595
    blk = np.full(18, 0x88, np.uint8)
    blk[:2] = f16b(2.0)
    blk[2] = 0xA3
    y = oracle.dequant_row_ref(2, blk, 32)
    assert y[0] == -10.0 and y[16] == 4.0 and (np.delete(y, [0, 16]) == 0).all()
    # Q2_K, :597-616
    blk = np.zeros(84, np.uint8)
    blk[0], blk[16] = 0x21, 3
    blk[80:82], blk[82:84] = f16b(0.5), f16b(0.25)
    y = oracle.dequant_row_ref(10, blk, 256)
    assert y[0] == 1.0 and y[1] == -0.5 and y[16] == 0.0
    # Q3_K, :618-636: all scales zero -> dl = 0.5 * (0 - 32) = -16; a CLEAR hmask bit subtracts 4
    blk = np.zeros(110, np.uint8)
    blk[0], blk[32] = 1, 1
    blk[108:110] = f16b(0.5)
    y = oracle.dequant_row_ref(11, blk, 256)
    assert y[0] == -16.0 and y[1] == 64.0 and y[128] == 64.0
    # Q5_0, :668-683
    blk = np.zeros(22, np.uint8)
    blk[:2] = f16b(0.5)
    blk[2], blk[4], blk[6] = 0x01, 0x01, 0x21
    y = oracle.dequant_row_ref(6, blk, 32)
    assert y[0] == 0.5 and y[16] == 1.0 and y[1] == -8.0 and y[31] == -8.0
    # Q5_K, :732-748
    blk = np.zeros(176, np.uint8)
    blk[:2], blk[2:4] = f16b(1.0), f16b(0.5)
    blk[4], blk[8], blk[16], blk[48] = 3, 2, 0x01, 0x01
    y = oracle.dequant_row_ref(13, blk, 256)
    assert y[0] == 50.0 and y[1] == -1.0
    # Q6_K, :750-766
    blk = np.zeros(210, np.uint8)
    blk[0], blk[192], blk[196] = 0x21, 2, 1
    blk[208:210] = f16b(0.25)
    y = oracle.dequant_row_ref(14, blk, 256)
    assert y[0] == -15.5 and y[64] == -7.5 and y[32] == 0.0


def test_q3k_scale_unpack_on_the_reference_pattern(oracle):
    # src/gguf/dequant.rs:641-666: scale bytes i*17, every lane different; with d = 1 and quants/hmask chosen so
    # that each element equals its scale: q = 1, hmask bit set -> value = scale - 32
    p = (np.arange(12) * 17 % 256).astype(np.uint8)
    blk = np.zeros(110, np.uint8)
    blk[:32] = 0xFF            # hmask set everywhere: nothing subtracted
    blk[32:96] = 0x55          # every 2-bit quant = 1
    blk[96:108] = p
    blk[108:110] = f16b(1.0)
    y = oracle.dequant_row_ref(11, blk, 256)
    w = lambda i: int.from_bytes(bytes(p[4 * i:4 * i + 4]), "little")
    k1, k2, a0, a1, t = 0x03030303, 0x0f0f0f0f, w(0), w(1), w(2)
    aux = [(a0 & k2) | (((t >> 0) & k1) << 4), (a1 & k2) | (((t >> 2) & k1) << 4),
           ((a0 >> 4) & k2) | (((t >> 4) & k1) << 4), ((a1 >> 4) & k2) | (((t >> 6) & k1) << 4)]
    scales = [(a >> (8 * k)) & 0xFF for a in aux for k in range(4)]
    assert all(s < 64 for s in scales)
    for nh in range(2):
        for j in range(4):
            for half in range(2):
                want = float(scales[nh * 8 + j * 2 + half] - 32)
                seg = y[nh * 128 + j * 32 + half * 16:][:16]
                assert (seg == want).all()


@pytest.mark.parametrize("ty", TYPES)
def test_adversarial_rows_oracle_equals_numpy(oracle, ty):
    # src/lowmem/pool.rs:1079-1195: the recipe, and the two independent decoders must agree bit for bit on it
    nb, rows = 8, 3
    adv = oracle.adversarial_rows(ty, nb, rows)
    bb, be = oracle.blk_bytes(ty), oracle.blk_elems(ty)
    blocks = adv.reshape(rows * nb, bb)
    d_off = {10: 80, 11: 108, 14: 208}.get(ty, 0)
    scale_bytes = [[0, 0], [1, 0], [255, 131], [255, 123]]
    for i, blk in enumerate(blocks):
        v = i % 4
        if v == 0:
            assert not blk.any()
        else:
            assert list(blk[d_off:d_off + 2]) == scale_bytes[v]
    cols = nb * be
    rb = oracle.row_bytes(ty, cols)
    seq = np.stack([oracle.dequant_row_ref(ty, adv[r * rb:(r + 1) * rb], cols) for r in range(rows)])
    with np.errstate(over="ignore", invalid="ignore"):
        ind = gguf_np.DECODERS[ty](adv).reshape(rows, cols)
    assert np.isfinite(seq).all() and np.abs(seq).max() > 1e5
    synth.assert_bits_equal(seq, ind, f"{gguf_np.NAMES[ty]}: C++ oracle vs numpy on the adversarial rows")


@pytest.mark.parametrize("ty", TYPES)
def test_random_blocks_oracle_equals_numpy(oracle, ty):
    bb, be = oracle.blk_bytes(ty), oracle.blk_elems(ty)
    nblk = 64
    raw = gguf_np.random_blocks(ty, nblk, seed=ty, blk_bytes=bb, scale_offsets=gguf_np.SCALE_OFFSETS[ty])
    seq = oracle.dequant_row_ref(ty, raw, nblk * be)
    ind = gguf_np.DECODERS[ty](raw)
    assert len(np.unique(seq)) > 50
    synth.assert_bits_equal(seq, ind, f"{gguf_np.NAMES[ty]}: C++ oracle vs numpy on random blocks")
    # gather of rows == decode of the same rows
    cols = 4 * be
    rb = oracle.row_bytes(ty, cols)
    ids = np.array([15, 0, 7, 7], np.uint32)
    g = oracle.embed_gather(raw, ty, 16, cols, ids, threads=2)
    synth.assert_bits_equal(g, seq.reshape(16, cols)[ids], "gather")
    with pytest.raises(ValueError):
        oracle.dequant_row_ref(ty, raw[:rb - 1], cols)


def test_types_outside_the_path_are_refused(oracle):
    for ty in (3, 7, 9, 15, 24, 28):  # Q4_1, Q5_1, Q8_1, Q8_K, I8, F64
        assert oracle.blk_elems(ty) == 0
        with pytest.raises(ValueError):
            oracle.dequant_row_ref(ty, np.zeros(64, np.uint8), 32)
