"""The codebook block types (IQ1_S, IQ1_M, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S) on the CPU: the committed
codebook fixture against the reference's own checksums, and the C++ oracle against an independent numpy reading of
the block layouts. The reference holds no hand vector for these types (its gate is GPU == CPU on the adversarial
recipe, src/lowmem/pool.rs:1079-1195), so two independent decoders agreeing is the pin. No GPU."""
import os

import numpy as np
import pytest

import gguf_np
import synth

GRIDS = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "iq_grids.npz"))
TYPES = sorted(gguf_np.GRID_DECODERS)


@pytest.fixture(scope="module")
def grid_oracle(oracle):
    oracle.set_iq_grids(GRIDS)
    return oracle


def iq_random_blocks(ty, n_blocks, seed):
    """Uniform random bytes with a finite, moderate f16 super-block scale (IQ1_M keeps it in four nibbles)."""
    rng = np.random.default_rng(seed)
    bb = gguf_np.GRID_BLOCK_BYTES[ty]
    b = rng.integers(0, 256, (n_blocks, bb), dtype=np.uint8)
    d = (np.abs(rng.standard_normal(n_blocks)) * 0.02 + 0.001).astype(np.float16).view(np.uint16)
    if ty == 29:
        for k in range(4):
            b[:, 49 + 2 * k] = (b[:, 49 + 2 * k] & 0x0F) | (((d >> (4 * k)) & 0x0F) << 4).astype(np.uint8)
    else:
        b[:, 0], b[:, 1] = (d & 0xFF).astype(np.uint8), (d >> 8).astype(np.uint8)
    return b.reshape(-1)


def test_codebook_fixture_matches_the_reference_checksums():
    # src/lowmem/iq_grids.rs:584-603: lengths and wrapping sums of the revision the tables were emitted from
    want = {"ksigns": (128, 16320), "iq2xxs": (256, 10026840302681211747), "iq2xs": (512, 3032300602630837921),
            "iq2s": (1024, 8502338067238609906), "iq3xxs": (256, 108356387642), "iq3s": (512, 53294177878),
            "iq1s": (2048, 7590341501443526924)}
    for key, (n, checksum) in want.items():
        a = GRIDS[key]
        assert a.size == n and sum(int(v) for v in a) % (1 << 64) == checksum, key
    assert GRIDS["iq3xxs"].dtype == np.uint32 and GRIDS["iq2s"].dtype == np.uint64
    # ksigns_iq2xs is derivable (7 bits plus an even-parity bit), so the library computes it instead of taking a table
    assert np.array_equal(gguf_np.KSIGNS, GRIDS["ksigns"])


def test_block_sizes(grid_oracle):
    # src/gguf/dequant.rs:94-114
    for ty, bb in gguf_np.GRID_BLOCK_BYTES.items():
        assert (grid_oracle.blk_elems(ty), grid_oracle.blk_bytes(ty)) == (256, bb)
    assert grid_oracle.row_bytes(16, 1024) == 264


def test_wrong_codebook_size_is_refused(oracle):
    with pytest.raises(ValueError):
        oracle.set_iq_grids({**{k: GRIDS[k] for k in oracle.GRID_ORDER}, "iq2xs": GRIDS["iq2xxs"]})
    oracle.set_iq_grids(GRIDS)


@pytest.mark.parametrize("ty", TYPES)
def test_adversarial_rows_oracle_equals_numpy(grid_oracle, ty):
    nb, rows = 8, 3
    adv = grid_oracle.adversarial_rows(ty, nb, rows)
    bb = grid_oracle.blk_bytes(ty)
    blocks = adv.reshape(rows * nb, bb)
    for i, blk in enumerate(blocks):
        if i % 4 == 0:
            assert not blk.any()
        elif ty != 29:
            assert list(blk[:2]) == [[0, 0], [1, 0], [255, 131], [255, 123]][i % 4]
    cols = nb * 256
    rb = grid_oracle.row_bytes(ty, cols)
    seq = np.stack([grid_oracle.dequant_row_ref(ty, adv[r * rb:(r + 1) * rb], cols) for r in range(rows)])
    ind = gguf_np.GRID_DECODERS[ty](adv, GRIDS).reshape(rows, cols)
    assert np.isfinite(seq).all() and np.abs(seq).max() > 1e5 and (seq == 0).mean() > 0.2
    synth.assert_bits_equal(seq, ind, f"{gguf_np.GRID_NAMES[ty]}: C++ oracle vs numpy on the adversarial rows")


@pytest.mark.parametrize("ty", TYPES)
def test_random_blocks_oracle_equals_numpy(grid_oracle, ty):
    nblk = 96
    raw = iq_random_blocks(ty, nblk, seed=ty)
    seq = grid_oracle.dequant_row_ref(ty, raw, nblk * 256)
    ind = gguf_np.GRID_DECODERS[ty](raw, GRIDS)
    assert np.isfinite(seq).all() and len(np.unique(seq)) > 100 and (seq < 0).mean() > 0.2
    synth.assert_bits_equal(seq, ind, f"{gguf_np.GRID_NAMES[ty]}: C++ oracle vs numpy on random blocks")
    ids = np.array([23, 0, 7, 7], np.uint32)
    g = grid_oracle.embed_gather(raw, ty, 24, 1024, ids, threads=2)
    synth.assert_bits_equal(g, seq.reshape(24, 1024)[ids], "gather")
