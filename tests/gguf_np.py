"""A second, independent reading of the GGUF block formats: vectorised numpy decoders written from the block
layouts (sizeof and field order as src/gguf/dequant.rs:94-114 lists them), used to cross-check the C++ oracle
before either is used to check the GPU. Every f32 multiply / subtract is a separate numpy f32 operation, so the rounding
sequence is the one the reference's expressions have. Returns f32 arrays of shape [n_blocks * elems]."""
import numpy as np

F32 = np.float32
KV = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.int32)  # IQ4 codebook


def _f16(b, off):
    return np.ascontiguousarray(b[:, off:off + 2]).view(np.float16).astype(F32)[:, 0]


def _blocks(raw, size):
    raw = np.ascontiguousarray(raw, np.uint8)
    assert raw.size % size == 0
    return raw.reshape(-1, size)


def _scale_min_k4(s):
    """12 packed bytes -> (8 six-bit scales, 8 six-bit mins) per block."""
    s = s.astype(np.uint32)
    sc = np.empty((s.shape[0], 8), np.uint32)
    mn = np.empty_like(sc)
    sc[:, :4] = s[:, 0:4] & 63
    mn[:, :4] = s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 0xF) | ((s[:, 0:4] >> 6) << 4)
    mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return sc, mn


def q8_0(raw):
    b = _blocks(raw, 34)
    return (b[:, 2:].view(np.int8).astype(F32) * _f16(b, 0)[:, None]).reshape(-1)


def q4_0(raw):
    b = _blocks(raw, 18)
    q = b[:, 2:].astype(np.int32)
    v = np.concatenate([(q & 15) - 8, (q >> 4) - 8], axis=1).astype(F32)
    return (v * _f16(b, 0)[:, None]).reshape(-1)


def q5_0(raw):
    b = _blocks(raw, 22)
    qh = np.ascontiguousarray(b[:, 2:6]).view("<u4")[:, 0].astype(np.uint64)
    j = np.arange(16, dtype=np.uint64)
    hi_lo = ((qh[:, None] >> j) & 1).astype(np.int32) << 4
    hi_hi = ((qh[:, None] >> (j + 16)) & 1).astype(np.int32) << 4
    q = b[:, 6:].astype(np.int32)
    v = np.concatenate([((q & 15) | hi_lo) - 16, ((q >> 4) | hi_hi) - 16], axis=1).astype(F32)
    return (v * _f16(b, 0)[:, None]).reshape(-1)


def iq4_nl(raw):
    b = _blocks(raw, 18)
    q = b[:, 2:].astype(np.int32)
    v = np.concatenate([KV[q & 15], KV[q >> 4]], axis=1).astype(F32)
    return (_f16(b, 0)[:, None] * v).reshape(-1)


def iq4_xs(raw):
    b = _blocks(raw, 136)
    d = _f16(b, 0)
    sh = np.ascontiguousarray(b[:, 2:4]).view("<u2")[:, 0].astype(np.int32)
    sl = b[:, 4:8].astype(np.int32)
    ib = np.arange(8)
    ls = ((sl[:, ib // 2] >> (4 * (ib % 2))) & 15) | (((sh[:, None] >> (2 * ib)) & 3) << 4)
    dl = d[:, None] * (ls - 32).astype(F32)                       # [nb, 8]
    q = b[:, 8:].reshape(-1, 8, 16).astype(np.int32)
    v = np.concatenate([KV[q & 15], KV[q >> 4]], axis=2).astype(F32)  # [nb, 8, 32]
    return (dl[:, :, None] * v).reshape(-1)


def q2_k(raw):
    b = _blocks(raw, 84)
    d, dmin = _f16(b, 80), _f16(b, 82)
    sc = b[:, :16].astype(np.int32).reshape(-1, 2, 4, 2)           # [nb, half128, field j, half16]
    qs = b[:, 16:80].astype(np.int32).reshape(-1, 2, 2, 16)        # [nb, half128, half16, l]
    j = np.arange(4).reshape(1, 1, 4, 1, 1)
    q = (qs[:, :, None, :, :] >> (2 * j)) & 3                      # [nb, 2, 4, 2, 16]
    dl = d[:, None, None, None] * (sc & 15).astype(F32)
    ml = dmin[:, None, None, None] * (sc >> 4).astype(F32)
    y = (dl[..., None] * q.astype(F32)).astype(F32) - ml[..., None]
    return y.astype(F32).reshape(-1)


def q3_k(raw):
    b = _blocks(raw, 110)
    d = _f16(b, 108)
    p = b[:, 96:108].astype(np.uint32)
    w = lambda i: p[:, 4 * i] | (p[:, 4 * i + 1] << 8) | (p[:, 4 * i + 2] << 16) | (p[:, 4 * i + 3] << 24)
    a0, a1, t = w(0), w(1), w(2)
    k1, k2 = np.uint32(0x03030303), np.uint32(0x0f0f0f0f)
    aux = [(a0 & k2) | (((t >> 0) & k1) << 4), (a1 & k2) | (((t >> 2) & k1) << 4),
           ((a0 >> 4) & k2) | (((t >> 4) & k1) << 4), ((a1 >> 4) & k2) | (((t >> 6) & k1) << 4)]
    scales = np.stack([(a >> (8 * k)) & 0xFF for a in aux for k in range(4)], axis=1).astype(np.int32) - 32  # [nb, 16]
    sc = scales.reshape(-1, 2, 4, 2)
    hm = b[:, :32].astype(np.int32).reshape(-1, 1, 1, 2, 16)
    qs = b[:, 32:96].astype(np.int32).reshape(-1, 2, 1, 2, 16)
    j = np.arange(4).reshape(1, 1, 4, 1, 1)
    nh = np.arange(2).reshape(1, 2, 1, 1, 1)
    q = (qs >> (2 * j)) & 3
    hi = np.where((hm >> (nh * 4 + j)) & 1, 0, 4)
    dl = d[:, None, None, None] * sc.astype(F32)
    return (dl[..., None] * (q - hi).astype(F32)).astype(F32).reshape(-1)


def q4_k(raw):
    b = _blocks(raw, 144)
    d, dmin = _f16(b, 0), _f16(b, 2)
    sc, mn = _scale_min_k4(b[:, 4:16])
    qs = b[:, 16:].astype(np.int32).reshape(-1, 4, 32)
    q = np.stack([qs & 15, qs >> 4], axis=2).reshape(-1, 8, 32)   # group order: low nibbles, then high nibbles
    dl = d[:, None] * sc.astype(F32)
    ml = dmin[:, None] * mn.astype(F32)
    return ((dl[:, :, None] * q.astype(F32)).astype(F32) - ml[:, :, None]).astype(F32).reshape(-1)


def q5_k(raw):
    b = _blocks(raw, 176)
    d, dmin = _f16(b, 0), _f16(b, 2)
    sc, mn = _scale_min_k4(b[:, 4:16])
    qh = b[:, 16:48].astype(np.int32)
    qs = b[:, 48:].astype(np.int32).reshape(-1, 4, 32)
    g = np.arange(4).reshape(1, 4, 1)
    lo = (qs & 15) + (((qh[:, None, :] >> (2 * g)) & 1) << 4)
    hi = (qs >> 4) + (((qh[:, None, :] >> (2 * g + 1)) & 1) << 4)
    q = np.stack([lo, hi], axis=2).reshape(-1, 8, 32)
    dl = d[:, None] * sc.astype(F32)
    ml = dmin[:, None] * mn.astype(F32)
    return ((dl[:, :, None] * q.astype(F32)).astype(F32) - ml[:, :, None]).astype(F32).reshape(-1)


def q6_k(raw):
    b = _blocks(raw, 210)
    d = _f16(b, 208)
    ql = b[:, :128].astype(np.int32).reshape(-1, 2, 2, 32)         # [nb, half128, lo/hi 32 bytes, l]
    qh = b[:, 128:192].astype(np.int32).reshape(-1, 2, 32)
    sc = b[:, 192:208].view(np.int8).astype(np.int32).reshape(-1, 2, 8)
    parts = []
    for k in range(4):  # sub-rows l, l+32, l+64, l+96 of each 128-element half
        nib = (ql[:, :, k & 1, :] & 15) if k < 2 else (ql[:, :, k & 1, :] >> 4)
        q = (nib | (((qh >> (2 * k)) & 3) << 4)) - 32
        s = np.repeat(sc[:, :, 2 * k:2 * k + 2], 16, axis=2)       # scale index is + 2k, is = l // 16
        parts.append((d[:, None, None] * s.astype(F32)).astype(F32) * q.astype(F32))
    return np.stack(parts, axis=2).astype(F32).reshape(-1)


# ---- codebook types: take the i-quant grids as a mapping (keys iq2xxs, iq2xs, iq2s, iq3xxs, iq3s, iq1s) ----

KSIGNS = np.array([i | ((bin(i).count("1") & 1) << 7) for i in range(128)], np.uint8)  # 7 bits + an even-parity bit


def _grid_bytes(grid, idx, width, signed=False):
    """Codebook entries grid[idx] split into `width` bytes, lowest first: shape idx.shape + (width,)."""
    g = np.asarray(grid)[idx].astype(np.uint64)
    by = ((g[..., None] >> (8 * np.arange(width, dtype=np.uint64))) & np.uint64(0xFF)).astype(np.uint8)
    return (by.view(np.int8) if signed else by).astype(F32)


def _sign_factors(sign_bytes):
    """Bit j of each byte set -> -1 for value j of the run: shape sign_bytes.shape + (8,)."""
    bits = (sign_bytes[..., None].astype(np.int32) >> np.arange(8)) & 1
    return np.where(bits == 1, F32(-1), F32(1)).astype(F32)


def _u32(b):
    return np.ascontiguousarray(b).view("<u4")


def iq2_xxs(raw, grids):
    b = _blocks(raw, 66)
    q = b[:, 2:].reshape(-1, 8, 8)                                  # per group: 4 grid bytes, then a u32
    a1 = _u32(q[:, :, 4:8])[:, :, 0].astype(np.int64)
    db = (_f16(b, 0)[:, None] * (F32(0.5) + (a1 >> 28).astype(F32))).astype(F32) * F32(0.25)
    signs = KSIGNS[(a1[:, :, None] >> (7 * np.arange(4))) & 127]
    g = _grid_bytes(grids["iq2xxs"], q[:, :, :4].astype(np.int64), 8)
    return ((db[:, :, None, None] * g).astype(F32) * _sign_factors(signs)).astype(F32).reshape(-1)


def _db_nibbles(d, sc):
    nib = np.stack([sc & 15, sc & 15, sc >> 4, sc >> 4], axis=2).astype(F32)  # runs 0,1 use the low nibble, 2,3 the high
    return (d[:, None, None] * (F32(0.5) + nib)).astype(F32) * F32(0.25)


def iq2_xs(raw, grids):
    b = _blocks(raw, 74)
    qv = np.ascontiguousarray(b[:, 2:66]).view("<u2").reshape(-1, 8, 4).astype(np.int64)
    db = _db_nibbles(_f16(b, 0), b[:, 66:74].astype(np.int32))
    g = _grid_bytes(grids["iq2xs"], qv & 511, 8)
    return ((db[..., None] * g).astype(F32) * _sign_factors(KSIGNS[qv >> 9])).astype(F32).reshape(-1)


def iq2_s(raw, grids):
    b = _blocks(raw, 82)
    lo = b[:, 2:34].reshape(-1, 8, 4).astype(np.int64)
    signs = b[:, 34:66].reshape(-1, 8, 4)
    qh = b[:, 66:74].astype(np.int64)
    db = _db_nibbles(_f16(b, 0), b[:, 74:82].astype(np.int32))
    gi = lo | ((qh[:, :, None] << (8 - 2 * np.arange(4))) & 0x300)
    g = _grid_bytes(grids["iq2s"], gi, 8)
    return ((db[..., None] * g).astype(F32) * _sign_factors(signs)).astype(F32).reshape(-1)


def iq3_xxs(raw, grids):
    b = _blocks(raw, 98)
    qs = b[:, 2:66].reshape(-1, 8, 4, 2).astype(np.int64)            # [group, run, half of the run]
    aux = _u32(b[:, 66:98]).astype(np.int64)                        # [nb, 8]
    db = (_f16(b, 0)[:, None] * (F32(0.5) + (aux >> 28).astype(F32))).astype(F32) * F32(0.5)
    signs = KSIGNS[(aux[:, :, None] >> (7 * np.arange(4))) & 127]
    g = _grid_bytes(grids["iq3xxs"], qs, 4).reshape(-1, 8, 4, 8)
    return ((db[:, :, None, None] * g).astype(F32) * _sign_factors(signs)).astype(F32).reshape(-1)


def iq3_s(raw, grids):
    b = _blocks(raw, 110)
    qs = b[:, 2:66].reshape(-1, 8, 4, 2).astype(np.int64)
    qh = b[:, 66:74].astype(np.int64)
    signs = b[:, 74:106].reshape(-1, 8, 4)
    scb = b[:, 106:110].astype(np.int32)
    sc = np.stack([scb & 15, scb >> 4], axis=2).reshape(-1, 8)       # group g: low nibble when g is even
    db = (_f16(b, 0)[:, None] * (1 + 2 * sc).astype(F32)).astype(F32)
    shift = 8 - 2 * np.arange(4)[:, None] - np.arange(2)[None, :]
    gi = qs | ((qh[:, :, None, None] << shift) & 256)
    g = _grid_bytes(grids["iq3s"], gi, 4).reshape(-1, 8, 4, 8)
    return ((db[:, :, None, None] * g).astype(F32) * _sign_factors(signs)).astype(F32).reshape(-1)


def iq1_s(raw, grids):
    b = _blocks(raw, 50)
    qs = b[:, 2:34].reshape(-1, 8, 4).astype(np.int64)
    qh = np.ascontiguousarray(b[:, 34:50]).view("<u2").astype(np.int64)  # [nb, 8]
    dl = (_f16(b, 0)[:, None] * (2 * ((qh >> 12) & 7) + 1).astype(F32)).astype(F32)
    delta = np.where(qh & 0x8000, F32(-0.125), F32(0.125)).astype(F32)
    gi = qs | (((qh[:, :, None] >> (3 * np.arange(4))) & 7) << 8)
    g = _grid_bytes(grids["iq1s"], gi, 8, signed=True)
    return (dl[:, :, None, None] * (g + delta[:, :, None, None]).astype(F32)).astype(F32).reshape(-1)


def iq1_m(raw, grids):
    b = _blocks(raw, 56)
    qs = b[:, :32].reshape(-1, 8, 4).astype(np.int64)
    qh = np.repeat(b[:, 32:48].reshape(-1, 8, 2), 2, axis=2).astype(np.int64)   # runs 0,1 share a byte, runs 2,3 the next
    sc = np.ascontiguousarray(b[:, 48:56]).view("<u2").astype(np.int64)          # [nb, 4]
    dbits = (sc[:, 0] >> 12) | ((sc[:, 1] >> 8) & 0x00F0) | ((sc[:, 2] >> 4) & 0x0F00) | (sc[:, 3] & 0xF000)
    d = dbits.astype(np.uint16).view(np.float16).astype(F32)
    ib, run = np.arange(8)[:, None], np.arange(4)[None, :]
    shift = 6 * (ib % 2) + np.where(run < 2, 0, 3)
    s = (np.repeat(sc, 2, axis=1)[:, :, None] >> shift) & 7           # group ib reads scale word ib // 2
    dl = (d[:, None, None] * (2 * s + 1).astype(F32)).astype(F32)
    even = (run % 2) == 0
    gi = qs | ((qh << np.where(even, 8, 4)) & 0x700)
    delta = np.where(qh & np.where(even, 0x08, 0x80), F32(-0.125), F32(0.125)).astype(F32)
    g = _grid_bytes(grids["iq1s"], gi, 8, signed=True)
    return (dl[..., None] * (g + delta[..., None]).astype(F32)).astype(F32).reshape(-1)


GRID_DECODERS = {16: iq2_xxs, 17: iq2_xs, 18: iq3_xxs, 19: iq1_s, 21: iq3_s, 22: iq2_s, 29: iq1_m}
GRID_NAMES = {16: "IQ2_XXS", 17: "IQ2_XS", 18: "IQ3_XXS", 19: "IQ1_S", 21: "IQ3_S", 22: "IQ2_S", 29: "IQ1_M"}
GRID_BLOCK_BYTES = {16: 66, 17: 74, 18: 98, 19: 50, 21: 110, 22: 82, 29: 56}

DECODERS = {2: q4_0, 6: q5_0, 8: q8_0, 10: q2_k, 11: q3_k, 12: q4_k, 13: q5_k, 14: q6_k, 20: iq4_nl, 23: iq4_xs}
NAMES = {2: "Q4_0", 6: "Q5_0", 8: "Q8_0", 10: "Q2_K", 11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 20: "IQ4_NL", 23: "IQ4_XS"}


def random_blocks(ty, n_blocks, seed, blk_bytes, scale_offsets):
    """Uniform random bytes with finite, moderate f16 scales at the given offsets (no inf / nan scales)."""
    rng = np.random.default_rng(seed)
    b = rng.integers(0, 256, (n_blocks, blk_bytes), dtype=np.uint8)
    for off in scale_offsets:
        v = (rng.standard_normal(n_blocks) * 0.02).astype(np.float16)
        b[:, off:off + 2] = v.view(np.uint8).reshape(n_blocks, 2)
    return b.reshape(-1)


SCALE_OFFSETS = {2: (0,), 6: (0,), 8: (0,), 10: (80, 82), 11: (108,), 12: (0, 2), 13: (0, 2), 14: (208,), 20: (0,), 23: (0,)}
