"""The GGUF container reader (lokal_gguf_*): the reference's container tests (src/gguf/container.rs:446-514) on
synthetic files built the way its test fixtures build them (src/gguf/testutil.rs:9-93), plus a small model-shaped
file whose token_embd.weight goes from the file through the gather on the GPU."""
import struct

import numpy as np
import pytest

import lokal_b200 as L
import synth
from lokal_b200 import GgufFile

E = L.capi


def put_str(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def kv(key, ty, payload):
    return put_str(key) + struct.pack("<I", ty) + payload


def tensor_info(name, ne, ty, offset):
    return put_str(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne) + struct.pack("<IQ", ty, offset)


def gguf_bytes(version, kvs, infos, data, align=32, n_tensors=None):
    b = b"GGUF" + struct.pack("<IQQ", version, len(infos) if n_tensors is None else n_tensors, len(kvs)) + b"".join(kvs) + b"".join(infos)
    b += b"\0" * (-len(b) % align)
    return b + data


def tiny_gguf(version, align=None):
    """One Q8_0 tensor "t" of ne = [32, 2]; optionally a general.alignment key (u32)."""
    kvs = [kv("general.architecture", 8, put_str("llama"))]
    if align is not None:
        kvs.append(kv("general.alignment", 4, struct.pack("<I", align)))
    return gguf_bytes(version, kvs, [tensor_info("t", [32, 2], 8, 0)], bytes(68), align or 32)


def mixed_lowbit_gguf():
    infos = [tensor_info(n, [256, 2], ty, 0) for n, ty in [("token_embd.weight", 9), ("blk.0.ffn_down.weight", 9), ("blk.0.attn_q.weight", 7),
                                                           ("blk.1.attn_q.weight", 3), ("output_norm.weight", 8)]]
    return gguf_bytes(3, [kv("general.architecture", 8, put_str("llama"))], infos, bytes(4096))


def open_err(tmp_path, data, name="x.gguf"):
    p = tmp_path / name
    p.write_bytes(data)
    with pytest.raises(L.LokalCudaError) as e:
        GgufFile(p)
    return e.value


def test_parses_the_synthetic_file(tmp_path):
    p = tmp_path / "parse.gguf"
    p.write_bytes(tiny_gguf(3))
    with GgufFile(p) as g:
        assert g.version == 3 and g.n_tensors() == 1
        assert g.get_str("general.architecture") == "llama"
        t = g.tensor("t")
        assert t.dims == (2, 32)  # ne reversed to row-major
        assert t.ggml_type == L.Q8_0 and t.nbytes == 68 and t.data.size == 68 and t.data_offset == 0
        assert g.data_start % 32 == 0 and [x.name for x in g.tensors()] == ["t"]
        with pytest.raises(L.LokalCudaError) as e:
            g.tensor("nope")
        assert e.value.status == E.ERR_NOT_FOUND and "tensor nope not in the GGUF file" in e.value.message


def test_respects_general_alignment(tmp_path):
    p = tmp_path / "align.gguf"
    p.write_bytes(tiny_gguf(2, 64))
    with GgufFile(p) as g:
        assert g.version == 2 and g.tensor("t").nbytes == 68 and g.data_start % 64 == 0
        assert g.get_usize("general.alignment") == 64
    for bad in (0, 48):
        e = open_err(tmp_path, tiny_gguf(3, bad))
        assert e.status == E.ERR_FORMAT and "general.alignment is invalid" in e.message


def test_rejects_big_endian_and_truncation(tmp_path):
    be = bytearray(tiny_gguf(3))
    be[4:8] = struct.pack(">I", 3)
    e = open_err(tmp_path, bytes(be))
    assert e.status == E.ERR_FORMAT and "big-endian" in e.message
    short = tiny_gguf(3)[:-40]
    e = open_err(tmp_path, short)
    assert "truncated" in e.message or "run past" in e.message
    e = open_err(tmp_path, tiny_gguf(3)[:30])  # cut inside the header
    assert "truncated" in e.message
    e = open_err(tmp_path, b"GGML" + tiny_gguf(3)[4:])
    assert "bad magic" in e.message
    e = open_err(tmp_path, tiny_gguf(4))
    assert "version 4 unsupported" in e.message
    with pytest.raises(L.LokalCudaError) as ex:
        GgufFile(tmp_path / "missing.gguf")
    assert ex.value.status == E.ERR_IO and "cannot open" in ex.value.message


def test_refusal_names_every_unsupported_type_at_once(tmp_path):
    e = open_err(tmp_path, mixed_lowbit_gguf())
    err = e.message
    assert e.status == E.ERR_UNSUPPORTED
    for want in ("Q8_1", "Q5_1", "Q4_1"):
        assert want in err
    assert "Q8_1 (2 tensors, e.g. token_embd.weight)" in err and "Q5_1 (1 tensor, e.g." in err
    assert "3 quantization type(s)" in err and "across 4 of 5 tensors" in err
    assert "Q8_0" not in err  # the supported type is not listed as a problem


def test_structural_errors(tmp_path):
    arch = [kv("general.architecture", 8, put_str("llama"))]
    dup = gguf_bytes(3, arch, [tensor_info("t", [32, 2], 8, 0), tensor_info("t", [32, 2], 8, 96)], bytes(256))
    assert "tensor t appears twice" in open_err(tmp_path, dup).message
    ragged = gguf_bytes(3, arch, [tensor_info("t", [48, 2], 8, 0)], bytes(256))
    assert "not a whole number" in open_err(tmp_path, ragged).message  # src/gguf/container.rs:220-226
    far = gguf_bytes(3, arch, [tensor_info("t", [32, 2], 8, 1 << 40)], bytes(256))
    assert "run past the file" in open_err(tmp_path, far).message
    five_d = gguf_bytes(3, arch, [tensor_info("t", [32, 1, 1, 1, 1], 8, 0)], bytes(256))
    assert "5 dimensions" in open_err(tmp_path, five_d).message
    bad_val = gguf_bytes(3, [kv("k", 13, b"")], [], b"")
    assert "value type 13 unsupported" in open_err(tmp_path, bad_val).message
    long_str = gguf_bytes(3, [struct.pack("<Q", 1 << 30) + b"abc"], [], b"")
    assert "corrupt length" in open_err(tmp_path, long_str).message


def model_file(tmp_path, vocab=64, hidden=64, layers=2, embed_type=L.Q8_0):
    """A model-shaped file: metadata of every value kind, token_embd.weight quantised, f32 norm weights and biases."""
    rng = np.random.default_rng(11)
    tensors = {"token_embd.weight": ([hidden, vocab], embed_type, synth.quant_table(embed_type, vocab, hidden, 3).tobytes()),
               "output_norm.weight": ([hidden], 0, rng.standard_normal(hidden).astype(np.float32).tobytes())}
    for i in range(layers):
        tensors[f"blk.{i}.attn_norm.weight"] = ([hidden], 0, rng.standard_normal(hidden).astype(np.float32).tobytes())
        tensors[f"blk.{i}.attn_q.bias"] = ([hidden], 1, rng.standard_normal(hidden).astype(np.float16).tobytes())
    infos, data = [], b""
    for name, (ne, ty, raw) in tensors.items():
        data += b"\0" * (-len(data) % 32)
        infos.append(tensor_info(name, ne, ty, len(data)))
        data += raw
    kvs = [kv("general.architecture", 8, put_str("qwen3")),
           kv("qwen3.block_count", 4, struct.pack("<I", layers)),
           kv("qwen3.embedding_length", 10, struct.pack("<Q", hidden)),
           kv("qwen3.attention.layer_norm_rms_epsilon", 6, struct.pack("<f", 1e-6)),
           kv("qwen3.rope.freq_base", 12, struct.pack("<d", 1e6)),
           kv("neg", 5, struct.pack("<i", -3)),
           kv("flag", 7, b"\x01"),
           kv("tokenizer.ggml.tokens", 9, struct.pack("<IQ", 8, 3) + put_str("a") + put_str("bc") + put_str("")),
           kv("tokenizer.ggml.token_type", 9, struct.pack("<IQ", 5, 3) + struct.pack("<iii", 1, -2, 3)),
           kv("recurrent_layers", 9, struct.pack("<IQ", 7, 4) + b"\x01\x00\x00\x01"),
           kv("scores", 9, struct.pack("<IQ", 6, 2) + struct.pack("<ff", 0.5, -1.5))]
    p = tmp_path / "model.gguf"
    p.write_bytes(gguf_bytes(3, kvs, infos, data))
    return p, tensors


def test_metadata_accessors_and_tensor_bytes(tmp_path):
    p, tensors = model_file(tmp_path)
    with GgufFile(p) as g:
        assert g.n_tensors() == len(tensors)
        assert g.get_str("general.architecture") == "qwen3" and g.get_usize("qwen3.block_count") == 2
        assert g.get_usize("qwen3.embedding_length") == 64
        assert g.get_f32("qwen3.attention.layer_norm_rms_epsilon") == np.float32(1e-6) and g.get_f32("qwen3.rope.freq_base") == 1e6
        assert g.get_arr_str("tokenizer.ggml.tokens") == ["a", "bc", ""]
        assert g.get_arr_i64("tokenizer.ggml.token_type") == [1, -2, 3]
        assert g.get_arr_i64("recurrent_layers") == [1, 0, 0, 1]  # bool arrays ride the int rail
        assert g.has_key("flag") and not g.has_key("nope")
        for key, call, what in [("neg", g.get_usize, "is a int, expected an integer"), ("qwen3.block_count", g.get_f32, "expected a float"),
                                ("qwen3.block_count", g.get_str, "expected a string"), ("scores", g.get_arr_i64, "is a float array"),
                                ("flag", g.get_usize, "is a bool")]:
            with pytest.raises(L.LokalCudaError) as e:
                call(key)
            assert e.value.status == E.ERR_BAD_ARG and what in e.value.message and key in e.value.message
        with pytest.raises(L.LokalCudaError) as e:
            g.get_usize("absent.key")
        assert e.value.status == E.ERR_NOT_FOUND and "absent.key is missing" in e.value.message
        for t in g.tensors():
            ne, ty, raw = tensors[t.name]
            assert t.dims == tuple(reversed(ne)) and t.ggml_type == ty and t.data.tobytes() == raw
            assert (g.data_start + t.data_offset) % 32 == 0
        emb = g.tensor("token_embd.weight")
        assert emb.dims == (64, 64) and emb.nbytes == L.row_bytes(L.Q8_0, 64 * 64)


def walk_everything(path):
    """Open, then touch every accessor and every tensor's bytes; a damaged file may be refused (an error with a
    message) or accepted, but what is accepted must be readable end to end."""
    try:
        g = GgufFile(path)
    except L.LokalCudaError as e:
        assert e.status in (E.ERR_FORMAT, E.ERR_IO, E.ERR_UNSUPPORTED) and e.message
        return False
    with g:
        g.version, g.data_start
        for t in g.tensors():
            assert t.data.nbytes == t.nbytes
            int(np.frombuffer(t.data, np.uint8).sum())  # every byte of the tensor is inside the mapping
        for key in ("general.architecture", "qwen3.block_count", "tokenizer.ggml.tokens", "tokenizer.ggml.token_type",
                    "recurrent_layers", "scores", "flag", "neg"):
            for call in (g.get_usize, g.get_f32, g.get_str, g.get_arr_i64, g.get_arr_str):
                try:
                    call(key)
                except L.LokalCudaError as e:
                    assert e.status in (E.ERR_BAD_ARG, E.ERR_NOT_FOUND)
    return True


def test_damaged_headers_are_refused_or_read_safely(tmp_path):
    """The reader's input is a file from outside. Every truncation of the header, every 8-byte field blown up to a huge
    count, and 1500 seeded byte flips: the reader must answer with an error or a file it can walk, never read outside
    the mapping (container.rs:248-288 bounds every tensor against the file length for the same reason)."""
    p, _ = model_file(tmp_path, vocab=8, hidden=32, layers=1)
    good = p.read_bytes()
    with GgufFile(p) as g:
        header = min(g.data_start + 64, len(good))  # the header and the first bytes of tensor data
    q = tmp_path / "damaged.gguf"
    assert walk_everything(p)
    accepted = 0
    for cut in range(0, header, 3):
        q.write_bytes(good[:cut])
        accepted += walk_everything(q)
    for off in range(4, header - 8, 4):
        for blow in (struct.pack("<Q", 0xFFFFFFFFFFFFFFFF), struct.pack("<Q", 1 << 40), struct.pack("<Q", 0x7FFFFFFF)):
            bad = bytearray(good)
            bad[off:off + 8] = blow
            q.write_bytes(bytes(bad))
            accepted += walk_everything(q)
    rng = np.random.default_rng(2024)
    for _ in range(1500):
        bad = bytearray(good)
        for _ in range(int(rng.integers(1, 4))):
            bad[int(rng.integers(0, header))] = int(rng.integers(0, 256))
        q.write_bytes(bytes(bad))
        accepted += walk_everything(q)
    assert accepted > 0  # some damage is harmless (a flipped byte inside a key name): those files must stay readable


def test_tiny_headers_cannot_ask_for_huge_allocations(tmp_path):
    """A 40-byte header that announces an array of 2^26 strings (or numbers) is refused before anything is reserved for
    it: an array cannot have more entries than the bytes left in the file can hold. And a tensor of exactly 2^62 F32
    elements, whose byte count wraps to zero in 64 bits, is an overflow, not an empty tensor."""
    import resource
    import time
    for et, each in ((8, 8), (4, 4), (10, 8), (7, 1)):
        n = 1 << 26
        blob = gguf_bytes(3, [kv("tokenizer.ggml.tokens", 9, struct.pack("<IQ", et, n))], [], b"")
        before = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss
        t0 = time.perf_counter()
        e = open_err(tmp_path, blob)
        assert e.status == E.ERR_FORMAT and "entries" in e.message and "left in the file" in e.message
        assert time.perf_counter() - t0 < 0.5
        assert resource.getrusage(resource.RUSAGE_SELF).ru_maxrss - before < 64 * 1024  # KiB: nowhere near the 0.5-2 GiB asked for
    # an array that does fit is still read
    ok = gguf_bytes(3, [kv("a", 9, struct.pack("<IQ", 4, 3) + struct.pack("<III", 7, 8, 9))], [], b"")
    p = tmp_path / "ok.gguf"
    p.write_bytes(ok)
    with GgufFile(p) as g:
        assert list(g.get_arr_i64("a")) == [7, 8, 9]
    for ne in ([1 << 62], [1 << 31, 1 << 31], [1 << 20, 1 << 21, 1 << 21]):
        e = open_err(tmp_path, gguf_bytes(3, [], [tensor_info("t", ne, 0, 0)], bytes(64)))
        assert e.status == E.ERR_FORMAT and ("overflow" in e.message or "past the file" in e.message)


@pytest.mark.gpu
@pytest.mark.parametrize("embed_type", [L.Q8_0, L.Q6_K, L.Q4_K])
def test_embedding_table_from_a_file_through_the_gather(tmp_path, ctx, dev, oracle, embed_type):
    vocab, hidden = 300, 512
    p, tensors = model_file(tmp_path, vocab=vocab, hidden=hidden, embed_type=embed_type)
    ids = synth.token_ids_uniform(vocab, 1000, seed=1)
    with GgufFile(p) as g:
        dptr, info = ctx.gguf_upload(g, "token_embd.weight")
        wptr, winfo = ctx.gguf_upload(g, "output_norm.weight")
        assert (info.dims[0], info.dims[1], info.ggml_type) == (vocab, hidden, embed_type) and winfo.nbytes == hidden * 4
    # the file is closed: the device copies stand on their own
    try:
        out = dev.empty((1000, hidden), synth.F32, fill=3.0)
        ctx.embed_gather(dptr, dev.put(ids), out, ggml_type=embed_type, vocab=vocab, dim=hidden, n=1000)
        y = dev.empty((1000, hidden), synth.F32, fill=0.0)
        ctx.rmsnorm(out, wptr, y, rows=1000, dim=hidden, eps=1e-6, dtype=synth.F32, w_dtype=synth.F32)
        ctx.stream_sync()
        raw = np.frombuffer(tensors["token_embd.weight"][2], np.uint8)
        want = oracle.embed_gather(raw, embed_type, vocab, hidden, ids)
        synth.assert_bits_equal(dev.get(out), want, "gather from a file's token_embd.weight")
        w = np.frombuffer(tensors["output_norm.weight"][2], np.float32)
        synth.check_f32(dev.get(y), np.stack([oracle.rmsnorm(r, w, 1e-6) for r in want]), "norm with a file's weights")
    finally:
        ctx.free(dptr)
        ctx.free(wptr)
    with pytest.raises(L.LokalCudaError) as e:
        with GgufFile(p) as g:
            ctx.gguf_upload(g, "blk.9.attn_norm.weight")
    assert e.value.status == E.ERR_NOT_FOUND
