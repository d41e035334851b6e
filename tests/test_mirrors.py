"""Mirror guards: every re-declaration of the C ABI must agree with include/lokal_cuda.h.

The reference re-declares its Metal parameter structs in Rust and guards the copies with a test that reads both sources
as text and compares them field for field (src/gpu/metal.rs:4448-4589). The same guard here, in two directions:

  * rust/lokal-cuda-sys/src/lib.rs (the FFI crate a `-b cuda` backend links): every struct of the header field for
    field (name, type, order), every function argument for argument (name, type, order, return type), every
    enumerator and #define by value;
  * lokal_b200/capi.py (the ctypes binding the tests and the benchmark use): every struct field for field, every
    function by arity and argument class.

The header is parsed once, from text; nothing is compiled and no GPU is needed.
"""
import ctypes as C
import os
import re

from lokal_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = open(os.path.join(ROOT, "include", "lokal_cuda.h")).read()
RUST = open(os.path.join(ROOT, "rust", "lokal-cuda-sys", "src", "lib.rs")).read()

OPAQUE = {"lokal_cuda_ctx", "lokal_cuda_graph", "lokal_gguf", "lokal_cuda_pass"}
SCALARS = {"int": "c_int", "int32_t": "i32", "uint32_t": "u32", "int64_t": "i64", "uint64_t": "u64", "size_t": "usize",
           "float": "f32", "uint8_t": "u8", "char": "c_char", "void": "c_void"}


def strip_comments(text):
    return re.sub(r"/\*.*?\*/", "", text, flags=re.S)


def camel(name):
    return "".join(p.capitalize() for p in name.split("_"))


# ---- the header, parsed into a neutral form: types are (base, [pointer constness...]) ----

def parse_c_type(text):
    """'const char* const**' -> ('char', ['const', 'const', 'mut']): base type, then one entry per '*', innermost first,
    saying whether what that pointer points AT is const."""
    toks = text.replace("*", " * ").split()
    i, const_pending = 0, False
    if toks[i] == "const":
        const_pending, i = True, i + 1
    base = toks[i]
    i += 1
    if i < len(toks) and toks[i] == "const":
        const_pending, i = True, i + 1
    ptrs = []
    while i < len(toks):
        assert toks[i] == "*", text
        ptrs.append("const" if const_pending else "mut")
        const_pending = False
        i += 1
        if i < len(toks) and toks[i] == "const":
            const_pending, i = True, i + 1
    return base, ptrs


def header_structs():
    out = {}
    for name, body in re.findall(r"typedef struct (\w+) \{(.*?)\} \1;", strip_comments(HEADER), flags=re.S):
        fields = []
        for stmt in body.split(";"):
            stmt = " ".join(stmt.split())
            if not stmt:
                continue
            m = re.match(r"((?:const )?\w+(?: const)?\s*\**)\s*(.*)$", stmt)
            ctype, names = m.group(1), m.group(2)
            for n in names.split(","):
                n = n.strip()
                arr = re.match(r"(\w+)\[(\d+)\]$", n)
                fields.append((arr.group(1), parse_c_type(ctype), int(arr.group(2))) if arr else (n, parse_c_type(ctype), 0))
        out[name] = fields
    return out


def header_functions():
    out = {}
    for ret, name, args in re.findall(r"^LOKAL_API\s+([\w \*]+?)\s*(\w+)\((.*?)\);", strip_comments(HEADER), flags=re.S | re.M):
        args = " ".join(args.split())
        params = []
        if args != "void":
            for a in args.split(","):
                m = re.match(r"(.*?)(\w+)$", a.strip())
                params.append((m.group(2), parse_c_type(m.group(1))))
        out[name] = (params, None if ret.strip() == "void" else parse_c_type(ret))
    return out


def header_constants():
    text = strip_comments(HEADER)
    vals = {n: int(v) for n, v in re.findall(r"\b(LOKAL_\w+) = (\d+)", text)}
    for n, v in re.findall(r"#define (LOKAL_\w+) \(?(\d+)u?\)?\s*$", text, flags=re.M):
        vals[n] = int(v)
    m = re.search(r"#define LOKAL_NOALLOC_TABLE_BYTES \((\d+)u << (\d+)\)", text)
    vals["LOKAL_NOALLOC_TABLE_BYTES"] = int(m.group(1)) << int(m.group(2))
    for n, v in re.findall(r"#define (LOKAL_\w+) (0x[0-9A-Fa-f]+)u?\s*$", text, flags=re.M):
        vals[n] = int(v, 16)
    return vals


# ---- the same declarations as the Rust source should spell them ----

def rust_type(ctype):
    base, ptrs = ctype
    if base == "lokal_cuda_stream":
        t = "LokalCudaStream"
    elif base in SCALARS:
        t = SCALARS[base]
    else:
        t = camel(base)
    for p in ptrs:
        t = ("*const " if p == "const" else "*mut ") + t
    return t


def rust_structs():
    out = {}
    for name, body in re.findall(r"#\[repr\(C\)\]\s*(?:#\[derive\([^\)]*\)\]\s*)?pub struct (\w+) \{(.*?)\n\}", RUST, flags=re.S):
        fields = []
        for line in body.splitlines():
            line = line.split("//")[0].strip().rstrip(",")
            if line:
                m = re.match(r"(?:pub )?(\w+): (.+)$", line)
                fields.append((m.group(1), m.group(2)))
        out[name] = fields
    return out


def rust_functions():
    block = re.search(r'extern "C" \{(.*?)\n\}', RUST, flags=re.S).group(1)
    out = {}
    for name, args, ret in re.findall(r"pub fn (\w+)\((.*?)\)(?:\s*->\s*([^;]+))?;", block, flags=re.S):
        params = []
        for a in " ".join(args.split()).split(", "):
            if a:
                n, t = a.split(": ", 1)
                params.append((n, t))
        out[name] = (params, ret.strip() if ret else None)
    return out


def test_rust_structs_mirror_the_header_field_for_field():
    hs, rs = header_structs(), rust_structs()
    assert set(hs) == {"lokal_qk_rope_params", "lokal_kv_layout", "lokal_gguf_tensor", "lokal_pass_config", "lokal_pass_weights",
                       "lokal_pass_inputs"}
    for cname, fields in hs.items():
        rname = camel(cname)
        assert rname in rs, f"{cname} has no #[repr(C)] mirror {rname} in lib.rs"
        want = [(n, f"[{rust_type(t)}; {arr}]" if arr else rust_type(t)) for n, t, arr in fields]
        assert rs[rname] == want, f"{rname} differs from {cname}"
    # the opaque handles are zero-sized #[repr(C)] structs, never dereferenced
    for cname in OPAQUE:
        assert rs[camel(cname)] == [("_opaque", "[u8; 0]")]
    assert set(rs) == {camel(n) for n in hs} | {camel(n) for n in OPAQUE}


def test_rust_functions_mirror_the_header_argument_for_argument():
    hf, rf = header_functions(), rust_functions()
    assert len(hf) >= 70
    assert list(rf) == list(hf), "lib.rs must declare exactly the header's functions, in the header's order"
    for name, (params, ret) in hf.items():
        want = ([(n, rust_type(t)) for n, t in params], rust_type(ret) if ret else None)
        assert rf[name] == want, f"{name}: lib.rs has {rf[name]}, the header says {want}"


def test_rust_constants_match_the_header():
    consts = {n: int(v) for n, v in re.findall(r"pub const (LOKAL_\w+): \w+ = (\d+);", RUST)}
    m = re.search(r"pub const LOKAL_NOALLOC_TABLE_BYTES: u32 = (\d+) << (\d+);", RUST)
    consts["LOKAL_NOALLOC_TABLE_BYTES"] = int(m.group(1)) << int(m.group(2))
    consts.update({n: int(v, 16) for n, v in re.findall(r"pub const (LOKAL_\w+): \w+ = (0x[0-9A-Fa-f]+);", RUST)})
    assert consts == header_constants()


# ---- the ctypes binding ----

CTYPES_SCALAR = {"int": C.c_int, "int32_t": C.c_int32, "uint32_t": C.c_uint32, "int64_t": C.c_int64, "uint64_t": C.c_uint64,
                 "size_t": C.c_size_t, "float": C.c_float}
CTYPES_STRUCTS = {"lokal_qk_rope_params": capi.QkRopeParams, "lokal_kv_layout": capi.KvLayout, "lokal_gguf_tensor": capi.GgufTensor,
                  "lokal_pass_config": capi.PassConfig, "lokal_pass_weights": capi.PassWeights, "lokal_pass_inputs": capi.PassInputs}


def ctypes_field_type(ctype, arr):
    base, ptrs = ctype
    if ptrs:
        t = C.c_char_p if (base == "char" and len(ptrs) == 1) else C.c_void_p
    else:
        t = CTYPES_SCALAR[base]
    return t * arr if arr else t


def test_ctypes_structs_mirror_the_header_field_for_field():
    for cname, fields in header_structs().items():
        mirror = CTYPES_STRUCTS[cname]
        got = [(n, t) for n, t in mirror._fields_]
        want = [(n, ctypes_field_type(t, arr)) for n, t, arr in fields]
        assert [n for n, _ in got] == [n for n, _ in want], f"{mirror.__name__}: field names or order differ from {cname}"
        for (n, g), (_, w) in zip(got, want):
            assert C.sizeof(g) == C.sizeof(w) and (g is w or (hasattr(g, "_length_") and g._length_ == w._length_ and g._type_ is w._type_)), \
                f"{mirror.__name__}.{n}: {g} against {w}"
    assert C.sizeof(capi.PassConfig) == 8 + 7 * 4 + 2 * 4 + 5 * 4 + 4 + 4 + 8  # with the padding before vocab
    assert C.sizeof(capi.PassInputs) == 14 * 8 and C.sizeof(capi.PassWeights) == 7 * 8 and C.sizeof(capi.KvLayout) == 32


def test_ctypes_signatures_agree_with_the_header_in_arity_and_argument_class():
    hf = header_functions()
    assert set(hf) == set(capi.SIGNATURES)
    for name, (params, ret) in hf.items():
        res, args = capi.SIGNATURES[name]
        assert len(args) == len(params), f"{name}: {len(args)} ctypes arguments, {len(params)} in the header"
        for (pname, (base, ptrs)), a in zip(params, args):
            is_pointer = bool(ptrs) or base == "lokal_cuda_stream"
            if is_pointer:
                assert a in (C.c_void_p, C.c_char_p) or hasattr(a, "contents") or getattr(a, "_type_", None) is not None, f"{name}.{pname}"
            else:
                assert C.sizeof(a) == C.sizeof(CTYPES_SCALAR[base]), f"{name}.{pname}: {a} against {base}"
        if ret is None:
            assert res is None, name
        elif ret[1]:
            assert res in (C.c_char_p, C.c_void_p), name
        else:
            assert C.sizeof(res) == C.sizeof(CTYPES_SCALAR[ret[0]]), name
