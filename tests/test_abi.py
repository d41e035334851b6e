"""The C ABI without a GPU: the library loads, exports every symbol the header declares, the ctypes
mirror of the parameter struct matches the header field for field, and host-only helpers behave."""
import ctypes as C
import os
import re

import pytest

import lokal_b200
from lokal_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = open(os.path.join(ROOT, "include", "lokal_cuda.h")).read()


def declared_functions():
    return re.findall(r"LOKAL_API\s+[\w\s\*]+?\b(lokal_(?:cuda|gguf)_\w+)\s*\(", HEADER)


def test_library_exports_every_declared_symbol():
    lib = capi.load()
    names = declared_functions()
    assert len(names) >= 30 and len(set(names)) == len(names)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/lokal_cuda.h but not exported"
    assert set(names) == set(capi.SIGNATURES), "ctypes signatures and the header disagree"


def test_param_struct_mirror_matches_header():
    # the same guard the reference keeps between its shader structs and their Rust mirrors
    # (src/gpu/metal.rs:4448-4589), here between the C header and the ctypes binding
    body = re.search(r"typedef struct lokal_qk_rope_params \{(.*?)\} lokal_qk_rope_params;", HEADER, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    ctype = {"void*": C.c_void_p, "const void*": C.c_void_p, "const float*": C.c_void_p, "const uint32_t*": C.c_void_p,
             "uint64_t": C.c_uint64, "uint32_t": C.c_uint32, "float": C.c_float, "int32_t": C.c_int32}
    for stmt in body.split(";"):
        stmt = " ".join(stmt.split())
        if not stmt:
            continue
        m = re.match(r"((?:const )?\w+\*?)\s+(.*)", stmt)
        ty, names = m.group(1), [n.strip() for n in m.group(2).split(",")]
        for n in names:
            fields.append((n, ctype[ty]))
    assert fields == [(n, t) for n, t in capi.QkRopeParams._fields_]
    assert C.sizeof(capi.QkRopeParams) == 10 * 8 + 8 + 4 * 4 + 4 * 8 + 4 + 3 * 4


def test_enums_match_header_and_gguf_ids():
    for name, val in re.findall(r"(LOKAL_(?:ERR_)?\w+) = (\d+)", HEADER):
        if name.startswith("LOKAL_ERR") or name == "LOKAL_OK":
            assert getattr(capi, name[len("LOKAL_"):]) == int(val)
    assert (capi.F32, capi.F16, capi.Q8_0, capi.Q4_K, capi.BF16) == (0, 1, 8, 12, 30)  # src/gguf/dequant.rs:21-41
    for name, val in re.findall(r"LOKAL_(I?Q\d\w+) = (\d+)", HEADER):
        assert getattr(capi, name) == int(val) and int(val) in capi.QUANT_TYPES + capi.GRID_TYPES
    assert len(capi.QUANT_TYPES) == 10 and len(capi.GRID_TYPES) == 7
    grids = dict(re.findall(r"LOKAL_GRID_(\w+) = (\d+)", HEADER))
    assert [k.lower() for k, v in sorted(grids.items(), key=lambda kv: int(kv[1]))] == list(capi.GRID_ORDER)


def test_block_geometry_matches_reference_table():
    # src/gguf/dequant.rs:567-577
    assert lokal_b200.blk_bytes(capi.Q8_0) == 34 and lokal_b200.blk_bytes(capi.Q4_K) == 144
    assert lokal_b200.blk_elems(capi.Q8_0) == 32 and lokal_b200.blk_elems(capi.Q4_K) == 256
    assert lokal_b200.row_bytes(capi.Q4_K, 512) == 288 and lokal_b200.row_bytes(capi.Q8_0, 896) == 952
    assert lokal_b200.row_bytes(capi.F16, 10) == 20 and lokal_b200.row_bytes(capi.BF16, 10) == 20
    want = {2: (32, 18), 6: (32, 22), 8: (32, 34), 10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176),
            14: (256, 210), 20: (32, 18), 23: (256, 136)}
    for ty, geom in want.items():
        assert (lokal_b200.blk_elems(ty), lokal_b200.blk_bytes(ty)) == geom
    grid_types = {16: 66, 17: 74, 18: 98, 19: 50, 21: 110, 22: 82, 29: 56}  # the codebook types
    for ty, bb in grid_types.items():
        assert (lokal_b200.blk_elems(ty), lokal_b200.blk_bytes(ty)) == (256, bb)
    for ty in (3, 7, 9, 15, 24, 28):  # Q4_1, Q5_1, Q8_1, Q8_K, I8, F64: refused by the reference too (src/gguf/dequant.rs:58-76)
        assert lokal_b200.blk_elems(ty) == 0 and lokal_b200.row_bytes(ty, 256) == 0


def test_shard_rows_partitions_every_row_once():
    for n_rows in (0, 1, 7, 8, 255, 256, 8192, 65536):
        for g in (1, 2, 3, 4, 8):
            spans = [lokal_b200.shard_rows(n_rows, g, r) for r in range(g)]
            assert sum(c for _, c in spans) == n_rows
            pos = 0
            for r0, c in spans:
                assert r0 == pos or c == 0
                pos += c
            assert max(c for _, c in spans) - min(c for _, c in spans) <= -(-n_rows // g)
    assert lokal_b200.shard_rows(8192, 8, 3) == (3072, 1024)
    with pytest.raises(lokal_b200.LokalCudaError):
        lokal_b200.shard_rows(10, 0, 0)
    with pytest.raises(lokal_b200.LokalCudaError):
        lokal_b200.shard_rows(10, 2, 2)


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    assert capi.load().lokal_cuda_device_count() == 0
    with pytest.raises(lokal_b200.LokalCudaError) as e:
        lokal_b200.Context(0)
    assert e.value.status == capi.ERR_NO_DEVICE


def test_null_context_is_refused_not_dereferenced():
    lib = capi.load()
    assert lib.lokal_cuda_stream_sync(None, None) == capi.ERR_BAD_ARG
    assert lib.lokal_cuda_swiglu(None, None, None, None, None, None, 0, 0, 0) == capi.ERR_BAD_ARG
    assert lib.lokal_cuda_last_error(None) == b"null context"
    assert b"sm_100a" in lib.lokal_cuda_version()


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "lokal_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("lm_dequant_oracle", ""), f"{f} mentions the oracle"


def test_header_is_plain_c_and_links_from_c(tmp_path):
    """The boundary is a C ABI: a C99 translation unit includes the header, links the library and calls the
    host-only entry points (no GPU needed), the way a cgo / bindgen / FFI consumer would."""
    import shutil
    import subprocess
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    capi.load()
    src = tmp_path / "use_abi.c"
    src.write_text(r'''
#include <stdio.h>
#include <string.h>
#include "lokal_cuda.h"
int main(void) {
    lokal_kv_layout lay;
    lokal_qk_rope_params p;
    size_t row0 = 0, count = 0;
    memset(&p, 0, sizeof p);
    if (lokal_cuda_blk_bytes(LOKAL_Q6_K) != 210 || lokal_cuda_row_bytes(LOKAL_Q8_0, 896) != 952) return 1;
    if (lokal_cuda_window_cfg(1024, 4, 512, &lay) != LOKAL_OK || lay.ring != 1536 || lokal_cuda_window_slot_of(&lay, 5) != 129) return 2;
    if (lokal_cuda_shard_rows(8192, 8, 3, &row0, &count) != LOKAL_OK || row0 != 3072 || count != 1024) return 3;
    if (lokal_cuda_stream_sync(NULL, NULL) != LOKAL_ERR_BAD_ARG) return 4;
    {
        lokal_gguf* g = NULL;
        char err[256];
        if (lokal_gguf_open("/nonexistent.gguf", &g, err, sizeof err) != LOKAL_ERR_IO || g != NULL || !strstr(err, "cannot open")) return 5;
    }
    printf("%s %zu\n", lokal_cuda_version(), sizeof p);
    return 0;
}
''')
    exe = tmp_path / "use_abi"
    libdir = os.path.dirname(capi.library_path())
    subprocess.run([cc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", libdir, "-llokal_cuda", f"-Wl,-rpath,{libdir}"], check=True, capture_output=True, text=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0, (res.returncode, res.stdout, res.stderr)
    assert "sm_100a" in res.stdout and res.stdout.split()[-1] == str(C.sizeof(capi.QkRopeParams))
