"""Writes tests/golden/iq_grids.npz: the i-quant codebooks the IQ1/IQ2/IQ3 row decoders index.

The codebooks are fitted tables, not formulas; the reference keeps them as data (src/lowmem/iq_grids.rs, emitted by
its benchmarks/extract_grids.py from ggml-common.h). The library never embeds them: a host application hands its own
tables to lokal_cuda_set_iq_grid. The tests need real values, so this script reads the numbers out of the
reference's data file (run where the reference tree is present), checks lengths and the wrapping checksums the
reference's own test holds (src/lowmem/iq_grids.rs:584-603), and stores them as a binary fixture.

    python tests/golden/make_iq_grids.py path/to/reference
"""
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
TABLES = {  # name in the data file -> (fixture key, dtype, length, wrapping sum)
    "KSIGNS_IQ2XS": ("ksigns", np.uint8, 128, 16320),
    "IQ2XXS_GRID": ("iq2xxs", np.uint64, 256, 10026840302681211747),
    "IQ2XS_GRID": ("iq2xs", np.uint64, 512, 3032300602630837921),
    "IQ2S_GRID": ("iq2s", np.uint64, 1024, 8502338067238609906),
    "IQ3XXS_GRID": ("iq3xxs", np.uint32, 256, 108356387642),
    "IQ3S_GRID": ("iq3s", np.uint32, 512, 53294177878),
    "IQ1S_GRID": ("iq1s", np.uint64, 2048, 7590341501443526924),
}


def wrapping_sum(a):
    return int(sum(int(v) for v in a) % (1 << 64))


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    ref = sys.argv[1]
    text = open(os.path.join(ref, "src", "lowmem", "iq_grids.rs")).read()
    out = {}
    for name, (key, dtype, n, checksum) in TABLES.items():
        m = re.search(r"const %s: \[\w+; (\d+)\] = \[(.*?)\];" % name, text, re.S)
        assert m and int(m.group(1)) == n, name
        vals = [int(v, 0) for v in re.findall(r"0x[0-9a-fA-F]+|\d+", m.group(2))]
        arr = np.array(vals, dtype=dtype)
        assert arr.size == n and wrapping_sum(arr) == checksum, (name, arr.size, wrapping_sum(arr))
        out[key] = arr
    path = os.path.join(HERE, "iq_grids.npz")
    np.savez_compressed(path, **out)
    print(path, {k: v.shape for k, v in out.items()}, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
