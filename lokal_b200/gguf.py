"""GgufFile: the ctypes handle over the library's GGUF container reader (lokal_gguf_*), named after the reference's
gguf::GgufFile (src/gguf/container.rs:152-384) and with its accessors: open / n_tensors / tensors / tensor /
get_usize / get_f32 / get_str / get_arr_str / get_arr_i64 / has_key. All parsing happens in the C++ library."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import capi
from .capi import GgufTensor, LokalCudaError


@dataclass
class Tensor:
    name: str
    dims: tuple[int, ...]   # row-major
    ggml_type: int
    data_offset: int
    nbytes: int
    data: np.ndarray        # uint8 view into the mapping; valid until the file is closed


class GgufFile:
    def __init__(self, path: str):
        self._lib = capi.load()
        h = C.c_void_p()
        err = C.create_string_buffer(2048)
        rc = self._lib.lokal_gguf_open(str(path).encode(), C.byref(h), err, len(err))
        if rc != capi.OK:
            raise LokalCudaError(rc, err.value.decode(errors="replace"))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            self._lib.lokal_gguf_close(self._h)
            self._h = None

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _check(self, rc):
        if rc != capi.OK:
            raise LokalCudaError(rc, self._lib.lokal_gguf_last_error(self._h).decode(errors="replace"))

    @property
    def handle(self):
        return self._h

    @property
    def version(self) -> int:
        return int(self._lib.lokal_gguf_version(self._h))

    @property
    def data_start(self) -> int:
        return int(self._lib.lokal_gguf_data_start(self._h))

    def n_tensors(self) -> int:
        return int(self._lib.lokal_gguf_n_tensors(self._h))

    def _wrap(self, t: GgufTensor) -> Tensor:
        buf = (C.c_uint8 * t.nbytes).from_address(t.data) if t.nbytes else (C.c_uint8 * 0)()
        return Tensor(t.name.decode(errors="replace"), tuple(int(t.dims[i]) for i in range(t.n_dims)), int(t.ggml_type), int(t.data_offset),
                      int(t.nbytes), np.frombuffer(buf, np.uint8))

    def tensors(self):
        for i in range(self.n_tensors()):
            t = GgufTensor()
            self._check(self._lib.lokal_gguf_tensor_at(self._h, i, C.byref(t)))
            yield self._wrap(t)

    def tensor(self, name: str) -> Tensor:
        t = GgufTensor()
        self._check(self._lib.lokal_gguf_find_tensor(self._h, name.encode(), C.byref(t)))
        return self._wrap(t)

    def has_key(self, key: str) -> bool:
        return bool(self._lib.lokal_gguf_has_key(self._h, key.encode()))

    def get_usize(self, key: str) -> int:
        v = C.c_uint64()
        self._check(self._lib.lokal_gguf_get_u64(self._h, key.encode(), C.byref(v)))
        return int(v.value)

    def get_f32(self, key: str) -> float:
        v = C.c_float()
        self._check(self._lib.lokal_gguf_get_f32(self._h, key.encode(), C.byref(v)))
        return float(v.value)

    def get_str(self, key: str) -> str:
        p, n = C.c_char_p(), C.c_size_t()
        self._check(self._lib.lokal_gguf_get_str(self._h, key.encode(), C.byref(p), C.byref(n)))
        return C.string_at(p, n.value).decode(errors="replace")

    def get_arr_i64(self, key: str) -> list[int]:
        p, n = C.POINTER(C.c_int64)(), C.c_size_t()
        self._check(self._lib.lokal_gguf_get_arr_i64(self._h, key.encode(), C.byref(p), C.byref(n)))
        return [int(p[i]) for i in range(n.value)]

    def get_arr_str(self, key: str) -> list[str]:
        p, n = C.POINTER(C.c_char_p)(), C.c_size_t()
        self._check(self._lib.lokal_gguf_get_arr_str(self._h, key.encode(), C.byref(p), C.byref(n)))
        return [p[i].decode(errors="replace") for i in range(n.value)]
