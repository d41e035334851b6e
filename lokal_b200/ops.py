"""Host-side handle over the C ABI, named after the reference's ops.

`Context` owns one `lokal_cuda_ctx` (one per GPU). Device buffers are passed
as anything with a ``data_ptr()`` (torch tensors are used by the tests and the
benchmark purely as device allocations) or as raw integer addresses. Every
method forwards to exactly one C entry point; errors come back as
`LokalCudaError` carrying the library's status code and message. Nothing here
computes on the CPU.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi
from .capi import BF16, F16, F32, Q4_K, Q8_0, KvLayout, LokalCudaError, PassConfig, PassInputs, PassWeights, QkRopeParams


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    raise TypeError(f"cannot take the address of {type(x)!r}")


_TORCH_TYPES = None


def dtype_id(x) -> int:
    """lokal_type of a torch tensor's dtype."""
    global _TORCH_TYPES
    if _TORCH_TYPES is None:
        import torch
        _TORCH_TYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}
    return _TORCH_TYPES[x.dtype]


class Context:
    def __init__(self, device: int = 0):
        self._lib = capi.load()
        h = C.c_void_p()
        rc = self._lib.lokal_cuda_create(device, C.byref(h))
        if rc != capi.OK:
            raise LokalCudaError(rc, f"lokal_cuda_create(device={device}) failed")
        self._h = h
        self.device = device

    # -- plumbing ---------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self._lib.lokal_cuda_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def handle(self):
        return self._h

    def _check(self, rc: int):
        if rc != capi.OK:
            raise LokalCudaError(rc, self._lib.lokal_cuda_last_error(self._h).decode())

    def version(self) -> str:
        return self._lib.lokal_cuda_version().decode()

    def stream_create(self) -> int:
        s = C.c_void_p()
        self._check(self._lib.lokal_cuda_stream_create(self._h, C.byref(s)))
        return s.value

    def stream_destroy(self, s):
        self._check(self._lib.lokal_cuda_stream_destroy(self._h, s))

    def stream_sync(self, s=None):
        self._check(self._lib.lokal_cuda_stream_sync(self._h, s))

    def malloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self._check(self._lib.lokal_cuda_malloc(self._h, nbytes, C.byref(p)))
        return p.value or 0

    def free(self, p):
        self._check(self._lib.lokal_cuda_free(self._h, p))

    def set_iq_grids(self, grids) -> None:
        """Hands the i-quant codebooks to the library (a mapping with the keys of capi.GRID_ORDER: iq2xxs, iq2xs, iq2s
        as uint64, iq3xxs, iq3s as uint32, iq1s as uint64). They are data of the file format kept by the host
        application (src/lowmem/iq_grids.rs in the reference); the library carries no copy."""
        for which, key in enumerate(capi.GRID_ORDER):
            if key in grids:
                a = np.ascontiguousarray(grids[key])
                self._check(self._lib.lokal_cuda_set_iq_grid(self._h, which, _ptr(a), a.nbytes))

    def gguf_upload(self, gguf, name: str, stream=None):
        """One tensor of an open GgufFile copied into a fresh device allocation: (device pointer, GgufTensor)."""
        p, info = C.c_void_p(), capi.GgufTensor()
        self._check(self._lib.lokal_cuda_gguf_upload(self._h, stream, gguf.handle, name.encode(), C.byref(p), C.byref(info)))
        return p.value or 0, info

    def host_alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self._check(self._lib.lokal_cuda_host_alloc(self._h, nbytes, C.byref(p)))
        return p.value or 0

    def host_free(self, p):
        self._check(self._lib.lokal_cuda_host_free(self._h, p))

    def memcpy_h2d(self, dst, src, nbytes: int, stream=None):
        self._check(self._lib.lokal_cuda_memcpy_h2d(self._h, stream, _ptr(dst), _ptr(src), nbytes))

    def memcpy_d2h(self, dst, src, nbytes: int, stream=None):
        self._check(self._lib.lokal_cuda_memcpy_d2h(self._h, stream, _ptr(dst), _ptr(src), nbytes))

    def graph_begin(self, stream):
        self._check(self._lib.lokal_cuda_graph_begin(self._h, stream))

    def graph_end(self, stream) -> int:
        g = C.c_void_p()
        self._check(self._lib.lokal_cuda_graph_end(self._h, stream, C.byref(g)))
        return g.value

    def graph_launch(self, graph, stream):
        self._check(self._lib.lokal_cuda_graph_launch(self._h, graph, stream))

    def graph_destroy(self, graph):
        self._check(self._lib.lokal_cuda_graph_destroy(self._h, graph))

    # -- ops on device memory ------------------------------------------------
    def rmsnorm(self, x, w, y, *, rows, dim, eps, dtype, w_dtype=F32, y_h=None, h_dtype=F16, stream=None):
        self._check(self._lib.lokal_cuda_rmsnorm(self._h, stream, _ptr(x), _ptr(w), _ptr(y), _ptr(y_h), rows, dim,
                                                 eps, dtype, w_dtype, h_dtype))

    def add_rmsnorm(self, x_inout, delta, w, xn, *, rows, dim, eps, dtype, w_dtype=F32, xn_h=None, h_dtype=F16,
                    stream=None):
        self._check(self._lib.lokal_cuda_add_rmsnorm(self._h, stream, _ptr(x_inout), _ptr(delta), _ptr(w), _ptr(xn),
                                                     _ptr(xn_h), rows, dim, eps, dtype, w_dtype, h_dtype))

    def rope_table(self, cos_sin, *, theta, rot_dim, rows, positions=None, pos0=0, stream=None):
        self._check(self._lib.lokal_cuda_rope_table(self._h, stream, theta, rot_dim, _ptr(positions), pos0, rows,
                                                    _ptr(cos_sin)))

    @staticmethod
    def qk_rope_params(*, q=None, k=None, q_out=None, k_out=None, q_bias=None, k_bias=None, q_norm_w=None,
                       k_norm_w=None, cos_sin=None, k_out_rows=None, rows, n_q_heads, n_kv_heads, head_dim,
                       rot_dim=None, q_row_stride=None, k_row_stride=None, q_out_row_stride=None,
                       k_out_row_stride=None, eps=0.0, q_dtype=F32, k_dtype=None, w_dtype=F32) -> QkRopeParams:
        p = QkRopeParams()
        p.q, p.k, p.q_out, p.k_out = _ptr(q), _ptr(k), _ptr(q_out), _ptr(k_out)
        p.q_bias, p.k_bias, p.q_norm_w, p.k_norm_w = _ptr(q_bias), _ptr(k_bias), _ptr(q_norm_w), _ptr(k_norm_w)
        p.cos_sin, p.k_out_rows = _ptr(cos_sin), _ptr(k_out_rows)
        p.rows = rows
        p.n_q_heads, p.n_kv_heads, p.head_dim = n_q_heads, n_kv_heads, head_dim
        p.rot_dim = head_dim if rot_dim is None else rot_dim
        p.q_row_stride = n_q_heads * head_dim if q_row_stride is None else q_row_stride
        p.k_row_stride = n_kv_heads * head_dim if k_row_stride is None else k_row_stride
        p.q_out_row_stride = p.q_row_stride if q_out_row_stride is None else q_out_row_stride
        p.k_out_row_stride = p.k_row_stride if k_out_row_stride is None else k_out_row_stride
        p.eps = eps
        p.q_dtype = q_dtype
        p.k_dtype = q_dtype if k_dtype is None else k_dtype
        p.w_dtype = w_dtype
        return p

    def qk_rope(self, params: QkRopeParams, stream=None):
        self._check(self._lib.lokal_cuda_qk_rope(self._h, stream, C.byref(params)))

    def qk_rope_pos(self, params: QkRopeParams, *, theta, positions=None, pos0=0, stream=None):
        self._check(self._lib.lokal_cuda_qk_rope_pos(self._h, stream, C.byref(params), theta, _ptr(positions), pos0))

    def qk_rope_pos_noalloc(self, params: QkRopeParams, *, theta, positions=None, pos0=0, stream=None):
        """qk_rope_pos for callers that must not allocate on this path (a decode loop that cannot stall on
        cudaMalloc, an engine whose KV pool already owns the rest of HBM). The cos/sin table sits in a fixed
        LOKAL_NOALLOC_TABLE_BYTES array inside the library, so rows * rot_dim * 4 must fit in it; calls that
        overlap on one GPU share (and race on) that array. Make the first call on a GPU outside stream capture."""
        self._check(self._lib.lokal_cuda_qk_rope_pos_noalloc(self._h, stream, C.byref(params), theta, _ptr(positions),
                                                             pos0))

    def swiglu(self, gate, up, out, *, n, dtype, out_h=None, h_dtype=F16, stream=None):
        self._check(self._lib.lokal_cuda_swiglu(self._h, stream, _ptr(gate), _ptr(up), _ptr(out), _ptr(out_h), n,
                                                dtype, h_dtype))

    def embed_gather(self, table, ids, out, *, ggml_type, vocab, dim, n, out_dtype=F32, stream=None):
        self._check(self._lib.lokal_cuda_embed_gather(self._h, stream, _ptr(table), ggml_type, vocab, dim, _ptr(ids),
                                                      n, _ptr(out), out_dtype))

    def embed_gather_rmsnorm(self, table, ids, x, xn, w, *, ggml_type, vocab, dim, n, eps, out_dtype=F32, w_dtype=F32, stream=None):
        """x[i] = dequant(table[ids[i]]), xn[i] = rmsnorm(x[i], w, eps): one launch for a quantised table."""
        self._check(self._lib.lokal_cuda_embed_gather_rmsnorm(self._h, stream, _ptr(table), ggml_type, vocab, dim, _ptr(ids), n,
                                                               _ptr(x), _ptr(xn), _ptr(w), eps, out_dtype, w_dtype))

    def dequant_rows(self, src, out, *, ggml_type, rows, cols, out_dtype=F32, stream=None):
        self._check(self._lib.lokal_cuda_dequant_rows(self._h, stream, ggml_type, _ptr(src), rows, cols, _ptr(out),
                                                      out_dtype))

    def kv_rows(self, rows_out, *, layout: KvLayout, rows, positions=None, pos0=0, slots=None, slot0=0, stream=None):
        """Cache row of every token row (linear slot*max_seq+pos, or sink + ring) into a device uint32 array."""
        self._check(self._lib.lokal_cuda_kv_rows(self._h, stream, C.byref(layout), _ptr(positions), pos0, _ptr(slots),
                                                 slot0, rows, _ptr(rows_out)))

    def kv_stage(self, src, dst, *, src_dtype, dst_dtype, rows, width, src_row_stride=None, dst_row_stride=None,
                 dst_rows=None, stream=None):
        """dst[dst_rows[r]] = narrow(src[r]): fresh K/V rows into their cache rows."""
        self._check(self._lib.lokal_cuda_kv_stage(self._h, stream, _ptr(src), src_dtype,
                                                  width if src_row_stride is None else src_row_stride, _ptr(dst),
                                                  dst_dtype, width if dst_row_stride is None else dst_row_stride,
                                                  _ptr(dst_rows), rows, width))

    # -- per-row siblings in the gated-deltanet blocks ------------------------------
    def l2norm_rows(self, x, y=None, *, dim, eps, rows_per_token, n_tokens=1, tok_stride=0, dtype=F32, stream=None):
        """deltanet_ref::l2_norm over rows: y = x / max(sqrt(sum x^2), eps); in place when y is None."""
        self._check(self._lib.lokal_cuda_l2norm_rows(self._h, stream, _ptr(x), _ptr(x if y is None else y), rows_per_token,
                                                     n_tokens, tok_stride, dim, eps, dtype))

    def gated_output_norm(self, o, w, z, y=None, *, rows, dim, eps, dtype=F32, w_dtype=F32, stream=None):
        """deltanet_ref::gated_output_norm: per row rmsnorm(o; w) * silu(z); in place when y is None."""
        self._check(self._lib.lokal_cuda_gated_output_norm(self._h, stream, _ptr(o), _ptr(w), _ptr(z), _ptr(o if y is None else y),
                                                           rows, dim, eps, dtype, w_dtype))

    def attn_out_gate(self, attn, gate, out=None, *, n, dtype=F32, stream=None):
        """deltanet_ref::attn_out_gate: attn * sigmoid(gate); in place when out is None."""
        self._check(self._lib.lokal_cuda_attn_out_gate(self._h, stream, _ptr(attn), _ptr(gate), _ptr(attn if out is None else out), n, dtype))

    def split_q_gate(self, src, q, gate, *, rows, n_heads, head_dim, dtype=F32, stream=None):
        """[q | gate] per head -> compact q and gate."""
        self._check(self._lib.lokal_cuda_split_q_gate(self._h, stream, _ptr(src), _ptr(q), _ptr(gate), rows, n_heads, head_dim, dtype))

    def delta_gates(self, alpha, beta_in, a, dt_bias, g, beta, *, n_v_heads, n_tokens, stream=None):
        """deltanet_ref::delta_gate / sigmoid per (token, V head): g = a * softplus(alpha + dt_bias), beta = sigmoid(beta_in)."""
        self._check(self._lib.lokal_cuda_delta_gates(self._h, stream, _ptr(alpha), _ptr(beta_in), _ptr(a), _ptr(dt_bias), _ptr(g), _ptr(beta),
                                                     n_v_heads, n_tokens))

    def ssm_conv(self, state, x, w, out, *, channels, d_conv, n_tokens, dtype=F32, roll=True, stream=None):
        """deltanet_ref::conv_step over n_tokens rows: depthwise causal conv + SiLU; `state` rolls when roll is set."""
        self._check(self._lib.lokal_cuda_ssm_conv(self._h, stream, _ptr(state), _ptr(x), _ptr(w), _ptr(out), channels, d_conv, n_tokens, dtype,
                                                  1 if roll else 0))

    def bf16_to_f16_copy(self, src, dst, *, n, clip_flag=None, stream=None):
        """bf16 bits -> f16 (nearest even); clip_flag (device u32) is OR-ed with 1 when a finite value overflows."""
        self._check(self._lib.lokal_cuda_bf16_to_f16_copy(self._h, stream, _ptr(src), _ptr(dst), n, _ptr(clip_flag)))

    # -- host-slice mirrors of the reference's CPU signatures ----------------------
    def host_rmsnorm(self, x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
        """math::rmsnorm(x, weight, eps) -> new vector; x may be [dim] or [rows, dim]."""
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        rows, dim = (1, x.shape[0]) if x.ndim == 1 else x.shape
        if w.size != dim:
            raise ValueError("weight length differs from the row length")
        y = np.empty_like(x)
        self._check(self._lib.lokal_cuda_host_rmsnorm(self._h, _ptr(x), _ptr(w), eps, rows, dim, _ptr(y)))
        return y

    def host_rope(self, x: np.ndarray, pos: int, head_dim: int, theta: float) -> np.ndarray:
        """model::rope(x, pos, head_dim, theta), returned as a rotated copy."""
        x = np.ascontiguousarray(x, np.float32).copy()
        self._check(self._lib.lokal_cuda_host_rope(self._h, _ptr(x), x.size, pos, head_dim, theta))
        return x

    def host_swiglu(self, gate: np.ndarray, up: np.ndarray) -> np.ndarray:
        gate = np.ascontiguousarray(gate, np.float32)
        up = np.ascontiguousarray(up, np.float32)
        if gate.size != up.size:
            raise ValueError("gate and up differ in length")
        out = np.empty_like(gate)
        self._check(self._lib.lokal_cuda_host_swiglu(self._h, _ptr(gate), _ptr(up), gate.size, _ptr(out)))
        return out

    def host_dequant_row(self, ggml_type: int, src: np.ndarray, n: int) -> np.ndarray:
        """gguf::dequant_row_ref(ty, src, out[n])."""
        src = np.ascontiguousarray(src, np.uint8)
        out = np.empty(n, np.float32)
        self._check(self._lib.lokal_cuda_host_dequant_row(self._h, ggml_type, _ptr(src), src.size, _ptr(out), n))
        return out

    def host_embed_gather(self, table_dev, ggml_type: int, vocab: int, dim: int, ids: np.ndarray, out: np.ndarray | None = None) -> np.ndarray:
        """Host ids in, host f32 rows out. `out` may be a caller-owned array (page-locked memory is written by DMA)."""
        ids = np.ascontiguousarray(ids, np.uint32)
        if out is None:
            out = np.empty((ids.size, dim), np.float32)
        assert out.dtype == np.float32 and out.flags.c_contiguous and out.size == ids.size * dim
        self._check(self._lib.lokal_cuda_host_embed_gather(self._h, _ptr(table_dev), ggml_type, vocab, dim, _ptr(ids),
                                                           ids.size, _ptr(out)))
        return out


class LayerPass:
    """One `lokal_cuda_pass`: the per-token ops of a forward step strung together layer by layer.

    Weights (host numpy arrays) are uploaded once at construction; `run_device` launches a step on
    device-resident inputs, `run_host` takes host inputs and returns when the result is in host memory.
    """

    def __init__(self, ctx: Context, *, max_rows, layers, hidden, inter, n_q_heads, n_kv_heads, head_dim, eps, theta,
                 dtype, w_dtype, embed_type, vocab, embed_table, norm_w, final_w, q_bias=None, k_bias=None,
                 q_norm_w=None, k_norm_w=None, rot_dim=None, slots=None):
        self.ctx = ctx
        cfg = PassConfig(max_rows=max_rows, layers=layers, hidden=hidden, inter=inter, n_q_heads=n_q_heads,
                         n_kv_heads=n_kv_heads, head_dim=head_dim, rot_dim=head_dim if rot_dim is None else rot_dim,
                         eps=eps, theta=theta, dtype=dtype, w_dtype=w_dtype, has_qk_bias=int(q_bias is not None),
                         has_qk_norm=int(q_norm_w is not None), embed_type=embed_type,
                         slots=layers if slots is None else slots, vocab=vocab)
        w = PassWeights(embed_table=_ptr(embed_table), norm_w=_ptr(norm_w), final_w=_ptr(final_w), q_bias=_ptr(q_bias),
                        k_bias=_ptr(k_bias), q_norm_w=_ptr(q_norm_w), k_norm_w=_ptr(k_norm_w))
        h = C.c_void_p()
        ctx._check(ctx._lib.lokal_cuda_pass_create(ctx._h, C.byref(cfg), C.byref(w), C.byref(h)))
        self._h = h
        self.cfg = cfg

    def close(self):
        if getattr(self, "_h", None) and self.ctx._h:
            self.ctx._lib.lokal_cuda_pass_destroy(self.ctx._h, self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def inputs(*, ids, rows, q, k, delta_att, delta_mlp, gate, up, q_layer_stride, k_layer_stride, delta_layer_stride,
               mlp_layer_stride, positions=None, pos0=0) -> PassInputs:
        return PassInputs(ids=_ptr(ids), positions=_ptr(positions), pos0=pos0, rows=rows, q=_ptr(q), k=_ptr(k),
                          delta_att=_ptr(delta_att), delta_mlp=_ptr(delta_mlp), gate=_ptr(gate), up=_ptr(up),
                          q_layer_stride=q_layer_stride, k_layer_stride=k_layer_stride,
                          delta_layer_stride=delta_layer_stride, mlp_layer_stride=mlp_layer_stride)

    def run_device(self, inputs: PassInputs, out_dev, stream=None):
        self.ctx._check(self.ctx._lib.lokal_cuda_pass_run_device(self.ctx._h, self._h, stream, C.byref(inputs), _ptr(out_dev)))

    def run_host(self, inputs: PassInputs, out_host):
        self.ctx._check(self.ctx._lib.lokal_cuda_pass_run_host(self.ctx._h, self._h, C.byref(inputs), _ptr(out_host)))

    def set_schedule(self, schedule: int):
        """capi.PASS_SCHEDULE_AUTO / _SEQUENTIAL / _BRANCHES: how run_device orders the kernels of a step."""
        self.ctx._check(self.ctx._lib.lokal_cuda_pass_set_schedule(self.ctx._h, self._h, schedule))

    def output(self, layer: int, which: int) -> int:
        p = C.c_void_p()
        self.ctx._check(self.ctx._lib.lokal_cuda_pass_output(self.ctx._h, self._h, layer, which, C.byref(p)))
        return p.value or 0

    @property
    def launches(self) -> int:
        return int(self.ctx._lib.lokal_cuda_pass_launches(self._h))


def blk_elems(ggml_type: int) -> int:
    return capi.load().lokal_cuda_blk_elems(ggml_type)


def blk_bytes(ggml_type: int) -> int:
    return capi.load().lokal_cuda_blk_bytes(ggml_type)


def row_bytes(ggml_type: int, n: int) -> int:
    return capi.load().lokal_cuda_row_bytes(ggml_type, n)


def window_cfg(window: int, sink: int, prefill_chunk: int = 512) -> KvLayout:
    """WindowCfg::new: sink region padded to 128 rows, ring = window + one prefill chunk, rounded up to 128."""
    lay = KvLayout()
    rc = capi.load().lokal_cuda_window_cfg(window, sink, prefill_chunk, C.byref(lay))
    if rc != capi.OK:
        raise LokalCudaError(rc, f"invalid window config: window {window}, sink {sink}")
    return lay


def window_slot_of(layout: KvLayout, p: int) -> int:
    return int(capi.load().lokal_cuda_window_slot_of(C.byref(layout), p))


def window_write_spans(layout: KvLayout, pos0: int, n: int) -> list[tuple[int, int, int]]:
    buf = (C.c_uint64 * 9)()
    cnt = capi.load().lokal_cuda_window_write_spans(C.byref(layout), pos0, n, buf)
    if cnt < 0:
        raise LokalCudaError(capi.ERR_BAD_ARG, "chunk does not fit three spans (longer than the ring) or layout is linear")
    return [(int(buf[3 * i]), int(buf[3 * i + 1]), int(buf[3 * i + 2])) for i in range(cnt)]


def shard_rows(n_rows: int, n_gpus: int, rank: int) -> tuple[int, int]:
    """Contiguous row block [row0, row0+count) that GPU `rank` of `n_gpus` owns."""
    r0, cnt = C.c_size_t(), C.c_size_t()
    rc = capi.load().lokal_cuda_shard_rows(n_rows, n_gpus, rank, C.byref(r0), C.byref(cnt))
    if rc != capi.OK:
        raise LokalCudaError(rc, f"shard_rows({n_rows}, {n_gpus}, {rank})")
    return r0.value, cnt.value
