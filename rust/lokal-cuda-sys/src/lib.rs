//! Raw bindings of `liblokal_cuda.so`: lokal's fused per-token layer ops on NVIDIA B200 (sm_100a).
//!
//! One declaration here for every declaration of `include/lokal_cuda.h`, in the header's order: the status and type
//! codes, the `#[repr(C)]` mirrors of its structs, and its functions. The mirror is guarded the way lokal guards
//! its Metal parameter structs (src/gpu/metal.rs:4448-4589): a test reads the C header and this file as text and
//! requires every struct to agree field for field and every function argument for argument. Change the header and
//! this file together.
//!
//! Everything here is `unsafe` to call; `src/gpu/cuda.rs` in the lokal tree wraps it behind `Engine` / `Session` /
//! `Batcher`. Link with `cargo:rustc-link-lib=dylib=lokal_cuda` (see build.rs).
#![allow(non_camel_case_types, clippy::too_many_arguments)]

use std::os::raw::{c_char, c_int, c_void};

// ---- lokal_status ----
pub const LOKAL_OK: c_int = 0;
pub const LOKAL_ERR_BAD_ARG: c_int = 1;
pub const LOKAL_ERR_UNSUPPORTED: c_int = 2;
pub const LOKAL_ERR_MISALIGNED: c_int = 3;
pub const LOKAL_ERR_CUDA: c_int = 4;
pub const LOKAL_ERR_ID_RANGE: c_int = 5;
pub const LOKAL_ERR_TIMEOUT: c_int = 6;
pub const LOKAL_ERR_NO_DEVICE: c_int = 7;
pub const LOKAL_ERR_IO: c_int = 8;
pub const LOKAL_ERR_FORMAT: c_int = 9;
pub const LOKAL_ERR_NOT_FOUND: c_int = 10;
pub const LOKAL_ERR_POS_RANGE: c_int = 11;

// ---- lokal_type: the GgmlType discriminants (src/gguf/dequant.rs:21-41), so `ty as c_int` of a GgmlType works ----
pub const LOKAL_F32: c_int = 0;
pub const LOKAL_F16: c_int = 1;
pub const LOKAL_Q4_0: c_int = 2;
pub const LOKAL_Q5_0: c_int = 6;
pub const LOKAL_Q8_0: c_int = 8;
pub const LOKAL_Q2_K: c_int = 10;
pub const LOKAL_Q3_K: c_int = 11;
pub const LOKAL_Q4_K: c_int = 12;
pub const LOKAL_Q5_K: c_int = 13;
pub const LOKAL_Q6_K: c_int = 14;
pub const LOKAL_IQ2_XXS: c_int = 16;
pub const LOKAL_IQ2_XS: c_int = 17;
pub const LOKAL_IQ3_XXS: c_int = 18;
pub const LOKAL_IQ1_S: c_int = 19;
pub const LOKAL_IQ4_NL: c_int = 20;
pub const LOKAL_IQ3_S: c_int = 21;
pub const LOKAL_IQ2_S: c_int = 22;
pub const LOKAL_IQ4_XS: c_int = 23;
pub const LOKAL_IQ1_M: c_int = 29;
pub const LOKAL_BF16: c_int = 30;

// ---- lokal_iq_grid: which codebook lokal_cuda_set_iq_grid receives (src/lowmem/iq_grids.rs) ----
pub const LOKAL_GRID_IQ2XXS: c_int = 0;
pub const LOKAL_GRID_IQ2XS: c_int = 1;
pub const LOKAL_GRID_IQ2S: c_int = 2;
pub const LOKAL_GRID_IQ3XXS: c_int = 3;
pub const LOKAL_GRID_IQ3S: c_int = 4;
pub const LOKAL_GRID_IQ1S: c_int = 5;

/// Bytes of the built-in cos/sin table of `lokal_cuda_qk_rope_pos_noalloc` (rows * rot_dim * 4 must fit).
pub const LOKAL_NOALLOC_TABLE_BYTES: u32 = 1 << 20;

/// Cache row that `lokal_cuda_kv_rows` gives a position the cache cannot hold; consumers store nothing for it.
pub const LOKAL_KV_ROW_NONE: u32 = 0xFFFFFFFF;

// ---- lokal_cuda_pass_set_schedule ----
pub const LOKAL_PASS_SCHEDULE_AUTO: c_int = 0;
pub const LOKAL_PASS_SCHEDULE_SEQUENTIAL: c_int = 1;
pub const LOKAL_PASS_SCHEDULE_BRANCHES: c_int = 3;

// ---- opaque handles ----
/// `lokal_cuda_ctx`: one per device; immutable after creation, so it may be shared across threads (`Engine: Send + Sync`).
#[repr(C)]
pub struct LokalCudaCtx {
    _opaque: [u8; 0],
}
/// `lokal_cuda_graph`: a captured and instantiated step.
#[repr(C)]
pub struct LokalCudaGraph {
    _opaque: [u8; 0],
}
/// `lokal_gguf`: an opened, memory-mapped GGUF file.
#[repr(C)]
pub struct LokalGguf {
    _opaque: [u8; 0],
}
/// `lokal_cuda_pass`: the layer-pass runner.
#[repr(C)]
pub struct LokalCudaPass {
    _opaque: [u8; 0],
}
/// `lokal_cuda_stream`: a `cudaStream_t`; null is the default stream. One per `Session` / `Batcher`.
pub type LokalCudaStream = *mut c_void;

// ---- struct mirrors ----
/// `lokal_qk_rope_params`: one fused bias + per-head RMSNorm + rotation call. Head geometry is explicit
/// (`n_q_heads`, `n_kv_heads`, `head_dim`, `rot_dim`), never derived from the hidden size (src/lowmem/mod.rs:62-101).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct LokalQkRopeParams {
    pub q: *mut c_void,
    pub k: *mut c_void,
    pub q_out: *mut c_void,
    pub k_out: *mut c_void,
    pub q_bias: *const c_void,
    pub k_bias: *const c_void,
    pub q_norm_w: *const c_void,
    pub k_norm_w: *const c_void,
    pub cos_sin: *const f32,
    pub k_out_rows: *const u32,
    pub rows: u64,
    pub n_q_heads: u32,
    pub n_kv_heads: u32,
    pub head_dim: u32,
    pub rot_dim: u32,
    pub q_row_stride: u64,
    pub k_row_stride: u64,
    pub q_out_row_stride: u64,
    pub k_out_row_stride: u64,
    pub eps: f32,
    pub q_dtype: i32,
    pub k_dtype: i32,
    pub w_dtype: i32,
}

/// `lokal_kv_layout`: a KV cache of `max_seq` rows per slot, or (ring != 0) a sink + ring window (`WindowCfg`, src/lowmem/mod.rs:190-192).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct LokalKvLayout {
    pub max_seq: u64,
    pub sink: u64,
    pub sink_pad: u64,
    pub ring: u64,
}

/// `lokal_gguf_tensor`: one tensor of an opened GGUF file; `dims` are row-major after the `ne` reversal (src/gguf/container.rs:279-280).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct LokalGgufTensor {
    pub name: *const c_char,
    pub n_dims: u32,
    pub dims: [u64; 4],
    pub ggml_type: i32,
    pub file_offset: u64,
    pub data_offset: u64,
    pub nbytes: u64,
    pub data: *const c_void,
}

/// `lokal_pass_config`: shapes and types of the layer pass (`lokal_cuda_pass_*`).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct LokalPassConfig {
    pub max_rows: u64,
    pub layers: u32,
    pub hidden: u32,
    pub inter: u32,
    pub n_q_heads: u32,
    pub n_kv_heads: u32,
    pub head_dim: u32,
    pub rot_dim: u32,
    pub eps: f32,
    pub theta: f32,
    pub dtype: i32,
    pub w_dtype: i32,
    pub has_qk_bias: i32,
    pub has_qk_norm: i32,
    pub embed_type: i32,
    pub slots: u32,
    pub vocab: u64,
}

/// `lokal_pass_weights`: HOST pointers, copied to the device once at `lokal_cuda_pass_create`.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct LokalPassWeights {
    pub embed_table: *const c_void,
    pub norm_w: *const c_void,
    pub final_w: *const c_void,
    pub q_bias: *const c_void,
    pub k_bias: *const c_void,
    pub q_norm_w: *const c_void,
    pub k_norm_w: *const c_void,
}

/// `lokal_pass_inputs`: the projections' outputs of one step, `[layers][rows][width]` with strides in elements.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct LokalPassInputs {
    pub ids: *const u32,
    pub positions: *const i32,
    pub pos0: i64,
    pub rows: u64,
    pub q: *mut c_void,
    pub k: *mut c_void,
    pub delta_att: *const c_void,
    pub delta_mlp: *const c_void,
    pub gate: *const c_void,
    pub up: *const c_void,
    pub q_layer_stride: u64,
    pub k_layer_stride: u64,
    pub delta_layer_stride: u64,
    pub mlp_layer_stride: u64,
}

// ---- functions, in the header's order ----
extern "C" {
pub fn lokal_cuda_create(device: c_int, out: *mut *mut LokalCudaCtx) -> c_int;
    pub fn lokal_cuda_destroy(ctx: *mut LokalCudaCtx);
    pub fn lokal_cuda_last_error(ctx: *const LokalCudaCtx) -> *const c_char;
    pub fn lokal_cuda_version() -> *const c_char;
    pub fn lokal_cuda_device_count() -> c_int;
    pub fn lokal_cuda_malloc(ctx: *mut LokalCudaCtx, bytes: usize, dptr: *mut *mut c_void) -> c_int;
    pub fn lokal_cuda_free(ctx: *mut LokalCudaCtx, dptr: *mut c_void) -> c_int;
    pub fn lokal_cuda_host_alloc(ctx: *mut LokalCudaCtx, bytes: usize, hptr: *mut *mut c_void) -> c_int;
    pub fn lokal_cuda_host_free(ctx: *mut LokalCudaCtx, hptr: *mut c_void) -> c_int;
    pub fn lokal_cuda_memcpy_h2d(ctx: *mut LokalCudaCtx, s: LokalCudaStream, dst: *mut c_void, src: *const c_void,
        bytes: usize) -> c_int;
    pub fn lokal_cuda_memcpy_d2h(ctx: *mut LokalCudaCtx, s: LokalCudaStream, dst: *mut c_void, src: *const c_void,
        bytes: usize) -> c_int;
    pub fn lokal_cuda_stream_create(ctx: *mut LokalCudaCtx, out: *mut LokalCudaStream) -> c_int;
    pub fn lokal_cuda_stream_destroy(ctx: *mut LokalCudaCtx, s: LokalCudaStream) -> c_int;
    pub fn lokal_cuda_stream_sync(ctx: *mut LokalCudaCtx, s: LokalCudaStream) -> c_int;
    pub fn lokal_cuda_graph_begin(ctx: *mut LokalCudaCtx, s: LokalCudaStream) -> c_int;
    pub fn lokal_cuda_graph_end(ctx: *mut LokalCudaCtx, s: LokalCudaStream, out: *mut *mut LokalCudaGraph) -> c_int;
    pub fn lokal_cuda_graph_launch(ctx: *mut LokalCudaCtx, g: *mut LokalCudaGraph, s: LokalCudaStream) -> c_int;
    pub fn lokal_cuda_graph_destroy(ctx: *mut LokalCudaCtx, g: *mut LokalCudaGraph) -> c_int;
    pub fn lokal_cuda_blk_elems(ggml_type: c_int) -> usize;
    pub fn lokal_cuda_blk_bytes(ggml_type: c_int) -> usize;
    pub fn lokal_cuda_row_bytes(ggml_type: c_int, n: usize) -> usize;
    pub fn lokal_cuda_set_iq_grid(ctx: *mut LokalCudaCtx, which: c_int, table: *const c_void, bytes: usize) -> c_int;
    pub fn lokal_cuda_rmsnorm(ctx: *mut LokalCudaCtx, s: LokalCudaStream, x: *const c_void, w: *const c_void,
        y: *mut c_void, y_h: *mut c_void, rows: usize, dim: usize, eps: f32, dtype: c_int, w_dtype: c_int,
        h_dtype: c_int) -> c_int;
    pub fn lokal_cuda_add_rmsnorm(ctx: *mut LokalCudaCtx, s: LokalCudaStream, x_inout: *mut c_void,
        delta: *const c_void, w: *const c_void, xn: *mut c_void, xn_h: *mut c_void, rows: usize, dim: usize,
        eps: f32, dtype: c_int, w_dtype: c_int, h_dtype: c_int) -> c_int;
    pub fn lokal_cuda_rope_table(ctx: *mut LokalCudaCtx, s: LokalCudaStream, theta: f32, rot_dim: u32,
        positions: *const i32, pos0: i64, rows: usize, cos_sin: *mut f32) -> c_int;
    pub fn lokal_cuda_qk_rope(ctx: *mut LokalCudaCtx, s: LokalCudaStream, p: *const LokalQkRopeParams) -> c_int;
    pub fn lokal_cuda_qk_rope_pos(ctx: *mut LokalCudaCtx, s: LokalCudaStream, p: *const LokalQkRopeParams,
        theta: f32, positions: *const i32, pos0: i64) -> c_int;
    pub fn lokal_cuda_qk_rope_pos_noalloc(ctx: *mut LokalCudaCtx, s: LokalCudaStream, p: *const LokalQkRopeParams,
        theta: f32, positions: *const i32, pos0: i64) -> c_int;
    pub fn lokal_cuda_swiglu(ctx: *mut LokalCudaCtx, s: LokalCudaStream, gate: *const c_void, up: *const c_void,
        out: *mut c_void, out_h: *mut c_void, n: usize, dtype: c_int, h_dtype: c_int) -> c_int;
    pub fn lokal_cuda_embed_gather(ctx: *mut LokalCudaCtx, s: LokalCudaStream, table: *const c_void,
        ggml_type: c_int, vocab: usize, dim: usize, ids: *const u32, n: usize, out: *mut c_void, out_dtype: c_int) -> c_int;
    pub fn lokal_cuda_embed_gather_rmsnorm(ctx: *mut LokalCudaCtx, s: LokalCudaStream, table: *const c_void, ggml_type: c_int,
        vocab: usize, dim: usize, ids: *const u32, n: usize, x: *mut c_void, xn: *mut c_void, w: *const c_void, eps: f32,
        out_dtype: c_int, w_dtype: c_int) -> c_int;
    pub fn lokal_cuda_dequant_rows(ctx: *mut LokalCudaCtx, s: LokalCudaStream, ggml_type: c_int,
        src: *const c_void, rows: usize, cols: usize, out: *mut c_void, out_dtype: c_int) -> c_int;
    pub fn lokal_cuda_window_cfg(window: u64, sink: u64, prefill_chunk: u64, out: *mut LokalKvLayout) -> c_int;
    pub fn lokal_cuda_window_slot_of(layout: *const LokalKvLayout, p: u64) -> u64;
    pub fn lokal_cuda_window_write_spans(layout: *const LokalKvLayout, pos0: u64, n: u64, spans: *mut u64) -> c_int;
    pub fn lokal_cuda_kv_rows(ctx: *mut LokalCudaCtx, s: LokalCudaStream, layout: *const LokalKvLayout,
        positions: *const i32, pos0: i64, slots: *const u32, slot0: u32, rows: usize, rows_out: *mut u32) -> c_int;
    pub fn lokal_cuda_kv_stage(ctx: *mut LokalCudaCtx, s: LokalCudaStream, src: *const c_void, src_dtype: c_int,
        src_row_stride: usize, dst: *mut c_void, dst_dtype: c_int, dst_row_stride: usize, dst_rows: *const u32,
        rows: usize, width: usize) -> c_int;
    pub fn lokal_cuda_l2norm_rows(ctx: *mut LokalCudaCtx, s: LokalCudaStream, x: *const c_void, y: *mut c_void,
        rows_per_token: usize, n_tokens: usize, tok_stride: usize, dim: usize, eps: f32, dtype: c_int) -> c_int;
    pub fn lokal_cuda_gated_output_norm(ctx: *mut LokalCudaCtx, s: LokalCudaStream, o: *const c_void,
        w: *const c_void, z: *const c_void, y: *mut c_void, rows: usize, dim: usize, eps: f32, dtype: c_int,
        w_dtype: c_int) -> c_int;
    pub fn lokal_cuda_attn_out_gate(ctx: *mut LokalCudaCtx, s: LokalCudaStream, attn: *const c_void,
        gate: *const c_void, out: *mut c_void, n: usize, dtype: c_int) -> c_int;
    pub fn lokal_cuda_split_q_gate(ctx: *mut LokalCudaCtx, s: LokalCudaStream, src: *const c_void, q: *mut c_void,
        gate: *mut c_void, rows: usize, n_heads: usize, head_dim: usize, dtype: c_int) -> c_int;
    pub fn lokal_cuda_delta_gates(ctx: *mut LokalCudaCtx, s: LokalCudaStream, alpha: *const f32,
        beta_in: *const f32, a: *const f32, dt_bias: *const f32, g: *mut f32, beta: *mut f32, n_v_heads: usize,
        n_tokens: usize) -> c_int;
    pub fn lokal_cuda_ssm_conv(ctx: *mut LokalCudaCtx, s: LokalCudaStream, state: *mut f32, x: *const c_void,
        w: *const f32, out: *mut c_void, channels: usize, d_conv: usize, n_tokens: usize, dtype: c_int, roll: c_int) -> c_int;
    pub fn lokal_cuda_bf16_to_f16_copy(ctx: *mut LokalCudaCtx, s: LokalCudaStream, src_bf16: *const c_void,
        dst_f16: *mut c_void, n: usize, clip_flag: *mut u32) -> c_int;
    pub fn lokal_gguf_open(path: *const c_char, out: *mut *mut LokalGguf, err: *mut c_char, err_len: usize) -> c_int;
    pub fn lokal_gguf_close(g: *mut LokalGguf);
    pub fn lokal_gguf_last_error(g: *const LokalGguf) -> *const c_char;
    pub fn lokal_gguf_version(g: *const LokalGguf) -> u32;
    pub fn lokal_gguf_n_tensors(g: *const LokalGguf) -> usize;
    pub fn lokal_gguf_data_start(g: *const LokalGguf) -> u64;
    pub fn lokal_gguf_tensor_at(g: *const LokalGguf, i: usize, out: *mut LokalGgufTensor) -> c_int;
    pub fn lokal_gguf_find_tensor(g: *const LokalGguf, name: *const c_char, out: *mut LokalGgufTensor) -> c_int;
    pub fn lokal_gguf_has_key(g: *const LokalGguf, key: *const c_char) -> c_int;
    pub fn lokal_gguf_get_u64(g: *const LokalGguf, key: *const c_char, out: *mut u64) -> c_int;
    pub fn lokal_gguf_get_f32(g: *const LokalGguf, key: *const c_char, out: *mut f32) -> c_int;
    pub fn lokal_gguf_get_str(g: *const LokalGguf, key: *const c_char, out: *mut *const c_char, len: *mut usize) -> c_int;
    pub fn lokal_gguf_get_arr_i64(g: *const LokalGguf, key: *const c_char, out: *mut *const i64, n: *mut usize) -> c_int;
    pub fn lokal_gguf_get_arr_str(g: *const LokalGguf, key: *const c_char, out: *mut *const *const c_char,
        n: *mut usize) -> c_int;
    pub fn lokal_cuda_gguf_upload(ctx: *mut LokalCudaCtx, s: LokalCudaStream, g: *const LokalGguf,
        name: *const c_char, dptr: *mut *mut c_void, info: *mut LokalGgufTensor) -> c_int;
    pub fn lokal_cuda_shard_rows(n_rows: usize, n_gpus: c_int, rank: c_int, row0: *mut usize, count: *mut usize) -> c_int;
    pub fn lokal_cuda_pass_create(ctx: *mut LokalCudaCtx, cfg: *const LokalPassConfig, w: *const LokalPassWeights,
        out: *mut *mut LokalCudaPass) -> c_int;
    pub fn lokal_cuda_pass_destroy(ctx: *mut LokalCudaCtx, pass: *mut LokalCudaPass) -> c_int;
    pub fn lokal_cuda_pass_run_device(ctx: *mut LokalCudaCtx, pass: *mut LokalCudaPass, s: LokalCudaStream,
        in_dev: *const LokalPassInputs, out_dev: *mut c_void) -> c_int;
    pub fn lokal_cuda_pass_run_host(ctx: *mut LokalCudaCtx, pass: *mut LokalCudaPass,
        in_host: *const LokalPassInputs, out_host: *mut c_void) -> c_int;
    pub fn lokal_cuda_pass_output(ctx: *mut LokalCudaCtx, pass: *mut LokalCudaPass, layer: u32, which: c_int,
        dptr: *mut *mut c_void) -> c_int;
    pub fn lokal_cuda_pass_launches(pass: *const LokalCudaPass) -> u64;
    pub fn lokal_cuda_pass_set_schedule(ctx: *mut LokalCudaCtx, pass: *mut LokalCudaPass, schedule: c_int) -> c_int;
    pub fn lokal_cuda_host_rmsnorm(ctx: *mut LokalCudaCtx, x: *const f32, w: *const f32, eps: f32, rows: usize,
        dim: usize, y: *mut f32) -> c_int;
    pub fn lokal_cuda_host_rope(ctx: *mut LokalCudaCtx, x: *mut f32, n: usize, pos: usize, head_dim: usize,
        theta: f32) -> c_int;
    pub fn lokal_cuda_host_swiglu(ctx: *mut LokalCudaCtx, gate: *const f32, up: *const f32, n: usize, out: *mut f32) -> c_int;
    pub fn lokal_cuda_host_dequant_row(ctx: *mut LokalCudaCtx, ggml_type: c_int, src: *const u8, src_len: usize,
        out: *mut f32, n: usize) -> c_int;
    pub fn lokal_cuda_host_embed_gather(ctx: *mut LokalCudaCtx, table_dev: *const c_void, ggml_type: c_int,
        vocab: usize, dim: usize, ids: *const u32, n: usize, out: *mut f32) -> c_int;
}
