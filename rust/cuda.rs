//! `-b cuda`: lokal's per-token layer ops on NVIDIA B200 through liblokal_cuda.
//!
//! Where this file goes: `src/gpu/cuda.rs` of the lokal tree, next to `metal.rs`, following the checklist of
//! src/gpu/mod.rs:3-13 — implement `Engine` + `Session` (+ `Batcher`), add one arm to `engine::create`
//! (src/engine.rs:83-110), gate it with a cargo feature:
//!
//! ```text
//! // Cargo.toml
//! [features]
//! cuda = ["dep:lokal-cuda-sys"]
//! [dependencies]
//! lokal-cuda-sys = { path = "lokal-cuda-sys", optional = true }
//!
//! // src/gpu/mod.rs
//! #[cfg(feature = "cuda")]
//! pub mod cuda;
//!
//! // src/engine.rs, inside `match backend`
//! #[cfg(feature = "cuda")]
//! "cuda" => Ok(Box::new(crate::gpu::cuda::CudaEngine::new(model)?)),
//! ```
//!
//! What the library owns: the fused per-token ops (embedding gather with GGUF row dequant, residual-add + RMSNorm,
//! q/k bias + per-head RMSNorm + RoPE, SwiGLU, K/V staging) on device buffers. What stays lokal's: the projections,
//! attention and the lm_head. They are behind the `DeviceMatmul` trait below so that this file reads top to bottom;
//! a maintainer plugs in cuBLAS or a kernel of their own there. This file has not been compiled (the image it was
//! written in has no Rust toolchain); the FFI declarations it uses are checked against the C header by a test.
//!
//! Invariants kept (src/gpu/mod.rs:9-13): weights are uploaded once at engine creation and stay on the device; a
//! whole step is encoded on one stream and waited for once (`lokal_cuda_stream_sync`); only token ids go up and
//! logits come down. Unsupported combinations are refused by name, never silently run elsewhere (src/main.rs:326-355).

use std::ffi::CStr;
use std::os::raw::{c_int, c_void};
use std::ptr::{null, null_mut};

use lokal_cuda_sys::*;

use crate::config::ModelConfig;
use crate::engine::{BatchRow, Batcher, Engine, Session};
use crate::model::Model;

/// Status code + the context's message -> `crate::Result`.
fn check(ctx: *mut LokalCudaCtx, rc: c_int) -> crate::Result<()> {
    if rc == LOKAL_OK {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(lokal_cuda_last_error(ctx)) }.to_string_lossy().into_owned();
    Err(format!("cuda backend: {msg} (status {rc})").into())
}

/// The contractions this backend does not take from liblokal_cuda. `a` is `[rows][in_dim]`, `w` the resident
/// `[out_dim][in_dim]` weight, `y` `[rows][out_dim]`, all device pointers, asynchronous on `stream`.
pub trait DeviceMatmul: Send + Sync {
    fn matmul(&self, stream: LokalCudaStream, a: *const c_void, w: DeviceWeight, rows: usize, y: *mut c_void) -> crate::Result<()>;
    /// Causal attention of `rows` query rows at positions `pos0..` against the cache rows of `slot`.
    fn attention(&self, stream: LokalCudaStream, q: *const c_void, layer: &LayerCache, slot: usize, pos0: usize, rows: usize,
                 out: *mut c_void) -> crate::Result<()>;
}

#[derive(Clone, Copy)]
pub struct DeviceWeight {
    pub ptr: *const c_void, // f16, [out_dim][in_dim]
    pub in_dim: usize,
    pub out_dim: usize,
}

/// One layer's resident tensors (uploaded once, src/gpu/metal.rs:965-1026 is the Metal twin).
struct LayerWeights {
    input_ln: *const c_void, // f16 [hidden]
    post_ln: *const c_void,
    q_bias: *const c_void,   // f16 [q_dim] or null (Qwen2)
    k_bias: *const c_void,
    v_bias: *const c_void,
    q_norm: *const c_void,   // f16 [head_dim] or null (qwen3)
    k_norm: *const c_void,
    q_proj: DeviceWeight,
    k_proj: DeviceWeight,
    v_proj: DeviceWeight,
    o_proj: DeviceWeight,
    gate_proj: DeviceWeight,
    up_proj: DeviceWeight,
    down_proj: DeviceWeight,
}

/// K and V of one layer: `[slots][max_seq][kv_dim]` f16 each, as the Metal batcher lays them out (src/engine.rs:36-41).
pub struct LayerCache {
    pub k: *mut c_void,
    pub v: *mut c_void,
}

pub struct CudaEngine {
    ctx: *mut LokalCudaCtx,
    cfg: ModelConfig,
    head_dim: usize, // from the checkpoint (Model::head_dim), never hidden / n_heads
    q_dim: usize,
    kv_dim: usize,
    embed: *const c_void, // f16 [vocab][hidden] (or raw GGUF rows with `embed_type`)
    embed_type: c_int,
    final_ln: *const c_void,
    lm_head: DeviceWeight,
    layers: Vec<LayerWeights>,
    mm: Box<dyn DeviceMatmul>,
}

// The context is immutable after creation and every mutable thing (streams, activations, caches) lives in a
// session or a batcher, as in the Metal backend (src/gpu/metal.rs:706-707).
unsafe impl Send for CudaEngine {}
unsafe impl Sync for CudaEngine {}

impl CudaEngine {
    pub fn new(model: Model) -> crate::Result<Self> {
        let mut ctx = null_mut();
        let rc = unsafe { lokal_cuda_create(0, &mut ctx) };
        if rc != LOKAL_OK {
            return Err(match rc {
                LOKAL_ERR_NO_DEVICE => "cuda backend: no CUDA device".into(),
                LOKAL_ERR_UNSUPPORTED => "cuda backend: liblokal_cuda holds sm_100a code only (B200); this GPU is older".into(),
                _ => format!("cuda backend: lokal_cuda_create failed (status {rc})").into(),
            });
        }
        let up_f16 = |v: &[f32]| -> crate::Result<*const c_void> {
            // f32 -> f16 on the host (half::f16::from_f32, as src/gpu/metal.rs:719-729), one upload per tensor
            let h: Vec<half::f16> = v.iter().map(|&x| half::f16::from_f32(x)).collect();
            let mut d = null_mut();
            check(ctx, unsafe { lokal_cuda_malloc(ctx, h.len() * 2, &mut d) })?;
            check(ctx, unsafe { lokal_cuda_memcpy_h2d(ctx, null_mut(), d, h.as_ptr().cast(), h.len() * 2) })?;
            check(ctx, unsafe { lokal_cuda_stream_sync(ctx, null_mut()) })?;
            Ok(d as *const c_void)
        };
        let up_opt = |v: &Option<Vec<f32>>| -> crate::Result<*const c_void> { v.as_ref().map_or(Ok(null()), |v| up_f16(v)) };
        let up_lin = |l: &crate::model::Linear| -> crate::Result<DeviceWeight> {
            Ok(DeviceWeight { ptr: up_f16(&l.w)?, in_dim: l.in_dim, out_dim: l.out_dim })
        };
        let mut layers = Vec::with_capacity(model.blocks.len());
        for b in &model.blocks {
            let f = b.ffn.dense();
            layers.push(LayerWeights {
                input_ln: up_f16(&b.input_layernorm)?,
                post_ln: up_f16(&b.post_attention_layernorm)?,
                q_bias: up_opt(&b.q_proj.bias)?,
                k_bias: up_opt(&b.k_proj.bias)?,
                v_bias: up_opt(&b.v_proj.bias)?,
                q_norm: up_opt(&b.q_norm)?,
                k_norm: up_opt(&b.k_norm)?,
                q_proj: up_lin(&b.q_proj)?,
                k_proj: up_lin(&b.k_proj)?,
                v_proj: up_lin(&b.v_proj)?,
                o_proj: up_lin(&b.o_proj)?,
                gate_proj: up_lin(&f.gate_proj)?,
                up_proj: up_lin(&f.up_proj)?,
                down_proj: up_lin(&f.down_proj)?,
            });
        }
        Ok(Self {
            ctx,
            head_dim: model.head_dim,
            q_dim: model.cfg.num_attention_heads * model.head_dim,
            kv_dim: model.kv_dim,
            embed: up_f16(&model.embed_tokens)?,
            embed_type: LOKAL_F16,
            final_ln: up_f16(&model.norm)?,
            lm_head: up_lin(&model.lm_head)?,
            layers,
            mm: crate::gpu::cuda_matmul::default_backend()?, // cuBLAS or the maintainer's own kernels
            cfg: model.cfg,
        })
    }
}

impl Drop for CudaEngine {
    fn drop(&mut self) {
        unsafe { lokal_cuda_destroy(self.ctx) } // resident tensors go with the process; a real engine frees them here
    }
}

impl Engine for CudaEngine {
    fn name(&self) -> &'static str {
        "cuda"
    }
    fn config(&self) -> &ModelConfig {
        &self.cfg
    }
    fn session(&self, max_seq: usize) -> crate::Result<Box<dyn Session + '_>> {
        Ok(Box::new(CudaSession { core: StepCore::new(self, 1, max_seq, max_seq.min(512))? }))
    }
    fn batcher(&self, n_slots: usize, max_seq: usize) -> Option<Box<dyn Batcher + '_>> {
        StepCore::new(self, n_slots, max_seq, n_slots.max(512)).ok().map(|core| Box::new(CudaBatcher { core }) as Box<dyn Batcher + '_>)
    }
}

/// Stream, activation buffers and KV cache shared by the session and the batcher: `max_rows` token rows per step.
struct StepCore<'e> {
    eng: &'e CudaEngine,
    stream: LokalCudaStream,
    layout: LokalKvLayout, // linear: slot * max_seq + pos
    cache: Vec<LayerCache>,
    max_rows: usize,
    // device activations, f32 as the Metal backend keeps them; f16 copies feed the projections
    x: *mut c_void,        // [max_rows][hidden] residual stream
    xn: *mut c_void,       // [max_rows][hidden] normed, f32
    xn_h: *mut c_void,     //   and its f16 copy
    q: *mut c_void,        // [max_rows][q_dim]
    k: *mut c_void,        // [max_rows][kv_dim]
    v: *mut c_void,
    att: *mut c_void,      // [max_rows][q_dim] attention output, then o_proj output in `delta`
    delta: *mut c_void,    // [max_rows][hidden]
    gate: *mut c_void,     // [max_rows][inter]
    up: *mut c_void,
    gate_h: *mut c_void,   // f16 copy of silu(gate) * up for the down projection
    logits: *mut c_void,   // [max_rows][vocab]
    ids: *mut u32,
    positions: *mut i32,
    slots: *mut u32,
    cache_rows: *mut u32,  // [max_rows] cache row of every token row (lokal_cuda_kv_rows)
    rope_table: *mut f32,  // [max_rows][head_dim] cos | sin
}

impl<'e> StepCore<'e> {
    fn new(eng: &'e CudaEngine, n_slots: usize, max_seq: usize, max_rows: usize) -> crate::Result<Self> {
        let ctx = eng.ctx;
        let mut stream = null_mut();
        check(ctx, unsafe { lokal_cuda_stream_create(ctx, &mut stream) })?;
        let alloc = |bytes: usize| -> crate::Result<*mut c_void> {
            let mut p = null_mut();
            check(ctx, unsafe { lokal_cuda_malloc(ctx, bytes, &mut p) })?;
            Ok(p)
        };
        let (h, i, qd, kd, v) = (eng.cfg.hidden_size, eng.cfg.intermediate_size, eng.q_dim, eng.kv_dim, eng.cfg.vocab_size);
        let mut cache = Vec::new();
        for _ in 0..eng.layers.len() {
            cache.push(LayerCache { k: alloc(n_slots * max_seq * kd * 2)?, v: alloc(n_slots * max_seq * kd * 2)? });
        }
        Ok(Self {
            eng,
            stream,
            layout: LokalKvLayout { max_seq: max_seq as u64, sink: 0, sink_pad: 0, ring: 0 },
            cache,
            max_rows,
            x: alloc(max_rows * h * 4)?,
            xn: alloc(max_rows * h * 4)?,
            xn_h: alloc(max_rows * h * 2)?,
            q: alloc(max_rows * qd * 4)?,
            k: alloc(max_rows * kd * 4)?,
            v: alloc(max_rows * kd * 4)?,
            att: alloc(max_rows * qd * 4)?,
            delta: alloc(max_rows * h * 4)?,
            gate: alloc(max_rows * i * 4)?,
            up: alloc(max_rows * i * 4)?,
            gate_h: alloc(max_rows * i * 2)?,
            logits: alloc(max_rows * v * 4)?,
            ids: alloc(max_rows * 4)?.cast(),
            positions: alloc(max_rows * 4)?.cast(),
            slots: alloc(max_rows * 4)?.cast(),
            cache_rows: alloc(max_rows * 4)?.cast(),
            rope_table: alloc(max_rows * eng.head_dim * 4)?.cast(),
        })
    }

    /// One step over `n` token rows: row r is token `ids[r]` at position `positions[r]` of KV slot `slots[r]`.
    /// The order is Model::forward's (src/model.rs:205-256); the Metal twin is MetalSession::run_from
    /// (src/gpu/metal.rs:2528-2669) and MetalBatcher::decode_step (:3681-3762). Returns logits of every row.
    fn step(&mut self, ids: &[u32], positions: &[i32], slots: &[u32]) -> crate::Result<Vec<Vec<f32>>> {
        let n = ids.len();
        if n == 0 || n > self.max_rows {
            return Err(format!("cuda backend: a step of {n} rows (capacity {})", self.max_rows).into());
        }
        let (e, ctx, s) = (self.eng, self.eng.ctx, self.stream);
        let (h, inter, eps) = (e.cfg.hidden_size, e.cfg.intermediate_size, e.cfg.rms_norm_eps);
        let (nq, nkv, hd) = (e.cfg.num_attention_heads as u32, e.cfg.num_key_value_heads as u32, e.head_dim as u32);
        unsafe {
            // ids, positions, slots up: the only host -> device traffic of the step
            check(ctx, lokal_cuda_memcpy_h2d(ctx, s, self.ids.cast(), ids.as_ptr().cast(), n * 4))?;
            check(ctx, lokal_cuda_memcpy_h2d(ctx, s, self.positions.cast(), positions.as_ptr().cast(), n * 4))?;
            check(ctx, lokal_cuda_memcpy_h2d(ctx, s, self.slots.cast(), slots.as_ptr().cast(), n * 4))?;
            // embedding rows (dequantised on the fly when the table is a GGUF block type), cos/sin of the step's
            // positions (shared by all heads and layers), the cache row of every token row
            check(ctx, lokal_cuda_embed_gather(ctx, s, e.embed, e.embed_type, e.cfg.vocab_size, h, self.ids, n, self.x, LOKAL_F32))?;
            check(ctx, lokal_cuda_rope_table(ctx, s, e.cfg.rope_theta, hd, self.positions, 0, n, self.rope_table))?;
            check(ctx, lokal_cuda_kv_rows(ctx, s, &self.layout, self.positions, 0, self.slots, 0, n, self.cache_rows))?;
            // first input norm, with the f16 copy the projections read; every later norm is fused with the residual add
            // that precedes it. (An engine that keeps 16-bit activations and needs no second copy takes gather and
            // norm as one launch: lokal_cuda_embed_gather_rmsnorm.)
            check(ctx, lokal_cuda_rmsnorm(ctx, s, self.x, e.layers[0].input_ln, self.xn, self.xn_h, n, h, eps, LOKAL_F32, LOKAL_F16, LOKAL_F16))?;
            for (l, w) in e.layers.iter().enumerate() {
                e.mm.matmul(s, self.xn_h, w.q_proj, n, self.q)?;
                e.mm.matmul(s, self.xn_h, w.k_proj, n, self.k)?;
                e.mm.matmul(s, self.xn_h, w.v_proj, n, self.v)?; // v bias, where there is one, rides in the GEMM epilogue
                // bias -> per-head RMSNorm -> RoPE of q and k in one pass, in place (f32 rows, f16 weights). With an
                // f16 k buffer, `k_out = cache[l].k` and `k_out_rows = cache_rows` would rotate k straight into its
                // cache rows and the first kv_stage below would go away.
                let p = LokalQkRopeParams {
                    q: self.q, k: self.k, q_out: null_mut(), k_out: null_mut(),
                    q_bias: w.q_bias, k_bias: w.k_bias, q_norm_w: w.q_norm, k_norm_w: w.k_norm,
                    cos_sin: self.rope_table, k_out_rows: null(),
                    rows: n as u64, n_q_heads: nq, n_kv_heads: nkv, head_dim: hd, rot_dim: hd, // explicit, never from hidden
                    q_row_stride: e.q_dim as u64, k_row_stride: e.kv_dim as u64, q_out_row_stride: 0, k_out_row_stride: 0,
                    eps, q_dtype: LOKAL_F32, k_dtype: LOKAL_F32, w_dtype: LOKAL_F16,
                };
                check(ctx, lokal_cuda_qk_rope(ctx, s, &p))?;
                // fresh K and V rows narrowed to f16 and scattered to (slot * max_seq + pos)
                check(ctx, lokal_cuda_kv_stage(ctx, s, self.k, LOKAL_F32, e.kv_dim, self.cache[l].k, LOKAL_F16, e.kv_dim, self.cache_rows, n, e.kv_dim))?;
                check(ctx, lokal_cuda_kv_stage(ctx, s, self.v, LOKAL_F32, e.kv_dim, self.cache[l].v, LOKAL_F16, e.kv_dim, self.cache_rows, n, e.kv_dim))?;
                e.mm.attention(s, self.q, &self.cache[l], slots[0] as usize, positions[0] as usize, n, self.att)?;
                e.mm.matmul(s, self.att, w.o_proj, n, self.delta)?;
                // x += att_out; xn = rmsnorm(x, post_ln): one launch
                check(ctx, lokal_cuda_add_rmsnorm(ctx, s, self.x, self.delta, w.post_ln, self.xn, self.xn_h, n, h, eps, LOKAL_F32, LOKAL_F16, LOKAL_F16))?;
                e.mm.matmul(s, self.xn_h, w.gate_proj, n, self.gate)?;
                e.mm.matmul(s, self.xn_h, w.up_proj, n, self.up)?;
                check(ctx, lokal_cuda_swiglu(ctx, s, self.gate, self.up, self.gate, self.gate_h, n * inter, LOKAL_F32, LOKAL_F16))?;
                e.mm.matmul(s, self.gate_h, w.down_proj, n, self.delta)?;
                // x += mlp_out; xn = rmsnorm(x, next layer's input_ln or the final norm)
                let next_ln = e.layers.get(l + 1).map_or(e.final_ln, |nx| nx.input_ln);
                check(ctx, lokal_cuda_add_rmsnorm(ctx, s, self.x, self.delta, next_ln, self.xn, self.xn_h, n, h, eps, LOKAL_F32, LOKAL_F16, LOKAL_F16))?;
            }
            e.mm.matmul(s, self.xn_h, e.lm_head, n, self.logits)?;
            // logits down, one wait for the whole step; an out-of-range token id or a device-side wait that gave
            // up surfaces here as LOKAL_ERR_ID_RANGE / LOKAL_ERR_TIMEOUT with its message
            let v = e.cfg.vocab_size;
            let mut out = vec![0f32; n * v];
            check(ctx, lokal_cuda_memcpy_d2h(ctx, s, out.as_mut_ptr().cast(), self.logits, n * v * 4))?;
            check(ctx, lokal_cuda_stream_sync(ctx, s))?;
            Ok(out.chunks(v).map(<[f32]>::to_vec).collect())
        }
    }
}

impl Drop for StepCore<'_> {
    fn drop(&mut self) {
        let ctx = self.eng.ctx;
        unsafe {
            lokal_cuda_stream_sync(ctx, self.stream);
            for p in [self.x, self.xn, self.xn_h, self.q, self.k, self.v, self.att, self.delta, self.gate, self.up, self.gate_h, self.logits,
                      self.ids.cast(), self.positions.cast(), self.slots.cast(), self.cache_rows.cast(), self.rope_table.cast()] {
                lokal_cuda_free(ctx, p);
            }
            for c in &self.cache {
                lokal_cuda_free(ctx, c.k);
                lokal_cuda_free(ctx, c.v);
            }
            lokal_cuda_stream_destroy(ctx, self.stream);
        }
    }
}

pub struct CudaSession<'e> {
    core: StepCore<'e>,
}

impl Session for CudaSession<'_> {
    fn forward(&mut self, token: u32, pos: usize) -> crate::Result<Vec<f32>> {
        Ok(self.core.step(&[token], &[pos as i32], &[0])?.pop().unwrap())
    }
    fn prefill(&mut self, ids: &[u32]) -> crate::Result<Vec<f32>> {
        let mut last = Vec::new();
        for (c, chunk) in ids.chunks(self.core.max_rows).enumerate() {
            let pos0 = c * self.core.max_rows;
            let positions: Vec<i32> = (0..chunk.len()).map(|i| (pos0 + i) as i32).collect();
            last = self.core.step(chunk, &positions, &vec![0; chunk.len()])?.pop().unwrap();
        }
        Ok(last)
    }
    fn forward_batch(&mut self, ids: &[u32], pos0: usize) -> crate::Result<Vec<Vec<f32>>> {
        let positions: Vec<i32> = (0..ids.len()).map(|i| (pos0 + i) as i32).collect();
        self.core.step(ids, &positions, &vec![0; ids.len()])
    }
}

pub struct CudaBatcher<'e> {
    core: StepCore<'e>,
}

// Lives on the scheduler thread (src/batch.rs:42); the raw pointers it holds are its own.
unsafe impl Send for CudaBatcher<'_> {}

impl Batcher for CudaBatcher<'_> {
    fn prefill(&mut self, slot: usize, ids: &[u32]) -> crate::Result<Vec<f32>> {
        let mut last = Vec::new();
        for (c, chunk) in ids.chunks(self.core.max_rows).enumerate() {
            let pos0 = c * self.core.max_rows;
            let positions: Vec<i32> = (0..chunk.len()).map(|i| (pos0 + i) as i32).collect();
            last = self.core.step(chunk, &positions, &vec![slot as u32; chunk.len()])?.pop().unwrap();
        }
        Ok(last)
    }
    fn decode_step(&mut self, rows: &[BatchRow]) -> crate::Result<Vec<Vec<f32>>> {
        let ids: Vec<u32> = rows.iter().map(|r| r.token).collect();
        let positions: Vec<i32> = rows.iter().map(|r| r.pos as i32).collect();
        let slots: Vec<u32> = rows.iter().map(|r| r.slot as u32).collect();
        self.core.step(&ids, &positions, &slots)
    }
}
