// Layer pass: the host-side runner that strings the per-token ops of one
// forward step together, layer by layer, the way the reference's step loop
// does around its projections (MetalSession::run_from, src/gpu/metal.rs:2528-2669;
// Model::forward, src/model.rs:205-256).
//
// Two ways to run a step:
//   * run_device: inputs already on the device, nothing but kernel launches on
//     the caller's stream (4 per layer + 3), so the whole step can be captured
//     into one CUDA graph.
//   * run_host: inputs in host memory. Layer l+1's six input blocks are copied
//     on a copy stream into a ring of layer slots while layer l's kernels run
//     on the compute stream; events order slot reuse. The final normed hidden
//     state is copied back and the call returns when it has landed.
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"

struct lokal_cuda_pass {
    lokal_pass_config cfg{};
    size_t es = 0, wes = 0;  // element sizes
    size_t q_dim = 0, kv_dim = 0;
    // resident weights
    void* embed_table = nullptr;
    void* norm_w = nullptr;
    void* final_w = nullptr;
    void* q_bias = nullptr;
    void* k_bias = nullptr;
    void* q_norm_w = nullptr;
    void* k_norm_w = nullptr;
    // per-step state
    void* x = nullptr;         // residual stream [max_rows][hidden]
    float* cos_sin = nullptr;  // [max_rows][rot_dim]
    uint32_t* ids = nullptr;   // staged ids (run_host)
    int32_t* positions = nullptr;
    void* out_dev = nullptr;   // final normed hidden (run_host)
    void* last_out = nullptr;  // where the last run put its result (the caller's buffer for run_device)
    // per-slot outputs and staged inputs
    void* xn0 = nullptr;    // [slots][max_rows][hidden]
    void* xn_att = nullptr; // [slots][max_rows][hidden]
    void* xn_mlp = nullptr; // [slots][max_rows][hidden]
    void* inner = nullptr;  // [slots][max_rows][inter]
    void* sq = nullptr;     // staged inputs (run_host only, allocated on first use)
    void* sk = nullptr;
    void* sda = nullptr;
    void* sdm = nullptr;
    void* sg = nullptr;
    void* su = nullptr;
    cudaStream_t copy_stream = nullptr, compute_stream = nullptr;
    std::vector<cudaEvent_t> filled, drained;  // per slot
    // run_device with op families on parallel branches (lokal_cuda_pass_set_schedule)
    int schedule = LOKAL_PASS_SCHEDULE_AUTO;
    cudaStream_t branch[3] = {nullptr, nullptr, nullptr};  // rotations, SwiGLU, norm chain (the last at high priority)
    cudaEvent_t fork_ev = nullptr, join_ev[3] = {nullptr, nullptr, nullptr};
    unsigned long long launches = 0;
    std::mutex mu;
};

namespace {

using lokal::DeviceGuard;

int dev_alloc(lokal_cuda_ctx* ctx, void** p, size_t bytes) {
    *p = nullptr;
    if (bytes == 0) return LOKAL_OK;
    LOKAL_CUDA_TRY(ctx, cudaMalloc(p, bytes));
    return LOKAL_OK;
}

int upload(lokal_cuda_ctx* ctx, void** dst, const void* src, size_t bytes) {
    int rc = dev_alloc(ctx, dst, bytes);
    if (rc != LOKAL_OK) return rc;
    LOKAL_CUDA_TRY(ctx, cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice));
    return LOKAL_OK;
}

char* at(void* base, size_t bytes) { return static_cast<char*>(base) + bytes; }
const char* at(const void* base, size_t bytes) { return static_cast<const char*>(base) + bytes; }

// The kernels of one layer. q/k/delta/gate/up point at this layer's blocks. Three op families, each on the stream
// it is given: rotation of q/k (s_rope), SwiGLU (s_mlp), and the two residual-add + RMSNorm calls that carry the
// residual stream from layer to layer (s_norm). With one stream for all three they are issued in the order of
// Model::forward (src/model.rs:207-255).
int layer_ops(lokal_cuda_ctx* ctx, lokal_cuda_pass* P, cudaStream_t s_rope, cudaStream_t s_norm, cudaStream_t s_mlp, bool branched,
              uint32_t l, size_t rows, void* q, void* k, const void* delta_att, const void* delta_mlp, const void* gate, const void* up) {
    const lokal_pass_config& c = P->cfg;
    const uint32_t slot = l % c.slots;
    const size_t hid_b = static_cast<size_t>(c.max_rows) * c.hidden * P->es;
    lokal_qk_rope_params rp{};
    rp.q = q;
    rp.k = k;
    rp.q_bias = P->q_bias ? at(P->q_bias, static_cast<size_t>(l) * P->q_dim * P->wes) : nullptr;
    rp.k_bias = P->k_bias ? at(P->k_bias, static_cast<size_t>(l) * P->kv_dim * P->wes) : nullptr;
    rp.q_norm_w = P->q_norm_w ? at(P->q_norm_w, static_cast<size_t>(l) * c.head_dim * P->wes) : nullptr;
    rp.k_norm_w = P->k_norm_w ? at(P->k_norm_w, static_cast<size_t>(l) * c.head_dim * P->wes) : nullptr;
    rp.cos_sin = P->cos_sin;
    rp.rows = rows;
    rp.n_q_heads = c.n_q_heads;
    rp.n_kv_heads = c.n_kv_heads;
    rp.head_dim = c.head_dim;
    rp.rot_dim = c.rot_dim;
    rp.q_row_stride = P->q_dim;
    rp.k_row_stride = P->kv_dim;
    rp.eps = c.eps;
    rp.q_dtype = rp.k_dtype = c.dtype;
    rp.w_dtype = c.w_dtype;
    int rc = lokal::launch_qk_rope(ctx, s_rope, rp, branched);
    if (rc != LOKAL_OK) return rc;
    const void* w_post = at(P->norm_w, (static_cast<size_t>(l) * 2 + 1) * c.hidden * P->wes);
    rc = lokal::launch_norm(ctx, s_norm, P->x, delta_att, w_post, at(P->xn_att, slot * hid_b), nullptr, rows, c.hidden, c.eps,
                            c.dtype, c.w_dtype, 0);
    if (rc != LOKAL_OK) return rc;
    rc = lokal::launch_swiglu(ctx, s_mlp, gate, up, at(P->inner, slot * static_cast<size_t>(c.max_rows) * c.inter * P->es), nullptr,
                              rows * c.inter, c.dtype, 0);
    if (rc != LOKAL_OK) return rc;
    const void* w_next = (l + 1 < c.layers) ? at(P->norm_w, (static_cast<size_t>(l + 1) * 2) * c.hidden * P->wes) : P->final_w;
    void* xn_next = (l + 1 < c.layers) ? at(P->xn_mlp, slot * hid_b) : P->out_dev;
    rc = lokal::launch_norm(ctx, s_norm, P->x, delta_mlp, w_next, xn_next, nullptr, rows, c.hidden, c.eps, c.dtype, c.w_dtype, 0);
    if (rc != LOKAL_OK) return rc;
    P->launches += 4;
    return LOKAL_OK;
}

// embed gather and first input norm (s_norm), rope table (s_rope)
int step_head(lokal_cuda_ctx* ctx, lokal_cuda_pass* P, cudaStream_t s_norm, cudaStream_t s_rope, const uint32_t* ids_dev,
              const int32_t* pos_dev, int64_t pos0, size_t rows) {
    const lokal_pass_config& c = P->cfg;
    // gather and first input norm: one launch for a quantised table
    int head_launches = 0;
    int rc = lokal::launch_gather_norm(ctx, s_norm, P->embed_table, c.embed_type, c.vocab, c.hidden, ids_dev, rows, P->x, c.dtype,
                                       P->norm_w, c.w_dtype, P->xn0, c.eps, &head_launches);
    if (rc != LOKAL_OK) return rc;
    rc = lokal::launch_rope_table(ctx, s_rope, c.theta, c.rot_dim, pos_dev, pos0, rows, P->cos_sin);
    if (rc != LOKAL_OK) return rc;
    P->launches += 1 + static_cast<unsigned>(head_launches);
    return LOKAL_OK;
}

int check_inputs(lokal_cuda_ctx* ctx, const lokal_cuda_pass* P, const lokal_pass_inputs* in) {
    if (!in) return ctx->fail(LOKAL_ERR_BAD_ARG, "pass: inputs are null");
    if (in->rows == 0 || in->rows > P->cfg.max_rows)
        return ctx->fail(LOKAL_ERR_BAD_ARG, "pass: %llu rows outside 1..%llu", (unsigned long long)in->rows,
                         (unsigned long long)P->cfg.max_rows);
    if (!in->ids || !in->q || !in->k || !in->delta_att || !in->delta_mlp || !in->gate || !in->up)
        return ctx->fail(LOKAL_ERR_BAD_ARG, "pass: an input pointer is null");
    if (in->q_layer_stride < in->rows * P->q_dim || in->k_layer_stride < in->rows * P->kv_dim ||
        in->delta_layer_stride < in->rows * P->cfg.hidden || in->mlp_layer_stride < in->rows * P->cfg.inter)
        return ctx->fail(LOKAL_ERR_BAD_ARG, "pass: a layer stride is smaller than one layer's block");
    if (!in->positions && in->pos0 < 0) return ctx->fail(LOKAL_ERR_BAD_ARG, "pass: pos0 is negative");
    return LOKAL_OK;
}

}  // namespace

extern "C" {

int lokal_cuda_pass_create(lokal_cuda_ctx* ctx, const lokal_pass_config* cfg, const lokal_pass_weights* w,
                           lokal_cuda_pass** out) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!cfg || !w || !out) return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_create: null argument");
    *out = nullptr;
    const lokal_pass_config& c = *cfg;
    if (!c.max_rows || !c.layers || !c.hidden || !c.inter || !c.n_q_heads || !c.n_kv_heads || !c.head_dim || !c.vocab)
        return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_create: a dimension is zero");
    if (c.rot_dim == 0 || (c.rot_dim & 1) || c.rot_dim > c.head_dim)
        return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_create: rot_dim %u must be even and <= head_dim %u", c.rot_dim, c.head_dim);
    if (!lokal::is_act_type(c.dtype) || !lokal::is_act_type(c.w_dtype))
        return ctx->fail(LOKAL_ERR_UNSUPPORTED, "pass_create: activation/weight type must be F32, F16 or BF16");
    const size_t rb = lokal_cuda_row_bytes(c.embed_type, c.hidden);
    if (rb == 0 || c.hidden % lokal_cuda_blk_elems(c.embed_type) != 0)
        return ctx->fail(LOKAL_ERR_UNSUPPORTED, "pass_create: embedding type %d cannot hold rows of %u elements", c.embed_type, c.hidden);
    if (c.slots == 0 || c.slots > c.layers) return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_create: slots must be in 1..layers");
    if (!w->embed_table || !w->norm_w || !w->final_w) return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_create: table or norm weights are null");
    if (c.has_qk_bias && (!w->q_bias || !w->k_bias)) return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_create: qk bias announced but null");
    if (c.has_qk_norm && (!w->q_norm_w || !w->k_norm_w)) return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_create: qk norm announced but null");

    lokal_cuda_pass* P = new (std::nothrow) lokal_cuda_pass();
    if (!P) return ctx->fail(LOKAL_ERR_CUDA, "out of host memory");
    P->cfg = c;
    P->es = lokal::type_size(c.dtype);
    P->wes = lokal::type_size(c.w_dtype);
    P->q_dim = static_cast<size_t>(c.n_q_heads) * c.head_dim;
    P->kv_dim = static_cast<size_t>(c.n_kv_heads) * c.head_dim;
    const size_t hid_b = static_cast<size_t>(c.max_rows) * c.hidden * P->es;
    int rc = upload(ctx, &P->embed_table, w->embed_table, static_cast<size_t>(c.vocab) * rb);
    if (rc == LOKAL_OK) rc = upload(ctx, &P->norm_w, w->norm_w, static_cast<size_t>(c.layers) * 2 * c.hidden * P->wes);
    if (rc == LOKAL_OK) rc = upload(ctx, &P->final_w, w->final_w, static_cast<size_t>(c.hidden) * P->wes);
    if (rc == LOKAL_OK && c.has_qk_bias) rc = upload(ctx, &P->q_bias, w->q_bias, static_cast<size_t>(c.layers) * P->q_dim * P->wes);
    if (rc == LOKAL_OK && c.has_qk_bias) rc = upload(ctx, &P->k_bias, w->k_bias, static_cast<size_t>(c.layers) * P->kv_dim * P->wes);
    if (rc == LOKAL_OK && c.has_qk_norm) rc = upload(ctx, &P->q_norm_w, w->q_norm_w, static_cast<size_t>(c.layers) * c.head_dim * P->wes);
    if (rc == LOKAL_OK && c.has_qk_norm) rc = upload(ctx, &P->k_norm_w, w->k_norm_w, static_cast<size_t>(c.layers) * c.head_dim * P->wes);
    if (rc == LOKAL_OK) rc = dev_alloc(ctx, &P->x, hid_b);
    if (rc == LOKAL_OK) rc = dev_alloc(ctx, reinterpret_cast<void**>(&P->cos_sin), static_cast<size_t>(c.max_rows) * c.rot_dim * 4);
    if (rc == LOKAL_OK) rc = dev_alloc(ctx, reinterpret_cast<void**>(&P->ids), static_cast<size_t>(c.max_rows) * 4);
    if (rc == LOKAL_OK) rc = dev_alloc(ctx, reinterpret_cast<void**>(&P->positions), static_cast<size_t>(c.max_rows) * 4);
    if (rc == LOKAL_OK) rc = dev_alloc(ctx, &P->out_dev, hid_b);
    if (rc == LOKAL_OK) rc = dev_alloc(ctx, &P->xn0, hid_b);
    if (rc == LOKAL_OK) rc = dev_alloc(ctx, &P->xn_att, hid_b * c.slots);
    if (rc == LOKAL_OK) rc = dev_alloc(ctx, &P->xn_mlp, hid_b * c.slots);
    if (rc == LOKAL_OK) rc = dev_alloc(ctx, &P->inner, static_cast<size_t>(c.max_rows) * c.inter * P->es * c.slots);
    if (rc == LOKAL_OK && cudaStreamCreateWithFlags(&P->copy_stream, cudaStreamNonBlocking) != cudaSuccess) rc = ctx->fail(LOKAL_ERR_CUDA, "cannot create the copy stream");
    if (rc == LOKAL_OK && cudaStreamCreateWithFlags(&P->compute_stream, cudaStreamNonBlocking) != cudaSuccess) rc = ctx->fail(LOKAL_ERR_CUDA, "cannot create the compute stream");
    // The norm chain is the only chain of dependent kernels through the layers, so it is the critical path of a
    // branched step: its stream gets the highest priority, so that its CTAs are placed ahead of CTAs of the others that
    // are still waiting for an SM. (With launches this short nearly all CTAs of all three families are resident at
    // once and nothing waits: measured on B200 the priority changes a step by less than the run-to-run spread.)
    int prio_least = 0, prio_greatest = 0;
    if (cudaDeviceGetStreamPriorityRange(&prio_least, &prio_greatest) != cudaSuccess) prio_least = prio_greatest = 0;
    if (lokal::tune_env("LOKAL_CUDA_PASS_PRIORITY", 1) == 0) prio_greatest = prio_least;
    for (int b = 0; rc == LOKAL_OK && b < 3; b++) {
        if (cudaStreamCreateWithPriority(&P->branch[b], cudaStreamNonBlocking, b == 2 ? prio_greatest : prio_least) != cudaSuccess ||
            cudaEventCreateWithFlags(&P->join_ev[b], cudaEventDisableTiming) != cudaSuccess)
            rc = ctx->fail(LOKAL_ERR_CUDA, "cannot create the branch streams");
    }
    if (rc == LOKAL_OK && cudaEventCreateWithFlags(&P->fork_ev, cudaEventDisableTiming) != cudaSuccess) rc = ctx->fail(LOKAL_ERR_CUDA, "cannot create events");
    for (uint32_t i = 0; rc == LOKAL_OK && i < c.slots; i++) {
        cudaEvent_t a = nullptr, b = nullptr;
        if (cudaEventCreateWithFlags(&a, cudaEventDisableTiming) != cudaSuccess || cudaEventCreateWithFlags(&b, cudaEventDisableTiming) != cudaSuccess)
            rc = ctx->fail(LOKAL_ERR_CUDA, "cannot create events");
        if (a) P->filled.push_back(a);
        if (b) P->drained.push_back(b);
    }
    if (rc != LOKAL_OK) {
        cudaGetLastError();
        lokal_cuda_pass_destroy(ctx, P);
        return rc;
    }
    *out = P;
    return LOKAL_OK;
}

int lokal_cuda_pass_destroy(lokal_cuda_ctx* ctx, lokal_cuda_pass* P) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    if (!P) return LOKAL_OK;
    DeviceGuard guard(ctx->device);
    cudaDeviceSynchronize();
    void* blocks[] = {P->embed_table, P->norm_w, P->final_w, P->q_bias, P->k_bias, P->q_norm_w, P->k_norm_w, P->x, P->cos_sin,
                      P->ids, P->positions, P->out_dev, P->xn0, P->xn_att, P->xn_mlp, P->inner, P->sq, P->sk, P->sda, P->sdm, P->sg, P->su};
    for (void* b : blocks)
        if (b) cudaFree(b);
    for (cudaEvent_t e : P->filled) cudaEventDestroy(e);
    for (cudaEvent_t e : P->drained) cudaEventDestroy(e);
    if (P->copy_stream) cudaStreamDestroy(P->copy_stream);
    if (P->compute_stream) cudaStreamDestroy(P->compute_stream);
    for (int b = 0; b < 3; b++) {
        if (P->branch[b]) cudaStreamDestroy(P->branch[b]);
        if (P->join_ev[b]) cudaEventDestroy(P->join_ev[b]);
    }
    if (P->fork_ev) cudaEventDestroy(P->fork_ev);
    delete P;
    return LOKAL_OK;
}

int lokal_cuda_pass_run_device(lokal_cuda_ctx* ctx, lokal_cuda_pass* P, lokal_cuda_stream stream, const lokal_pass_inputs* in,
                               void* out_dev) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!P || !out_dev) return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_run_device: null argument");
    int rc = check_inputs(ctx, P, in);
    if (rc != LOKAL_OK) return rc;
    std::lock_guard<std::mutex> g(P->mu);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const lokal_pass_config& c = P->cfg;
    P->launches = 0;
    void* saved_out = P->out_dev;
    P->out_dev = out_dev;
    // Schedule. Every input of the step is given up front, so the only chain through the layers is the residual
    // stream x (norm -> norm); the rotations read and write q/k and the table only, SwiGLU reads gate/up and writes
    // inner only. With three branches those families run side by side (fork and join through events, which a stream
    // capture turns into graph edges): the ramp and drain of one family's short kernels is covered by the others.
    // AUTO is the branched schedule: measured on B200 it is the shorter one at every batch size (8192 rows of the
    // 0.6B shapes: 1.60 against 1.84 ms; 1024 rows: 0.27 against 0.37 ms).
    int branches = P->schedule;
    if (branches == LOKAL_PASS_SCHEDULE_AUTO) branches = LOKAL_PASS_SCHEDULE_BRANCHES;
    cudaStream_t s_rope = s, s_mlp = s, s_norm = s;
    if (branches == LOKAL_PASS_SCHEDULE_BRANCHES) {
        s_rope = P->branch[0];
        s_mlp = P->branch[1];
        s_norm = P->branch[2];
        LOKAL_CUDA_TRY(ctx, cudaEventRecord(P->fork_ev, s));
        for (int b = 0; b < 3; b++) LOKAL_CUDA_TRY(ctx, cudaStreamWaitEvent(P->branch[b], P->fork_ev, 0));
    }
    rc = step_head(ctx, P, s_norm, s_rope, in->ids, in->positions, in->pos0, in->rows);
    for (uint32_t l = 0; rc == LOKAL_OK && l < c.layers; l++) {
        rc = layer_ops(ctx, P, s_rope, s_norm, s_mlp, branches == LOKAL_PASS_SCHEDULE_BRANCHES, l, in->rows, at(in->q, l * in->q_layer_stride * P->es), at(in->k, l * in->k_layer_stride * P->es),
                       at(in->delta_att, l * in->delta_layer_stride * P->es), at(in->delta_mlp, l * in->delta_layer_stride * P->es),
                       at(in->gate, l * in->mlp_layer_stride * P->es), at(in->up, l * in->mlp_layer_stride * P->es));
    }
    if (branches == LOKAL_PASS_SCHEDULE_BRANCHES) {  // joined even after a failed launch, so that a capture stays well formed
        cudaError_t e = cudaSuccess;
        for (int b = 0; b < 3 && e == cudaSuccess; b++) {
            e = cudaEventRecord(P->join_ev[b], P->branch[b]);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(s, P->join_ev[b], 0);
        }
        if (e != cudaSuccess && rc == LOKAL_OK) rc = ctx->fail(LOKAL_ERR_CUDA, "pass_run_device: joining the branches failed: %s", cudaGetErrorString(e));
    }
    P->out_dev = saved_out;
    P->last_out = out_dev;
    return rc;
}

int lokal_cuda_pass_run_host(lokal_cuda_ctx* ctx, lokal_cuda_pass* P, const lokal_pass_inputs* in, void* out_host) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!P || !out_host) return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_run_host: null argument");
    int rc = check_inputs(ctx, P, in);
    if (rc != LOKAL_OK) return rc;
    std::lock_guard<std::mutex> g(P->mu);
    const lokal_pass_config& c = P->cfg;
    const size_t R = c.max_rows, rows = in->rows;
    if (!P->sq) {  // staged-input ring, allocated on the first host run
        rc = dev_alloc(ctx, &P->sq, R * P->q_dim * P->es * c.slots);
        if (rc == LOKAL_OK) rc = dev_alloc(ctx, &P->sk, R * P->kv_dim * P->es * c.slots);
        if (rc == LOKAL_OK) rc = dev_alloc(ctx, &P->sda, R * c.hidden * P->es * c.slots);
        if (rc == LOKAL_OK) rc = dev_alloc(ctx, &P->sdm, R * c.hidden * P->es * c.slots);
        if (rc == LOKAL_OK) rc = dev_alloc(ctx, &P->sg, R * c.inter * P->es * c.slots);
        if (rc == LOKAL_OK) rc = dev_alloc(ctx, &P->su, R * c.inter * P->es * c.slots);
        if (rc != LOKAL_OK) return rc;
    }
    cudaStream_t cs = P->copy_stream, ks = P->compute_stream;
    P->launches = 0;
    P->last_out = P->out_dev;
    // ids / positions, then the head of the step
    LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(P->ids, in->ids, rows * 4, cudaMemcpyHostToDevice, ks));
    if (in->positions) LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(P->positions, in->positions, rows * 4, cudaMemcpyHostToDevice, ks));
    rc = step_head(ctx, P, ks, ks, P->ids, in->positions ? P->positions : nullptr, in->pos0, rows);
    if (rc != LOKAL_OK) return rc;
    for (uint32_t l = 0; l < c.layers; l++) {
        const uint32_t slot = l % c.slots;
        void* dq = at(P->sq, slot * R * P->q_dim * P->es);
        void* dk = at(P->sk, slot * R * P->kv_dim * P->es);
        void* dda = at(P->sda, slot * R * c.hidden * P->es);
        void* ddm = at(P->sdm, slot * R * c.hidden * P->es);
        void* dg = at(P->sg, slot * R * c.inter * P->es);
        void* du = at(P->su, slot * R * c.inter * P->es);
        // the slot may be refilled once the kernels of layer l - slots have drained it
        if (l >= c.slots) LOKAL_CUDA_TRY(ctx, cudaStreamWaitEvent(cs, P->drained[slot], 0));
        LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(dq, at(in->q, l * in->q_layer_stride * P->es), rows * P->q_dim * P->es, cudaMemcpyHostToDevice, cs));
        LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(dk, at(in->k, l * in->k_layer_stride * P->es), rows * P->kv_dim * P->es, cudaMemcpyHostToDevice, cs));
        LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(dda, at(in->delta_att, l * in->delta_layer_stride * P->es), rows * c.hidden * P->es, cudaMemcpyHostToDevice, cs));
        LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(dg, at(in->gate, l * in->mlp_layer_stride * P->es), rows * c.inter * P->es, cudaMemcpyHostToDevice, cs));
        LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(du, at(in->up, l * in->mlp_layer_stride * P->es), rows * c.inter * P->es, cudaMemcpyHostToDevice, cs));
        LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(ddm, at(in->delta_mlp, l * in->delta_layer_stride * P->es), rows * c.hidden * P->es, cudaMemcpyHostToDevice, cs));
        LOKAL_CUDA_TRY(ctx, cudaEventRecord(P->filled[slot], cs));
        LOKAL_CUDA_TRY(ctx, cudaStreamWaitEvent(ks, P->filled[slot], 0));
        rc = layer_ops(ctx, P, ks, ks, ks, false, l, rows, dq, dk, dda, ddm, dg, du);
        if (rc != LOKAL_OK) return rc;
        LOKAL_CUDA_TRY(ctx, cudaEventRecord(P->drained[slot], ks));
    }
    LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(out_host, P->out_dev, rows * c.hidden * P->es, cudaMemcpyDeviceToHost, ks));
    LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(ks));
    LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(cs));
    // device-side error word (out-of-range ids, bounded waits)
    LOKAL_CUDA_TRY(ctx, cudaMemcpy(ctx->err_word_host, ctx->err_word, sizeof(unsigned), cudaMemcpyDeviceToHost));
    const unsigned bits = *ctx->err_word_host;
    if (bits) {
        LOKAL_CUDA_TRY(ctx, cudaMemset(ctx->err_word, 0, sizeof(unsigned)));
        if (bits & lokal::kErrTimeout) return ctx->fail(LOKAL_ERR_TIMEOUT, "a device-side wait on a staged copy gave up");
        if (bits & lokal::kErrPosRange) return ctx->fail(LOKAL_ERR_POS_RANGE, "a position was negative or beyond the KV cache (its row was not stored)");
        return ctx->fail(LOKAL_ERR_ID_RANGE, "a token id was out of range for the table (its row was zero-filled)");
    }
    return LOKAL_OK;
}

int lokal_cuda_pass_output(lokal_cuda_ctx* ctx, lokal_cuda_pass* P, uint32_t layer, int which, void** dptr) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    if (!P || !dptr || layer >= P->cfg.layers) return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_output: bad argument");
    const lokal_pass_config& c = P->cfg;
    const size_t slot = layer % c.slots, R = c.max_rows;
    switch (which) {
        case 0: *dptr = at(P->xn_att, slot * R * c.hidden * P->es); break;
        case 1: *dptr = (layer + 1 < c.layers) ? at(P->xn_mlp, slot * R * c.hidden * P->es) : P->last_out; break;
        case 2: *dptr = at(P->inner, slot * R * c.inter * P->es); break;
        case 3: *dptr = P->sq ? at(P->sq, slot * R * P->q_dim * P->es) : nullptr; break;
        case 4: *dptr = P->sk ? at(P->sk, slot * R * P->kv_dim * P->es) : nullptr; break;
        default: return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_output: unknown output %d", which);
    }
    return LOKAL_OK;
}

uint64_t lokal_cuda_pass_launches(const lokal_cuda_pass* P) { return P ? P->launches : 0; }

int lokal_cuda_pass_set_schedule(lokal_cuda_ctx* ctx, lokal_cuda_pass* P, int schedule) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    if (!P) return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_set_schedule: pass is null");
    if (schedule != LOKAL_PASS_SCHEDULE_AUTO && schedule != LOKAL_PASS_SCHEDULE_SEQUENTIAL && schedule != LOKAL_PASS_SCHEDULE_BRANCHES)
        return ctx->fail(LOKAL_ERR_BAD_ARG, "pass_set_schedule: unknown schedule %d", schedule);
    std::lock_guard<std::mutex> g(P->mu);
    P->schedule = schedule;
    return LOKAL_OK;
}

}  // extern "C"
