// The C ABI: argument validation, handle lifetime, launch sequencing.
// No entry point below allocates after shrike_moe_create / shrike_pool_create /
// shrike_residency_create.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "internal.h"

using namespace shrike;

namespace {

thread_local std::string g_create_error;

int fail(shrike_moe* m, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (m) m->err = buf; else g_create_error = buf;
    return code;
}

int cuda_fail(shrike_moe* m, cudaError_t e, const char* what) {
    return fail(m, SHRIKE_EIO, "%s: %s", what, cudaGetErrorString(e));
}

#define CU(call)                                                  \
    do {                                                          \
        cudaError_t e_ = (call);                                  \
        if (e_ != cudaSuccess) return cuda_fail(m, e_, #call);    \
    } while (0)

bool valid_config(const shrike_moe_config& c, std::string& why) {
    auto bad = [&](const char* s) { why = s; return false; };
    if (c.d == 0 || c.d % 64 != 0 || c.d > 2944) return bad("d must be a multiple of 64, at most 2944");
    if (c.f == 0 || c.f % 64 != 0) return bad("f must be a multiple of 64");
    if (c.num_experts == 0 || c.num_experts > SHRIKE_MAX_EXPERTS) return bad("num_experts must be 1..256");
    if (c.top_k == 0 || c.top_k > SHRIKE_MAX_TOP_K || c.top_k > c.num_experts) return bad("top_k must be 1..8 and <= num_experts");
    if (c.weight_bits != 4 && c.weight_bits != 8) return bad("weight_bits must be 4 or 8");
    if (c.group_size != 32 && c.group_size != 64) return bad("group_size must be 32 or 64");
    if (c.meta_dtype > SHRIKE_DTYPE_FP16) return bad("meta_dtype must be BF16 or FP16");
    if (c.act_dtype > SHRIKE_DTYPE_FP32) return bad("act_dtype must be BF16, FP16 or FP32");
    if (c.activation > SHRIKE_ACT_CLAMPED_SWIGLU) return bad("unknown activation");
    if (c.router_kind > SHRIKE_ROUTER_SIGMOID) return bad("unknown router_kind");
    if (c.router_weight_bits != 0 && c.router_weight_bits != 4 && c.router_weight_bits != 8) return bad("router_weight_bits must be 0, 4 or 8");
    if (c.has_shared && (c.shared_f == 0 || c.shared_f % 64 != 0)) return bad("shared_f must be a multiple of 64");
    if (c.shared_gated && !c.has_shared) return bad("shared_gated needs has_shared");
    if (c.max_tokens == 0 || c.max_tokens > 65536) return bad("max_tokens must be 1..65536");
    if (c.y_dtype > SHRIKE_DTYPE_FP32) return bad("y_dtype must be BF16, FP16 or FP32");
    return true;
}

void make_offsets(const shrike_moe_config& c, bool shared, shrike_expert_offsets& o, uint64_t& bytes) {
    const uint32_t f = shared ? c.shared_f : c.f;
    const uint32_t rows[3] = {f, f, c.d}, cols[3] = {c.d, c.d, f};
    uint32_t w[3], s[3], b[3], ab[3];
    uint64_t cur = 0;
    for (int p = 0; p < 3; ++p) {
        const uint64_t wb = (uint64_t)rows[p] * (cols[p] * c.weight_bits / 8);
        const uint64_t mb = (uint64_t)rows[p] * (cols[p] / c.group_size) * 2;
        w[p] = (uint32_t)cur; cur += wb;
        s[p] = (uint32_t)cur; cur += mb;
        b[p] = (uint32_t)cur; cur += mb;
        if (c.expert_bias) { ab[p] = (uint32_t)cur; cur += rows[p] * 2; } else ab[p] = 0;
    }
    o.gate_w = w[0]; o.gate_s = s[0]; o.gate_b = b[0]; o.gate_ab = ab[0];
    o.up_w = w[1]; o.up_s = s[1]; o.up_b = b[1]; o.up_ab = ab[1];
    o.down_w = w[2]; o.down_s = s[2]; o.down_b = b[2]; o.down_ab = ab[2];
    bytes = cur;
}

bool offsets_aligned(const shrike_expert_offsets& o) {
    const uint32_t* p = &o.gate_w;
    for (int i = 0; i < 12; ++i)
        if (p[i] % 16 != 0) return false;
    return true;
}

// Every encode call launches on the current device against this handle's workspace and pool.
int check_device(shrike_moe* m) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != m->device)
        return fail(m, SHRIKE_EINVAL, "the handle lives on device %d but device %d is current", m->device, dev);
    return SHRIKE_OK;
}

bool aligned_to(const void* p, uintptr_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

// Makes `device` current for the scope and puts the caller's device back afterwards.
struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int device) {
        cudaGetDevice(&prev);
        if (prev != device) cudaSetDevice(device);
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

}  // namespace

namespace shrike {
// What the router kernels' vector loads rely on; `why` receives the first violation.
bool router_operands_aligned(const shrike_moe_config& c, const shrike_router_operands& o, const void* hidden,
                             const char** why) {
    auto bad = [&](const char* s) { *why = s; return false; };
    if (!aligned_to(hidden, c.act_dtype == SHRIKE_DTYPE_FP32 ? 16 : 8))
        return bad("hidden must be 16-byte aligned (fp32) or 8-byte aligned (16-bit activations)");
    if (!aligned_to(o.weights, 16)) return bad("router weights must be 16-byte aligned");
    if (o.shared_gate && !aligned_to(o.shared_gate, 16)) return bad("shared_gate must be 16-byte aligned");
    if (o.effective_scale && !aligned_to(o.effective_scale, 8)) return bad("effective_scale must be 8-byte aligned");
    if (!aligned_to(o.scales, 2) || !aligned_to(o.biases, 2) || !aligned_to(o.logit_bias, 2) ||
        !aligned_to(o.per_expert_scale, 2))
        return bad("scales, biases, logit_bias and per_expert_scale must be 2-byte aligned");
    return true;
}
}  // namespace shrike

namespace {

template <typename P>
cudaError_t dev_alloc(P** p, size_t bytes) {
    return cudaMalloc((void**)p, bytes ? bytes : 16);
}

void free_workspace(Workspace& w) {
    void* ptrs[] = {w.fused_logits, w.fused_acts, w.fused_epoch, w.yacc, w.xs, w.chunk_inst, w.n_chunk_inst, w.done_counter, w.xsum, w.logits, w.xh, w.acts, w.acts_shared, w.sorted, w.inst, w.n_inst, w.status, w.block_hist,
                    w.expert_offsets, w.expert_counts, w.slot_of_expert, w.x_dev, w.y_dev,
                    w.ids_dev, w.w_dev, w.gate_dev, w.slots_dev, w.counts_dev};
    for (void* p : ptrs)
        if (p) cudaFree(p);
    free(w.tensor_maps);
    free(w.fused_geom);
    free(w.fused_maps);
    w = Workspace();
}

int fill_expert_args(shrike_moe* m, const shrike_pool* pool, const shrike_expert_offsets* ro,
                     const shrike_shared_expert* shared, const float* weights, const float* shared_gate,
                     ExpertArgs& a, bool check_gate = true) {
    const shrike_moe_config& c = m->cfg;
    if (!pool || !ro) return fail(m, SHRIKE_EINVAL, "pool and routed_offsets are required");
    if (!offsets_aligned(*ro)) return fail(m, SHRIKE_EINVAL, "routed offsets must be multiples of 16 bytes");
    if (c.has_shared) {
        if (!shared || !shared->block) return fail(m, SHRIKE_EINVAL, "this handle was created with a shared expert; pass it");
        if (!offsets_aligned(shared->offsets) || ((uintptr_t)shared->block & 15))
            return fail(m, SHRIKE_EINVAL, "shared expert block and offsets must be 16-byte aligned");
    }
    if (check_gate && shared_gate && !c.shared_gated) return fail(m, SHRIKE_EINVAL, "shared_gate given but the handle is not shared_gated");
    if (check_gate && c.shared_gated && !shared_gate) return fail(m, SHRIKE_EINVAL, "shared_gated handle needs the router's shared_gate output");
    memset(&a, 0, sizeof a);
    a.pool = pool->view;
    a.routed = to_offsets3(*ro);
    if (c.has_shared) {
        a.shared = to_offsets3(shared->offsets);
        a.shared_block = (const uint8_t*)shared->block;
    }
    a.d = c.d; a.f = c.f; a.f_shared = c.has_shared ? c.shared_f : 0; a.top_k = c.top_k;
    a.activation = c.activation; a.expert_bias = c.expert_bias; a.act_dtype = c.act_dtype; a.y_dtype = c.y_dtype;
    a.inst = m->ws.inst; a.n_inst = m->ws.n_inst; a.sorted = m->ws.sorted; a.xh = m->ws.xh;
    a.xsum = m->ws.xsum;
    a.acts = m->ws.acts; a.acts_shared = m->ws.acts_shared; a.yacc = m->ws.yacc;
    a.route_w = weights; a.shared_gate = shared_gate; a.status = m->ws.status;
#ifdef SHRIKE_TRACE
    a.trace = m->trace;
#endif
    return SHRIKE_OK;
}


// The prefill call with the status word of a streamed batch (moe.metal:36-39, 918-921): when io_status is
// given and the word is neither READY nor 3, the routed experts are skipped and y is the shared term alone.
int encode_prefill(shrike_moe* m, void* stream, const shrike_pool* pool,
                   const shrike_expert_offsets* routed_offsets, const uint32_t* topk_indices,
                   const uint32_t* resolved_slots, const float* routing_weights, const void* x,
                   uint32_t query_count, const shrike_shared_expert* shared, const float* shared_gate,
                   const uint32_t* io_status, void* y, void* hidden) {
    if (!m) return SHRIKE_EINVAL;
    if (!topk_indices || !resolved_slots || !routing_weights || !x || !y)
        return fail(m, SHRIKE_EINVAL, "prefill: null operand");
    if (query_count > m->cfg.max_tokens) return fail(m, SHRIKE_ERANGE, "query_count exceeds max_tokens");
    if (m->cfg.max_tokens <= SHRIKE_MAX_DECODE_TOKENS)
        return fail(m, SHRIKE_EINVAL, "handle was created for decode only (max_tokens <= %u)", SHRIKE_MAX_DECODE_TOKENS);
    if (query_count == 0) return SHRIKE_OK;
    ExpertArgs a;
    int rc = fill_expert_args(m, pool, routed_offsets, shared, routing_weights, shared_gate, a);
    if (rc) return rc;
    if ((rc = check_device(m))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t mi = max_instances(m->cfg, query_count);
    // The expert-grouped GEMM runs on the tcgen05 tensor cores. Shapes whose K is not a multiple of 64 keep
    // every expert on the 8-row warp-MMA tiles (the decode kernels); SHRIKE_PREFILL_PATH=mma in the
    // environment of shrike_moe_create forces them for a handle (a test switch).
    const bool warp_mma = m->force_warp_mma || !umma_supported(m->cfg);
    // fp32 rows out and no residual to add: the down epilogue adds straight into y (zeroed by the plan; x is read
    // after that, so not when y is x) and no pass over the rows follows
    const bool direct = m->cfg.y_dtype == SHRIKE_DTYPE_FP32 && !hidden && y != x;
    if (direct) a.yacc = (float*)y;
    CU(launch_prefill_plan(m, st, topk_indices, resolved_slots, x, query_count, m->cfg.has_shared != 0,
                           pool->view.cells, warp_mma, io_status, nullptr, nullptr, direct ? (float*)y : nullptr));
    if (warp_mma) {
        CU(launch_phase1(m, st, a, mi, false));
        CU(launch_phase2_accumulate(m, st, a, mi));
    } else {
        CU(launch_umma_prefill(m, st, a, query_count, pool->view.cells));
    }
    if (!direct) CU(launch_prefill_combine(m, st, query_count, y, hidden));
    return SHRIKE_OK;
}

}  // namespace

namespace shrike {
size_t act_bytes(uint32_t dt) { return dt == SHRIKE_DTYPE_FP32 ? 4 : 2; }
}

extern "C" {

const char* shrike_last_error(const shrike_moe* moe) {
    return moe ? moe->err.c_str() : g_create_error.c_str();
}

int shrike_expert_offsets_make(const shrike_moe_config* config, int shared, shrike_expert_offsets* out,
                               uint64_t* block_bytes) {
    std::string why;
    if (!config || !out) return fail(nullptr, SHRIKE_EINVAL, "null argument");
    if (!valid_config(*config, why)) return fail(nullptr, SHRIKE_EINVAL, "%s", why.c_str());
    if (shared && !config->has_shared) return fail(nullptr, SHRIKE_EINVAL, "config has no shared expert");
    uint64_t bytes;
    make_offsets(*config, shared != 0, *out, bytes);
    if (block_bytes) *block_bytes = bytes;
    return SHRIKE_OK;
}

int shrike_moe_create(const shrike_moe_config* config, int device, shrike_moe** out) {
    if (!config || !out) return fail(nullptr, SHRIKE_EINVAL, "null argument");
    *out = nullptr;
    std::string why;
    if (!valid_config(*config, why)) return fail(nullptr, SHRIKE_EINVAL, "%s", why.c_str());
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(nullptr, SHRIKE_EIO, "no CUDA device: %s (this library has no CPU path)",
                    cudaGetErrorString(e));
    if (device < 0 || device >= count) return fail(nullptr, SHRIKE_ERANGE, "device %d out of range", device);
    int caller_device = device;
    cudaGetDevice(&caller_device);
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaSetDevice");
    // the caller's current device is put back on every way out
    struct Restore { int dev; ~Restore() { cudaSetDevice(dev); } } restore{caller_device};
    shrike_moe* m = new (std::nothrow) shrike_moe();
    if (!m) return fail(nullptr, SHRIKE_ENOMEM, "host allocation failed");
    m->cfg = *config;
    m->device = device;
    cudaDeviceGetAttribute(&m->sm_count, cudaDevAttrMultiProcessorCount, device);
    // switches for tests and diagnostics, read once here and never on the per-layer path
    m->no_pdl = getenv("SHRIKE_NO_PDL") != nullptr;
    m->single_stream = getenv("SHRIKE_SINGLE_STREAM") != nullptr;
    const char* path = getenv("SHRIKE_PREFILL_PATH");
    m->force_warp_mma = path && strcmp(path, "mma") == 0;
    const shrike_moe_config& c = m->cfg;
    Workspace& w = m->ws;
    const size_t T = c.max_tokens, K = c.top_k;
    w.max_inst = max_instances(c, c.max_tokens);
    const size_t ab = act_bytes(c.act_dtype), yb = act_bytes(c.y_dtype);
    bool ok = true;
    auto A = [&](auto** p, size_t bytes) { if (ok && dev_alloc(p, bytes) != cudaSuccess) ok = false; };
    A(&w.logits, T * c.num_experts * 4);
    A(&w.xh, T * c.d * 2);
    A(&w.xsum, T * (c.d / c.group_size) * 4);
    A(&w.acts, T * K * c.f * 2);
    A(&w.acts_shared, c.has_shared ? T * c.shared_f * 2 : 0);
    A(&w.sorted, T * K * 4);
    A(&w.inst, (size_t)w.max_inst * sizeof(Instance));
    A(&w.n_inst, 4);
    A(&w.status, 4);
    A(&w.done_counter, 4);
    A(&w.block_hist, ((T + 127) / 128) * c.num_experts * 4);
    A(&w.expert_offsets, c.num_experts * 4);
    A(&w.expert_counts, c.num_experts * 4);
    A(&w.slot_of_expert, c.num_experts * 4);
    A(&w.yacc, T > SHRIKE_MAX_DECODE_TOKENS ? T * c.d * 4 : 0);
    A(&w.chunk_inst, T > SHRIKE_MAX_DECODE_TOKENS ? umma_max_chunk_instances(c, c.max_tokens) * umma_chunk_instance_bytes() : 0);
    A(&w.n_chunk_inst, 8);
    A(&w.xs, T > SHRIKE_MAX_DECODE_TOKENS ? T * K * c.d * 2 : 0);
    A(&w.x_dev, T * c.d * ab);
    A(&w.y_dev, T * c.d * yb);
    A(&w.ids_dev, T * K * 4);
    A(&w.w_dev, T * K * 4);
    A(&w.gate_dev, T * 4);
    A(&w.slots_dev, T * K * 4);
    A(&w.counts_dev, 8);
    // the one-row layer kernel: sizes of its shared-memory ring, and its hand-over buffers
    int smem_optin = 0;
    cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    w.fused_geom = malloc(fused_geom_bytes());
    w.fused_maps = calloc(1, fused_map_cache_bytes());
    if (w.fused_geom && w.fused_maps && fused_geometry(c, m->sm_count, smem_optin, *(FusedGeom*)w.fused_geom)) {
        A((uint8_t**)&w.fused_logits, fused_logits_bytes(c));
        A(&w.fused_acts, fused_acts_bytes(c));
        A(&w.fused_epoch, 4);
    } else {
        free(w.fused_geom);
        free(w.fused_maps);
        w.fused_geom = nullptr;
        w.fused_maps = nullptr;
    }
    if (!ok) {
        free_workspace(w);
        delete m;
        cudaGetLastError();
        return fail(nullptr, SHRIKE_ENOMEM, "device allocation of the workspace failed");
    }
    if (w.fused_geom) {
        // no logit carries the first epoch's tag, no activation has been published
        cudaMemset(w.fused_logits, 0xff, fused_logits_bytes(c));
        cudaMemset(w.fused_acts, 0xff, fused_acts_bytes(c));
        cudaMemset(w.fused_epoch, 0, 4);
    }
    if (T <= SHRIKE_MAX_DECODE_TOKENS) {   // decode-only handle: no prefill operands
        cudaFree(w.xs);
        w.xs = nullptr;
    } else {
        w.tensor_maps = aligned_alloc(64, umma_tensor_map_bytes());
        const cudaError_t me = w.tensor_maps ? umma_prepare(m) : cudaErrorMemoryAllocation;
        if (me != cudaSuccess) {
            free_workspace(w);
            delete m;
            cudaGetLastError();
            return fail(nullptr, SHRIKE_EIO, "TMA descriptors of the prefill operands: %s", cudaGetErrorString(me));
        }
    }
    cudaMemset(w.status, 0, 4);
    cudaMemset(w.done_counter, 0, 4);
    cudaMemset(w.n_inst, 0, 4);
    *out = m;
    return SHRIKE_OK;
}

void shrike_moe_destroy(shrike_moe* moe) {
    if (!moe) return;
    DeviceGuard guard(moe->device);
    free_workspace(moe->ws);
    if (moe->residency) cudaFree(moe->residency);
    delete moe;
}

int shrike_moe_status(shrike_moe* m, void* stream) {
    if (!m) return SHRIKE_EINVAL;
    CU(cudaStreamSynchronize((cudaStream_t)stream));
    uint32_t st = 0;
    CU(cudaMemcpy(&st, m->ws.status, 4, cudaMemcpyDeviceToHost));
    if (st != kStatusOk) {
        cudaMemset(m->ws.status, 0, 4);
        if (st == kStatusWaitTimeout) return fail(m, SHRIKE_ETIMEDOUT, "a device-side wait gave up");
        if (st == kStatusOperandRange)
            return fail(m, SHRIKE_ERANGE, "an activation beyond the fp16 operand range (|x| > 65504) was clamped");
        return fail(m, SHRIKE_ERANGE, "a kernel met a slot id outside the pool");
    }
    return SHRIKE_OK;
}

#ifdef SHRIKE_TRACE
int shrike_debug_set_trace(shrike_moe* m, uint64_t* trace_device_buffer) {
    if (!m) return SHRIKE_EINVAL;
    m->trace = trace_device_buffer;
    return SHRIKE_OK;
}
#endif

// ---- pool -------------------------------------------------------------------

int shrike_pool_create(shrike_moe* m, uint32_t cells, uint64_t cell_stride, uint32_t chunks,
                       shrike_pool** out) {
    if (!m || !out) return SHRIKE_EINVAL;
    *out = nullptr;
    if (cells == 0 || chunks == 0 || chunks > SHRIKE_MAX_POOL_CHUNKS)
        return fail(m, SHRIKE_EINVAL, "cells must be > 0 and chunks 1..8");
    if (cell_stride == 0 || cell_stride % 256 != 0)
        return fail(m, SHRIKE_EINVAL, "cell_stride must be a positive multiple of 256 bytes");
    DeviceGuard guard(m->device);
    shrike_pool* p = new (std::nothrow) shrike_pool();
    if (!p) return fail(m, SHRIKE_ENOMEM, "host allocation failed");
    memset(p, 0, sizeof *p);
    p->owner = m;
    p->chunks = chunks;
    p->view.cells = cells;
    p->view.stride = cell_stride;
    p->view.cells_per_chunk = (cells + chunks - 1) / chunks;
    for (uint32_t i = 0; i < SHRIKE_MAX_POOL_CHUNKS; ++i) p->view.base[i] = nullptr;
    for (uint32_t i = 0; i < chunks; ++i) {
        const uint64_t first = (uint64_t)i * p->view.cells_per_chunk;
        if (first >= cells) { p->chunks = i; break; }
        const uint64_t n = (first + p->view.cells_per_chunk <= cells) ? p->view.cells_per_chunk : cells - first;
        cudaError_t e = cudaMalloc(&p->chunk[i], n * cell_stride);
        if (e != cudaSuccess) {
            for (uint32_t j = 0; j < i; ++j) cudaFree(p->chunk[j]);
            delete p;
            cudaGetLastError();
            return fail(m, SHRIKE_ENOMEM, "pool chunk of %llu bytes: %s", (unsigned long long)(n * cell_stride),
                        cudaGetErrorString(e));
        }
        p->view.base[i] = (const uint8_t*)p->chunk[i];
    }
    *out = p;
    return SHRIKE_OK;
}

void shrike_pool_destroy(shrike_pool* pool) {
    if (!pool) return;
    DeviceGuard guard(pool->owner->device);
    for (uint32_t i = 0; i < pool->chunks; ++i)
        if (pool->chunk[i]) cudaFree(pool->chunk[i]);
    delete pool;
}

int shrike_pool_cell_address(const shrike_pool* pool, uint32_t cell, void** out) {
    if (!pool || !out) return SHRIKE_EINVAL;
    if (cell >= pool->view.cells) return fail(pool->owner, SHRIKE_ERANGE, "cell %u out of range", cell);
    *out = (void*)pool_cell_base(pool->view, cell);
    return SHRIKE_OK;
}

int shrike_pool_upload(shrike_pool* pool, uint32_t cell, const void* block_host, uint64_t bytes, void* stream) {
    if (!pool || !block_host) return SHRIKE_EINVAL;
    shrike_moe* m = pool->owner;
    if (cell >= pool->view.cells) return fail(m, SHRIKE_ERANGE, "cell %u out of range", cell);
    if (bytes > pool->view.stride) return fail(m, SHRIKE_ERANGE, "block larger than the cell stride");
    CU(cudaMemcpyAsync((void*)pool_cell_base(pool->view, cell), block_host, bytes, cudaMemcpyHostToDevice,
                       (cudaStream_t)stream));
    return SHRIKE_OK;
}

int shrike_pool_download(shrike_pool* pool, uint32_t cell, void* block_host, uint64_t bytes, void* stream) {
    if (!pool || !block_host) return SHRIKE_EINVAL;
    shrike_moe* m = pool->owner;
    if (cell >= pool->view.cells) return fail(m, SHRIKE_ERANGE, "cell %u out of range", cell);
    if (bytes > pool->view.stride) return fail(m, SHRIKE_ERANGE, "block larger than the cell stride");
    CU(cudaMemcpyAsync(block_host, pool_cell_base(pool->view, cell), bytes, cudaMemcpyDeviceToHost,
                       (cudaStream_t)stream));
    CU(cudaStreamSynchronize((cudaStream_t)stream));
    return SHRIKE_OK;
}

int shrike_pool_fill_synthetic(shrike_moe* m, shrike_pool* pool, uint32_t first_cell, uint32_t count,
                               uint64_t seed, uint32_t layer, uint32_t first_expert, int shared, void* stream) {
    if (!m || !pool) return SHRIKE_EINVAL;
    if ((uint64_t)first_cell + count > pool->view.cells) return fail(m, SHRIKE_ERANGE, "cells out of range");
    if (shared && !m->cfg.has_shared) return fail(m, SHRIKE_EINVAL, "no shared expert in this config");
    shrike_expert_offsets o;
    uint64_t bytes;
    make_offsets(m->cfg, shared != 0, o, bytes);
    if (bytes > pool->view.stride) return fail(m, SHRIKE_ERANGE, "block larger than the cell stride");
    if (count == 0) return SHRIKE_OK;
    CU(launch_synth_fill(m, (cudaStream_t)stream, pool->view, first_cell, count, seed, layer, first_expert,
                         shared != 0, to_offsets3(o)));
    return SHRIKE_OK;
}

// ---- residency ----------------------------------------------------------------

int shrike_residency_create(shrike_moe* m, uint32_t layers, uint64_t** table_out) {
    if (!m || layers == 0) return SHRIKE_EINVAL;
    DeviceGuard guard(m->device);
    if (m->residency) { cudaFree(m->residency); m->residency = nullptr; }
    const size_t n = (size_t)layers * m->cfg.num_experts;
    cudaError_t e = cudaMalloc((void**)&m->residency, n * 8);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(m, SHRIKE_ENOMEM, "residency table: %s", cudaGetErrorString(e)); }
    // every entry: state 0 (absent)
    CU(cudaMemset(m->residency, 0, n * 8));
    m->residency_layers = layers;
    if (table_out) *table_out = m->residency;
    return SHRIKE_OK;
}

__global__ void residency_identity_kernel(uint64_t* row, uint32_t ne, uint32_t first_cell) {
    const uint32_t e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < ne) row[e] = ((uint64_t)2 << 32) | (uint64_t)(first_cell + e);
}

__global__ void residency_set_kernel(uint64_t* word, uint64_t value) {
    // one 64-bit store: the reader sees the old or the new {slot, state}, never a mix
    *(volatile uint64_t*)word = value;
}

int shrike_residency_set(shrike_moe* m, uint32_t layer, uint32_t expert, uint32_t slot, uint32_t state,
                         void* stream) {
    if (!m || !m->residency) return SHRIKE_EINVAL;
    if (layer >= m->residency_layers || expert >= m->cfg.num_experts)
        return fail(m, SHRIKE_ERANGE, "layer %u / expert %u out of range", layer, expert);
    const uint64_t v = ((uint64_t)state << 32) | slot;
    residency_set_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(
        m->residency + (size_t)layer * m->cfg.num_experts + expert, v);
    CU(cudaGetLastError());
    return SHRIKE_OK;
}

int shrike_residency_set_layer_identity(shrike_moe* m, uint32_t layer, uint32_t first_cell, void* stream) {
    if (!m || !m->residency) return SHRIKE_EINVAL;
    if (layer >= m->residency_layers) return fail(m, SHRIKE_ERANGE, "layer %u out of range", layer);
    residency_identity_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(
        m->residency + (size_t)layer * m->cfg.num_experts, m->cfg.num_experts, first_cell);
    CU(cudaGetLastError());
    return SHRIKE_OK;
}

// ---- the path -------------------------------------------------------------------

// Argument checks shared by the router entry points: operands, counts, stride, alignment.
static int check_router_call(shrike_moe* m, const shrike_router_operands* ops, const void* hidden,
                             uint32_t query_count, uint32_t limit, uint32_t hidden_stride_elements,
                             bool need_gate_out, const void* out_shared_gate) {
    const shrike_moe_config& c = m->cfg;
    if (!ops || !ops->weights || !hidden) return fail(m, SHRIKE_EINVAL, "router: null operand");
    if (c.router_weight_bits != 0 && (!ops->scales || !ops->biases))
        return fail(m, SHRIKE_EINVAL, "router: affine weights need scales and biases");
    if (query_count > limit) return fail(m, SHRIKE_ERANGE, "query_count %u exceeds %u", query_count, limit);
    if (hidden_stride_elements < c.d || hidden_stride_elements % 4 != 0)
        return fail(m, SHRIKE_EINVAL, "hidden stride must be >= d and a multiple of 4 elements");
    if (c.shared_gated && (!ops->shared_gate || (need_gate_out && !out_shared_gate)))
        return fail(m, SHRIKE_EINVAL, "router: a shared_gated handle needs shared_gate and out_shared_gate");
    const char* why = nullptr;
    if (!router_operands_aligned(c, *ops, hidden, &why)) return fail(m, SHRIKE_EINVAL, "router: %s", why);
    return SHRIKE_OK;
}

int shrike_encode_router(shrike_moe* m, void* stream, const shrike_router_operands* ops, const void* hidden,
                         uint32_t query_count, uint32_t hidden_stride_elements, uint32_t* out_indices,
                         float* out_weights, float* out_shared_gate) {
    if (!m) return SHRIKE_EINVAL;
    if (query_count == 0) return SHRIKE_OK;
    if (!out_indices || !out_weights) return fail(m, SHRIKE_EINVAL, "router: null operand");
    int rc = check_router_call(m, ops, hidden, query_count, m->cfg.max_tokens, hidden_stride_elements, true,
                               out_shared_gate);
    if (rc) return rc;
    if ((rc = check_device(m))) return rc;
    CU(launch_router(m, (cudaStream_t)stream, *ops, hidden, query_count, hidden_stride_elements, out_indices,
                     out_weights, out_shared_gate));
    return SHRIKE_OK;
}

int shrike_encode_residency_classification(shrike_moe* m, void* stream, const uint32_t* topk_indices,
                                           const uint64_t* residency_table_row, uint32_t query_count,
                                           uint32_t* resolved_slots, uint32_t* counts,
                                           uint32_t* miss_positions, uint32_t* miss_experts) {
    if (!m) return SHRIKE_EINVAL;
    if (!topk_indices || !residency_table_row || !resolved_slots)
        return fail(m, SHRIKE_EINVAL, "classification: null operand");
    if (query_count > m->cfg.max_tokens) return fail(m, SHRIKE_ERANGE, "query_count exceeds max_tokens");
    if (int rc = check_device(m)) return rc;
    if (query_count == 0) {
        if (counts) CU(cudaMemsetAsync(counts, 0, 8, (cudaStream_t)stream));
        return SHRIKE_OK;
    }
    CU(launch_classify(m, (cudaStream_t)stream, topk_indices, residency_table_row, query_count, resolved_slots,
                       counts, miss_positions, miss_experts));
    return SHRIKE_OK;
}

int shrike_encode_decode_plan(shrike_moe* m, void* stream, const shrike_pool* pool,
                              const uint32_t* resolved_slots, const void* x, uint32_t query_count,
                              const uint32_t* io_status) {
    if (!m) return SHRIKE_EINVAL;
    if (!pool || !resolved_slots || !x) return fail(m, SHRIKE_EINVAL, "decode plan: null operand");
    if (query_count == 0 || query_count > SHRIKE_MAX_DECODE_TOKENS || query_count > m->cfg.max_tokens)
        return fail(m, SHRIKE_ERANGE, "decode handles 1..%u rows (max_tokens %u); use the prefill call",
                    SHRIKE_MAX_DECODE_TOKENS, m->cfg.max_tokens);
    if (int rc = check_device(m)) return rc;
    CU(launch_decode_plan(m, (cudaStream_t)stream, resolved_slots, x, query_count, io_status,
                          m->cfg.has_shared != 0, pool->view.cells));
    return SHRIKE_OK;
}

int shrike_encode_phase1(shrike_moe* m, void* stream, const shrike_pool* pool,
                         const shrike_expert_offsets* routed_offsets, const shrike_shared_expert* shared,
                         uint32_t query_count) {
    if (!m) return SHRIKE_EINVAL;
    if (query_count == 0 || query_count > SHRIKE_MAX_DECODE_TOKENS || query_count > m->cfg.max_tokens)
        return fail(m, SHRIKE_ERANGE, "phase 1: query_count out of range");
    ExpertArgs a;
    int rc = fill_expert_args(m, pool, routed_offsets, shared, nullptr, nullptr, a, false);
    if (rc) return rc;
    if ((rc = check_device(m))) return rc;
    CU(launch_phase1(m, (cudaStream_t)stream, a, max_instances(m->cfg, query_count), false));
    return SHRIKE_OK;
}

int shrike_encode_phase2_reduce(shrike_moe* m, void* stream, const shrike_pool* pool,
                                const shrike_expert_offsets* routed_offsets, const float* routing_weights,
                                const shrike_shared_expert* shared, const float* shared_gate,
                                uint32_t query_count, void* y, void* hidden) {
    if (!m) return SHRIKE_EINVAL;
    if (!routing_weights || !y) return fail(m, SHRIKE_EINVAL, "phase 2: null operand");
    if (query_count == 0 || query_count > SHRIKE_MAX_DECODE_TOKENS || query_count > m->cfg.max_tokens)
        return fail(m, SHRIKE_ERANGE, "phase 2: query_count out of range");
    ExpertArgs a;
    int rc = fill_expert_args(m, pool, routed_offsets, shared, routing_weights, shared_gate, a, true);
    if (rc) return rc;
    if ((rc = check_device(m))) return rc;
    CU(launch_phase2(m, (cudaStream_t)stream, a, query_count, max_instances(m->cfg, query_count), y, hidden, false));
    return SHRIKE_OK;
}

int shrike_encode_moe_decode(shrike_moe* m, void* stream, const shrike_pool* pool,
                             const shrike_expert_offsets* routed_offsets, const uint32_t* resolved_slots,
                             const float* routing_weights, const void* x, uint32_t query_count,
                             const shrike_shared_expert* shared, const float* shared_gate,
                             const uint32_t* io_status, void* y, void* hidden) {
    if (!m) return SHRIKE_EINVAL;
    if (query_count == 0) return SHRIKE_OK;
    if (!resolved_slots || !routing_weights || !x || !y) return fail(m, SHRIKE_EINVAL, "decode: null operand");
    int rc = shrike_encode_decode_plan(m, stream, pool, resolved_slots, x, query_count, io_status);
    if (rc) return rc;
    rc = shrike_encode_phase1(m, stream, pool, routed_offsets, shared, query_count);
    if (rc) return rc;
    return shrike_encode_phase2_reduce(m, stream, pool, routed_offsets, routing_weights, shared, shared_gate,
                                       query_count, y, hidden);
}

int shrike_encode_route_decode(shrike_moe* m, void* stream, const shrike_router_operands* ops,
                               const uint64_t* residency_table_row, const shrike_pool* pool,
                               const void* hidden, uint32_t query_count, uint32_t hidden_stride_elements,
                               const uint32_t* io_status, uint32_t* out_indices, float* out_weights,
                               float* out_shared_gate, uint32_t* out_resolved_slots, uint32_t* out_counts) {
    if (!m) return SHRIKE_EINVAL;
    if (query_count == 0) return SHRIKE_OK;
    if (!out_indices || !out_weights || !residency_table_row || !pool)
        return fail(m, SHRIKE_EINVAL, "route_decode: null operand");
    const uint32_t limit = m->cfg.max_tokens < SHRIKE_MAX_DECODE_TOKENS ? m->cfg.max_tokens : SHRIKE_MAX_DECODE_TOKENS;
    int rc = check_router_call(m, ops, hidden, query_count, limit, hidden_stride_elements, true, out_shared_gate);
    if (rc) return rc;
    if ((rc = check_device(m))) return rc;
    CU(launch_route_fused(m, (cudaStream_t)stream, *ops, hidden, query_count, hidden_stride_elements,
                          residency_table_row, pool->view.cells, io_status, out_indices, out_weights,
                          out_shared_gate, out_resolved_slots, out_counts, !m->no_pdl));
    return SHRIKE_OK;
}

int shrike_encode_decode_layer(shrike_moe* m, void* stream, const shrike_pool* pool,
                               const shrike_expert_offsets* routed_offsets,
                               const uint64_t* residency_table_row, const shrike_router_operands* router,
                               const shrike_shared_expert* shared, const void* x, uint32_t query_count,
                               const uint32_t* io_status, uint32_t* out_indices, float* out_weights, void* y,
                               void* hidden) {
    if (!m) return SHRIKE_EINVAL;
    if (query_count == 0) return SHRIKE_OK;
    if (!x || !y) return fail(m, SHRIKE_EINVAL, "decode_layer: null operand");
    Workspace& w = m->ws;
    uint32_t* ids = out_indices ? out_indices : w.ids_dev;
    float* wt = out_weights ? out_weights : w.w_dev;
    float* gate = m->cfg.shared_gated ? w.gate_dev : nullptr;
    // A few dozen rows on a handle that owns the prefill operands: the expert-grouped tensor-core call reads
    // every expert once for all its rows, where the 8-row tiles read it once per 8 (gpt-oss shape, 64 rows:
    // 279 us per layer against 740).
    if (query_count > 16 && w.xs && umma_supported(m->cfg) && !m->force_warp_mma) {
        int rcg = shrike_encode_router(m, stream, router, x, query_count, m->cfg.d, ids, wt, gate);
        if (rcg) return rcg;
        rcg = shrike_encode_residency_classification(m, stream, ids, residency_table_row, query_count, w.slots_dev,
                                                     nullptr, nullptr, nullptr);
        if (rcg) return rcg;
        return encode_prefill(m, stream, pool, routed_offsets, ids, w.slots_dev, wt, x, query_count, shared, gate,
                              io_status, y, hidden);
    }
    if (query_count == 1 && w.fused_geom) {
        // one row: router, selection, lookup, both projections and the combine in ONE launch (fused_layer.cu)
        if (!residency_table_row || !pool) return fail(m, SHRIKE_EINVAL, "decode_layer: null operand");
        int rcf = check_router_call(m, router, x, 1, 1, m->cfg.d, false, nullptr);
        if (rcf) return rcf;
        if (!aligned_to(y, 16) || (hidden && !aligned_to(hidden, 16)))
            return fail(m, SHRIKE_EINVAL, "decode_layer: y and hidden must be 16-byte aligned");
        ExpertArgs ea;
        rcf = fill_expert_args(m, pool, routed_offsets, shared, wt, gate, ea);
        if (rcf) return rcf;
        if ((rcf = check_device(m))) return rcf;
        const cudaError_t fe = launch_fused_layer(m, (cudaStream_t)stream, ea, *router, residency_table_row,
                                                  pool->view.cells, io_status, x, ids, wt, w.slots_dev, gate, y, hidden);
        if (fe == cudaSuccess) return SHRIKE_OK;
        if (fe != cudaErrorNotSupported) return cuda_fail(m, fe, "launch_fused_layer");
        // a block layout the tiled copies cannot describe: the three launches below
    }
    int rc = shrike_encode_route_decode(m, stream, router, residency_table_row, pool, x, query_count, m->cfg.d,
                                        io_status, ids, wt, gate, w.slots_dev, nullptr);
    if (rc) return rc;
    ExpertArgs a;
    rc = fill_expert_args(m, pool, routed_offsets, shared, wt, gate, a);
    if (rc) return rc;
    const uint32_t mi = max_instances(m->cfg, query_count);
    // phase 1 and phase 2 may start before their predecessor has drained
    CU(launch_phase1(m, (cudaStream_t)stream, a, mi, !m->no_pdl));
    CU(launch_phase2(m, (cudaStream_t)stream, a, query_count, mi, y, hidden, !m->no_pdl));
    return SHRIKE_OK;
}

int shrike_encode_moe_prefill(shrike_moe* m, void* stream, const shrike_pool* pool,
                              const shrike_expert_offsets* routed_offsets, const uint32_t* topk_indices,
                              const uint32_t* resolved_slots, const float* routing_weights, const void* x,
                              uint32_t query_count, const shrike_shared_expert* shared,
                              const float* shared_gate, void* y, void* hidden) {
    return encode_prefill(m, stream, pool, routed_offsets, topk_indices, resolved_slots, routing_weights, x,
                          query_count, shared, shared_gate, nullptr, y, hidden);
}

int shrike_encode_group_pairs(shrike_moe* m, void* stream, const uint32_t* topk_indices,
                              const float* routing_weights, uint32_t query_count, uint32_t* sorted_pairs,
                              uint32_t* per_expert_offsets, uint32_t* per_expert_counts) {
    if (!m) return SHRIKE_EINVAL;
    if (!topk_indices || !sorted_pairs || !per_expert_offsets || !per_expert_counts)
        return fail(m, SHRIKE_EINVAL, "group_pairs: null operand");
    if (query_count > m->cfg.max_tokens) return fail(m, SHRIKE_ERANGE, "query_count exceeds max_tokens");
    CU(launch_group_pairs(m, (cudaStream_t)stream, topk_indices, routing_weights, query_count, sorted_pairs,
                          per_expert_offsets, per_expert_counts));
    return SHRIKE_OK;
}

// ---- expert parallelism ---------------------------------------------------------

int shrike_ep_encode_dispatch(shrike_moe* m, void* stream, const void* x, const uint32_t* topk_indices,
                              const float* routing_weights, uint32_t query_count, uint32_t world,
                              uint32_t experts_per_rank, uint32_t capacity_rows, void* send_x, uint32_t* send_ids,
                              float* send_weights, uint32_t* send_counts, int32_t* row_of) {
    if (!m) return SHRIKE_EINVAL;
    if (!x || !topk_indices || !routing_weights || !send_x || !send_ids || !send_weights || !send_counts || !row_of)
        return fail(m, SHRIKE_EINVAL, "ep dispatch: null operand");
    if (world == 0 || world > 64 || experts_per_rank == 0 || (uint64_t)world * experts_per_rank < m->cfg.num_experts)
        return fail(m, SHRIKE_EINVAL, "ep dispatch: world x experts_per_rank must cover num_experts");
    if (query_count > m->cfg.max_tokens) return fail(m, SHRIKE_ERANGE, "query_count exceeds max_tokens");
    if (capacity_rows < query_count)
        return fail(m, SHRIKE_ERANGE, "ep dispatch: capacity_rows must be at least query_count (a row goes to a rank at most once)");
    if (query_count == 0) {
        CU(cudaMemsetAsync(send_counts, 0, world * 4, (cudaStream_t)stream));
        return SHRIKE_OK;
    }
    CU(launch_ep_dispatch(m, (cudaStream_t)stream, x, topk_indices, routing_weights, query_count, world,
                          experts_per_rank, capacity_rows, send_x, send_ids, send_weights, send_counts, row_of));
    return SHRIKE_OK;
}

int shrike_ep_encode_local_slots(shrike_moe* m, void* stream, const uint32_t* recv_ids,
                                 const uint64_t* residency_table_row, uint32_t rows, uint32_t* resolved_slots) {
    if (!m) return SHRIKE_EINVAL;
    if (!recv_ids || !residency_table_row || !resolved_slots) return fail(m, SHRIKE_EINVAL, "ep local slots: null operand");
    if (rows == 0) return SHRIKE_OK;
    CU(launch_ep_local_slots(m, (cudaStream_t)stream, recv_ids, residency_table_row, rows, resolved_slots));
    return SHRIKE_OK;
}

int shrike_ep_encode_combine(shrike_moe* m, void* stream, const void* recv_y, const int32_t* row_of,
                             const void* y_home, uint32_t query_count, uint32_t world, uint32_t capacity_rows,
                             void* y, void* hidden) {
    if (!m) return SHRIKE_EINVAL;
    if (!recv_y || !row_of || !y) return fail(m, SHRIKE_EINVAL, "ep combine: null operand");
    if (query_count == 0) return SHRIKE_OK;
    CU(launch_ep_combine(m, (cudaStream_t)stream, recv_y, row_of, y_home, query_count, world, capacity_rows, y,
                         hidden));
    return SHRIKE_OK;
}

int shrike_moe_layer_forward_host(shrike_moe* m, void* stream, const shrike_pool* pool,
                                  const shrike_expert_offsets* routed_offsets,
                                  const uint64_t* residency_table_row, const shrike_router_operands* router,
                                  const shrike_shared_expert* shared, const void* x_host,
                                  uint32_t query_count, void* y_host, uint32_t* ids_host, float* weights_host) {
    if (!m) return SHRIKE_EINVAL;
    if (!x_host || !y_host || !router || !residency_table_row) return fail(m, SHRIKE_EINVAL, "forward_host: null operand");
    const shrike_moe_config& c = m->cfg;
    if (query_count == 0) return SHRIKE_OK;
    if (query_count > c.max_tokens) return fail(m, SHRIKE_ERANGE, "query_count exceeds max_tokens");
    cudaStream_t st = (cudaStream_t)stream;
    Workspace& w = m->ws;
    const size_t bytes = (size_t)query_count * c.d * act_bytes(c.act_dtype);
    CU(cudaMemcpyAsync(w.x_dev, x_host, bytes, cudaMemcpyHostToDevice, st));
    float* gate = c.shared_gated ? w.gate_dev : nullptr;
    int rc;
    if (query_count <= SHRIKE_MAX_DECODE_TOKENS) {
        rc = shrike_encode_decode_layer(m, stream, pool, routed_offsets, residency_table_row, router, shared,
                                        w.x_dev, query_count, nullptr, w.ids_dev, w.w_dev, w.y_dev, nullptr);
    } else {
        rc = shrike_encode_router(m, stream, router, w.x_dev, query_count, c.d, w.ids_dev, w.w_dev, gate);
        if (rc) return rc;
        rc = shrike_encode_residency_classification(m, stream, w.ids_dev, residency_table_row, query_count,
                                                    w.slots_dev, w.counts_dev, nullptr, nullptr);
        if (rc) return rc;
        rc = shrike_encode_moe_prefill(m, stream, pool, routed_offsets, w.ids_dev, w.slots_dev, w.w_dev, w.x_dev,
                                       query_count, shared, gate, w.y_dev, nullptr);
    }
    if (rc) return rc;
    CU(cudaMemcpyAsync(y_host, w.y_dev, bytes, cudaMemcpyDeviceToHost, st));
    if (ids_host) CU(cudaMemcpyAsync(ids_host, w.ids_dev, (size_t)query_count * c.top_k * 4, cudaMemcpyDeviceToHost, st));
    if (weights_host) CU(cudaMemcpyAsync(weights_host, w.w_dev, (size_t)query_count * c.top_k * 4, cudaMemcpyDeviceToHost, st));
    return shrike_moe_status(m, stream);
}

int shrike_dequant_affine_rows(void* stream, const void* packed, const void* scales, const void* biases,
                               uint32_t bits, uint32_t group, uint32_t meta_dtype, uint32_t rows, uint32_t cols,
                               float* out) {
    if (!packed || !scales || !biases || !out) return SHRIKE_EINVAL;
    if ((bits != 4 && bits != 8) || (group != 32 && group != 64) || cols == 0 || cols % group != 0 ||
        (meta_dtype != SHRIKE_DTYPE_BF16 && meta_dtype != SHRIKE_DTYPE_FP16))
        return SHRIKE_EINVAL;
    if (((uintptr_t)scales & 1) || ((uintptr_t)biases & 1) || ((uintptr_t)out & 3)) return SHRIKE_EINVAL;
    if (rows == 0) return SHRIKE_OK;
    if ((uint64_t)rows * cols > 0x7fffffffull * 256) return SHRIKE_ERANGE;
    return launch_dequant_affine_rows((cudaStream_t)stream, packed, scales, biases, bits, group, meta_dtype, rows, cols,
                                      out) == cudaSuccess ? SHRIKE_OK : SHRIKE_EIO;
}

// ---- expert parallelism over peer memory ---------------------------------------------------------------

struct shrike_ep {
    shrike_moe* home;
    shrike_moe* routed;
    uint32_t rank, world, cap, epr, t_max;
    EpLayout lay;
    uint8_t* mine = nullptr;
    uint8_t* peer[SHRIKE_EP_MAX_WORLD] = {};
    bool opened[SHRIKE_EP_MAX_WORLD] = {};
    bool connected = false;
    // local scratch
    uint32_t* ids = nullptr; float* w = nullptr; float* gate = nullptr; int32_t* row_of = nullptr;
    uint32_t* send_counts = nullptr; uint32_t* miss_slots = nullptr;
    uint32_t* c_ids = nullptr; float* c_w = nullptr; uint32_t* c_slots = nullptr; uint32_t* row_map = nullptr;
    uint32_t* prefix = nullptr; uint32_t* n_rows = nullptr;
    void* y_home = nullptr;
    cudaStream_t side = nullptr;
    cudaEvent_t ev_routed = nullptr, ev_shared = nullptr;
    uint32_t epoch = 0;
    uint32_t max_polls = 1000000;   // ~1 us per poll
};

static void ep_free(shrike_ep* ep) {
    for (uint32_t g = 0; g < SHRIKE_EP_MAX_WORLD; ++g)
        if (ep->opened[g] && ep->peer[g]) cudaIpcCloseMemHandle(ep->peer[g]);
    void* ptrs[] = {ep->mine, ep->ids, ep->w, ep->gate, ep->row_of, ep->send_counts, ep->miss_slots, ep->c_ids, ep->c_w,
                    ep->c_slots, ep->row_map, ep->prefix, ep->n_rows, ep->y_home};
    for (void* p : ptrs)
        if (p) cudaFree(p);
    if (ep->side) cudaStreamDestroy(ep->side);
    if (ep->ev_routed) cudaEventDestroy(ep->ev_routed);
    if (ep->ev_shared) cudaEventDestroy(ep->ev_shared);
    delete ep;
}

int shrike_ep_create(shrike_moe* home, shrike_moe* routed, uint32_t rank, uint32_t world, uint32_t rows_per_call,
                     shrike_ep** out) {
    if (!home || !routed || !out) return SHRIKE_EINVAL;
    shrike_moe* m = home;
    *out = nullptr;
    const shrike_moe_config& c = home->cfg;
    const shrike_moe_config& r = routed->cfg;
    if (world == 0 || world > SHRIKE_EP_MAX_WORLD || rank >= world)
        return fail(m, SHRIKE_EINVAL, "ep: world must be 1..%u and rank below it", SHRIKE_EP_MAX_WORLD);
    if (c.num_experts % world != 0 || r.num_experts != c.num_experts / world)
        return fail(m, SHRIKE_EINVAL, "ep: the routed handle must hold num_experts / world experts");
    // weight_bits, group_size and meta_dtype may differ: the home handle's describe the shared expert's block, the
    // routed handle's the routed experts' (an int8 shared expert beside int4 routed experts,
    // SharedExpertInt8.swift:55-227)
    if (r.d != c.d || r.f != c.f || r.top_k != c.top_k || r.act_dtype != c.act_dtype || r.y_dtype != c.y_dtype ||
        r.activation != c.activation || r.expert_bias != c.expert_bias || r.has_shared || home->device != routed->device)
        return fail(m, SHRIKE_EINVAL, "ep: the routed handle must share the layer's shape, dtypes and device and have no shared expert");
    if ((r.weight_bits != c.weight_bits || r.group_size != c.group_size || r.meta_dtype != c.meta_dtype) && !c.has_shared)
        return fail(m, SHRIKE_EINVAL, "ep: the handles' weight formats differ but the home handle has no shared expert to describe");
    if (rows_per_call == 0 || rows_per_call > c.max_tokens)
        return fail(m, SHRIKE_ERANGE, "ep: rows_per_call must be 1..max_tokens of the home handle");
    const uint32_t t_max = world * rows_per_call;
    if (r.max_tokens < t_max || r.max_tokens <= SHRIKE_MAX_DECODE_TOKENS)
        return fail(m, SHRIKE_ERANGE, "ep: the routed handle needs max_tokens >= max(65, world * rows_per_call)");
    DeviceGuard guard(home->device);
    shrike_ep* ep = new (std::nothrow) shrike_ep();
    if (!ep) return fail(m, SHRIKE_ENOMEM, "host allocation failed");
    ep->home = home; ep->routed = routed; ep->rank = rank; ep->world = world; ep->cap = rows_per_call;
    ep->epr = r.num_experts; ep->t_max = t_max;
    ep->lay = ep_layout(c, world, rows_per_call);
    const size_t T = rows_per_call, K = c.top_k;
    bool ok = true;
    auto A = [&](auto** p, size_t bytes) { if (ok && dev_alloc(p, bytes) != cudaSuccess) ok = false; };
    A(&ep->mine, ep->lay.bytes);
    A(&ep->ids, T * K * 4); A(&ep->w, T * K * 4); A(&ep->gate, T * 4); A(&ep->row_of, T * world * 4);
    A(&ep->send_counts, SHRIKE_EP_MAX_WORLD * 4); A(&ep->miss_slots, T * K * 4);
    A(&ep->c_ids, (size_t)t_max * K * 4); A(&ep->c_w, (size_t)t_max * K * 4); A(&ep->c_slots, (size_t)t_max * K * 4);
    A(&ep->row_map, (size_t)t_max * 4); A(&ep->prefix, (SHRIKE_EP_MAX_WORLD + 1) * 4); A(&ep->n_rows, 4);
    A((uint8_t**)&ep->y_home, c.has_shared ? T * c.d * act_bytes(c.y_dtype) : 0);
    if (ok && (cudaStreamCreateWithFlags(&ep->side, cudaStreamNonBlocking) != cudaSuccess ||
               cudaEventCreateWithFlags(&ep->ev_routed, cudaEventDisableTiming) != cudaSuccess ||
               cudaEventCreateWithFlags(&ep->ev_shared, cudaEventDisableTiming) != cudaSuccess))
        ok = false;
    if (!ok) {
        ep_free(ep);
        cudaGetLastError();
        return fail(m, SHRIKE_ENOMEM, "ep: allocation of the exchange buffers failed");
    }
    // no arrival word carries the first epoch's tag; the shared-only call of the home rows sees every pick miss
    cudaMemset(ep->mine, 0, ep->lay.bytes);
    cudaMemset(ep->miss_slots, 0xff, T * K * 4);
    ep->peer[rank] = ep->mine;
    ep->connected = world == 1;
    *out = ep;
    return SHRIKE_OK;
}

void shrike_ep_destroy(shrike_ep* ep) {
    if (!ep) return;
    DeviceGuard guard(ep->home->device);
    cudaDeviceSynchronize();
    ep_free(ep);
}

int shrike_ep_export(shrike_ep* ep, void* handle_out) {
    if (!ep || !handle_out) return SHRIKE_EINVAL;
    shrike_moe* m = ep->home;
    static_assert(sizeof(cudaIpcMemHandle_t) == SHRIKE_EP_HANDLE_BYTES, "token size");
    DeviceGuard guard(m->device);
    cudaIpcMemHandle_t h;
    CU(cudaIpcGetMemHandle(&h, ep->mine));
    memcpy(handle_out, &h, sizeof h);
    return SHRIKE_OK;
}

int shrike_ep_connect(shrike_ep* ep, const void* all_handles) {
    if (!ep || !all_handles) return SHRIKE_EINVAL;
    shrike_moe* m = ep->home;
    DeviceGuard guard(m->device);
    for (uint32_t g = 0; g < ep->world; ++g) {
        if (g == ep->rank || ep->peer[g]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t*)all_handles + (size_t)g * SHRIKE_EP_HANDLE_BYTES, sizeof h);
        void* p = nullptr;
        CU(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        ep->peer[g] = (uint8_t*)p;
        ep->opened[g] = true;
    }
    ep->connected = true;
    return SHRIKE_OK;
}

int shrike_ep_buffer(shrike_ep* ep, void** base_out, uint64_t* bytes_out) {
    if (!ep || !base_out) return SHRIKE_EINVAL;
    *base_out = ep->mine;
    if (bytes_out) *bytes_out = ep->lay.bytes;
    return SHRIKE_OK;
}

int shrike_ep_connect_pointers(shrike_ep* ep, void* const* peer_bases) {
    if (!ep || !peer_bases) return SHRIKE_EINVAL;
    for (uint32_t g = 0; g < ep->world; ++g) {
        if (g == ep->rank) continue;
        if (!peer_bases[g]) return fail(ep->home, SHRIKE_EINVAL, "ep: peer %u has no buffer", g);
        ep->peer[g] = (uint8_t*)peer_bases[g];
    }
    ep->connected = true;
    return SHRIKE_OK;
}

int shrike_ep_set_wait_polls(shrike_ep* ep, uint32_t wait_polls) {
    if (!ep) return SHRIKE_EINVAL;
    ep->max_polls = wait_polls ? wait_polls : 1000000;
    return SHRIKE_OK;
}

int shrike_ep_forward(shrike_ep* ep, void* stream, const shrike_pool* local_pool,
                      const shrike_expert_offsets* routed_offsets, const uint64_t* local_residency_row,
                      const shrike_router_operands* router, const shrike_shared_expert* shared, const void* x,
                      uint32_t query_count, void* y, void* hidden) {
    if (!ep) return SHRIKE_EINVAL;
    shrike_moe* m = ep->home;
    shrike_moe* r = ep->routed;
    if (!ep->connected) return fail(m, SHRIKE_EINVAL, "ep: connect the ranks' buffers first");
    if (!local_pool || !routed_offsets || !local_residency_row || !router || !y || (query_count && !x))
        return fail(m, SHRIKE_EINVAL, "ep forward: null operand");
    if (query_count > ep->cap) return fail(m, SHRIKE_ERANGE, "ep forward: query_count exceeds rows_per_call");
    const shrike_moe_config& c = m->cfg;
    cudaStream_t st = (cudaStream_t)stream;
    int rc;
    if ((rc = check_device(m))) return rc;
    const uint32_t epoch = ++ep->epoch;
    const uint32_t T = query_count;
    float* gate = c.shared_gated ? ep->gate : nullptr;
    if (T) {
        rc = shrike_encode_router(m, stream, router, x, T, c.d, ep->ids, ep->w, gate);
        if (rc) return rc;
    }
    // the shared expert of the home rows depends on the router's gate only: second stream, beside the exchange
    const bool with_shared = c.has_shared && T > 0;
    if (with_shared) {
        CU(cudaEventRecord(ep->ev_routed, st));
        CU(cudaStreamWaitEvent(ep->side, ep->ev_routed, 0));
        if (T <= SHRIKE_MAX_DECODE_TOKENS)
            rc = shrike_encode_moe_decode(m, ep->side, local_pool, routed_offsets, ep->miss_slots, ep->w, x, T, shared, gate,
                                          nullptr, ep->y_home, nullptr);
        else
            rc = encode_prefill(m, ep->side, local_pool, routed_offsets, ep->ids, ep->miss_slots, ep->w, x, T, shared, gate,
                                nullptr, ep->y_home, nullptr);
        if (rc) return rc;
        CU(cudaEventRecord(ep->ev_shared, ep->side));
    }
    CU(launch_ep_dispatch_peer(m, st, x, ep->ids, ep->w, T, ep->world, ep->rank, ep->epr, ep->cap, ep->peer, ep->lay, epoch,
                               ep->send_counts, ep->row_of));
    CU(launch_ep_receive(r, st, ep->mine, ep->lay, ep->world, ep->cap, epoch, local_residency_row, ep->t_max, ep->prefix,
                         ep->n_rows, ep->c_ids, ep->c_w, ep->c_slots, ep->row_map, ep->max_polls));
    {   // local experts on the received rows (read in place through the row map), accumulated per row
        ExpertArgs a;
        rc = fill_expert_args(r, local_pool, routed_offsets, nullptr, ep->c_w, nullptr, a);
        if (rc) { m->err = r->err; return rc; }
        const bool warp_mma = r->force_warp_mma || !umma_supported(r->cfg);
        CU(launch_prefill_plan(r, st, ep->c_ids, ep->c_slots, ep->mine + ep->lay.off_recv_x, ep->t_max, false,
                               local_pool->view.cells, warp_mma, nullptr, ep->row_map, ep->n_rows));
        if (warp_mma) {
            const uint32_t mi = max_instances(r->cfg, ep->t_max);
            CU(launch_phase1(r, st, a, mi, false));
            CU(launch_phase2_accumulate(r, st, a, mi));
        } else {
            CU(launch_umma_prefill(r, st, a, ep->t_max, local_pool->view.cells));
        }
    }
    CU(launch_ep_return(r, st, ep->row_map, ep->n_rows, ep->t_max, ep->world, ep->rank, ep->cap, ep->peer, ep->lay, epoch));
    CU(launch_ep_wait_returns(m, st, ep->mine, ep->lay, ep->world, ep->cap, epoch, ep->max_polls));
    if (with_shared) CU(cudaStreamWaitEvent(st, ep->ev_shared, 0));
    if (T)
        CU(launch_ep_combine(m, st, ep->mine + ep->lay.off_ret, ep->row_of, with_shared ? ep->y_home : nullptr, T, ep->world,
                             ep->cap, y, hidden));
    return SHRIKE_OK;
}

int shrike_ep_status(shrike_ep* ep, void* stream) {
    if (!ep) return SHRIKE_EINVAL;
    int rc = shrike_moe_status(ep->home, stream);
    const int rc2 = shrike_moe_status(ep->routed, stream);
    if (!rc && rc2) {
        ep->home->err = ep->routed->err;
        rc = rc2;
    }
    return rc;
}

int shrike_ep_last_counts(shrike_ep* ep, uint32_t* sent_per_rank, uint32_t* rows_received, uint64_t* bytes_stored) {
    if (!ep) return SHRIKE_EINVAL;
    shrike_moe* m = ep->home;
    uint32_t sent[SHRIKE_EP_MAX_WORLD] = {};
    uint32_t n = 0;
    CU(cudaMemcpy(sent, ep->send_counts, ep->world * 4, cudaMemcpyDeviceToHost));
    CU(cudaMemcpy(&n, ep->n_rows, 4, cudaMemcpyDeviceToHost));
    uint64_t rows_out = 0;
    for (uint32_t g = 0; g < ep->world; ++g) {
        if (sent_per_rank) sent_per_rank[g] = sent[g];
        if (g != ep->rank) rows_out += sent[g];
    }
    if (rows_received) *rows_received = n;
    if (bytes_stored) {
        const shrike_moe_config& c = m->cfg;
        // rows + ids + weights out, partial rows back (the rows this rank received from others), 8-byte words
        uint32_t own = 0;
        uint32_t pre[SHRIKE_EP_MAX_WORLD + 1] = {};
        CU(cudaMemcpy(pre, ep->prefix, (ep->world + 1) * 4, cudaMemcpyDeviceToHost));
        own = pre[ep->rank + 1] - pre[ep->rank];
        *bytes_stored = rows_out * ((uint64_t)c.d * act_bytes(c.act_dtype) + (uint64_t)c.top_k * 8) +
                        (uint64_t)(n - own) * c.d * act_bytes(c.y_dtype) + (uint64_t)(ep->world - 1) * 16;
    }
    return SHRIKE_OK;
}

struct shrike_decode_stack {
    std::vector<shrike_stack_layer> layers;
    uint32_t max_rows;
    void* stream_dev = nullptr;   // [(layers + 1) x max_rows x d]
};

int shrike_decode_stack_create(const shrike_stack_layer* layers, uint32_t layer_count, uint32_t max_rows,
                               shrike_decode_stack** out) {
    if (!layers || layer_count == 0 || !layers[0].moe || !out) return SHRIKE_EINVAL;
    *out = nullptr;
    shrike_moe* m = layers[0].moe;
    const shrike_moe_config& c = m->cfg;
    if (max_rows == 0 || max_rows > SHRIKE_MAX_DECODE_TOKENS)
        return fail(m, SHRIKE_ERANGE, "decode_stack: max_rows must be 1..%u", SHRIKE_MAX_DECODE_TOKENS);
    for (uint32_t l = 0; l < layer_count; ++l) {
        const shrike_moe* ml = layers[l].moe;
        if (!ml || ml->device != m->device || ml->cfg.d != c.d || ml->cfg.act_dtype != c.act_dtype)
            return fail(m, SHRIKE_EINVAL, "decode_stack: layer %u does not share device, d and act_dtype with layer 0", l);
        if (max_rows > ml->cfg.max_tokens) return fail(m, SHRIKE_ERANGE, "decode_stack: max_rows exceeds layer %u's max_tokens", l);
        if (!layers[l].pool || !layers[l].routed_offsets || !layers[l].residency_table_row || !layers[l].router)
            return fail(m, SHRIKE_EINVAL, "decode_stack: layer %u has a null operand", l);
    }
    DeviceGuard guard(m->device);
    shrike_decode_stack* s = new (std::nothrow) shrike_decode_stack();
    if (!s) return fail(m, SHRIKE_ENOMEM, "host allocation failed");
    s->layers.assign(layers, layers + layer_count);
    s->max_rows = max_rows;
    const size_t bytes = (size_t)(layer_count + 1) * max_rows * c.d * act_bytes(c.act_dtype);
    if (cudaMalloc(&s->stream_dev, bytes) != cudaSuccess) {
        delete s;
        cudaGetLastError();
        return fail(m, SHRIKE_ENOMEM, "decode_stack: residual stream of %zu bytes", bytes);
    }
    *out = s;
    return SHRIKE_OK;
}

void shrike_decode_stack_destroy(shrike_decode_stack* stack) {
    if (!stack) return;
    DeviceGuard guard(stack->layers[0].moe->device);
    cudaFree(stack->stream_dev);
    delete stack;
}

int shrike_decode_stack_forward_host(shrike_decode_stack* stack, void* stream, const void* rows_host,
                                     uint32_t query_count, void* out_host) {
    if (!stack) return SHRIKE_EINVAL;
    shrike_moe* m = stack->layers[0].moe;
    if (!rows_host || !out_host) return fail(m, SHRIKE_EINVAL, "decode_stack: null operand");
    if (query_count == 0) return SHRIKE_OK;
    if (query_count > stack->max_rows) return fail(m, SHRIKE_ERANGE, "decode_stack: query_count exceeds max_rows");
    const shrike_moe_config& c = m->cfg;
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t L = (uint32_t)stack->layers.size();
    const size_t block = (size_t)query_count * c.d * act_bytes(c.act_dtype);
    uint8_t* dev = (uint8_t*)stack->stream_dev;
    CU(cudaMemcpyAsync(dev, rows_host, (size_t)(L + 1) * block, cudaMemcpyHostToDevice, st));
    for (uint32_t l = 0; l < L; ++l) {
        const shrike_stack_layer& ly = stack->layers[l];
        const int rc = shrike_encode_decode_layer(ly.moe, stream, ly.pool, ly.routed_offsets, ly.residency_table_row,
                                                  ly.router, ly.shared, dev + (size_t)l * block, query_count, nullptr, nullptr,
                                                  nullptr, ly.moe->ws.y_dev, dev + (size_t)(l + 1) * block);
        if (rc) {
            if (ly.moe != m) m->err = ly.moe->err;
            return rc;
        }
    }
    CU(cudaMemcpyAsync(out_host, dev + (size_t)L * block, block, cudaMemcpyDeviceToHost, st));
    CU(cudaStreamSynchronize(st));
    return SHRIKE_OK;
}

}  // extern "C"
