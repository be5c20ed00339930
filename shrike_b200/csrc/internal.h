// Internals of the opaque handles and the launch entry points the C ABI calls.
#pragma once

#include <string>

#include "common.cuh"

namespace shrike {

// One unit of expert work: up to 8 rows (tokens) that all use one expert block.
struct Instance {
    uint32_t kind;   // 0 = routed (block = pool cell `slot`), 1 = shared expert
    uint32_t slot;   // pool cell (routed)
    uint32_t first;  // routed: index into the sorted pair list; shared: first token
    uint32_t count;  // 1..8
    uint32_t pair[8];  // routed: row*top_k + rank of each of the `count` rows; shared: the row
};

// PoolBases (moe.metal:297-300) by value as a kernel argument.
struct PoolView {
    const uint8_t* base[SHRIKE_MAX_POOL_CHUNKS];
    uint32_t cells_per_chunk;
    uint32_t cells;
    uint64_t stride;
};

__host__ __device__ __forceinline__ const uint8_t* pool_cell_base(const PoolView& p, uint32_t cell) {
    return p.base[cell / p.cells_per_chunk] + (uint64_t)(cell % p.cells_per_chunk) * p.stride;
}

struct Offsets3 {  // gate / up / down
    uint32_t w[3], s[3], b[3], ab[3];
};

inline Offsets3 to_offsets3(const shrike_expert_offsets& o) {
    Offsets3 r;
    r.w[0] = o.gate_w; r.s[0] = o.gate_s; r.b[0] = o.gate_b; r.ab[0] = o.gate_ab;
    r.w[1] = o.up_w;   r.s[1] = o.up_s;   r.b[1] = o.up_b;   r.ab[1] = o.up_ab;
    r.w[2] = o.down_w; r.s[2] = o.down_s; r.b[2] = o.down_b; r.ab[2] = o.down_ab;
    return r;
}

// Everything the expert kernels need that does not change between launches of
// one call.
struct ExpertArgs {
    PoolView pool;
    Offsets3 routed;
    Offsets3 shared;
    const uint8_t* shared_block;
    uint32_t d, f, f_shared, top_k;
    uint32_t activation, expert_bias;
    uint32_t act_dtype;           // dtype of x and hidden
    uint32_t y_dtype;             // dtype of y
    const Instance* inst;
    const uint32_t* n_inst;
    const uint32_t* sorted;       // sorted pair ids (token*top_k + rank)
    const uint16_t* xh;           // fp16 operand copy of x, [tokens x d]
    const float* xsum;            // per-group sums of xh, [tokens x d/group]
    uint16_t* acts;               // fp16 operand copy of the routed activations [pairs x f]
    uint16_t* acts_shared;        // [tokens x f_shared]
    float* yacc;                  // prefill: fp32 output accumulator [tokens x d]
    const float* route_w;         // [tokens x top_k]
    const float* shared_gate;     // [tokens] or NULL
    uint32_t* status;
#ifdef SHRIKE_TRACE
    uint64_t* trace;              // debug builds: per-block timestamps, or NULL
#endif
};

struct Workspace {
    float* logits = nullptr;        // [max_tokens x num_experts]
    uint16_t* xh = nullptr;
    float* xsum = nullptr;
    uint16_t* acts = nullptr;
    uint16_t* acts_shared = nullptr;
    uint32_t* sorted = nullptr;     // [max_tokens x top_k]
    Instance* inst = nullptr;
    uint32_t* n_inst = nullptr;
    uint32_t* status = nullptr;     // device status word
    uint32_t* done_counter = nullptr; // blocks finished, fused route kernel
    uint32_t* block_hist = nullptr; // prefill grouping scratch
    uint32_t* expert_offsets = nullptr;
    uint32_t* expert_counts = nullptr;
    uint32_t* slot_of_expert = nullptr;
    float* yacc = nullptr;          // prefill: fp32 output accumulator [max_tokens x d]
    void* chunk_inst = nullptr;     // prefill: instances of up to 256 rows (tensor-core path)
    uint32_t* n_chunk_inst = nullptr; // [0] instances, [1] sorted rows
    uint16_t* xs = nullptr;         // prefill: fp16 activation rows in expert-sorted order [max_tokens x top_k x d]
    void* tensor_maps = nullptr;    // host: the TMA descriptors of xs, acts, xh, acts_shared
    // one-row decode layer in one launch (fused_layer.cu)
    void* fused_geom = nullptr;       // host: sizes of the shared-memory ring, or NULL when the shape does not fit
    void* fused_maps = nullptr;       // host: cached tensor maps of the last call's pool and shared block
    void* fused_logits = nullptr;     // [num_experts + 1] {epoch, logit} words
    uint16_t* fused_acts = nullptr;   // two activation hand-over buffers
    uint32_t* fused_epoch = nullptr;
    // forward_host staging
    void* x_dev = nullptr; void* y_dev = nullptr;
    uint32_t* ids_dev = nullptr; float* w_dev = nullptr; float* gate_dev = nullptr;
    uint32_t* slots_dev = nullptr; uint32_t* counts_dev = nullptr;
    uint32_t max_inst = 0;
};

}  // namespace shrike

struct shrike_pool {
    shrike_moe* owner;
    shrike::PoolView view;
    void* chunk[SHRIKE_MAX_POOL_CHUNKS];
    uint32_t chunks;
};

struct shrike_moe {
    shrike_moe_config cfg;
    int device;
    std::string err;
    shrike::Workspace ws;
    uint64_t* residency = nullptr;
    uint32_t residency_layers = 0;
    int sm_count = 148;
    bool no_pdl = false;          // SHRIKE_NO_PDL was set when the handle was created (diagnostics)
    bool single_stream = false;   // SHRIKE_SINGLE_STREAM was set when the handle was created: nothing else runs on the GPU
                                  // beside this handle's stream, so the one-launch layer need not be a cooperative launch
    bool force_warp_mma = false;  // SHRIKE_PREFILL_PATH=mma was set when the handle was created (test switch)
#ifdef SHRIKE_TRACE
    uint64_t* trace = nullptr;
#endif
};

#ifdef SHRIKE_TRACE
// Debug builds only (-DSHRIKE_TRACE): device buffer that receives per-block timestamps; NULL switches it off.
extern "C" int shrike_debug_set_trace(shrike_moe* moe, uint64_t* trace_device_buffer);
#endif

namespace shrike {

size_t act_bytes(uint32_t dt);

// Most instances a decode call of T rows can have: one per distinct expert, one more per 8 further
// rows of an expert, and the shared expert's.
inline uint32_t max_instances(const shrike_moe_config& c, uint32_t T) {
    const uint32_t pairs = T * c.top_k;
    uint32_t routed = c.num_experts + pairs / 8;
    if (routed > pairs) routed = pairs;
    return routed + (c.has_shared ? (T + 7) / 8 : 0);
}

// api.cu: what the router kernels' vector loads rely on; `why` receives the first violation
bool router_operands_aligned(const shrike_moe_config& c, const shrike_router_operands& o, const void* hidden,
                             const char** why);
// router.cu
cudaError_t launch_router(const shrike_moe* m, cudaStream_t st, const shrike_router_operands& ops,
                          const void* hidden, uint32_t T, uint32_t stride, uint32_t* ids,
                          float* weights, float* shared_gate);
cudaError_t launch_route_fused(const shrike_moe* m, cudaStream_t st, const shrike_router_operands& ops,
                               const void* hidden, uint32_t T, uint32_t stride, const uint64_t* table,
                               uint32_t pool_cells, const uint32_t* io_status, uint32_t* ids, float* weights,
                               float* shared_gate, uint32_t* slots, uint32_t* counts, bool pdl,
                               bool no_tail = false);
cudaError_t launch_classify(const shrike_moe* m, cudaStream_t st, const uint32_t* ids,
                            const uint64_t* table, uint32_t T, uint32_t* slots, uint32_t* counts,
                            uint32_t* miss_pos, uint32_t* miss_exp);
// plan.cu
cudaError_t launch_decode_plan(const shrike_moe* m, cudaStream_t st, const uint32_t* slots,
                               const void* x, uint32_t T, const uint32_t* io_status,
                               bool with_shared, uint32_t pool_cells);
cudaError_t launch_group_pairs(const shrike_moe* m, cudaStream_t st, const uint32_t* ids,
                               const float* weights, uint32_t T, uint32_t* sorted_pairs,
                               uint32_t* offsets, uint32_t* counts);
// decode.cu
cudaError_t launch_phase1(const shrike_moe* m, cudaStream_t st, const ExpertArgs& a,
                          uint32_t max_inst, bool pdl);
cudaError_t launch_phase2(const shrike_moe* m, cudaStream_t st, const ExpertArgs& a, uint32_t T,
                          uint32_t max_inst, void* y, void* hidden, bool pdl);
// synth.cu
cudaError_t launch_synth_fill(const shrike_moe* m, cudaStream_t st, const PoolView& pool,
                              uint32_t first_cell, uint32_t count, uint64_t seed, uint32_t layer,
                              uint32_t first_expert, bool shared, const Offsets3& off);

}  // namespace shrike

namespace shrike {
cudaError_t launch_phase2_accumulate(const shrike_moe* m, cudaStream_t st, const ExpertArgs& a,
                                     uint32_t max_inst);
// prefill.cu
cudaError_t launch_prefill_plan(const shrike_moe* m, cudaStream_t st, const uint32_t* ids,
                                const uint32_t* slots, const void* x, uint32_t T, bool with_shared,
                                uint32_t pool_cells, bool warp_mma_instances, const uint32_t* io_status,
                                const uint32_t* row_map = nullptr, const uint32_t* n_rows = nullptr,
                                float* accumulator = nullptr);
cudaError_t launch_prefill_combine(const shrike_moe* m, cudaStream_t st, uint32_t T, void* y, void* hidden);
}  // namespace shrike

namespace shrike {
// ep.cu
struct EpLayout {   // byte offsets inside a rank's exchange buffer
    size_t off_recv_x, off_recv_ids, off_recv_w, off_ret, off_arrive, off_ret_arrive, bytes;
};
EpLayout ep_layout(const shrike_moe_config& c, uint32_t world, uint32_t cap);
cudaError_t launch_ep_dispatch_peer(const shrike_moe* m, cudaStream_t st, const void* x, const uint32_t* ids,
                                    const float* weights, uint32_t T, uint32_t world, uint32_t rank,
                                    uint32_t experts_per_rank, uint32_t cap, uint8_t* const* peer_base,
                                    const EpLayout& lay, uint32_t epoch, uint32_t* send_counts, int32_t* row_of);
cudaError_t launch_ep_receive(const shrike_moe* routed, cudaStream_t st, const uint8_t* mine, const EpLayout& lay,
                              uint32_t world, uint32_t cap, uint32_t epoch, const uint64_t* table, uint32_t t_max,
                              uint32_t* prefix, uint32_t* n_rows, uint32_t* c_ids, float* c_w, uint32_t* c_slots,
                              uint32_t* row_map, uint32_t max_polls);
cudaError_t launch_ep_return(const shrike_moe* routed, cudaStream_t st, const uint32_t* row_map, const uint32_t* n_rows,
                             uint32_t t_max, uint32_t world, uint32_t rank, uint32_t cap, uint8_t* const* peer_base,
                             const EpLayout& lay, uint32_t epoch);
cudaError_t launch_ep_wait_returns(const shrike_moe* home, cudaStream_t st, const uint8_t* mine, const EpLayout& lay,
                                   uint32_t world, uint32_t cap, uint32_t epoch, uint32_t max_polls);
cudaError_t launch_ep_dispatch(const shrike_moe* m, cudaStream_t st, const void* x, const uint32_t* ids,
                               const float* weights, uint32_t T, uint32_t world, uint32_t experts_per_rank,
                               uint32_t cap, void* send_x, uint32_t* send_ids, float* send_w,
                               uint32_t* send_counts, int32_t* row_of);
cudaError_t launch_ep_local_slots(const shrike_moe* m, cudaStream_t st, const uint32_t* recv_ids,
                                  const uint64_t* table, uint32_t rows, uint32_t* slots);
cudaError_t launch_ep_combine(const shrike_moe* m, cudaStream_t st, const void* recv_y, const int32_t* row_of,
                              const void* y_home, uint32_t T, uint32_t world, uint32_t cap, void* y, void* hidden);
}  // namespace shrike

namespace shrike {
// fused_layer.cu
struct FusedGeom;
bool fused_geometry(const shrike_moe_config& c, int sm_count, int max_smem_optin, FusedGeom& g);
size_t fused_geom_bytes();
size_t fused_map_cache_bytes();
size_t fused_logits_bytes(const shrike_moe_config& c);
size_t fused_acts_bytes(const shrike_moe_config& c);
cudaError_t launch_dequant_affine_rows(cudaStream_t st, const void* packed, const void* scales, const void* biases,
                                       uint32_t bits, uint32_t group, uint32_t meta_dtype, uint32_t rows, uint32_t cols,
                                       float* out);
cudaError_t launch_fused_layer(const shrike_moe* m, cudaStream_t st, const ExpertArgs& ea,
                               const shrike_router_operands& ops, const uint64_t* table, uint32_t pool_cells,
                               const uint32_t* io_status, const void* x, uint32_t* ids, float* weights,
                               uint32_t* slots, float* gate, void* y, void* hidden);
}  // namespace shrike

namespace shrike {
// umma_gemm.cu
uint32_t umma_max_chunk_instances(const shrike_moe_config& c, uint32_t T);
size_t umma_chunk_instance_bytes();
size_t umma_tensor_map_bytes();
cudaError_t umma_prepare(shrike_moe* m);
bool umma_supported(const shrike_moe_config& c);
cudaError_t launch_umma_prefill(const shrike_moe* m, cudaStream_t st, const ExpertArgs& a, uint32_t T,
                                uint32_t pool_cells);
}  // namespace shrike
