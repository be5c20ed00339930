/*
 * shrike_b200 — C ABI of the B200 (sm_100a) implementation of Shrike's
 * quantised routed-expert MoE feed-forward.
 *
 * This header is what the reference's `ShrikeKernelsC` SwiftPM target would
 * include in place of the Metal encode calls of `sources/Shrike/Kernels/MoE`
 * and `sources/Shrike/Kernels/Prefill/MoE`. Conventions follow the reference's
 * own C interface (sources/ShrikeKernelsC/include/shrike_expert_io.h:33-72):
 * opaque handles, `create` hands the handle back through an out-pointer, every
 * call returns an int (0 = success, otherwise an errno-style code), nothing
 * throws or aborts across the boundary. All data pointers are plain device
 * pointers unless a parameter name ends in `_host`; `stream` is a
 * `cudaStream_t` passed as `void*` (NULL = the legacy default stream).
 * Calls only enqueue work; device-side failures surface as a non-zero
 * `shrike_moe_status` after the stream is synchronised.
 *
 * Threading: one host thread per handle at a time (the reference's runner is
 * single-owner, RealForwardRunner.swift:95-101). One handle per GPU; every
 * encode call must be made with the handle's device current (checked:
 * SHRIKE_EINVAL otherwise). shrike_moe_create leaves the caller's current
 * device as it found it.
 *
 * Operand precision: the expert tiles multiply on the tensor cores with fp16
 * operands and fp32 accumulation (the reference's matrix path does the same,
 * tensorops.metal:106). bf16 and fp16 activations convert exactly; an fp32
 * activation is rounded to fp16 (2^-11 relative) before the expert
 * projections -- the router reads x at full precision. An activation whose
 * magnitude exceeds 65504 is clamped to it and the call's status becomes
 * SHRIKE_ERANGE (shrike_moe_status) instead of an infinity propagating.
 *
 * Alignment (checked at the call, SHRIKE_EINVAL otherwise): x / hidden given
 * to a router or layer call 16 bytes when fp32, 8 bytes when 16-bit, with a row
 * stride that is a multiple of 4 elements; router weights and the shared gate
 * row 16 bytes; effective_scale 8 bytes; the other bf16 operand vectors, scales
 * and biases 2 bytes; expert sub-tensor offsets and the shared block 16 bytes;
 * cell stride 256 bytes.
 */
#ifndef SHRIKE_B200_H
#define SHRIKE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SHRIKE_MAX_TOP_K 8u          /* MoE.maxStreamedExperts, MoE.swift:42 */
#define SHRIKE_MAX_EXPERTS 256u      /* MoE.swift:263 */
#define SHRIKE_MAX_POOL_CHUNKS 8u    /* PoolBases.base[8], moe.metal:297-300 */
#define SHRIKE_MAX_DECODE_TOKENS 64u /* largest query_count of the decode entry points */
#define SHRIKE_STATIC_ROUTER_MAX_ROWS 64u /* rows the allocation-free router accepts per call */
#define SHRIKE_SLOT_MISS 0xffffffffu /* resolved_slots sentinel, moe.metal:146 */
#define SHRIKE_EP_MAX_WORLD 16u      /* most ranks of one expert-parallel group (the GPUs of one box) */
#define SHRIKE_EP_HANDLE_BYTES 64u   /* size of the token a rank exports for its exchange buffer */

enum { SHRIKE_DTYPE_BF16 = 0, SHRIKE_DTYPE_FP16 = 1, SHRIKE_DTYPE_FP32 = 2 };
enum { SHRIKE_ACT_SILU = 0, SHRIKE_ACT_GELU_TANH = 1, SHRIKE_ACT_CLAMPED_SWIGLU = 2 };
enum { SHRIKE_ROUTER_SOFTMAX = 0, SHRIKE_ROUTER_SIGMOID = 1 };
enum { SHRIKE_IO_PENDING = 0, SHRIKE_IO_READY = 1, SHRIKE_IO_FAILED = 2 };

enum {
    SHRIKE_OK = 0,
    SHRIKE_EINVAL = 22,     /* bad argument or unsupported shape */
    SHRIKE_ENOMEM = 12,     /* device or host allocation failed */
    SHRIKE_ERANGE = 34,     /* slot / expert / token count out of range */
    SHRIKE_EIO = 5,         /* CUDA runtime error; text in shrike_last_error */
    SHRIKE_ETIMEDOUT = 110  /* a bounded device-side wait gave up */
};

/* Replaces the arguments of `MoE.init` (MoE.swift:94-106) plus the dtypes the
 * Metal build fixes at compile time. */
typedef struct shrike_moe_config {
    uint32_t d;                 /* hidden size, multiple of 64 */
    uint32_t f;                 /* routed expert intermediate size, multiple of 64 */
    uint32_t num_experts;       /* <= 256 */
    uint32_t top_k;             /* 1..8 */
    uint32_t weight_bits;       /* 4 or 8 (routedWeightBits) */
    uint32_t group_size;        /* 64 (the reference's only value) or 32 */
    uint32_t meta_dtype;        /* dtype of scales and zero-point biases: BF16 (reference) or FP16 */
    uint32_t act_dtype;         /* dtype of x and hidden: BF16, FP16 or FP32 */
    uint32_t activation;        /* SHRIKE_ACT_* (siluActivation / clampedSwiGLU) */
    uint32_t expert_bias;       /* expertAdditiveBiases */
    uint32_t router_kind;       /* SHRIKE_ROUTER_* (sigmoidRouterScores) */
    float    routed_scaling;    /* routedScalingFactor */
    uint32_t router_weight_bits;/* 0 = fp32 rows, 4 or 8 = affine g64 bf16 (routerWeightBits) */
    uint32_t round_route_weights_f16; /* round route weights through fp16 as the shader does */
    uint32_t has_shared;        /* a shared expert is passed to the moe calls */
    uint32_t shared_gated;      /* shared output is multiplied by sigmoid(gate . x) */
    uint32_t shared_f;          /* shared expert intermediate size */
    uint32_t max_tokens;        /* largest query_count of any call; sizes the workspace */
    uint32_t y_dtype;           /* dtype of y: BF16, FP16 or FP32, independent of act_dtype. The sums are
                                 * formed in fp32; FP32 here returns them unrounded (bf16 x in, fp32 y out is
                                 * the configuration the 1e-3 relative-L2 parity bar is stated for), a 16-bit
                                 * type rounds once on store as moe_phase2_finish does (moe.metal:889-893).
                                 * hidden += y adds the value as stored in y and rounds to act_dtype. */
} shrike_moe_config;

/* Field-for-field `MoEExpertOffsets` (MoE.swift:4-39) = `ExpertOffsets`
 * (moe.metal:240-255): byte offsets inside one packed expert block. */
typedef struct shrike_expert_offsets {
    uint32_t gate_w, gate_s, gate_b;
    uint32_t up_w, up_s, up_b;
    uint32_t down_w, down_s, down_b;
    uint32_t gate_ab, up_ab, down_ab;
} shrike_expert_offsets;

/* Operands of `MoE.encodeRouter` (MoE.swift:249-261). `weights` is fp32
 * [num_experts x d] when router_weight_bits == 0, else packed affine rows with
 * bf16 `scales`/`biases` [num_experts x d/64]. The three bf16 vectors may be
 * NULL (ones / ones / zeros). `shared_gate` is the shared expert's scalar gate
 * row, fp32 [d], or NULL. */
typedef struct shrike_router_operands {
    const void*     weights;
    const uint16_t* scales;
    const uint16_t* biases;
    const uint16_t* effective_scale;   /* bf16 [d] */
    const uint16_t* per_expert_scale;  /* bf16 [num_experts] */
    const uint16_t* logit_bias;        /* bf16 [num_experts] */
    const float*    shared_gate;       /* fp32 [d] */
} shrike_router_operands;

/* The resident shared expert (SharedExpertRuntime, SharedExpertInt4.swift:251-342):
 * one packed block in the routed experts' format with its own offsets. */
typedef struct shrike_shared_expert {
    const void*           block;
    shrike_expert_offsets offsets;
} shrike_shared_expert;

typedef struct shrike_moe shrike_moe;     /* replaces `final class MoE` + PrefillGroupedRoutedMoE */
typedef struct shrike_pool shrike_pool;   /* replaces ExpertCellArena (ExpertCellArena.swift:16-132) */

/* ---- lifetime ---------------------------------------------------------- */

/* MoE.init (MoE.swift:94-143). Allocates the workspace for max_tokens; no
 * later call allocates. */
int shrike_moe_create(const shrike_moe_config* config, int device, shrike_moe** out);
void shrike_moe_destroy(shrike_moe* moe);

/* Text of the last failure on this handle (or of the last failed create when
 * moe is NULL). Never NULL. */
const char* shrike_last_error(const shrike_moe* moe);

/* Synchronises `stream`, then returns SHRIKE_OK, SHRIKE_ETIMEDOUT when a
 * kernel's bounded wait gave up, or SHRIKE_EIO for a CUDA error
 * (the reference inspects commandBuffer.error, RealForwardRunner.swift:5360-5363). */
int shrike_moe_status(shrike_moe* moe, void* stream);

/* CPUExpertFFN.Offsets (CPUExpertFFN.swift:34-61) / Model.routedExpertOffsets
 * (ModelExpertIO.swift:69-94): offsets and unpadded size of one block. */
int shrike_expert_offsets_make(const shrike_moe_config* config, int shared,
                               shrike_expert_offsets* out, uint64_t* block_bytes);

/* ---- HBM slot pool ------------------------------------------------------ */

/* ExpertCellArena.init: `cells` cells of `cell_stride` bytes (multiple of 256)
 * in `chunks` (1..8) device allocations. */
int shrike_pool_create(shrike_moe* moe, uint32_t cells, uint64_t cell_stride, uint32_t chunks,
                       shrike_pool** out);
void shrike_pool_destroy(shrike_pool* pool);
/* Copies one unmodified packed expert block from host memory into a cell. */
int shrike_pool_upload(shrike_pool* pool, uint32_t cell, const void* block_host, uint64_t bytes,
                       void* stream);
int shrike_pool_download(shrike_pool* pool, uint32_t cell, void* block_host, uint64_t bytes,
                         void* stream);
/* pool_cell_base (moe.metal:302-305): device address of a cell. */
int shrike_pool_cell_address(const shrike_pool* pool, uint32_t cell, void** out);
/* Benchmark/test utility: fills `count` cells starting at `first_cell` with
 * seeded synthetic blocks of experts first_expert.. of `layer` (counter-mode
 * SplitMix64; nibbles uniform, scale U(0.5,1.5)*0.02/7.5, bias -8*scale). */
int shrike_pool_fill_synthetic(shrike_moe* moe, shrike_pool* pool, uint32_t first_cell,
                               uint32_t count, uint64_t seed, uint32_t layer,
                               uint32_t first_expert, int shared, void* stream);

/* Affine rows -> fp32, on the device: out[r][c] = q[r][c] * scale[r][c / group] + bias[r][c / group], one rounding
 * (fmaf). For operands this library takes as fp32 and a `.gturbo` file holds packed: the shared expert's scalar
 * gate row -- int8 [1 x d] with g64 scales and biases, multiplied by the Metal host with its own int8 GEMV
 * (SharedExpertInt8.swift:55-227, RealForwardRunner.swift:5447-5467) -- is uploaded verbatim and turned into the
 * `shared_gate` operand of shrike_router_operands once per layer, at load time. No handle, no allocation.
 * bits 4 or 8 (nibbles low first); group 32 or 64; meta_dtype SHRIKE_DTYPE_BF16 or _FP16; cols a multiple of
 * group; packed rows are cols * bits / 8 bytes, scale and bias rows cols / group elements, all dense. */
int shrike_dequant_affine_rows(void* stream, const void* packed, const void* scales, const void* biases,
                               uint32_t bits, uint32_t group, uint32_t meta_dtype, uint32_t rows, uint32_t cols,
                               float* out);

/* ---- residency table ----------------------------------------------------- */

/* ExpertResidencyEntry (ExpertResidencyTable.swift:4-19): one u64 per expert,
 * slot in the low 32 bits, state in the high 32 (2 = resident). `table` is a
 * device array of `layers * num_experts` words owned by the handle. */
int shrike_residency_create(shrike_moe* moe, uint32_t layers, uint64_t** table_out);
int shrike_residency_set(shrike_moe* moe, uint32_t layer, uint32_t expert, uint32_t slot,
                         uint32_t state, void* stream);
/* Marks experts [0, num_experts) of `layer` resident in cells first_cell.. */
int shrike_residency_set_layer_identity(shrike_moe* moe, uint32_t layer, uint32_t first_cell,
                                        void* stream);

/* ---- the path ------------------------------------------------------------ */

/* MoE.encodeRouter (MoE.swift:249-316: router_gemv_r4 + router_topk_select_k8,
 * moe.metal:324-582) and PrefillRouter.encodeBlock (PrefillRouter.swift:75-152)
 * for `query_count` rows of `hidden` spaced `hidden_stride_elements` apart.
 * Writes ids u32 [query_count x top_k], weights fp32 [query_count x top_k] and,
 * when operands->shared_gate is set, sigmoid(gate . x) fp32 [query_count]. */
int shrike_encode_router(shrike_moe* moe, void* stream, const shrike_router_operands* operands,
                         const void* hidden, uint32_t query_count,
                         uint32_t hidden_stride_elements, uint32_t* out_indices,
                         float* out_weights, float* out_shared_gate);

/* MoE.encodeResidencyClassification (MoE.swift:552-613;
 * moe_classify_expert_residency_spec, moe.metal:194-231) for query_count rows.
 * resolved_slots u32 [query_count x top_k]; counts[0] = hits, counts[1] =
 * misses; miss_positions / miss_experts hold (row*top_k+rank, expert) per miss
 * in row order (either may be NULL). */
int shrike_encode_residency_classification(shrike_moe* moe, void* stream,
                                           const uint32_t* topk_indices,
                                           const uint64_t* residency_table_row,
                                           uint32_t query_count, uint32_t* resolved_slots,
                                           uint32_t* counts, uint32_t* miss_positions,
                                           uint32_t* miss_experts);

/* Decode, query_count <= SHRIKE_MAX_DECODE_TOKENS rows. One call stands for
 * encodeSharedExpertWork (RealForwardRunner.swift:5436-5497),
 * MoE.encodeSpecPhase1U16Load (MoE.swift:906-948) and
 * MoE.encodeSpecPhase2Reduce (MoE.swift:992-1049):
 *   y[t] = sg[t] * shared(x[t]) + sum_k w[t,k] * expert(slot[t,k])(x[t]);
 *   hidden[t] += y[t]   (hidden may be NULL)
 * A row whose slot is SHRIKE_SLOT_MISS contributes nothing. When io_status is
 * given and *io_status is neither READY nor 3, y is the shared term alone
 * (moe.metal:36-39, 918-921). shared may be NULL when has_shared == 0;
 * shared_gate is the router call's out_shared_gate (NULL = ungated). */
int shrike_encode_moe_decode(shrike_moe* moe, void* stream, const shrike_pool* pool,
                             const shrike_expert_offsets* routed_offsets,
                             const uint32_t* resolved_slots, const float* routing_weights,
                             const void* x, uint32_t query_count,
                             const shrike_shared_expert* shared, const float* shared_gate,
                             const uint32_t* io_status, void* y, void* hidden);

/* The three steps of the decode call, for hosts that encode them separately as
 * the reference does. They must run in this order on one stream with the same
 * pool, offsets, shared expert and query_count; the handle's workspace carries
 * the work lists and activations from one to the next.
 *   plan:    resolved_slots -> per-expert work lists (the slot lookup at the top
 *            of the spec kernels, moe.metal:980-984), x -> operand layout
 *   phase 1: MoE.encodeSpecPhase1U16Load (MoE.swift:906-948) + shared gate/up
 *   phase 2: MoE.encodeSpecPhase2Reduce (MoE.swift:992-1049) + shared down */
int shrike_encode_decode_plan(shrike_moe* moe, void* stream, const shrike_pool* pool,
                              const uint32_t* resolved_slots, const void* x, uint32_t query_count,
                              const uint32_t* io_status);
int shrike_encode_phase1(shrike_moe* moe, void* stream, const shrike_pool* pool,
                         const shrike_expert_offsets* routed_offsets,
                         const shrike_shared_expert* shared, uint32_t query_count);
int shrike_encode_phase2_reduce(shrike_moe* moe, void* stream, const shrike_pool* pool,
                                const shrike_expert_offsets* routed_offsets,
                                const float* routing_weights, const shrike_shared_expert* shared,
                                const float* shared_gate, uint32_t query_count, void* y, void* hidden);

/* Decode fast path, query_count <= SHRIKE_MAX_DECODE_TOKENS: encodeRouter +
 * encodeResidencyClassification + the work lists of the decode plan in ONE
 * launch (the block that finishes its logits last does the selection; no block
 * waits on another). Same outputs as the three separate calls, bit for bit;
 * out_resolved_slots and out_counts may be NULL. Must be followed by
 * shrike_encode_phase1 / shrike_encode_phase2_reduce on the same handle. */
int shrike_encode_route_decode(shrike_moe* moe, void* stream, const shrike_router_operands* operands,
                               const uint64_t* residency_table_row, const shrike_pool* pool,
                               const void* hidden, uint32_t query_count,
                               uint32_t hidden_stride_elements, const uint32_t* io_status,
                               uint32_t* out_indices, float* out_weights, float* out_shared_gate,
                               uint32_t* out_resolved_slots, uint32_t* out_counts);

/* One decode layer in three launches chained with programmatic dependent
 * launch (route -> phase 1 -> phase 2; each starts its weight fetch while its
 * predecessor drains): what encodeDecodeTailStage's router + classification
 * (RealForwardRunner.swift:2834) and encodeSpeculativeRouted
 * (RealForwardRunner.swift:5520-5572) encode for one routed layer.
 * out_indices / out_weights may be NULL. With more than 16 rows, no io_status
 * and a handle created for prefill (max_tokens > 64) the call runs the router,
 * the classification and the expert-grouped tensor-core path instead: the same
 * result within the parity tolerance, every expert read once for all its rows. */
int shrike_encode_decode_layer(shrike_moe* moe, void* stream, const shrike_pool* pool,
                               const shrike_expert_offsets* routed_offsets,
                               const uint64_t* residency_table_row,
                               const shrike_router_operands* router,
                               const shrike_shared_expert* shared, const void* x, uint32_t query_count,
                               const uint32_t* io_status, uint32_t* out_indices, float* out_weights,
                               void* y, void* hidden);

/* Prefill, any query_count <= max_tokens. Stands for buildPrefillRoutes
 * (RealForwardRunner.swift:4305), encodeGroupedExpertGEMMs
 * (PrefillGroupedRoutedMoE.swift:925-1035), PrefillSharedExpert.encodeChunk
 * (PrefillSharedExpert.swift:105-161), encodeReduceTokenMajor (PrefillMoE.swift:11-20)
 * and the two residual adds (RealForwardRunner.swift:4658-4665). Same
 * arithmetic contract as the decode call; rows are grouped by topk_indices
 * (the expert ids), and every pair of one expert must resolve to one cell. */
int shrike_encode_moe_prefill(shrike_moe* moe, void* stream, const shrike_pool* pool,
                              const shrike_expert_offsets* routed_offsets,
                              const uint32_t* topk_indices, const uint32_t* resolved_slots,
                              const float* routing_weights,
                              const void* x, uint32_t query_count,
                              const shrike_shared_expert* shared, const float* shared_gate,
                              void* y, void* hidden);

/* PrefillMoEGrouping.groupTokenExpertPairs (PrefillMoEGrouping.swift:269-370)
 * on the device: sorts the query_count*top_k (token, expert, rank, weight bits)
 * pairs by (expert, token, rank). sorted_pairs: 4 u32 per pair
 * (PrefillTokenExpertPair, PrefillRouter.swift:5-28); offsets/counts u32
 * [num_experts] (offset 0xffffffff for an unrouted expert).
 * A row's top_k ids must be distinct (a router never picks an expert twice);
 * a row that names an expert twice, or an id >= num_experts other than the
 * expert-parallel sentinel 0xffffffff, is reported through the status word
 * (SHRIKE_ERANGE) by this call and by shrike_encode_moe_prefill. */
int shrike_encode_group_pairs(shrike_moe* moe, void* stream, const uint32_t* topk_indices,
                              const float* routing_weights, uint32_t query_count,
                              uint32_t* sorted_pairs, uint32_t* per_expert_offsets,
                              uint32_t* per_expert_counts);

/* ---- expert parallelism (no counterpart in the reference, which runs on one
 * device): rank r owns experts [r*experts_per_rank, (r+1)*experts_per_rank).
 * The three calls bracket the host's two all-to-all exchanges (NCCL).
 *
 * dispatch: packs, per destination rank g, the rows that have an expert on g --
 * one copy per (row, rank), in row order -- into send_x[g][0..count_g) with the
 * expert ids local to g (0xffffffff for the row's other experts) and the route
 * weights. Buffers are [world x capacity_rows x ...] so that the exchange is a
 * fixed-size all-to-all; capacity_rows >= query_count always suffices.
 * row_of[row*world + g] = the row's index at g, or -1. */
int shrike_ep_encode_dispatch(shrike_moe* moe, void* stream, const void* x, const uint32_t* topk_indices,
                              const float* routing_weights, uint32_t query_count, uint32_t world,
                              uint32_t experts_per_rank, uint32_t capacity_rows, void* send_x,
                              uint32_t* send_ids, float* send_weights, uint32_t* send_counts,
                              int32_t* row_of);
/* On the receiving rank (`moe` is the handle of its local experts): received
 * local ids -> pool cells through the residency table; invalid ids miss. */
int shrike_ep_encode_local_slots(shrike_moe* moe, void* stream, const uint32_t* recv_ids,
                                 const uint64_t* residency_table_row, uint32_t rows,
                                 uint32_t* resolved_slots);
/* Back on the home rank: y = y_home (the shared-expert term, may be NULL) + the
 * partial rows returned by every rank, in rank order; hidden += y. */
int shrike_ep_encode_combine(shrike_moe* moe, void* stream, const void* recv_y, const int32_t* row_of,
                             const void* y_home, uint32_t query_count, uint32_t world,
                             uint32_t capacity_rows, void* y, void* hidden);

/* ---- the expert-parallel layer as one call (no counterpart in the reference) ---------------------------
 *
 * The exchange needs no collective library: every rank owns one exchange buffer, exports a token for it,
 * the host hands every rank all tokens (over whatever transport it has), and from then on the kernels of
 * shrike_ep_forward store rows straight into the destination rank's buffer over NVLink and wait on its
 * arrival words -- plain peer loads and stores, bounded waits. Only the rows routed to a rank move.
 *
 *   shrike_ep_create   `home` is this rank's handle for the router and the shared expert (config of the whole
 *                      layer, max_tokens >= rows_per_call); `routed` is the handle of its local experts
 *                      (num_experts = experts per rank, no shared expert, max_tokens >= max(65, world *
 *                      rows_per_call)). rows_per_call bounds query_count of every forward on every rank.
 *   shrike_ep_export   SHRIKE_EP_HANDLE_BYTES bytes to give to the other ranks (a CUDA IPC handle).
 *   shrike_ep_connect  all ranks' tokens, [world x SHRIKE_EP_HANDLE_BYTES], in rank order (its own is skipped).
 *                      One process per GPU. A process that drives several GPUs itself passes the buffers'
 *                      device addresses (shrike_ep_buffer) to shrike_ep_connect_pointers instead, with peer
 *                      access enabled between the devices.
 *   shrike_ep_forward  router -> dispatch -> (shared expert on a second stream meanwhile) -> local experts ->
 *                      return -> combine for this rank's query_count rows; every rank of the group calls it
 *                      once per layer step. The call enqueues on `stream` and on the handle's own second
 *                      stream (joined before it returns control of `stream`'s order); it is not capturable
 *                      in a CUDA graph (the epoch of the arrival words is a host counter).
 *                      A rank whose peer never arrives waits about a second per exchange, then the next
 *                      shrike_ep_status returns SHRIKE_ETIMEDOUT; the rows of that peer are missing from y.
 *   wait_polls         0 = the default limit (about one second); tests pass a small number. */
typedef struct shrike_ep shrike_ep;
int shrike_ep_create(shrike_moe* home, shrike_moe* routed, uint32_t rank, uint32_t world, uint32_t rows_per_call,
                     shrike_ep** out);
void shrike_ep_destroy(shrike_ep* ep);
int shrike_ep_export(shrike_ep* ep, void* handle_out);
int shrike_ep_connect(shrike_ep* ep, const void* all_handles);
int shrike_ep_buffer(shrike_ep* ep, void** base_out, uint64_t* bytes_out);
int shrike_ep_connect_pointers(shrike_ep* ep, void* const* peer_bases);
int shrike_ep_set_wait_polls(shrike_ep* ep, uint32_t wait_polls);
int shrike_ep_forward(shrike_ep* ep, void* stream, const shrike_pool* local_pool,
                      const shrike_expert_offsets* routed_offsets, const uint64_t* local_residency_row,
                      const shrike_router_operands* router, const shrike_shared_expert* shared, const void* x,
                      uint32_t query_count, void* y, void* hidden);
/* Synchronises `stream`; SHRIKE_OK, or the first failure either handle recorded. */
int shrike_ep_status(shrike_ep* ep, void* stream);
/* Counters of the last forward, read after a synchronise: rows this rank sent to each rank
 * [world], rows it received in total, bytes it stored into peers' buffers (both directions). */
int shrike_ep_last_counts(shrike_ep* ep, uint32_t* sent_per_rank, uint32_t* rows_received, uint64_t* bytes_stored);

/* The router for callers that cannot allocate. No counterpart in the reference.
 * Creating a handle sizes a workspace with cudaMalloc; a host that has already
 * given all free HBM to its expert pool, that fixes its memory plan before the
 * first token, or that must not take cudaMalloc's device-wide synchronisation
 * inside its decode loop cannot do that. This call needs no handle: it takes
 * the configuration by pointer (d, num_experts, top_k, act_dtype, router_kind,
 * routed_scaling, router_weight_bits and round_route_weights_f16 are read) and
 * keeps its one piece of scratch, the logits, in a 64 KiB device array built
 * into the library (resident on every GPU that loads it, until exit). It calls
 * no cudaMalloc, cudaFree or other allocating routine. Same outputs as
 * shrike_encode_router, bit for bit.
 *   - Limits: query_count <= SHRIKE_STATIC_ROUTER_MAX_ROWS and num_experts <=
 *     SHRIKE_MAX_EXPERTS; anything larger is refused with SHRIKE_ERANGE.
 *   - The device to run on must be current. The first call on a device looks up
 *     the array's device address (cudaGetSymbolAddress); make that first call
 *     before any stream capture begins.
 *   - Every call on a device shares the one array, which keeps the previous
 *     call's logits (each call overwrites the rows it uses before reading them,
 *     so nothing needs clearing). Two calls whose kernels overlap on the GPU --
 *     different streams without an ordering between them -- race on it.
 *   - Errors come back as the return code and, when error_text is given, as
 *     text in that buffer (there is no handle to hold a message). */
int shrike_encode_router_static(const shrike_moe_config* config, void* stream,
                                const shrike_router_operands* operands, const void* hidden,
                                uint32_t query_count, uint32_t hidden_stride_elements,
                                uint32_t* out_indices, float* out_weights, float* out_shared_gate,
                                char* error_text, size_t error_text_bytes);

/* End-to-end convenience for hosts that keep activations in host memory:
 * copies x_host in, runs router -> classification -> decode/prefill for one
 * layer, copies y (and hidden) back, and synchronises. */
int shrike_moe_layer_forward_host(shrike_moe* moe, void* stream, const shrike_pool* pool,
                                  const shrike_expert_offsets* routed_offsets,
                                  const uint64_t* residency_table_row,
                                  const shrike_router_operands* router,
                                  const shrike_shared_expert* shared,
                                  const void* x_host, uint32_t query_count, void* y_host,
                                  uint32_t* ids_host, float* weights_host);

/* One layer of a decode stack, as shrike_moe_decode_stack_forward_host takes them. */
typedef struct shrike_stack_layer {
    shrike_moe*                  moe;                 /* the layer's handle (its own work lists) */
    const shrike_pool*           pool;
    const shrike_expert_offsets* routed_offsets;
    const uint64_t*              residency_table_row;
    const shrike_router_operands* router;
    const shrike_shared_expert*  shared;              /* NULL without a shared expert */
} shrike_stack_layer;

/* A decode step through stacked MoE layers with host activations in and out: what produceToken's per-layer
 * encodeRoutedLayer calls (RealForwardRunner.swift:2205-2313) amount to for this path when only the MoE
 * halves of the layers are present. The stack owns a device copy of the residual stream,
 * [(layer_count + 1) x max_rows x d] in act_dtype.
 *
 *   rows_host   [(layer_count + 1) x query_count x d]: block 0 is the row set entering layer 0; block l >= 1 is
 *               what the rest of transformer block l (attention, normalisation -- not part of this library)
 *               contributes to the residual stream between MoE layer l-1 and MoE layer l.
 *   forward     copies rows_host to the device (one copy), then for every layer l runs
 *               shrike_encode_decode_layer with x = block l and hidden = block l+1, so that
 *               block l+1 = rows_host block l+1 + y_l is the next layer's input; copies the last block
 *               into out_host [query_count x d] and synchronises the stream.
 * Every handle must share device, d and act_dtype; query_count <= max_rows <= SHRIKE_MAX_DECODE_TOKENS and
 * <= every handle's max_tokens. Pinned host memory makes the copies asynchronous up to the final wait. */
typedef struct shrike_decode_stack shrike_decode_stack;
int shrike_decode_stack_create(const shrike_stack_layer* layers, uint32_t layer_count, uint32_t max_rows,
                               shrike_decode_stack** out);
void shrike_decode_stack_destroy(shrike_decode_stack* stack);
int shrike_decode_stack_forward_host(shrike_decode_stack* stack, void* stream, const void* rows_host,
                                     uint32_t query_count, void* out_host);

#ifdef __cplusplus
}
#endif
#endif /* SHRIKE_B200_H */
