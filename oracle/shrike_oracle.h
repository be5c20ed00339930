/*
 * CPU oracle for the quantised routed-expert MoE feed-forward.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the reference's
 * CPU/C expert dequant-FFN and of the shader maths around it (router, top-k,
 * shared expert, combine). Only the test-suite, the smoke check and the
 * benchmark's CPU-baseline leg may call it; the product library never does.
 *
 * Parity pin: the int4/g64 GEMV is checked against the reference's own
 * `shrike_int4_affine_gemv` compiled unmodified (oracle/_ref), and the whole
 * file against the known-answer cases of the reference's test-suite
 * (tests/test_oracle_*.py).
 *
 * Reference files followed (paths inside the reference project):
 *   sources/ShrikeKernelsC/int4_affine_gemv.c:28-135      affine int4 GEMV
 *   sources/Shrike/Kernels/CPU/CPUExpertFFN.swift:34-140   offsets, accumulate
 *   sources/Shrike/Metal/MoE/moe.metal:46-54               generic-bits unpack
 *   sources/Shrike/Metal/MoE/moe.metal:233-288             activation, GLU, additive biases
 *   sources/Shrike/Metal/MoE/moe.metal:324-364             router GEMV
 *   sources/Shrike/Metal/MoE/moe.metal:419-491             top-k selection
 *   sources/Shrike/Metal/MoE/moe.metal:121-151             residency classification
 *   sources/Shrike/Metal/MoE/moe.metal:889-941             combine
 *   sources/Shrike/Metal/Quant/dequant_int4.metal:247-331  shared expert tail
 *   sources/Shrike/Metal/Prefill/prefill.metal:624-645     token-major reduce
 *   sources/Shrike/Kernels/Prefill/MoE/PrefillMoEGrouping.swift:269-370  pair grouping
 *   sources/Shrike/Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:104-153 wave planning
 */
#ifndef SHRIKE_ORACLE_H
#define SHRIKE_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { SO_ACT_SILU = 0, SO_ACT_GELU_TANH = 1, SO_ACT_CLAMPED_SWIGLU = 2 };
enum { SO_META_BF16 = 0, SO_META_FP16 = 1 };
enum { SO_ROUTER_SOFTMAX = 0, SO_ROUTER_SIGMOID = 1 };
enum { SO_ROUTER_W_F32 = 0, SO_ROUTER_W_INT4 = 4, SO_ROUTER_W_INT8 = 8 };

typedef struct {
    uint32_t d;            /* hidden size */
    uint32_t f;            /* expert intermediate size */
    uint32_t bits;         /* 4 or 8 */
    uint32_t group;        /* 32 or 64 */
    uint32_t meta_dtype;   /* SO_META_* : dtype of scales / zero-point biases */
    uint32_t activation;   /* SO_ACT_* */
    uint32_t expert_bias;  /* additive bf16 biases on gate/up/down present */
} so_expert_cfg;

/* Byte offsets of the sub-tensors of one packed expert block; index 0/1/2 =
 * gate/up/down. Same twelve offsets as the reference's MoEExpertOffsets. */
typedef struct {
    uint32_t w[3];
    uint32_t s[3];
    uint32_t b[3];
    uint32_t ab[3];
    uint32_t stride;  /* unpadded block size */
} so_offsets;

typedef struct {
    uint32_t num_experts;
    uint32_t top_k;
    uint32_t kind;          /* SO_ROUTER_SOFTMAX / SIGMOID */
    uint32_t weight_kind;   /* SO_ROUTER_W_* */
    float    scaling;       /* routedScalingFactor; used by the sigmoid router */
    uint32_t round_weights_f16; /* round route weights through fp16 like the shader */
} so_router_cfg;

typedef void (*so_int4_gemv_fn)(const uint8_t*, const uint16_t*, const uint16_t*,
                                const float*, size_t, size_t, float*);

/* Install the reference's own compiled `shrike_int4_affine_gemv` for the
 * int4 / group 64 / bf16 case (NULL restores the restatement). */
void so_set_reference_int4_gemv(so_int4_gemv_fn fn);

float so_bf16_to_f32(uint16_t bits);
uint16_t so_f32_to_bf16(float x);
float so_f16_to_f32(uint16_t bits);
uint16_t so_f32_to_f16(float x);
float so_exp_det(float x);

void so_offsets_make(const so_expert_cfg* cfg, so_offsets* out);

/* out[r] = sum_i (q[r][i]*scale[r][g(i)] + bias[r][g(i)]) * x[i], factored per
 * group as scale*sum(q*x) + bias*sum(x). out is written, not accumulated. */
void so_affine_gemv(const uint8_t* weights, const uint16_t* scales, const uint16_t* biases,
                    const float* x, size_t rows, size_t n, uint32_t bits, uint32_t group,
                    uint32_t meta_dtype, float* out);

float so_glu(float gate, float up, uint32_t activation);

/* scratch: 2*f + d floats. out[r] += route_weight * ffn(x)[r]. */
void so_expert_ffn_accumulate(const uint8_t* block, const so_expert_cfg* cfg,
                              const so_offsets* off, const float* x, float route_weight,
                              float* scratch, float* out);

/* Router logits, fp32 weights [ne x d]; summation order: 32 lane accumulators,
 * lane l takes float4 chunks l, l+32, ... in order with fused multiply-adds,
 * then a butterfly (xor 16, 8, 4, 2, 1). */
void so_router_logits_f32(const float* w, const float* x, uint32_t ne, uint32_t d, float* logits);

/* Router logits, affine int8/int4 g64 weights, lane order of the shader:
 * lane l takes elements g*64 + 2l, 2l+1 of every group, same butterfly. */
void so_router_logits_affine(const uint8_t* w, const uint16_t* scales, const uint16_t* biases,
                             uint32_t bits, const float* x, const float* effective_scale,
                             uint32_t ne, uint32_t d, float* logits);

/* Top-k with ties to the lower expert id; weights per router kind. bias and
 * per_expert_scale may be NULL (zeros / ones). */
void so_router_select(const float* logits, const float* bias, const float* per_expert_scale,
                      const so_router_cfg* cfg, uint32_t* ids, float* weights);

/* Residency table lookup: word = slot | state<<32, hit iff state==2 && slot!=~0. */
uint32_t so_classify_residency(const uint32_t* topk, const uint64_t* table, uint32_t top_k,
                               uint32_t num_experts, uint32_t* resolved_slots,
                               uint32_t* hit_positions, uint32_t* miss_positions,
                               uint32_t* miss_experts);

typedef struct {
    so_expert_cfg expert;      /* routed experts */
    uint32_t has_shared;
    uint32_t shared_gated;     /* multiply the shared output by sigmoid(gate . x) */
    so_expert_cfg shared;      /* shared expert geometry (f may differ) */
} so_layer_cfg;

/* One MoE layer for T tokens given routing: y[t] = shared(x[t]) + sum_k w*ffn_k(x[t]).
 * blocks[e] points at expert e's packed block (only selected ones are read).
 * shared_gate_w: fp32 [d] or NULL. threads<=1 runs inline. */
void so_moe_layer(const so_layer_cfg* cfg, const uint8_t* const* blocks,
                  const uint8_t* shared_block, const float* shared_gate_w,
                  const float* x, uint32_t tokens, const uint32_t* ids, const float* weights,
                  uint32_t top_k, float* y, uint32_t threads);

/* h2[t,d] = sum_r w[t,r] * partials[(t*top_k+r)*d + d']. */
void so_reduce_token_major(const float* partials, const float* weights, uint32_t tokens,
                           uint32_t top_k, uint32_t d, float* h2);

/* Stable grouping of (token, expert, rank) pairs by (expert, token, rank).
 * pairs_in/out: 4 u32 per pair (token, expert, rank, weight bits).
 * offsets[e] = first sorted index or 0xffffffff, counts[e]. Returns 0, or a
 * negative code for an out-of-range / duplicate pair. */
int so_group_pairs(const uint32_t* pairs_in, uint32_t n_pairs, uint32_t tokens, uint32_t top_k,
                   uint32_t num_experts, uint32_t* pairs_out, uint32_t* offsets, uint32_t* counts);

/* Wave planner without the tail tile: blocks of 5 u32 (slot, pairStart, rows,
 * stagingRow, rowTileStart); wave_of_block[i] = wave index. Returns block count
 * or -1 when max_blocks is too small / staging_rows is not a multiple of tile. */
int so_plan_expert_waves(const uint32_t* range_expert_slot, const uint32_t* range_pair_start,
                         const uint32_t* range_pair_count, uint32_t n_ranges,
                         uint32_t staging_rows, uint32_t row_tile, uint32_t* blocks,
                         uint32_t* wave_of_block, uint32_t* wave_padded_rows, uint32_t max_blocks);

/* Seeded synthetic expert block (counter-mode SplitMix64), the same function
 * the library's device-side pool fill computes. */
uint64_t so_splitmix64_at(uint64_t key, uint64_t index);
uint64_t so_synth_block_key(uint64_t seed, uint32_t layer, uint32_t expert);
void so_synth_fill_block(const so_expert_cfg* cfg, const so_offsets* off, uint64_t key,
                         uint8_t* block);

#ifdef __cplusplus
}
#endif
#endif
