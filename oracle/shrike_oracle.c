/*
 * CPU oracle (test infrastructure, not product code) — see shrike_oracle.h for
 * the list of reference files each function restates.
 *
 * Build with -ffp-contract=off: every fused multiply-add below is written as
 * fmaf() on purpose and every plain a*b+c must stay two roundings, so that the
 * summation orders documented in the header are the ones that run.
 */
#include "shrike_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------- scalars */

float so_bf16_to_f32(uint16_t bits) {
    union { uint32_t u; float f; } c;
    c.u = ((uint32_t)bits) << 16;
    return c.f;
}

/* Round-half-to-even, no NaN special case: Quantization.swift:16-23. */
uint16_t so_f32_to_bf16(float x) {
    union { uint32_t u; float f; } c;
    c.f = x;
    uint32_t lsb = (c.u >> 16) & 1u;
    return (uint16_t)((c.u + 0x7FFFu + lsb) >> 16);
}

float so_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    union { uint32_t u; float f; } c;
    if (exp == 0) {
        if (man == 0) { c.u = sign; return c.f; }
        /* subnormal: value = man * 2^-24 */
        float v = (float)man * (1.0f / 16777216.0f);
        return sign ? -v : v;
    }
    if (exp == 31) { c.u = sign | 0x7F800000u | (man << 13); return c.f; }
    c.u = sign | ((exp + 112u) << 23) | (man << 13);
    return c.f;
}

uint16_t so_f32_to_f16(float x) {
    union { uint32_t u; float f; } c;
    c.f = x;
    uint32_t sign = (c.u >> 16) & 0x8000u;
    uint32_t a = c.u & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | ((a > 0x7F800000u) ? 0x200u : 0));
    if (a >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (a < 0x33000001u) return (uint16_t)sign; /* < 2^-25 (or == 2^-25 ties to 0) */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
    if (e < -14) {
        /* subnormal half: shift so that the unit is 2^-24 */
        uint32_t shift = (uint32_t)(-14 - e) + 13u;
        uint32_t q = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1u);
        if (rem > half || (rem == half && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t q = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3FFu);
    uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
    return (uint16_t)(sign | q);
}

static inline float meta_to_f32(uint16_t bits, uint32_t meta_dtype) {
    return meta_dtype == SO_META_FP16 ? so_f16_to_f32(bits) : so_bf16_to_f32(bits);
}
static inline uint16_t f32_to_meta(float x, uint32_t meta_dtype) {
    return meta_dtype == SO_META_FP16 ? so_f32_to_f16(x) : so_f32_to_bf16(x);
}

/* ---------------------------------------------------------------- offsets */

/* CPUExpertFFN.Offsets (CPUExpertFFN.swift:34-61) generalised to any bit
 * width / group size and to the additive-bias slices the packer appends after
 * each projection's zero-point biases (RepackPlanner.swift:735-826). */
void so_offsets_make(const so_expert_cfg* cfg, so_offsets* o) {
    const uint32_t d = cfg->d, f = cfg->f;
    const uint32_t rows[3] = { f, f, d };
    const uint32_t cols[3] = { d, d, f };
    uint32_t cursor = 0;
    for (int p = 0; p < 3; ++p) {
        const uint32_t wbytes = rows[p] * (cols[p] * cfg->bits / 8u);
        const uint32_t mbytes = rows[p] * (cols[p] / cfg->group) * 2u;
        o->w[p] = cursor; cursor += wbytes;
        o->s[p] = cursor; cursor += mbytes;
        o->b[p] = cursor; cursor += mbytes;
        if (cfg->expert_bias) { o->ab[p] = cursor; cursor += rows[p] * 2u; }
        else o->ab[p] = 0;
    }
    o->stride = cursor;
}

/* ------------------------------------------------------------------ GEMV */

static so_int4_gemv_fn g_ref_int4_gemv = NULL;
void so_set_reference_int4_gemv(so_int4_gemv_fn fn) { g_ref_int4_gemv = fn; }

/* moe.metal:46-54 — value `element` of a row packed at `bits` per value. */
static inline uint32_t affine_value(const uint8_t* packed, uint32_t element, uint32_t bits) {
    const uint32_t bit = element * bits;
    const uint32_t byte = bit >> 3, shift = bit & 7u;
    uint32_t word = packed[byte];
    if (shift + bits > 8u) word |= ((uint32_t)packed[byte + 1u]) << 8;
    return (word >> shift) & ((1u << bits) - 1u);
}

/* Portable branch of int4_affine_gemv.c:117-133, with the group size, bit
 * width and meta dtype as parameters. For int4 the pair order inside a byte is
 * the reference's: dot += lo*x0 + hi*x1; xsum += x0 + x1. */
void so_affine_gemv(const uint8_t* weights, const uint16_t* scales, const uint16_t* biases,
                    const float* x, size_t rows, size_t n, uint32_t bits, uint32_t group,
                    uint32_t meta_dtype, float* out) {
    if (bits == 4 && group == 64 && meta_dtype == SO_META_BF16 && g_ref_int4_gemv) {
        g_ref_int4_gemv(weights, scales, biases, x, rows, n, out);
        return;
    }
    const size_t groups = n / group;
    const size_t row_bytes = n * bits / 8;
    for (size_t r = 0; r < rows; ++r) {
        const uint8_t* w_row = weights + r * row_bytes;
        float acc = 0.0f;
        for (size_t g = 0; g < groups; ++g) {
            const float* xg = x + g * group;
            float dot = 0.0f, xsum = 0.0f;
            if (bits == 4) {
                const uint8_t* wg = w_row + g * (group / 2);
                for (size_t k = 0; k < group / 2; ++k) {
                    const float x0 = xg[k * 2], x1 = xg[k * 2 + 1];
                    dot += (float)(wg[k] & 0x0F) * x0 + (float)(wg[k] >> 4) * x1;
                    xsum += x0 + x1;
                }
            } else {
                for (size_t k = 0; k < group; k += 2) {
                    const float x0 = xg[k], x1 = xg[k + 1];
                    const float q0 = (float)affine_value(w_row, (uint32_t)(g * group + k), bits);
                    const float q1 = (float)affine_value(w_row, (uint32_t)(g * group + k + 1), bits);
                    dot += q0 * x0 + q1 * x1;
                    xsum += x0 + x1;
                }
            }
            acc += meta_to_f32(scales[r * groups + g], meta_dtype) * dot
                 + meta_to_f32(biases[r * groups + g], meta_dtype) * xsum;
        }
        out[r] = acc;
    }
}

/* --------------------------------------------------------------- expert */

/* moe.metal:99-106 (gelu), :233-238 (silu), :280-288 (GLU incl. the clamped
 * SwiGLU, limit 7, alpha 1.702); CPUExpertFFN.swift:93-95 for silu. */
float so_glu(float gate, float up, uint32_t activation) {
    if (activation == SO_ACT_CLAMPED_SWIGLU) {
        const float g = fminf(gate, 7.0f);
        const float u = fmaxf(-7.0f, fminf(up, 7.0f));
        return (g / (1.0f + expf(-1.702f * g))) * (u + 1.0f);
    }
    if (activation == SO_ACT_GELU_TANH) {
        const float x3 = gate * gate * gate;
        float inner = 0.7978845608028654f * (gate + 0.044715f * x3);
        inner = fmaxf(-20.0f, fminf(inner, 20.0f));
        return (0.5f * gate * (1.0f + tanhf(inner))) * up;
    }
    return (gate / (1.0f + expf(-gate))) * up;
}

/* ffn(x) into scratch[2f .. 2f+d) (unweighted, additive down bias applied). */
static void expert_ffn(const uint8_t* block, const so_expert_cfg* cfg, const so_offsets* off,
                       const float* x, float* scratch) {
    const uint32_t d = cfg->d, f = cfg->f;
    float* gate_out = scratch;
    float* up_out = scratch + f;
    float* down_out = scratch + 2 * f;
    so_affine_gemv(block + off->w[0], (const uint16_t*)(block + off->s[0]),
                   (const uint16_t*)(block + off->b[0]), x, f, d, cfg->bits, cfg->group,
                   cfg->meta_dtype, gate_out);
    so_affine_gemv(block + off->w[1], (const uint16_t*)(block + off->s[1]),
                   (const uint16_t*)(block + off->b[1]), x, f, d, cfg->bits, cfg->group,
                   cfg->meta_dtype, up_out);
    const uint16_t* gab = (const uint16_t*)(block + off->ab[0]);
    const uint16_t* uab = (const uint16_t*)(block + off->ab[1]);
    const uint16_t* dab = (const uint16_t*)(block + off->ab[2]);
    for (uint32_t i = 0; i < f; ++i) {
        float g = gate_out[i], u = up_out[i];
        if (cfg->expert_bias) { g += so_bf16_to_f32(gab[i]); u += so_bf16_to_f32(uab[i]); }
        gate_out[i] = so_glu(g, u, cfg->activation);
    }
    so_affine_gemv(block + off->w[2], (const uint16_t*)(block + off->s[2]),
                   (const uint16_t*)(block + off->b[2]), gate_out, d, f, cfg->bits, cfg->group,
                   cfg->meta_dtype, down_out);
    if (cfg->expert_bias)
        for (uint32_t r = 0; r < d; ++r) down_out[r] += so_bf16_to_f32(dab[r]);
}

/* CPUExpertFFN.accumulate (CPUExpertFFN.swift:102-140). */
void so_expert_ffn_accumulate(const uint8_t* block, const so_expert_cfg* cfg,
                              const so_offsets* off, const float* x, float route_weight,
                              float* scratch, float* out) {
    expert_ffn(block, cfg, off, x, scratch);
    const float* down_out = scratch + 2 * cfg->f;
    for (uint32_t r = 0; r < cfg->d; ++r) out[r] += route_weight * down_out[r];
}

/* --------------------------------------------------------------- router */

static float butterfly32(float* lane) {
    for (int m = 16; m >= 1; m >>= 1) {
        float next[32];
        for (int l = 0; l < 32; ++l) next[l] = lane[l] + lane[l ^ m];
        memcpy(lane, next, sizeof next);
    }
    return lane[0];
}

void so_router_logits_f32(const float* w, const float* x, uint32_t ne, uint32_t d, float* logits) {
    const uint32_t chunks = d / 4;
    for (uint32_t e = 0; e < ne; ++e) {
        const float* row = w + (size_t)e * d;
        float lane[32];
        for (uint32_t l = 0; l < 32; ++l) {
            float acc = 0.0f;
            for (uint32_t c = l; c < chunks; c += 32) {
                acc = fmaf(row[4 * c + 0], x[4 * c + 0], acc);
                acc = fmaf(row[4 * c + 1], x[4 * c + 1], acc);
                acc = fmaf(row[4 * c + 2], x[4 * c + 2], acc);
                acc = fmaf(row[4 * c + 3], x[4 * c + 3], acc);
            }
            lane[l] = acc;
        }
        logits[e] = butterfly32(lane);
    }
}

/* router_gemv_body, moe.metal:324-364: per lane and group
 *   acc = fma(s, q0*x0 + q1*x1, acc); acc = fma(b, x0 + x1, acc)
 * with x = hidden * effective_scale; the cross-lane sum is this build's
 * butterfly (the shader's simd_sum order is unspecified). */
void so_router_logits_affine(const uint8_t* w, const uint16_t* scales, const uint16_t* biases,
                             uint32_t bits, const float* x, const float* effective_scale,
                             uint32_t ne, uint32_t d, float* logits) {
    const uint32_t groups = d / 64;
    const uint32_t row_bytes = d * bits / 8;
    for (uint32_t e = 0; e < ne; ++e) {
        const uint8_t* row = w + (size_t)e * row_bytes;
        float lane[32];
        for (uint32_t l = 0; l < 32; ++l) {
            float acc = 0.0f;
            for (uint32_t g = 0; g < groups; ++g) {
                const float s = so_bf16_to_f32(scales[e * groups + g]);
                const float b = so_bf16_to_f32(biases[e * groups + g]);
                const uint32_t idx = g * 64 + l * 2;
                const float q0 = (float)affine_value(row, idx, bits);
                const float q1 = (float)affine_value(row, idx + 1, bits);
                const float es0 = effective_scale ? effective_scale[idx] : 1.0f;
                const float es1 = effective_scale ? effective_scale[idx + 1] : 1.0f;
                const float x0 = x[idx] * es0, x1 = x[idx + 1] * es1;
                acc = fmaf(s, q0 * x0 + q1 * x1, acc);
                acc = fmaf(b, x0 + x1, acc);
            }
            lane[l] = acc;
        }
        logits[e] = butterfly32(lane);
    }
}

/* exp() as a fixed sequence of IEEE fp32 operations, so that router scores and
 * weights come out bit-identical on the CPU and on the GPU (the library expf
 * differs between the two in the last place). The shader uses its own
 * fast::exp (moe.metal:477); neither is pinned by the reference. */
float so_exp_det(float x) {
    x = fminf(88.0f, fmaxf(-87.0f, x));
    const float n = rintf(x * 1.4426950408889634f);
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.428606765330187e-06f, r);
    float p = 1.0f / 720.0f;
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    union { uint32_t u; float f; } c;
    c.u = (uint32_t)((int)n + 127) << 23;
    return p * c.f;
}

static inline float sigmoidf_(float x) { return 1.0f / (1.0f + so_exp_det(-x)); }

/* router_topk_select_body, moe.metal:419-491. */
void so_router_select(const float* logits, const float* bias, const float* per_expert_scale,
                      const so_router_cfg* cfg, uint32_t* ids, float* weights) {
    const uint32_t ne = cfg->num_experts, k = cfg->top_k;
    const int sig = cfg->kind == SO_ROUTER_SIGMOID;
    uint32_t top_idx[8];
    float top_score[8];
    for (int i = 0; i < 8; ++i) { top_idx[i] = 0; top_score[i] = -INFINITY; }
    for (uint32_t e = 0; e < ne; ++e) {
        const float raw = logits[e];
        const float s = (sig ? sigmoidf_(raw) : raw) + (bias ? bias[e] : 0.0f);
        if (s < top_score[k - 1]) continue;
        uint32_t pos = k;
        for (uint32_t i = 0; i < k; ++i) {
            if (s > top_score[i] || (s == top_score[i] && e < top_idx[i])) { pos = i; break; }
        }
        if (pos >= k) continue;
        for (uint32_t i = k - 1; i > pos; --i) {
            top_idx[i] = top_idx[i - 1];
            top_score[i] = top_score[i - 1];
        }
        top_idx[pos] = e;
        top_score[pos] = s;
    }
    float w[8];
    if (sig) {
        float orig[8], sum = 0.0f;
        for (uint32_t i = 0; i < k; ++i) { orig[i] = sigmoidf_(logits[top_idx[i]]); sum += orig[i]; }
        const float inv = cfg->scaling / (sum + 1e-20f);
        for (uint32_t i = 0; i < k; ++i) w[i] = orig[i] * inv;
    } else {
        const float max_s = top_score[0];
        float exps[8], sum = 0.0f;
        for (uint32_t i = 0; i < k; ++i) { exps[i] = so_exp_det(top_score[i] - max_s); sum += exps[i]; }
        for (uint32_t i = 0; i < k; ++i) w[i] = exps[i] / sum;
    }
    for (uint32_t i = 0; i < k; ++i) {
        float v = w[i] * (per_expert_scale ? per_expert_scale[top_idx[i]] : 1.0f);
        if (cfg->round_weights_f16) v = so_f16_to_f32(so_f32_to_f16(v));
        ids[i] = top_idx[i];
        weights[i] = v;
    }
}

/* moe_classify_residency_body, moe.metal:121-151. */
uint32_t so_classify_residency(const uint32_t* topk, const uint64_t* table, uint32_t top_k,
                               uint32_t num_experts, uint32_t* resolved_slots,
                               uint32_t* hit_positions, uint32_t* miss_positions,
                               uint32_t* miss_experts) {
    uint32_t hits = 0, misses = 0;
    for (uint32_t p = 0; p < top_k; ++p) {
        uint32_t e = topk[p] < num_experts - 1u ? topk[p] : num_experts - 1u;
        const uint64_t word = table[e];
        const uint32_t slot = (uint32_t)(word & 0xffffffffu);
        const uint32_t state = (uint32_t)(word >> 32);
        if (state == 2u && slot != 0xffffffffu) {
            hit_positions[hits++] = p;
            resolved_slots[p] = slot;
        } else {
            miss_positions[misses] = p;
            miss_experts[misses] = e;
            ++misses;
            resolved_slots[p] = 0xffffffffu;
        }
    }
    return misses;
}

/* ---------------------------------------------------------------- layer */

typedef struct {
    const so_layer_cfg* cfg;
    const uint8_t* const* blocks;
    const uint8_t* shared_block;
    const float* x;
    const uint32_t* ids;
    uint32_t top_k, per_token, n_tasks, d;
    so_offsets off_routed, off_shared;
    float* contrib;          /* n_tasks x d, unweighted ffn outputs */
    volatile uint32_t next;
    pthread_mutex_t mu;
} layer_job;

static void* layer_worker(void* arg) {
    layer_job* j = (layer_job*)arg;
    const so_layer_cfg* c = j->cfg;
    const uint32_t fmax = c->expert.f > c->shared.f ? c->expert.f : c->shared.f;
    float* scratch = (float*)malloc(sizeof(float) * (2 * fmax + j->d));
    for (;;) {
        pthread_mutex_lock(&j->mu);
        uint32_t t = j->next++;
        pthread_mutex_unlock(&j->mu);
        if (t >= j->n_tasks) break;
        const uint32_t tok = t / j->per_token, r = t % j->per_token;
        const float* x = j->x + (size_t)tok * j->d;
        if (r < j->top_k) {
            const uint32_t e = j->ids[tok * j->top_k + r];
            expert_ffn(j->blocks[e], &c->expert, &j->off_routed, x, scratch);
            memcpy(j->contrib + (size_t)t * j->d, scratch + 2 * c->expert.f, sizeof(float) * j->d);
        } else {
            expert_ffn(j->shared_block, &c->shared, &j->off_shared, x, scratch);
            memcpy(j->contrib + (size_t)t * j->d, scratch + 2 * c->shared.f, sizeof(float) * j->d);
        }
    }
    free(scratch);
    return NULL;
}

/* Decode dataflow of the reference: h1 = [sigmoid(g.x)] * shared(x)
 * (RealForwardRunner.swift:5436-5467), y = h1 + sum_k w_k * down_k in rank
 * order (moe.metal:936-940; CPUExpertFFN.swift:137-139). */
void so_moe_layer(const so_layer_cfg* cfg, const uint8_t* const* blocks,
                  const uint8_t* shared_block, const float* shared_gate_w,
                  const float* x, uint32_t tokens, const uint32_t* ids, const float* weights,
                  uint32_t top_k, float* y, uint32_t threads) {
    layer_job j;
    memset(&j, 0, sizeof j);
    j.cfg = cfg; j.blocks = blocks; j.shared_block = shared_block; j.x = x; j.ids = ids;
    j.top_k = top_k; j.d = cfg->expert.d;
    j.per_token = top_k + (cfg->has_shared ? 1u : 0u);
    j.n_tasks = tokens * j.per_token;
    so_offsets_make(&cfg->expert, &j.off_routed);
    if (cfg->has_shared) so_offsets_make(&cfg->shared, &j.off_shared);
    j.contrib = (float*)malloc(sizeof(float) * (size_t)j.n_tasks * j.d);
    pthread_mutex_init(&j.mu, NULL);
    if (threads <= 1) {
        layer_worker(&j);
    } else {
        if (threads > 256) threads = 256;
        pthread_t th[256];
        for (uint32_t i = 0; i < threads; ++i) pthread_create(&th[i], NULL, layer_worker, &j);
        for (uint32_t i = 0; i < threads; ++i) pthread_join(th[i], NULL);
    }
    pthread_mutex_destroy(&j.mu);
    const uint32_t d = j.d;
    for (uint32_t t = 0; t < tokens; ++t) {
        float* out = y + (size_t)t * d;
        const float* xt = x + (size_t)t * d;
        if (cfg->has_shared) {
            const float* sh = j.contrib + ((size_t)t * j.per_token + top_k) * d;
            float gate = 1.0f;
            if (cfg->shared_gated) {
                float acc = 0.0f;
                for (uint32_t i = 0; i < d; ++i) acc += shared_gate_w[i] * xt[i];
                gate = sigmoidf_(acc);
            }
            for (uint32_t r = 0; r < d; ++r) out[r] = cfg->shared_gated ? sh[r] * gate : sh[r];
        } else {
            for (uint32_t r = 0; r < d; ++r) out[r] = 0.0f;
        }
        for (uint32_t k = 0; k < top_k; ++k) {
            const float w = weights[t * top_k + k];
            const float* c = j.contrib + ((size_t)t * j.per_token + k) * d;
            for (uint32_t r = 0; r < d; ++r) out[r] += w * c[r];
        }
    }
    free(j.contrib);
}

/* prefill_moe_reduce_token_major, prefill.metal:624-645. */
void so_reduce_token_major(const float* partials, const float* weights, uint32_t tokens,
                           uint32_t top_k, uint32_t d, float* h2) {
    for (uint32_t t = 0; t < tokens; ++t)
        for (uint32_t i = 0; i < d; ++i) {
            float acc = 0.0f;
            for (uint32_t r = 0; r < top_k; ++r)
                acc = fmaf(weights[t * top_k + r], partials[((size_t)t * top_k + r) * d + i], acc);
            h2[(size_t)t * d + i] = acc;
        }
}

/* ------------------------------------------------------------- grouping */

typedef struct { uint32_t token, expert, rank, wbits; } so_pair;

static int pair_cmp(const void* a, const void* b) {
    const so_pair* p = (const so_pair*)a; const so_pair* q = (const so_pair*)b;
    if (p->expert != q->expert) return p->expert < q->expert ? -1 : 1;
    if (p->token != q->token) return p->token < q->token ? -1 : 1;
    if (p->rank != q->rank) return p->rank < q->rank ? -1 : 1;
    return 0;
}

/* PrefillMoEGrouping.groupTokenExpertPairs, PrefillMoEGrouping.swift:269-370
 * (without the custom expert order, which only serves SSD-fetch scheduling). */
int so_group_pairs(const uint32_t* pairs_in, uint32_t n_pairs, uint32_t tokens, uint32_t top_k,
                   uint32_t num_experts, uint32_t* pairs_out, uint32_t* offsets, uint32_t* counts) {
    if (n_pairs != tokens * top_k) return -1;
    uint8_t* seen = (uint8_t*)calloc((size_t)tokens * top_k + 1, 1);
    const so_pair* in = (const so_pair*)pairs_in;
    for (uint32_t i = 0; i < n_pairs; ++i) {
        if (in[i].token >= tokens) { free(seen); return -2; }
        if (in[i].rank >= top_k) { free(seen); return -3; }
        if (in[i].expert >= num_experts) { free(seen); return -4; }
        uint8_t* s = &seen[(size_t)in[i].token * top_k + in[i].rank];
        if (*s) { free(seen); return -5; }
        *s = 1;
    }
    free(seen);
    memcpy(pairs_out, pairs_in, sizeof(so_pair) * n_pairs);
    qsort(pairs_out, n_pairs, sizeof(so_pair), pair_cmp);
    for (uint32_t e = 0; e < num_experts; ++e) { offsets[e] = 0xffffffffu; counts[e] = 0; }
    const so_pair* out = (const so_pair*)pairs_out;
    for (uint32_t i = 0; i < n_pairs; ++i) {
        if (counts[out[i].expert] == 0) offsets[out[i].expert] = i;
        counts[out[i].expert]++;
    }
    return 0;
}

/* planExpertWaves without the tail tile, PrefillGroupedRoutedMoE.swift:104-153. */
int so_plan_expert_waves(const uint32_t* range_expert_slot, const uint32_t* range_pair_start,
                         const uint32_t* range_pair_count, uint32_t n_ranges,
                         uint32_t staging_rows, uint32_t row_tile, uint32_t* blocks,
                         uint32_t* wave_of_block, uint32_t* wave_padded_rows, uint32_t max_blocks) {
    if (staging_rows < row_tile || staging_rows % row_tile != 0) return -1;
    uint32_t n = 0, wave = 0, cursor = 0, wave_has = 0;
    for (uint32_t i = 0; i < n_ranges; ++i) {
        uint32_t consumed = 0;
        while (consumed < range_pair_count[i]) {
            if (cursor == staging_rows) {
                wave_padded_rows[wave] = cursor; wave++; cursor = 0; wave_has = 0;
            }
            uint32_t rows = range_pair_count[i] - consumed;
            if (rows > staging_rows - cursor) rows = staging_rows - cursor;
            if (n >= max_blocks) return -1;
            uint32_t* b = blocks + 5 * n;
            b[0] = range_expert_slot[i];
            b[1] = range_pair_start[i] + consumed;
            b[2] = rows;
            b[3] = cursor;
            b[4] = cursor / row_tile;
            wave_of_block[n] = wave;
            n++; wave_has = 1;
            cursor += (rows + row_tile - 1) / row_tile * row_tile;
            consumed += rows;
        }
    }
    if (wave_has) wave_padded_rows[wave] = cursor;
    return (int)n;
}

/* ------------------------------------------------------- synthetic blocks */

static inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* Output number `index` of a SplitMix64 stream seeded with `key`
 * (SplitMix64.swift: state += golden; mix(state)). */
uint64_t so_splitmix64_at(uint64_t key, uint64_t index) {
    return mix64(key + (index + 1) * 0x9E3779B97F4A7C15ull);
}

uint64_t so_synth_block_key(uint64_t seed, uint32_t layer, uint32_t expert) {
    return mix64(seed ^ mix64((((uint64_t)layer << 32) | expert) + 0x9E3779B97F4A7C15ull));
}

/* nibbles/bytes uniform; scale = (0.02 / (2^bits-1)/2) * U(0.5,1.5) rounded to
 * the meta dtype; zero-point bias = -2^(bits-1) * scale (exact); additive
 * biases: sum of four 16-bit uniforms scaled to unit variance times 0.1. */
void so_synth_fill_block(const so_expert_cfg* cfg, const so_offsets* off, uint64_t key,
                         uint8_t* block) {
    const uint32_t rows[3] = { cfg->f, cfg->f, cfg->d };
    const uint32_t cols[3] = { cfg->d, cfg->d, cfg->f };
    const float base = cfg->bits == 4 ? (0.02f / 7.5f) : (0.02f / 127.5f);
    const float zp = cfg->bits == 4 ? -8.0f : -128.0f;
    for (uint32_t p = 0; p < 3; ++p) {
        const uint32_t wwords = rows[p] * (cols[p] * cfg->bits / 8u) / 8u;
        uint8_t* w = block + off->w[p];
        for (uint32_t i = 0; i < wwords; ++i) {
            uint64_t r = so_splitmix64_at(key ^ (0x1000u + p), i);
            memcpy(w + 8 * (size_t)i, &r, 8);
        }
        const uint32_t n_meta = rows[p] * (cols[p] / cfg->group);
        uint16_t* s = (uint16_t*)(block + off->s[p]);
        uint16_t* b = (uint16_t*)(block + off->b[p]);
        for (uint32_t i = 0; i < n_meta; ++i) {
            uint64_t r = so_splitmix64_at(key ^ (0x2000u + p), i);
            float u = (float)(r >> 40) * (1.0f / 16777216.0f);
            float t = 0.5f + u;
            float sc = base * t;
            uint16_t sb = f32_to_meta(sc, cfg->meta_dtype);
            s[i] = sb;
            b[i] = f32_to_meta(zp * meta_to_f32(sb, cfg->meta_dtype), cfg->meta_dtype);
        }
        if (cfg->expert_bias) {
            uint16_t* ab = (uint16_t*)(block + off->ab[p]);
            for (uint32_t i = 0; i < rows[p]; ++i) {
                uint64_t r = so_splitmix64_at(key ^ (0x3000u + p), i);
                uint32_t sum = (uint32_t)(r & 0xFFFF) + (uint32_t)((r >> 16) & 0xFFFF)
                             + (uint32_t)((r >> 32) & 0xFFFF) + (uint32_t)((r >> 48) & 0xFFFF);
                float v = ((float)sum - 131070.0f) * 2.6429e-6f;
                ab[i] = so_f32_to_bf16(v);
            }
        }
    }
}
