// Decode-time expert kernels: dequant-fused skinny GEMMs, one 16-row weight
// tile against up to 8 activation rows, HBM-bound.
//
//   phase 1: acts[pair, f] = GLU(gate[f,:].x + b, up[f,:].x + b)
//            (moe_phase1_gate_up_act_spec_u16load, moe.metal:950-998; shared
//            expert: dequant_int4_shared_gate_up_gemv_simd, dequant_int4.metal:206)
//   phase 2: y[t, d] = sg[t]*shared_down[d,:].acts + sum_k w[t,k]*(down_k[d,:].acts_k + b)
//            hidden[t, d] += y[t, d]
//            (moe_phase2_down_reduce_spec_k8, moe.metal:1008-1057;
//            dequant_int4_shared_down_fused, dequant_int4.metal:247-331)
//
// Arithmetic. The reference factors each group's dot product as
// scale*sum(q*x) + bias*sum(x) (int4_affine_gemv.c:108-111, moe.metal:752-755).
// Here sum((q-Z)*x) and sum(x) come out of the tensor cores exactly: the
// packed values are turned into the fp16 integers q-Z (Z = 8 or 128) with one
// logic op and one packed subtract per pair, x is an fp16 copy of the
// activation row, products and sums accumulate in fp32, and each group then
// costs one fused multiply-add with the scale and one with bias + Z*scale.
// Weight bytes are streamed once, straight from global memory into registers
// (8- or 16-byte loads per thread, 32 contiguous bytes per row and quad);
// the tile's scales and zero-point biases are staged in shared memory by the
// TMA engine (1-D bulk copies completing on an mbarrier).
#include "internal.h"

namespace shrike {


template <int BITS, int GROUP>
struct QT {
    static constexpr int kWords = GROUP * BITS / 128;  // u32 per thread, row and group
    static constexpr int kMmas = GROUP / 16;           // k16 steps per group
    static constexpr int kBRegs = GROUP / 8;           // u32 of activations per thread and group
    // groups whose weights a thread has in flight together: 16 bytes per row. (Measured at 4 and 16 rows of the
    // Qwen shape: 32 bytes per row cost 125 registers and two gate/up blocks per SM; with 16 the kernel takes 80,
    // three blocks fit, and a layer is 3 to 6 % faster -- these kernels wait on latencies, not on bytes in flight.)
    static constexpr int kBatch = kWords >= 4 ? 1 : 4 / kWords;
    // The tiles multiply (1024 + q): sum((1024 + q) x) = 1024 sum(x) + sum(q x), so a group contributes
    // scale * c + (bias - 1024 * scale) * sum(x); products and sums stay exact in fp32 (|c| < 2^24 * ulp).
    static constexpr float kOffset = -1024.0f;
};

template <int W>
__device__ __forceinline__ void load_words(const uint8_t* p, uint32_t (&w)[W]) {
    if constexpr (W == 1) {
        w[0] = ldg_stream_u32(p);
    } else if constexpr (W == 2) {
        const uint2 v = ldg_stream_u64(p);
        w[0] = v.x; w[1] = v.y;
    } else {
        const uint4 v = ldg_stream_u128(p);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    }
}

// The two A registers (k 2t..2t+1 and k 2t+8..2t+9) of k16 step `m` of a group.
template <int BITS, int W>
__device__ __forceinline__ void unpack_step(const uint32_t (&w)[W], int m, uint32_t& lo, uint32_t& hi) {
    if constexpr (BITS == 4) {
        const uint32_t v = w[m >> 1] >> ((m & 1) * 8);
        // (1024 + n_i, 1024 + n_{i+4}) as fp16, exact: the 1024 is taken out again per group together
        // with the zero point (QT::kOffset), which saves the packed subtract per register
        lo = lop3_and_or(v, 0x000F000Fu, 0x64006400u);
        hi = lop3_and_or(v >> 4, 0x000F000Fu, 0x64006400u);
    } else {
        const uint32_t v = w[m];
        // (1024 + b0, 1024 + b1)
        lo = prmt(v, 0x64646464u, 0x5140u);
        hi = prmt(v, 0x64646464u, 0x5342u);
    }
}

template <int G>
__device__ __forceinline__ void load_bfrag(const uint16_t* p, uint32_t (&b)[G / 8]) {
    const uint4 v0 = __ldg((const uint4*)p);
    b[0] = v0.x; b[1] = v0.y; b[2] = v0.z; b[3] = v0.w;
    if constexpr (G == 64) {
        const uint4 v1 = __ldg((const uint4*)p + 1);
        b[4] = v1.x; b[5] = v1.y; b[6] = v1.z; b[7] = v1.w;
    }
}

// One group of NMAT matrices (rows g and g+8 of each) against one B fragment.
// c[mat] = sum((1024+q)*x); with ONES also xs = column sums of x (identical in
// every row), otherwise the caller supplies them.
template <int BITS, int GROUP, int NMAT, bool ONES>
__device__ __forceinline__ void group_mma(const uint32_t (&raw)[NMAT][2][QT<BITS, GROUP>::kWords],
                                          const uint32_t (&b)[QT<BITS, GROUP>::kBRegs],
                                          float (&c)[NMAT][4], float (&xs)[4]) {
    constexpr uint32_t kOnes = 0x3C003C00u;
#pragma unroll
    for (int m = 0; m < QT<BITS, GROUP>::kMmas; ++m) {
        const uint32_t b0 = b[2 * m], b1 = b[2 * m + 1];
        if constexpr (ONES) mma_16816(xs, kOnes, kOnes, kOnes, kOnes, b0, b1);
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat) {
            uint32_t lo0, hi0, lo1, hi1;
            unpack_step<BITS>(raw[mat][0], m, lo0, hi0);
            unpack_step<BITS>(raw[mat][1], m, lo1, hi1);
            mma_16816(c[mat], lo0, lo1, hi0, hi1, b0, b1);
        }
    }
}

// Weight words of up to kBatch groups (g0, g0+gstep, ... < gend) of NMAT
// matrices, rows g and g+8: all loads are issued before any is used.
template <int BITS, int GROUP, int NMAT>
__device__ __forceinline__ void load_batch(const uint8_t* (&wrow)[NMAT][2], uint32_t g0, uint32_t gstep,
                                           uint32_t gend,
                                           uint32_t (&raw)[QT<BITS, GROUP>::kBatch][NMAT][2][QT<BITS, GROUP>::kWords]) {
    using Q = QT<BITS, GROUP>;
    constexpr uint32_t kGroupBytes = GROUP * BITS / 8;
#pragma unroll
    for (int i = 0; i < Q::kBatch; ++i) {
        const uint32_t grp = g0 + i * gstep;
        if (grp < gend) {
#pragma unroll
            for (int mat = 0; mat < NMAT; ++mat) {
                load_words<Q::kWords>(wrow[mat][0] + (size_t)grp * kGroupBytes, raw[i][mat][0]);
                load_words<Q::kWords>(wrow[mat][1] + (size_t)grp * kGroupBytes, raw[i][mat][1]);
            }
        }
    }
}

// The activation fragments of the same groups.
template <int BITS, int GROUP>
__device__ __forceinline__ void load_bfrags(const uint16_t* xrow, uint32_t g0, uint32_t gstep, uint32_t gend,
                                            uint32_t t,
                                            uint32_t (&bf)[QT<BITS, GROUP>::kBatch][QT<BITS, GROUP>::kBRegs]) {
#pragma unroll
    for (int i = 0; i < QT<BITS, GROUP>::kBatch; ++i) {
        const uint32_t grp = g0 + i * gstep;
        if (grp < gend) load_bfrag<GROUP>(xrow + (size_t)grp * GROUP + t * (GROUP / 4), bf[i]);
    }
}

// tot += scale * sum((1024+q)x) + (bias - 1024*scale) * sum(x) for every group of the batch.
// s_sm/b_sm[mat]: the tile's [16 x G] scales / biases in shared memory.
template <int BITS, int GROUP, int META, int NMAT, bool ONES>
__device__ __forceinline__ void compute_batch(
    const uint32_t (&raw)[QT<BITS, GROUP>::kBatch][NMAT][2][QT<BITS, GROUP>::kWords],
    const uint32_t (&bf)[QT<BITS, GROUP>::kBatch][QT<BITS, GROUP>::kBRegs],
    const float (&xsv)[QT<BITS, GROUP>::kBatch][2], const uint16_t* (&s_sm)[NMAT],
    const uint16_t* (&b_sm)[NMAT], uint32_t G, uint32_t g0, uint32_t gstep, uint32_t gend, uint32_t g,
    float (&tot)[NMAT][4]) {
    using Q = QT<BITS, GROUP>;
#pragma unroll
    for (int i = 0; i < Q::kBatch; ++i) {
        const uint32_t grp = g0 + i * gstep;
        if (grp < gend) {
            float c[NMAT][4];
            float xs[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (!ONES) { xs[0] = xsv[i][0]; xs[1] = xsv[i][1]; }
#pragma unroll
            for (int mat = 0; mat < NMAT; ++mat) c[mat][0] = c[mat][1] = c[mat][2] = c[mat][3] = 0.f;
            group_mma<BITS, GROUP, NMAT, ONES>(raw[i], bf[i], c, xs);
#pragma unroll
            for (int mat = 0; mat < NMAT; ++mat) {
                const float s0 = meta_to_f32<META>(s_sm[mat][g * G + grp]);
                const float s1 = meta_to_f32<META>(s_sm[mat][(g + 8) * G + grp]);
                const float z0 = fmaf(Q::kOffset, s0, meta_to_f32<META>(b_sm[mat][g * G + grp]));
                const float z1 = fmaf(Q::kOffset, s1, meta_to_f32<META>(b_sm[mat][(g + 8) * G + grp]));
                tot[mat][0] = fmaf(z0, xs[0], fmaf(s0, c[mat][0], tot[mat][0]));
                tot[mat][1] = fmaf(z0, xs[1], fmaf(s0, c[mat][1], tot[mat][1]));
                tot[mat][2] = fmaf(z1, xs[0], fmaf(s1, c[mat][2], tot[mat][2]));
                tot[mat][3] = fmaf(z1, xs[1], fmaf(s1, c[mat][3], tot[mat][3]));
            }
        }
    }
}

// Accumulates groups gbeg, gbeg+gstep, ... < gend of NMAT matrices into tot.
// wrow[mat][r]: this thread's byte pointer into row g+8r of the tile at group 0.
// With `preloaded` the first batch's weight words are already in `raw`.
// ONES: the per-group activation sums come out of the tensor cores; otherwise
// they are read from the tables xs0 / xs1 (one fp32 per group, for the two
// columns this thread accumulates).
template <int BITS, int GROUP, int META, int NMAT, bool ONES>
__device__ __forceinline__ void tile_accumulate(
    const uint8_t* (&wrow)[NMAT][2], const uint16_t* (&s_sm)[NMAT], const uint16_t* (&b_sm)[NMAT],
    const uint16_t* xrow, uint32_t G, uint32_t gbeg, uint32_t gend, uint32_t gstep, uint32_t g, uint32_t t,
    uint64_t* bar, uint32_t parity, uint32_t* status, float (&tot)[NMAT][4], bool preloaded,
    uint32_t (&raw)[QT<BITS, GROUP>::kBatch][NMAT][2][QT<BITS, GROUP>::kWords], const float* xs0 = nullptr,
    const float* xs1 = nullptr) {
    using Q = QT<BITS, GROUP>;
    bool waited = false;
    for (uint32_t g0 = gbeg; g0 < gend; g0 += gstep * Q::kBatch) {
        if (!(preloaded && g0 == gbeg)) load_batch<BITS, GROUP, NMAT>(wrow, g0, gstep, gend, raw);
        uint32_t bf[Q::kBatch][Q::kBRegs];
        load_bfrags<BITS, GROUP>(xrow, g0, gstep, gend, t, bf);
        float xsv[Q::kBatch][2];
        if constexpr (!ONES) {
#pragma unroll
            for (int i = 0; i < Q::kBatch; ++i) {
                const uint32_t grp = g0 + i * gstep;
                if (grp < gend) { xsv[i][0] = __ldg(xs0 + grp); xsv[i][1] = __ldg(xs1 + grp); }
            }
        }
        if (!waited) {
            // the scales arrive (TMA) while the weight loads are in flight
            if (!mbar_wait_bounded(bar, parity)) report_status(status, kStatusWaitTimeout);
            waited = true;
        }
        compute_batch<BITS, GROUP, META, NMAT, ONES>(raw, bf, xsv, s_sm, b_sm, G, g0, gstep, gend, g, tot);
    }
    if (!waited && !mbar_wait_bounded(bar, parity)) report_status(status, kStatusWaitTimeout);
}

constexpr int kP1Warps = 8;

__device__ __forceinline__ Instance load_instance(const Instance* p) {
    const uint4* q = (const uint4*)p;
    const uint4 a = q[0], b = q[1], c = q[2];
    Instance in;
    in.kind = a.x; in.slot = a.y; in.first = a.z; in.count = a.w;
    in.pair[0] = b.x; in.pair[1] = b.y; in.pair[2] = b.z; in.pair[3] = b.w;
    in.pair[4] = c.x; in.pair[5] = c.y; in.pair[6] = c.z; in.pair[7] = c.w;
    return in;
}

__device__ __forceinline__ uint32_t pick(const uint32_t (&v)[8], uint32_t i) {
    uint32_t r = v[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) r = i == (uint32_t)j ? v[j] : r;
    return r;
}

// grid (max(f, f_shared)/16, max instances); block 256. The eight warps split
// K by groups (warp w takes groups w, w+8, ...).
template <int BITS, int GROUP, int META>
__global__ void __launch_bounds__(kP1Warps * 32, 3) phase1_kernel(const ExpertArgs a) {
    using Q = QT<BITS, GROUP>;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t ii = blockIdx.y;
    // the work lists come from the kernel launched just before this one
    pdl_wait();
    const uint32_t n_inst = *a.n_inst;
    const Instance in = load_instance(a.inst + ii);
    if (ii >= n_inst) return;
    pdl_launch_dependents();
    const bool shared = in.kind == 1;
    const uint32_t F = shared ? a.f_shared : a.f;
    const uint32_t f0 = blockIdx.x * 16;
    if (f0 >= F) return;
    const Offsets3& off = shared ? a.shared : a.routed;
    const uint8_t* base = shared ? a.shared_block : pool_cell_base(a.pool, in.slot);
    const uint32_t D = a.d, G = D / GROUP;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

    // weight words first: they are the long pole
    const size_t row_bytes = (size_t)D * BITS / 8;
    const uint32_t toff = t * Q::kWords * 4;
    const uint8_t* wrow[2][2];
#pragma unroll
    for (int mat = 0; mat < 2; ++mat) {
        wrow[mat][0] = base + off.w[mat] + (size_t)(f0 + g) * row_bytes + toff;
        wrow[mat][1] = base + off.w[mat] + (size_t)(f0 + g + 8) * row_bytes + toff;
    }
    uint32_t raw[Q::kBatch][2][2][Q::kWords];
    load_batch<BITS, GROUP, 2>(wrow, warp, kP1Warps, G, raw);

    // shared memory: [gate s][gate b][up s][up b] (16*G u16 each) | ab gate, ab up (16 u16 each)
    // | mbarrier | cross-warp reduction buffer
    const uint32_t meta_bytes = 32 * G;
    uint16_t* s_gate = (uint16_t*)smem;
    uint16_t* b_gate = (uint16_t*)(smem + meta_bytes);
    uint16_t* s_up = (uint16_t*)(smem + 2 * meta_bytes);
    uint16_t* b_up = (uint16_t*)(smem + 3 * meta_bytes);
    uint16_t* ab_gate = (uint16_t*)(smem + 4 * meta_bytes);
    uint16_t* ab_up = ab_gate + 16;
    uint64_t* bar = (uint64_t*)(smem + 4 * meta_bytes + 64);
    float* red = (float*)(smem + 4 * meta_bytes + 80);

    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
        const uint32_t ab_bytes = a.expert_bias ? 64u : 0u;
        mbar_expect_tx(bar, 4 * meta_bytes + ab_bytes);
        const size_t moff = (size_t)f0 * G * 2;
        bulk_g2s(s_gate, base + off.s[0] + moff, meta_bytes, bar);
        bulk_g2s(b_gate, base + off.b[0] + moff, meta_bytes, bar);
        bulk_g2s(s_up, base + off.s[1] + moff, meta_bytes, bar);
        bulk_g2s(b_up, base + off.b[1] + moff, meta_bytes, bar);
        if (a.expert_bias) {
            bulk_g2s(ab_gate, base + off.ab[0] + (size_t)f0 * 2, 32, bar);
            bulk_g2s(ab_up, base + off.ab[1] + (size_t)f0 * 2, 32, bar);
        }
    }
    __syncthreads();  // the barrier word is initialised before anyone polls it

    // B operand: column n = g is row `n` of this instance (columns past the
    // count repeat row 0; their results are never stored).
    const uint32_t pair = pick(in.pair, g < in.count ? g : 0);
    const uint32_t token = shared ? pair : pair / a.top_k;
    const uint16_t* xrow = a.xh + (size_t)token * D;

    const uint16_t* s_sm[2] = {s_gate, s_up};
    const uint16_t* b_sm[2] = {b_gate, b_up};
    float tot[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    // per-group sums of x for the two columns this thread accumulates
    const uint32_t p0 = pick(in.pair, 2 * t < in.count ? 2 * t : 0);
    const uint32_t p1 = pick(in.pair, 2 * t + 1 < in.count ? 2 * t + 1 : 0);
    const float* xs0 = a.xsum + (size_t)(shared ? p0 : p0 / a.top_k) * G;
    const float* xs1 = a.xsum + (size_t)(shared ? p1 : p1 / a.top_k) * G;
    tile_accumulate<BITS, GROUP, META, 2, true>(wrow, s_sm, b_sm, xrow, G, warp, G, kP1Warps, g, t, bar, 0,
                                                a.status, tot, true, raw, xs0, xs1);

    // split-K reduction across the warps, fixed order
#pragma unroll
    for (int mat = 0; mat < 2; ++mat) {
        float* r = red + ((warp * 2 + mat) * 16) * 8;
        r[g * 8 + 2 * t] = tot[mat][0];
        r[g * 8 + 2 * t + 1] = tot[mat][1];
        r[(g + 8) * 8 + 2 * t] = tot[mat][2];
        r[(g + 8) * 8 + 2 * t + 1] = tot[mat][3];
    }
    __syncthreads();
    if (tid < 128) {
        const uint32_t row = tid >> 3, c = tid & 7;
        if (c < in.count) {
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < kP1Warps; ++w) {
                gate += red[((w * 2 + 0) * 16 + row) * 8 + c];
                up += red[((w * 2 + 1) * 16 + row) * 8 + c];
            }
            if (a.expert_bias) {
                gate += bf16_bits_to_f32(ab_gate[row]);
                up += bf16_bits_to_f32(ab_up[row]);
            }
            const float act = glu(gate, up, a.activation);
            const uint32_t fi = perm_index(f0 + row, BITS == 4);
            uint16_t* dst = shared ? a.acts_shared : a.acts;
            dst[(size_t)pick(in.pair, c) * F + fi] = act_to_half_bits(act, a.status);
        }
    }
}

constexpr int kP2Warps = 24;  // most warps a block uses; fewer when shared memory is short

// grid d/16; block 768. Warps take (instance, k-split) units round-robin and
// add their weighted tiles into private accumulators; a fixed-order sum over
// the warps finishes y. When the launch carries the programmatic-dependency
// attribute the warp's first unit fetches its weights and scales before it
// waits for phase 1 (the work lists were complete before phase 1 began).
template <int BITS, int GROUP, int META>
__global__ void __launch_bounds__(kP2Warps * 32) phase2_kernel(const ExpertArgs a, uint32_t T,
                                                               uint32_t ksplit, uint32_t gmax,
                                                               void* __restrict__ y,
                                                               void* __restrict__ hidden) {
    using Q = QT<BITS, GROUP>;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t d0 = blockIdx.x * 16;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

    // shared memory: per warp [s][b] (16*gmax u16 each) + ab (16 u16) + mbarrier,
    // then the per-warp accumulators [T][16] fp32.
    const uint32_t meta_bytes = 32 * gmax;
    const uint32_t per_warp = 2 * meta_bytes + 32 + 16;
    uint8_t* mine = smem + warp * per_warp;
    uint16_t* s_sm0 = (uint16_t*)mine;
    uint16_t* b_sm0 = (uint16_t*)(mine + meta_bytes);
    uint16_t* ab_sm = (uint16_t*)(mine + 2 * meta_bytes);
    uint64_t* bar = (uint64_t*)(mine + 2 * meta_bytes + 32);
    const uint32_t nw = blockDim.x >> 5;
    float* yacc_all = (float*)(smem + nw * per_warp);
    float* yacc = yacc_all + (size_t)warp * T * 16;

    for (uint32_t i = lane; i < T * 16; i += 32) yacc[i] = 0.f;
    if (lane == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncwarp();

    // The work lists were complete before phase 1 began (its own dependency wait saw them), so they can
    // be read, and this warp's first weights fetched, while phase 1 is still running.
    bool first = true;
    const uint32_t n_inst = *a.n_inst;
    const uint32_t units = n_inst * ksplit;
    uint32_t parity = 0;
    for (uint32_t u = warp; u < units; u += nw) {
        const uint32_t ii = u / ksplit, ks = u % ksplit;
        const Instance in = load_instance(a.inst + ii);
        const bool shared = in.kind == 1;
        const uint32_t F = shared ? a.f_shared : a.f;
        const uint32_t G = F / GROUP;
        const Offsets3& off = shared ? a.shared : a.routed;
        const uint8_t* base = shared ? a.shared_block : pool_cell_base(a.pool, in.slot);
        const uint32_t gbeg = G * ks / ksplit;          // G * ksplit is far below 2^32: no 64-bit division
        const uint32_t gend = G * (ks + 1) / ksplit;
        const bool add_bias = a.expert_bias && ks == 0;

        const size_t row_bytes = (size_t)F * BITS / 8;
        const uint32_t toff = t * Q::kWords * 4;
        const uint8_t* wrow[1][2];
        wrow[0][0] = base + off.w[2] + (size_t)(d0 + g) * row_bytes + toff;
        wrow[0][1] = base + off.w[2] + (size_t)(d0 + g + 8) * row_bytes + toff;
        uint32_t raw[Q::kBatch][1][2][Q::kWords];
        load_batch<BITS, GROUP, 1>(wrow, gbeg, 1, gend, raw);

        if (lane == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            const uint32_t mb = 32 * G;
            mbar_expect_tx(bar, 2 * mb + (add_bias ? 32u : 0u));
            const size_t moff = (size_t)d0 * G * 2;
            bulk_g2s(s_sm0, base + off.s[2] + moff, mb, bar);
            bulk_g2s(b_sm0, base + off.b[2] + moff, mb, bar);
            if (add_bias) bulk_g2s(ab_sm, base + off.ab[2] + (size_t)d0 * 2, 32, bar);
        }
        if (first) {
            pdl_wait();  // the activations of phase 1
            pdl_launch_dependents();
            first = false;
        }

        const uint32_t bpair = pick(in.pair, g < in.count ? g : 0);
        const uint16_t* brow = (shared ? a.acts_shared : a.acts) + (size_t)bpair * F;
        const uint16_t* s_sm[1] = {s_sm0};
        const uint16_t* b_sm[1] = {b_sm0};
        float tot[1][4] = {{0.f, 0.f, 0.f, 0.f}};
        tile_accumulate<BITS, GROUP, META, 1, true>(wrow, s_sm, b_sm, brow, G, gbeg, gend, 1, g, t, bar, parity,
                                              a.status, tot, true, raw);
        parity ^= 1;

        const float ab0 = add_bias ? bf16_bits_to_f32(ab_sm[g]) : 0.f;
        const float ab1 = add_bias ? bf16_bits_to_f32(ab_sm[g + 8]) : 0.f;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const uint32_t cc = 2 * t + c;
            if (cc < in.count) {
                const uint32_t pair = pick(in.pair, cc);
                uint32_t token;
                float w;
                if (shared) {
                    token = pair;
                    w = a.shared_gate ? a.shared_gate[token] : 1.0f;
                } else {
                    token = pair / a.top_k;
                    w = a.route_w[pair];
                }
                yacc[token * 16 + g] += w * (tot[0][c] + ab0);
                yacc[token * 16 + g + 8] += w * (tot[0][2 + c] + ab1);
            }
        }
        __syncwarp();
    }
    if (first) {
        pdl_wait();
        pdl_launch_dependents();
    }
    // the residual of this thread's first output is requested before the barrier: its round trip
    // would otherwise be the last thing the block waits for
    float h_first = 0.f;
    if (hidden && tid < T * 16) h_first = load_act(hidden, (size_t)(tid >> 4) * a.d + d0 + (tid & 15), a.act_dtype);
    __syncthreads();
    // y = sum over warps; hidden += y (moe_phase2_finish, moe.metal:889-893)
    for (uint32_t i = tid; i < T * 16; i += nw * 32) {
        const uint32_t token = i >> 4, row = i & 15;
        float acc = 0.f;
        for (uint32_t w = 0; w < nw; ++w) acc += yacc_all[(size_t)w * T * 16 + i];
        const size_t o = (size_t)token * a.d + d0 + row;
        store_act(y, o, a.y_dtype, acc);
        if (hidden) {
            const float h = (i == tid ? h_first : load_act(hidden, o, a.act_dtype)) + round_act(a.y_dtype, acc);
            store_act(hidden, o, a.act_dtype, h);
        }
    }
}

constexpr int kP2pWarps = 8;

// Prefill form of the down projection (prefill_grouped_routed_moe_batched_down, prefill.metal:693, with
// the weighted reduce of prefill_moe_reduce_token_major folded in): grid (d/16, ceil(max instances / 8)),
// one instance per warp; every row's output, additive down bias included, is multiplied by its route
// weight (the shared expert's by its gate) and added into the token's fp32 accumulator row.
template <int BITS, int GROUP, int META>
__global__ void __launch_bounds__(kP2pWarps * 32) phase2_accumulate_kernel(const ExpertArgs a, uint32_t gmax) {
    using Q = QT<BITS, GROUP>;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t d0 = blockIdx.x * 16;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const uint32_t ii = blockIdx.y * kP2pWarps + warp;
    if (ii >= *a.n_inst) return;
    const uint32_t meta_bytes = 32 * gmax;
    const uint32_t per_warp = 2 * meta_bytes + 32 + 16;
    uint8_t* mine = smem + warp * per_warp;
    uint16_t* s_sm0 = (uint16_t*)mine;
    uint16_t* b_sm0 = (uint16_t*)(mine + meta_bytes);
    uint16_t* ab_sm = (uint16_t*)(mine + 2 * meta_bytes);
    uint64_t* bar = (uint64_t*)(mine + 2 * meta_bytes + 32);

    const Instance in = load_instance(a.inst + ii);
    const bool shared = in.kind == 1;
    const uint32_t F = shared ? a.f_shared : a.f;
    const uint32_t G = F / GROUP;
    const Offsets3& off = shared ? a.shared : a.routed;
    const uint8_t* base = shared ? a.shared_block : pool_cell_base(a.pool, in.slot);
    if (lane == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
        const uint32_t mb = 32 * G;
        mbar_expect_tx(bar, 2 * mb + (a.expert_bias ? 32u : 0u));
        const size_t moff = (size_t)d0 * G * 2;
        bulk_g2s(s_sm0, base + off.s[2] + moff, mb, bar);
        bulk_g2s(b_sm0, base + off.b[2] + moff, mb, bar);
        if (a.expert_bias) bulk_g2s(ab_sm, base + off.ab[2] + (size_t)d0 * 2, 32, bar);
    }
    __syncwarp();
    const uint32_t bpair = pick(in.pair, g < in.count ? g : 0);
    const uint16_t* brow = (shared ? a.acts_shared : a.acts) + (size_t)bpair * F;
    const size_t row_bytes = (size_t)F * BITS / 8;
    const uint32_t toff = t * Q::kWords * 4;
    const uint8_t* wrow[1][2];
    wrow[0][0] = base + off.w[2] + (size_t)(d0 + g) * row_bytes + toff;
    wrow[0][1] = base + off.w[2] + (size_t)(d0 + g + 8) * row_bytes + toff;
    const uint16_t* s_sm[1] = {s_sm0};
    const uint16_t* b_sm[1] = {b_sm0};
    float tot[1][4] = {{0.f, 0.f, 0.f, 0.f}};
    uint32_t raw[Q::kBatch][1][2][Q::kWords];
    tile_accumulate<BITS, GROUP, META, 1, true>(wrow, s_sm, b_sm, brow, G, 0, G, 1, g, t, bar, 0, a.status, tot, false,
                                          raw);
    const float ab0 = a.expert_bias ? bf16_bits_to_f32(ab_sm[g]) : 0.f;
    const float ab1 = a.expert_bias ? bf16_bits_to_f32(ab_sm[g + 8]) : 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const uint32_t cc = 2 * t + c;
        if (cc < in.count) {
            const uint32_t pair = pick(in.pair, cc);
            const uint32_t token = shared ? pair : pair / a.top_k;
            const float w = shared ? (a.shared_gate ? a.shared_gate[token] : 1.0f) : a.route_w[pair];
            float* out = a.yacc + (size_t)token * a.d;
            atomicAdd(out + d0 + g, w * (tot[0][c] + ab0));
            atomicAdd(out + d0 + g + 8, w * (tot[0][2 + c] + ab1));
        }
    }
}

// ---- launchers -------------------------------------------------------------

template <typename K, typename... Args>
static cudaError_t launch_kernel(K kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                                 Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = pdl ? attr : nullptr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

static inline uint32_t p1_smem(uint32_t G) { return 4 * 32 * G + 80 + kP1Warps * 2 * 128 * 4; }
static inline uint32_t p2_smem(uint32_t gmax, uint32_t T, uint32_t warps) {
    return warps * (2 * 32 * gmax + 48) + warps * T * 16 * 4;
}

template <int BITS, int GROUP, int META>
static cudaError_t launch_p1_t(cudaStream_t st, const ExpertArgs& a, uint32_t max_inst, bool pdl) {
    const uint32_t fmax = a.f_shared > a.f ? a.f_shared : a.f;
    const uint32_t smem = p1_smem(a.d / GROUP);
    auto k = phase1_kernel<BITS, GROUP, META>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    return launch_kernel(k, dim3(fmax / 16, max_inst), dim3(kP1Warps * 32), smem, st, pdl, a);
}

template <int BITS, int GROUP, int META>
static cudaError_t launch_p2_t(cudaStream_t st, const ExpertArgs& a, uint32_t T, uint32_t max_inst, void* y,
                               void* hidden, bool pdl) {
    const uint32_t fmax = a.f_shared > a.f ? a.f_shared : a.f;
    const uint32_t gmax = fmax / GROUP;
    const uint32_t gmin = (a.f_shared && a.f_shared < a.f ? a.f_shared : a.f) / GROUP;
    // few instances (small batches): split K so that every warp has a unit of about one batch
    uint32_t warps = kP2Warps;
    while (warps > 4 && p2_smem(gmax, T, warps) > 200 * 1024) warps -= 4;
    uint32_t ksplit = warps / (max_inst ? max_inst : 1);
    const uint32_t most = gmin / QT<BITS, GROUP>::kBatch;
    if (ksplit > most) ksplit = most;
    if (ksplit < 1) ksplit = 1;
    // no more warps than units: the registers left over let the next launch's blocks start (and fetch
    // their weights) on the same SMs while this one runs
    if (max_inst * ksplit < warps) warps = max_inst * ksplit;
    const uint32_t smem = p2_smem(gmax, T, warps);
    auto k = phase2_kernel<BITS, GROUP, META>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    return launch_kernel(k, dim3(a.d / 16), dim3(warps * 32), smem, st, pdl, a, T, ksplit, gmax, y, hidden);
}

template <int BITS, int GROUP, int META>
static cudaError_t launch_p2p_t(cudaStream_t st, const ExpertArgs& a, uint32_t max_inst) {
    const uint32_t fmax = a.f_shared > a.f ? a.f_shared : a.f;
    const uint32_t gmax = fmax / GROUP;
    const uint32_t smem = kP2pWarps * (2 * 32 * gmax + 48);
    auto k = phase2_accumulate_kernel<BITS, GROUP, META>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    k<<<dim3(a.d / 16, (max_inst + kP2pWarps - 1) / kP2pWarps), kP2pWarps * 32, smem, st>>>(a, gmax);
    return cudaGetLastError();
}

#define SHRIKE_DISPATCH(FN, ...)                                                          \
    do {                                                                                  \
        const uint32_t bits = m->cfg.weight_bits, grp = m->cfg.group_size;                \
        const bool f16 = m->cfg.meta_dtype == SHRIKE_DTYPE_FP16;                          \
        if (bits == 4 && grp == 64 && !f16) return FN<4, 64, SHRIKE_DTYPE_BF16>(__VA_ARGS__); \
        if (bits == 4 && grp == 64 && f16) return FN<4, 64, SHRIKE_DTYPE_FP16>(__VA_ARGS__);  \
        if (bits == 4 && grp == 32 && !f16) return FN<4, 32, SHRIKE_DTYPE_BF16>(__VA_ARGS__); \
        if (bits == 4 && grp == 32 && f16) return FN<4, 32, SHRIKE_DTYPE_FP16>(__VA_ARGS__);  \
        if (bits == 8 && grp == 64 && !f16) return FN<8, 64, SHRIKE_DTYPE_BF16>(__VA_ARGS__); \
        if (bits == 8 && grp == 64 && f16) return FN<8, 64, SHRIKE_DTYPE_FP16>(__VA_ARGS__);  \
        if (bits == 8 && grp == 32 && !f16) return FN<8, 32, SHRIKE_DTYPE_BF16>(__VA_ARGS__); \
        if (bits == 8 && grp == 32 && f16) return FN<8, 32, SHRIKE_DTYPE_FP16>(__VA_ARGS__);  \
        return cudaErrorInvalidValue;                                                     \
    } while (0)


cudaError_t launch_phase1(const shrike_moe* m, cudaStream_t st, const ExpertArgs& a, uint32_t max_inst,
                          bool pdl) {
    SHRIKE_DISPATCH(launch_p1_t, st, a, max_inst, pdl);
}

cudaError_t launch_phase2(const shrike_moe* m, cudaStream_t st, const ExpertArgs& a, uint32_t T,
                          uint32_t max_inst, void* y, void* hidden, bool pdl) {
    SHRIKE_DISPATCH(launch_p2_t, st, a, T, max_inst, y, hidden, pdl);
}

cudaError_t launch_phase2_accumulate(const shrike_moe* m, cudaStream_t st, const ExpertArgs& a,
                                     uint32_t max_inst) {
    SHRIKE_DISPATCH(launch_p2p_t, st, a, max_inst);
}

}  // namespace shrike
