// Seeded synthetic expert blocks written straight into pool cells: what the
// benchmark and the full-size parity checks run on (no checkpoint is
// available offline). Counter-mode SplitMix64 (the PRNG of the reference's
// test fixtures, sources/ShrikeValidation/Support/PRNG/SplitMix64.swift), so any
// word of any block can be recomputed on the host.
#include "internal.h"

namespace shrike {

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__host__ __device__ __forceinline__ uint64_t splitmix64_at(uint64_t key, uint64_t index) {
    return mix64(key + (index + 1) * 0x9E3779B97F4A7C15ull);
}
__host__ __device__ __forceinline__ uint64_t block_key(uint64_t seed, uint32_t layer, uint32_t expert) {
    return mix64(seed ^ mix64((((uint64_t)layer << 32) | expert) + 0x9E3779B97F4A7C15ull));
}

struct SynthShape {
    Offsets3 off;
    uint32_t wwords[3];   // 8-byte words of packed weights per projection
    uint32_t nmeta[3];    // scales (= biases) per projection
    uint32_t nab[3];      // additive biases per projection (0 when absent)
    uint32_t bits, meta_dtype;
    uint32_t total;       // work items per block
};

__device__ __forceinline__ uint16_t to_meta(float v, uint32_t meta_dtype) {
    return meta_dtype == SHRIKE_DTYPE_FP16 ? __half_as_ushort(__float2half_rn(v))
                                           : __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float from_meta(uint16_t b, uint32_t meta_dtype) {
    return meta_dtype == SHRIKE_DTYPE_FP16 ? f16_bits_to_f32(b) : bf16_bits_to_f32(b);
}

__global__ void __launch_bounds__(256)
synth_fill_kernel(PoolView pool, uint32_t first_cell, uint64_t seed, uint32_t layer,
                  uint32_t first_expert, SynthShape sh) {
    const uint32_t cell = first_cell + blockIdx.y;
    uint8_t* block = const_cast<uint8_t*>(pool_cell_base(pool, cell));
    const uint64_t key = block_key(seed, layer, first_expert + blockIdx.y);
    const float base = sh.bits == 4 ? (0.02f / 7.5f) : (0.02f / 127.5f);
    const float zp = sh.bits == 4 ? -8.0f : -128.0f;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < sh.total; i += gridDim.x * blockDim.x) {
        uint32_t j = i;
        bool done = false;
#pragma unroll
        for (uint32_t p = 0; p < 3 && !done; ++p) {
            if (j < sh.wwords[p]) {
                ((uint64_t*)(block + sh.off.w[p]))[j] = splitmix64_at(key ^ (0x1000u + p), j);
                done = true;
            } else j -= sh.wwords[p];
        }
#pragma unroll
        for (uint32_t p = 0; p < 3 && !done; ++p) {
            if (j < sh.nmeta[p]) {
                const uint64_t r = splitmix64_at(key ^ (0x2000u + p), j);
                const float u = __fmul_rn((float)(r >> 40), 1.0f / 16777216.0f);
                const float sc = __fmul_rn(base, __fadd_rn(0.5f, u));
                const uint16_t sb = to_meta(sc, sh.meta_dtype);
                ((uint16_t*)(block + sh.off.s[p]))[j] = sb;
                ((uint16_t*)(block + sh.off.b[p]))[j] =
                    to_meta(__fmul_rn(zp, from_meta(sb, sh.meta_dtype)), sh.meta_dtype);
                done = true;
            } else j -= sh.nmeta[p];
        }
#pragma unroll
        for (uint32_t p = 0; p < 3 && !done; ++p) {
            if (j < sh.nab[p]) {
                const uint64_t r = splitmix64_at(key ^ (0x3000u + p), j);
                const uint32_t sum = (uint32_t)(r & 0xFFFF) + (uint32_t)((r >> 16) & 0xFFFF) +
                                     (uint32_t)((r >> 32) & 0xFFFF) + (uint32_t)((r >> 48) & 0xFFFF);
                const float v = __fmul_rn(__fsub_rn((float)sum, 131070.0f), 2.6429e-6f);
                ((uint16_t*)(block + sh.off.ab[p]))[j] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
                done = true;
            } else j -= sh.nab[p];
        }
    }
}

cudaError_t launch_synth_fill(const shrike_moe* m, cudaStream_t st, const PoolView& pool,
                              uint32_t first_cell, uint32_t count, uint64_t seed, uint32_t layer,
                              uint32_t first_expert, bool shared, const Offsets3& off) {
    const shrike_moe_config& c = m->cfg;
    const uint32_t f = shared ? c.shared_f : c.f;
    const uint32_t rows[3] = {f, f, c.d}, cols[3] = {c.d, c.d, f};
    SynthShape sh;
    sh.off = off;
    sh.bits = c.weight_bits;
    sh.meta_dtype = c.meta_dtype;
    sh.total = 0;
    for (int p = 0; p < 3; ++p) {
        sh.wwords[p] = rows[p] * (cols[p] * c.weight_bits / 8) / 8;
        sh.nmeta[p] = rows[p] * (cols[p] / c.group_size);
        sh.nab[p] = c.expert_bias ? rows[p] : 0;
        sh.total += sh.wwords[p] + sh.nmeta[p] + sh.nab[p];
    }
    uint32_t done = 0;
    while (done < count) {
        const uint32_t n = count - done > 32768 ? 32768 : count - done;
        synth_fill_kernel<<<dim3(64, n), 256, 0, st>>>(pool, first_cell + done, seed, layer,
                                                       first_expert + done, sh);
        done += n;
    }
    return cudaGetLastError();
}

}  // namespace shrike
