// Batched routed-expert GEMMs on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
//
// For every expert e with its n_e tokens (pairs sorted by expert, "slots"):
//   up   : G[h, t] = W1_e[h, :] . x_t,  U[h, t] = W3_e[h, :] . x_t,  mid[slot, h] = silu(G) * U
//   down : y[slot, o] = w_pair * W2_e[o, :] . mid[slot, :]
// Weights are the MMA's A operand (M = 128 weight rows per tile), tokens its B operand (N = 16 .. 128 tokens),
// so a weight tile is read from HBM and dequantised ONCE for all tokens of the expert.
//
// Numbers.  Operands are fp16, products and sums FP32 in the tensor core.
//   * weights: E2M1 * 2^(s - c_row), c_row = largest E8M0 byte of the row (computed in-kernel from the row's own
//     scale bytes, which are read once and cached in shared memory).  E2M1 times a power of two is exact in fp16
//     down to 2^-24, i.e. blocks up to 2^23 times smaller than the row's largest are exact, smaller ones vanish.
//   * activations: x_t * 2^-e_t with the token's largest magnitude in [1, 2)  (moe_prep.cuh).
//   * mid is stored as silu(G) * U * 2^(-2 e_t) in fp16: since |silu(g)| <= |g| its magnitude is bounded by the
//     product of two dot products of normalised activations with weight rows, whatever the scale of x.
// The powers of two are multiplied back in the epilogues, in FP32.
//
// CTA = 17 warps: warps 0..15 dequantise the weight tiles and copy the token tile into a ring of shared-memory
// stages (K-major, 128-byte swizzle), one lane of warp 16 issues the MMAs and releases stages through
// tcgen05.commit; warps 0..3 then read the accumulators.  Persistent grid, one CTA per SM, static tile striding.
// Every wait is bounded (stream_ring.cuh).
#pragma once

#include "moe_prep.cuh"
#include "stream_ring.cuh"
#include "tc05.cuh"

namespace dsv4 {

constexpr int kGemmProducers = 512;             // 16 producer warps
constexpr int kGemmThreads = kGemmProducers + 32;
constexpr int kGemmKBlock = 64;                 // K values per stage (128 bytes of fp16 per row)
constexpr uint32_t kGemmTileBytes = 128 * 128;  // one operand tile of 128 rows

struct MoeGemmArgs {
    const uint8_t* wa_p; const uint8_t* wb_p;   // up: W1, W3 packed; down: W2 (wb unused)
    const uint8_t* wa_s; const uint8_t* wb_s;   // their E8M0 scales
    long long stride_p, stride_s;               // bytes per expert
    int rows;                                   // weight rows per expert in this stage
    int K;                                      // reduction length of this stage (multiple of 256)
    int n_experts, k_top;
    const __half* act;                          // up: normalised x [T, K]; down: mid [P, K]
    const int* xexp;                            // [T] exponent removed from x
    const float* pair_w;                        // [P] router weight of pair t * k + j (down)
    MoeGroups g;
    __half* mid;                                // up output [P, rows]
    float* y;                                   // down output [P, rows]
};

template <int MODE>   // 0 = up (two weight matrices), 1 = down
struct MoeGemmLayout {
    static constexpr int kMats = MODE == 0 ? 2 : 1;
    static constexpr int kStages = MODE == 0 ? 3 : 4;
    static constexpr uint32_t kStageBytes = (kMats + 1) * kGemmTileBytes;
    static constexpr uint32_t kScaleCache = kStages * kStageBytes;          // kMats * 128 rows * (K / 32) bytes
    static uint32_t bytes(int K) { return kScaleCache + kMats * 128 * (K / 32) + 1024; }
};

// 2^d (d <= 0) as fp16 bits, exact down to 2^-24, 0 below.
__device__ __forceinline__ uint32_t half_pow2_bits(int d) {
    if (d >= -14) return (uint32_t)(15 + d) << 10;
    if (d >= -24) return 1u << (d + 24);
    return 0u;
}

// 2^e as float for |e| well inside the FP32 range.
__device__ __forceinline__ float float_pow2(int e) {
    e = min(max(e, -126), 127);
    return __uint_as_float((uint32_t)(e + 127) << 23);
}

// 16 packed bytes (32 E2M1 values of one scale block) -> 32 fp16 values times `mult2`, into chunks
// 4 * half .. 4 * half + 3 of row `row` of a swizzled tile.
__device__ __forceinline__ void dequant_block_to_tile(const uint4& w, uint32_t mult_bits, uint8_t* tile, int row,
                                                      int half) {
    const uint32_t m2 = mult_bits | (mult_bits << 16);
    const __half2 mult = *reinterpret_cast<const __half2*>(&m2);
    const uint32_t word[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h[4];
        e2m1x8_to_h2x4(word[i], h);
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __hmul2(h[j], mult);
        *reinterpret_cast<uint4*>(tile + tc05_sw128_offset(row, 4 * half + i)) = *reinterpret_cast<const uint4*>(h);
    }
}

}  // namespace dsv4
