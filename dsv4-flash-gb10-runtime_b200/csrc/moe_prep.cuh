// Small kernels around the batched routed-expert GEMMs: activations to normalised fp16, grouping of
// (token, expert) pairs by expert, and the final per-token sum.
#pragma once

#include "gemv_engine.cuh"

namespace dsv4 {

constexpr int kMoeMaxExperts = 1024;
constexpr int kMoeTileRows = 128;      // weight rows per tensor-core tile (the MMA's M)
constexpr int kMoeTileTokens = 128;    // tokens per tile at most (fp16 path; the MMA's N)

// Work descriptors written by the grouping kernel, read by the GEMM kernels.
struct MoeGroups {
    int* offsets;        // [E + 1] first slot of every expert (slots = pairs sorted by expert)
    int* tiles_up;       // [E + 1] prefix sum of gate/up tiles per expert
    int* tiles_down;     // [E + 1] prefix sum of down tiles per expert
    int* slot_pair;      // [P] slot -> pair index t * k + j
    int* pair_slot;      // [P] pair index -> slot
};

// One warp per token: x (bf16) -> x * 2^-e as fp16 with the largest magnitude in [1, 2), e stored per token.
// Rows of all-zero tokens get e = 0.
__global__ void moe_token_fp16_kernel(const __nv_bfloat16* __restrict__ x, int n_tokens, int K,
                                      __half* __restrict__ xh, int* __restrict__ xexp) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    const __nv_bfloat16* row = x + (size_t)t * K;
    uint32_t m = 0;
    for (int c = lane; c < K / 8; c += 32) {
        float v[8];
        load8_as_float(row + 8 * c, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) m = max(m, __float_as_uint(v[i]) & 0x7fffffffu);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = max(m, __shfl_xor_sync(kFullMask, m, off));
    int e = (int)(m >> 23) - 127;                      // floor(log2(amax)); -127 for zero / subnormal rows
    if (m == 0) e = 0;
    e = min(max(e, -100), 100);
    const float inv = __uint_as_float((uint32_t)(127 - e) << 23);
    for (int c = lane; c < K / 8; c += 32) {
        float v[8];
        load8_as_float(row + 8 * c, v);
        __half2 h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i] * inv, v[2 * i + 1] * inv);
        *reinterpret_cast<uint4*>(xh + (size_t)t * K + 8 * c) = *reinterpret_cast<const uint4*>(h);
    }
    if (lane == 0) xexp[t] = e;
}

// Single CTA: counting sort of the P = n_tokens * k pairs by expert id.  The order of pairs inside an expert is
// arbitrary (it only decides which accumulator column a token uses, not any arithmetic).  tok_up / tok_down and
// m_tiles_up / m_tiles_down: tokens per tile and row tiles per expert of the GEMM kernels that will read the tables.
__global__ void __launch_bounds__(1024) moe_group_kernel(const int* __restrict__ ids, int n_pairs, int n_experts,
                                                         int m_tiles_up, int m_tiles_down, int tok_up, int tok_down,
                                                         MoeGroups g, int* __restrict__ status) {
    __shared__ int count[kMoeMaxExperts];
    __shared__ int cursor[kMoeMaxExperts];
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    // a single CTA is latency-bound: keep eight independent loads of ids in flight per thread
    constexpr int kBatch = 8;
    for (int p0 = threadIdx.x; p0 < n_pairs; p0 += blockDim.x * kBatch) {
        int e[kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
            const int p = p0 + i * blockDim.x;
            e[i] = p < n_pairs ? __ldg(ids + p) : -1;
        }
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
            if (e[i] >= 0 && e[i] < n_experts) atomicAdd(&count[e[i]], 1);
            else if (e[i] >= n_experts) atomicExch(status, 3);   // id past the bank: dropped and reported
            // (a negative id marks a pair that is not this bank's: dropped silently, e.g. another rank's expert)
        }
    }
    __syncthreads();
    // exclusive prefix sums over the experts (thread e owns expert e; blockDim.x == kMoeMaxExperts): pair counts,
    // gate/up tiles and down tiles, scanned together
    {
        __shared__ int warp_sums[3][32];
        const int e = threadIdx.x, lane = e & 31, wid = e >> 5;
        const int c = e < n_experts ? count[e] : 0;
        int v[3] = {c, ((c + tok_up - 1) / tok_up) * m_tiles_up, ((c + tok_down - 1) / tok_down) * m_tiles_down};
        int inc[3];
#pragma unroll
        for (int q = 0; q < 3; ++q) {
            int x = v[q];
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int y = __shfl_up_sync(kFullMask, x, off);
                if (lane >= off) x += y;
            }
            inc[q] = x;
            if (lane == 31) warp_sums[q][wid] = x;
        }
        __syncthreads();
        if (wid == 0) {
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                int x = warp_sums[q][lane];
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const int y = __shfl_up_sync(kFullMask, x, off);
                    if (lane >= off) x += y;
                }
                warp_sums[q][lane] = x;                  // inclusive over warps
            }
        }
        __syncthreads();
        int exc[3];
#pragma unroll
        for (int q = 0; q < 3; ++q) exc[q] = inc[q] - v[q] + (wid > 0 ? warp_sums[q][wid - 1] : 0);
        if (e < n_experts) {
            g.offsets[e] = exc[0]; g.tiles_up[e] = exc[1]; g.tiles_down[e] = exc[2];
            cursor[e] = exc[0];
        }
        if (e == n_experts - 1) {
            g.offsets[n_experts] = exc[0] + v[0]; g.tiles_up[n_experts] = exc[1] + v[1];
            g.tiles_down[n_experts] = exc[2] + v[2];
        }
    }
    __syncthreads();
    for (int p0 = threadIdx.x; p0 < n_pairs; p0 += blockDim.x * kBatch) {
        int e[kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
            const int p = p0 + i * blockDim.x;
            e[i] = p < n_pairs ? __ldg(ids + p) : -1;
        }
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
            const int p = p0 + i * blockDim.x;
            if (e[i] >= 0 && e[i] < n_experts) {
                const int slot = atomicAdd(&cursor[e[i]], 1);
                g.slot_pair[slot] = p;
                g.pair_slot[p] = slot;
            } else if (p < n_pairs) {
                g.pair_slot[p] = -1;
            }
        }
    }
}

// out[t, :] = bf16( sum_j y[slot(t, j), :] ), j in the router's order (fixed summation order).
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pair_slot, int n_tokens,
                                   int k, int O, __nv_bfloat16* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int o = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (o >= O) return;
    for (int t = blockIdx.y; t < n_tokens; t += gridDim.y) {         // grid.y is capped at 65 535
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < k; ++j) {
            const int slot = pair_slot[t * k + j];
            if (slot < 0) continue;
            const float4 v = __ldcs(reinterpret_cast<const float4*>(y + (size_t)slot * O + o));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(out + (size_t)t * O + o) = packed;
    }
}

// Expert parallel: where the per-token sums of a rank go.  Token t of the gathered batch belongs to rank
// t / tokens_per_rank; its partial row is stored straight into THAT rank's receive buffer (a peer pointer: plain
// stores over NVLink, no collective), at [my_rank][t % tokens_per_rank][O].
constexpr int kMoeMaxRanks = 16;
struct MoePeerOut {
    __nv_bfloat16* recv[kMoeMaxRanks];     // receive buffer of every rank, [world][tokens_per_rank][O] bf16
    int world, my_rank, tokens_per_rank;
};

// Expert parallel, input side: the tokens of the gathered batch are not copied together first; rank r's tokens
// are read where they are, from the buffers rank r published (peer pointers: plain loads over NVLink).
struct MoePeerIn {
    const __nv_bfloat16* x[kMoeMaxRanks];      // [tokens_per_rank, K] bf16 of every rank
    const int* ids[kMoeMaxRanks];              // [tokens_per_rank, k] GLOBAL expert ids
    const float* w[kMoeMaxRanks];              // [tokens_per_rank, k] router weights
    int world, my_rank, tokens_per_rank, experts_per_rank;
};

// ids / weights of all ranks -> this rank's view of the gathered batch: local expert index, or -1 where the
// expert lives on another rank (a pair the layer skips).
__global__ void moe_ep_gather_meta_kernel(const MoePeerIn in, int k, int* __restrict__ ids_local,
                                          float* __restrict__ w_local) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_rank = in.tokens_per_rank * k;
    const int n = in.world * per_rank;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int r = i / per_rank, j = i - r * per_rank;
        const int e = __ldcg(in.ids[r] + j) - in.my_rank * in.experts_per_rank;
        ids_local[i] = (e >= 0 && e < in.experts_per_rank) ? e : -1;
        w_local[i] = __ldcg(in.w[r] + j);
    }
}

// moe_combine_kernel with the peer destination above: the exchange is the kernel's own stores, row by row.
__global__ void moe_combine_peer_kernel(const float* __restrict__ y, const int* __restrict__ pair_slot, int n_tokens,
                                        int k, int O, const MoePeerOut peer) {
    pdl_launch_dependents();
    pdl_wait();
    const int o = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (o >= O) return;
    for (int t = blockIdx.y; t < n_tokens; t += gridDim.y) {         // grid.y is capped at 65 535
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        bool any = false;
        for (int j = 0; j < k; ++j) {
            const int slot = pair_slot[t * k + j];
            if (slot < 0) continue;
            any = true;
            const float4 v = __ldcs(reinterpret_cast<const float4*>(y + (size_t)slot * O + o));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (!any) continue;                 // none of the token's experts lives here: the home rank skips this slice
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        const int home = t / peer.tokens_per_rank, tl = t - home * peer.tokens_per_rank;
        __nv_bfloat16* dst = peer.recv[home] + ((size_t)peer.my_rank * peer.tokens_per_rank + tl) * O + o;
        *reinterpret_cast<uint2*>(dst) = packed;
    }
}

// out[t, :] = bf16( sum_r recv[r][t, :] ), ranks in ascending order (fixed summation order), over the ranks that
// own at least one of the token's experts (ids [n_tokens, k] global, experts_per_rank per rank): the others wrote
// nothing.
__global__ void moe_ep_sum_kernel(const __nv_bfloat16* __restrict__ recv, const int* __restrict__ ids, int k,
                                  int experts_per_rank, int world, int n_tokens, int O,
                                  __nv_bfloat16* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t n4 = (size_t)n_tokens * O / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / (size_t)(O / 4));
        uint32_t owners = 0;
        for (int j = 0; j < k; ++j) {
            const int e = ids[t * k + j];
            if (e >= 0 && e / experts_per_rank < world) owners |= 1u << (e / experts_per_rank);
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < world; ++r) {
            if (!((owners >> r) & 1u)) continue;
            const uint2 q = __ldcs(reinterpret_cast<const uint2*>(recv + (size_t)r * n_tokens * O) + i);
            acc.x += __uint_as_float(q.x << 16); acc.y += __uint_as_float(q.x & 0xffff0000u);
            acc.z += __uint_as_float(q.y << 16); acc.w += __uint_as_float(q.y & 0xffff0000u);
        }
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(out)[i] = packed;
    }
}

// Rows of activations -> three MXFP4 terms whose sum reproduces the row to ~12 bits:
//   v ~ q1 * 2^e1 + q2 * 2^e2 + q3 * 2^e3   per 32-element block, q E2M1, 2^e the smallest power of two with
// amax(what is left) <= 6 * 2^e (no saturation),
// each term the round-to-nearest E2M1 quantisation of the residual the previous terms left.  The tensor cores
// multiply FP4 by FP4; three terms are what keeps the layer inside its tolerance (one term: cosine 0.993).
// Output: q [3][rows][K / 2] packed (low nibble = even element), s [3][rows][K / 32] E8M0 bytes.
// A lane owns eight neighbouring elements, four lanes own a block, a warp 256 consecutive elements of a row
// (K must be a multiple of 256): 16- or 32-byte loads, one 4-byte store per lane and term.
// With PEER the rows are not in `src` but in the per-rank buffers of `in` (row t = row t % tokens_per_rank of rank
// t / tokens_per_rank).
// rows_used (device, may be null): only rows [0, *rows_used) are converted (the intermediate of an expert-parallel
// rank holds rows for its own pairs only).  row_ids / k (may be null): row t is converted only if one of
// row_ids[t * k .. t * k + k) is >= 0 (a token none of whose experts lives on this rank is never read).
template <class Elem, bool PEER = false>
__global__ void moe_quantize_mxfp4x3_kernel(const Elem* __restrict__ src, long long rows, int K,
                                            uint8_t* __restrict__ q, uint8_t* __restrict__ s, const MoePeerIn in = {},
                                            const int* __restrict__ rows_used = nullptr,
                                            const int* __restrict__ row_ids = nullptr, int k = 0) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long live_rows = rows_used ? min(rows, (long long)__ldg(rows_used)) : rows;
    const long long n_chunks = live_rows * (K / 256);
    const long long term_q = rows * (K / 2), term_s = rows * (K / 32);
    for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < n_chunks;
         w += (long long)gridDim.x * (blockDim.x >> 5)) {
        const long long e0 = w * 256 + 8 * lane;                    // first of this lane's eight elements (row-major)
        if (row_ids) {
            const long long row = e0 / K;
            bool wanted = false;
            for (int j = 0; j < k; ++j) wanted |= __ldg(row_ids + row * k + j) >= 0;
            if (!wanted) continue;                                   // warp-uniform: a warp works on one row
        }
        float v[8];
        if constexpr (sizeof(Elem) == 2) {
            const Elem* from = src + e0;
            if constexpr (PEER) {
                const long long row = e0 / K;
                const int r = (int)(row / in.tokens_per_rank);
                from = reinterpret_cast<const Elem*>(in.x[r]) + (row - (long long)r * in.tokens_per_rank) * K + (e0 - row * K);
            }
            const uint4 u = __ldcs(reinterpret_cast<const uint4*>(from));
            const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[2 * i] = __uint_as_float(uu[i] << 16);
                v[2 * i + 1] = __uint_as_float(uu[i] & 0xffff0000u);
            }
        } else {
            const float4 f0 = __ldcs(reinterpret_cast<const float4*>(src + e0));
            const float4 f1 = __ldcs(reinterpret_cast<const float4*>(src + e0) + 1);
            v[0] = f0.x; v[1] = f0.y; v[2] = f0.z; v[3] = f0.w;
            v[4] = f1.x; v[5] = f1.y; v[6] = f1.z; v[7] = f1.w;
        }
#pragma unroll
        for (int t = 0; t < 3; ++t) {
            uint32_t m = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) m = max(m, __float_as_uint(v[i]) & 0x7fffffffu);
            m = max(m, __shfl_xor_sync(kFullMask, m, 1));
            m = max(m, __shfl_xor_sync(kFullMask, m, 2));            // 4-lane block
            int e = (int)(m >> 23) - 127 - 2;                       // amax / 2^e in [4, 8)
            if ((m & 0x007fffffu) > 0x00400000u) e += 1;             // above 6 * 2^e the E2M1 grid would saturate
            e = min(max(e, -127), 127);
            if (m == 0) e = -127;
            const float inv = __uint_as_float((uint32_t)min(max(127 - e, 1), 254) << 23);
            const float sc = __uint_as_float((uint32_t)max(e + 127, 1) << 23);                     // 2^e (>= 2^-126)
            uint32_t word = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint16_t packed;
                asm("{\n .reg .b8 b;\n cvt.rn.satfinite.e2m1x2.f32 b, %2, %1;\n mov.b16 %0, {b, 0};\n}"
                    : "=h"(packed) : "f"(v[2 * i] * inv), "f"(v[2 * i + 1] * inv));
                const float2 back = e2m1x2_to_float2(packed);
                v[2 * i] -= back.x * sc;
                v[2 * i + 1] -= back.y * sc;
                word |= (uint32_t)(packed & 0xff) << (8 * i);
            }
            *reinterpret_cast<uint32_t*>(q + t * term_q + (e0 >> 1)) = word;
            if ((lane & 3) == 0) s[t * term_s + (e0 >> 5)] = (uint8_t)(e + 127);
        }
    }
}

}  // namespace dsv4
