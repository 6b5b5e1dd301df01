// The tensor-core kernel of the batched routed-expert path (see moe_gemm.cuh for the design).
#pragma once

#include "moe_gemm.cuh"

namespace dsv4 {

template <int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1) moe_gemm_kernel(const MoeGemmArgs a) {
    using L = MoeGemmLayout<MODE>;
    constexpr int S = L::kStages;
    constexpr int MATS = L::kMats;
    extern __shared__ __align__(1024) uint8_t gemm_smem[];
    __shared__ __align__(8) uint64_t bar_full[S], bar_empty[S], bar_accum;
    __shared__ uint32_t tmem_holder;
    __shared__ int row_exp[2][128];          // largest E8M0 byte of every weight row of the tile (-1: none)
    __shared__ int tok_exp[128];             // exponent removed from the token of every accumulator column
    __shared__ int tok_row[128];             // activation row of every column (token index / slot)
    __shared__ float tok_w[128];             // router weight of every column (down)
    pdl_launch_dependents();

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int kProducerWarps = kGemmProducers / 32;
    const bool producer = warp < kProducerWarps;
    const int n_kb = a.K / kGemmKBlock;
    const int scale_row = a.K / 32;          // scale bytes per weight row
    uint8_t* scale_cache = gemm_smem + L::kScaleCache;

    if (warp == kProducerWarps) tc05_alloc(smem_u32(&tmem_holder), 256);
    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(smem_u32(&bar_full[s]), kProducerWarps); mbar_init(smem_u32(&bar_empty[s]), 1); }
        mbar_init(smem_u32(&bar_accum), 1);
        mbar_init_fence();
    }
    pdl_wait();
    tc05_fence_before_sync();
    __syncthreads();
    tc05_fence_after_sync();
    const uint32_t tmem = tmem_holder;

    const int* tiles = MODE == 0 ? a.g.tiles_up : a.g.tiles_down;
    const int n_tiles = tiles[a.n_experts];
    const int m_tiles = a.rows / kMoeTileRows;
    uint32_t it = 0;                          // stages produced / consumed so far (same count in both roles)
    uint32_t tile_count = 0;
    bool alive = true;

    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tile_count) {
        // expert of this tile: last e with tiles[e] <= tile
        int lo = 0, hi = a.n_experts;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (tiles[mid] <= tile) lo = mid; else hi = mid;
        }
        const int e = lo;
        const int local = tile - tiles[e];
        const int nt = local / m_tiles, mt = local - nt * m_tiles;
        const int slot0 = a.g.offsets[e] + nt * kMoeTileTokens;
        const int n_valid = min(kMoeTileTokens, a.g.offsets[e + 1] - slot0);
        const int n_mma = (n_valid + 15) & ~15;
        const int m0 = mt * kMoeTileRows;

        if (producer) {
            // ---- tile set-up: scale rows -> shared memory, row exponents, per-column token data
            const uint8_t* sc_src[2] = {a.wa_s + e * a.stride_s + (long long)m0 * scale_row,
                                        MODE == 0 ? a.wb_s + e * a.stride_s + (long long)m0 * scale_row : nullptr};
            const int vec_per_mat = 128 * scale_row / 16;
#pragma unroll
            for (int m = 0; m < MATS; ++m)
                for (int i = tid; i < vec_per_mat; i += kGemmProducers)
                    reinterpret_cast<uint4*>(scale_cache + m * 128 * scale_row)[i] =
                        ldg_stream_v4(sc_src[m] + (size_t)i * 16);
            if (tid < n_valid) {
                const int slot = slot0 + tid;
                const int pair = a.g.slot_pair[slot];
                const int token = pair / a.k_top;
                tok_exp[tid] = a.xexp[token];
                tok_row[tid] = MODE == 0 ? token : slot;
                if (MODE == 1) tok_w[tid] = a.pair_w[pair];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kGemmProducers) : "memory");
            if (tid < 128 * MATS) {
                const int m = tid >> 7, r = tid & 127;
                // scale rows are a multiple of 8 bytes (K is a multiple of 256)
                const uint2* p = reinterpret_cast<const uint2*>(scale_cache + (m * 128 + r) * scale_row);
                uint32_t best = 0;
                bool any = false;
                for (int i = 0; i < scale_row / 8; ++i) {
                    const uint2 q = p[i];
                    const uint32_t w[2] = {q.x, q.y};
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const uint32_t is_ff = __vcmpeq4(w[j], 0xffffffffu);
                        any = any || (is_ff != 0xffffffffu);
                        best = __vmaxu4(best, w[j] & ~is_ff);
                    }
                }
                const uint32_t b = max(max(best & 0xff, (best >> 8) & 0xff), max((best >> 16) & 0xff, best >> 24));
                row_exp[m][r] = any ? (int)b : -1;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kGemmProducers) : "memory");

            // ---- main loop: a thread owns one 32-value block (row, half) of ONE weight tile and 2 chunks of the
            // token tile (with one weight matrix only half of the producers have a weight block)
            const int mat = (tid >> 8) & 1;
            const bool has_a = mat < MATS;
            const int row = (tid & 255) >> 1, half = tid & 1;
            const uint8_t* wbase = (mat == 0 || MODE != 0) ? a.wa_p : a.wb_p;
            const uint8_t* wsrc = wbase + e * a.stride_p + (long long)(m0 + row) * (a.K >> 1) + half * 16;
            const uint8_t* my_scale = scale_cache + ((has_a ? mat : 0) * 128 + row) * scale_row + half;
            const int my_exp = row_exp[has_a ? mat : 0][row];
            const __half* bsrc[2];
            bool bok[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int idx = tid + kGemmProducers * q;
                const int n = idx >> 3, c = idx & 7;
                bok[q] = n < n_valid;
                bsrc[q] = a.act + (size_t)(bok[q] ? tok_row[n] : 0) * a.K + c * 8;
            }
            uint4 ring_a[4];
            uint4 ring_b[2][2];
            auto load_a = [&](int kb, uint4& dst) {
                if (has_a) dst = ldg_stream_v4(wsrc + (size_t)kb * 32);
            };
            auto load_b = [&](int kb, uint4 (&dst)[2]) {
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    dst[q] = bok[q] ? __ldcg(reinterpret_cast<const uint4*>(bsrc[q] + (size_t)kb * kGemmKBlock))
                                    : make_uint4(0, 0, 0, 0);
            };
#pragma unroll
            for (int d = 0; d < 3; ++d)
                if (d < n_kb) load_a(d, ring_a[d]);
            load_b(0, ring_b[0]);
            for (int kb0 = 0; kb0 < n_kb; kb0 += 4) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int kb = kb0 + u;
                    if (kb + 3 < n_kb) load_a(kb + 3, ring_a[(u + 3) & 3]);
                    if (kb + 1 < n_kb) load_b(kb + 1, ring_b[(u + 1) & 1]);
                    const uint32_t s = it % S;
                    if (it >= (uint32_t)S && alive)
                        alive = mbar_wait_bounded(smem_u32(&bar_empty[s]), ((it / S) - 1) & 1, 4);
                    uint8_t* stage = gemm_smem + s * L::kStageBytes;
                    if (has_a) {
                        const int sb = my_scale[kb * 2];
                        const uint32_t mult = (sb == 255 || my_exp < 0) ? 0u : half_pow2_bits(sb - my_exp);
                        dequant_block_to_tile(ring_a[u & 3], mult, stage + mat * kGemmTileBytes, row, half);
                    }
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const int idx = tid + kGemmProducers * q;
                        if ((idx >> 3) < n_mma)
                            *reinterpret_cast<uint4*>(stage + MATS * kGemmTileBytes + tc05_sw128_offset(idx >> 3, idx & 7)) =
                                ring_b[u & 1][q];
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bar_full[s])) : "memory");
                    ++it;
                }
            }
        } else {
            // ---- last warp: issue the MMAs of every stage; a stage is released when its MMAs have completed
            const uint32_t idesc = tc05_idesc_f16(128, n_mma);
            for (int kb = 0; kb < n_kb; ++kb, ++it) {
                const uint32_t s = it % S;
                if (alive) alive = mbar_wait_bounded(smem_u32(&bar_full[s]), (it / S) & 1, 5);
                tc05_fence_after_sync();
                if (lane == 0 && alive) {
                    const uint32_t stage = smem_u32(gemm_smem) + s * L::kStageBytes;
#pragma unroll
                    for (int j = 0; j < kGemmKBlock / 16; ++j) {
                        const uint64_t db = tc05_desc_k_sw128(stage + MATS * kGemmTileBytes + 32 * j);
#pragma unroll
                        for (int m = 0; m < MATS; ++m)
                            tc05_mma_f16(tmem + m * 128, tc05_desc_k_sw128(stage + m * kGemmTileBytes + 32 * j), db, idesc,
                                         (kb > 0 || j > 0) ? 1u : 0u);
                    }
                    tc05_commit(smem_u32(&bar_empty[s]));
                    if (kb == n_kb - 1) tc05_commit(smem_u32(&bar_accum));
                }
                __syncwarp();
            }
        }

        // ---- epilogue: warps 0..3 own accumulator rows 32 w .. 32 w + 31
        if (warp < 4) {
            if (alive) alive = mbar_wait_bounded(smem_u32(&bar_accum), tile_count & 1, 6);
            tc05_fence_after_sync();
            const int r = tid;                                   // accumulator row = weight row m0 + r
            const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
            const float sa = row_exp[0][r] < 0 ? 0.f : float_pow2(row_exp[0][r] - 127);
            const float sb = (MODE == 0) ? (row_exp[1][r] < 0 ? 0.f : float_pow2(row_exp[1][r] - 127)) : 0.f;
            for (int c0 = 0; c0 < n_mma && alive; c0 += 16) {
                float g[16], u[16];
                tc05_ld16(trow + c0, g);
                if (MODE == 0) tc05_ld16(trow + 128 + c0, u);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int n = c0 + i;
                    if (n < n_valid) {
                        const int ex = tok_exp[n];
                        if (MODE == 0) {
                            // g = gn * 2^ex, u = un * 2^ex; silu(g) * u / 2^(2 ex) = gn * sigmoid(g) * un: stored without
                            // the token's scale (squared), bounded whatever the scale of x
                            const float gn = g[i] * sa, un = u[i] * sb;
                            const float stored = gn * (1.0f / (1.0f + __expf(-gn * float_pow2(ex)))) * un;
                            a.mid[(size_t)(slot0 + n) * a.rows + m0 + r] =
                                __float2half_rn(fminf(fmaxf(stored, -65504.f), 65504.f));
                        } else {
                            a.y[(size_t)(slot0 + n) * a.rows + m0 + r] =
                                g[i] * sa * float_pow2(ex) * float_pow2(ex) * tok_w[n];
                        }
                    }
                }
            }
        }
        tc05_fence_before_sync();
        __syncthreads();            // accumulators read, token tables free: the next tile may start
        tc05_fence_after_sync();
    }
    __syncthreads();
    if (warp == kProducerWarps) tc05_dealloc(tmem, 256);
}

}  // namespace dsv4
