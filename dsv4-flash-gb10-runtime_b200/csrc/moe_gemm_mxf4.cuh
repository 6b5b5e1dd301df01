// Batched routed-expert GEMMs with BLOCK-SCALED tensor-core MMAs (tcgen05 kind::mxf4, UE8M0 scales in tensor
// memory): the MXFP4 weights go from HBM to shared memory to the tensor cores exactly as the checkpoint stores them
// (packed nibbles + E8M0 bytes) - no dequantisation instruction is executed, and a weight costs half a byte of
// shared-memory traffic instead of the four bytes the fp16 path (moe_gemm_kernel.cuh) pays.
//
// The tensor cores multiply FP4 by FP4, so the activations are given as three MXFP4 terms (moe_prep.cuh) and every
// weight tile is multiplied by each of them, accumulating into the same FP32 accumulator:
//   D = W * (q1 + q2 + q3) = W q1 + W q2 + W q3.
//
// Tiles: 128 weight rows (M) x up to 128 tokens (N); a stage covers 256 K-elements (one 128-byte swizzled row per
// operand row = 4 MMAs of K = 64).  Per stage the 16 producer warps copy: the packed weight rows (one or two
// matrices), the three packed activation terms of the tile's tokens, and the scale bytes re-arranged into
// 512-byte scale atoms; one lane of the last warp copies the atoms into tensor memory (tcgen05.cp) and issues the
// MMAs; tcgen05.commit releases the stage.  Persistent grid, one CTA per SM.  Every wait is bounded.
#pragma once

#include "moe_gemm.cuh"

namespace dsv4 {

constexpr int kQKBlock = 256;                        // K-elements per stage
constexpr int kQTerms = 3;                           // activation terms
constexpr uint32_t kQTile = 128 * 128;               // bytes of one packed operand tile (128 rows x 128 B)
constexpr uint32_t kQAtoms = 2 * 512;                // scale bytes of one operand per stage (2 atoms)

struct MoeQGemmArgs {
    const uint8_t* wa_p; const uint8_t* wb_p;        // up: W1, W3 packed; down: W2
    const uint8_t* wa_s; const uint8_t* wb_s;
    long long stride_p, stride_s;                    // bytes per expert
    int rows, K, n_experts, k_top;
    const uint8_t* act_q;                            // [3][act_rows][K / 2]
    const uint8_t* act_s;                            // [3][act_rows][K / 32]
    long long act_rows;                              // rows of the activation matrix (tokens for up, pairs for down)
    const float* pair_w;                             // [P] router weights (down)
    MoeGroups g;
    float* mid;                                      // up output [P, rows] FP32
    float* y;                                        // down output [P, rows] FP32
};

template <int MODE>
struct MoeQGemmLayout {
    static constexpr int kMats = MODE == 0 ? 2 : 1;
    static constexpr int kStages = MODE == 0 ? 2 : 3;
    static constexpr uint32_t kOffB = kMats * kQTile;
    static constexpr uint32_t kOffSfA = kOffB + kQTerms * kQTile;
    static constexpr uint32_t kOffSfB = kOffSfA + kMats * kQAtoms;
    static constexpr uint32_t kStageBytes = kOffSfB + kQTerms * kQAtoms;     // 87 040 (up) / 69 632 (down)
    static constexpr uint32_t kBytes = kStages * kStageBytes + 1024;
    // tensor memory: accumulators first, then per stage the scale columns of every operand (8 columns each)
    static constexpr uint32_t kAccCols = kMats * 128;
    static constexpr uint32_t kSfColsPerStage = (kMats + kQTerms) * 8;
    static_assert(kStageBytes % 1024 == 0, "stage size must keep tiles 1024-byte aligned");
    static_assert(kAccCols + kStages * kSfColsPerStage <= 512, "tensor memory overflow");
};

template <int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1) moe_gemm_mxf4_kernel(const MoeQGemmArgs a) {
    using L = MoeQGemmLayout<MODE>;
    constexpr int S = L::kStages;
    constexpr int MATS = L::kMats;
    constexpr int kProducerWarps = kGemmProducers / 32;
    extern __shared__ __align__(1024) uint8_t gemm_smem[];
    __shared__ __align__(8) uint64_t bar_full[S], bar_empty[S], bar_accum;
    __shared__ uint32_t tmem_holder;
    __shared__ int tok_row[128];             // activation row of every accumulator column
    __shared__ float tok_w[128];             // router weight of every column (down)
    pdl_launch_dependents();

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool producer = warp < kProducerWarps;
    const int n_kb = a.K / kQKBlock;
    const int row_p = a.K >> 1, row_s = a.K >> 5;

    if (warp == kProducerWarps) tc05_alloc(smem_u32(&tmem_holder), 512);
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
    uint32_t it = 0, tile_count = 0;
    bool alive = true;

    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tile_count) {
        int lo = 0, hi = a.n_experts;
        while (hi - lo > 1) {
            const int md = (lo + hi) >> 1;
            if (tiles[md] <= tile) lo = md; else hi = md;
        }
        const int e = lo;
        const int local = tile - tiles[e];
        const int nt = local / m_tiles, mt = local - nt * m_tiles;
        const int slot0 = a.g.offsets[e] + nt * kMoeTileTokens;
        const int n_valid = min(kMoeTileTokens, a.g.offsets[e + 1] - slot0);
        const int n_mma = (n_valid + 15) & ~15;
        const int m0 = mt * kMoeTileRows;

        if (producer) {
            if (tid < n_valid) {
                const int slot = slot0 + tid;
                const int pair = a.g.slot_pair[slot];
                tok_row[tid] = MODE == 0 ? pair / a.k_top : slot;
                if (MODE == 1) tok_w[tid] = a.pair_w[pair];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kGemmProducers) : "memory");

            // what this thread copies in every stage
            // weights: chunk (row, c) of each matrix; 128 rows x 8 chunks = 1024 per matrix, 2 per thread
            // activations: chunk (n, c) of each term; scales: one row of 8 bytes per 128 threads and operand
            const int wr[2] = {tid >> 3, (tid + kGemmProducers) >> 3};
            const int wc = tid & 7;
            const uint8_t* wsrc[2][2];
#pragma unroll
            for (int m = 0; m < MATS; ++m)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    wsrc[m][h] = (m == 0 ? a.wa_p : a.wb_p) + e * a.stride_p + (long long)(m0 + wr[h]) * row_p + wc * 16;
            const uint8_t* bsrc[2];
            bool bok[2], bwrite[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                bok[h] = wr[h] < n_valid;
                bwrite[h] = wr[h] < n_mma;
                bsrc[h] = a.act_q + (long long)(bok[h] ? tok_row[wr[h]] : 0) * row_p + wc * 16;
            }
            // scale rows: threads 0..127 matrix A rows, 128..255 matrix B rows (up), then 3 x 128 for the terms
            const int sf_op = tid >> 7, sf_row = tid & 127;               // operand index 0 .. 3 (4 x 128 threads)
            const uint8_t* sfsrc[2] = {nullptr, nullptr};                  // up to two operands per thread
            uint32_t sfdst[2] = {0, 0};
            bool sfok[2] = {false, false};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int op = sf_op + 4 * h;                              // 0 .. MATS-1 weights, then the terms
                if (op < MATS) {
                    sfsrc[h] = (op == 0 ? a.wa_s : a.wb_s) + e * a.stride_s + (long long)(m0 + sf_row) * row_s;
                    sfdst[h] = L::kOffSfA + op * kQAtoms;
                    sfok[h] = true;
                } else if (op < MATS + kQTerms) {
                    const int t = op - MATS;
                    sfok[h] = true;
                    sfdst[h] = L::kOffSfB + t * kQAtoms;
                    sfsrc[h] = sf_row < n_valid
                                   ? a.act_s + (long long)t * a.act_rows * row_s + (long long)tok_row[sf_row] * row_s
                                   : nullptr;                              // padding columns: scale 1, data 0
                }
            }

            for (int kb = 0; kb < n_kb; ++kb, ++it) {
                // ---- requests first (they are what takes long), stores after the stage is free
                uint4 wv[MATS][2], bv[kQTerms][2];
                uint2 sv[2];
#pragma unroll
                for (int m = 0; m < MATS; ++m)
#pragma unroll
                    for (int h = 0; h < 2; ++h) wv[m][h] = ldg_stream_v4(wsrc[m][h] + (size_t)kb * 128);
#pragma unroll
                for (int t = 0; t < kQTerms; ++t)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        bv[t][h] = bok[h] ? __ldcg(reinterpret_cast<const uint4*>(bsrc[h] + (long long)t * a.act_rows * row_p +
                                                                                    (size_t)kb * 128))
                                          : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    sv[h] = make_uint2(0x7f7f7f7fu, 0x7f7f7f7fu);
                    if (sfok[h] && sfsrc[h]) sv[h] = __ldcg(reinterpret_cast<const uint2*>(sfsrc[h] + (size_t)kb * 8));
                }
                const uint32_t s = it % S;
                if (it >= (uint32_t)S && alive)
                    alive = mbar_wait_bounded(smem_u32(&bar_empty[s]), ((it / S) - 1) & 1, 4);
                uint8_t* stage = gemm_smem + s * L::kStageBytes;
#pragma unroll
                for (int m = 0; m < MATS; ++m)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        *reinterpret_cast<uint4*>(stage + m * kQTile + tc05_sw128_offset(wr[h], wc)) = wv[m][h];
#pragma unroll
                for (int t = 0; t < kQTerms; ++t)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        if (bwrite[h])
                            *reinterpret_cast<uint4*>(stage + L::kOffB + t * kQTile + tc05_sw128_offset(wr[h], wc)) = bv[t][h];
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    if (sfok[h]) {
                        // scales 0..3 -> atom 0, 4..7 -> atom 1; the four bytes of a row are one aligned word
                        *reinterpret_cast<uint32_t*>(stage + sfdst[h] + tc05_scale_atom_offset(sf_row, 0)) = sv[h].x;
                        *reinterpret_cast<uint32_t*>(stage + sfdst[h] + 512 + tc05_scale_atom_offset(sf_row, 0)) = sv[h].y;
                    }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bar_full[s])) : "memory");
            }
        } else {
            // ---- last warp: scale atoms into tensor memory, then the MMAs of the stage
            for (int kb = 0; kb < n_kb; ++kb, ++it) {
                const uint32_t s = it % S;
                if (alive) alive = mbar_wait_bounded(smem_u32(&bar_full[s]), (it / S) & 1, 5);
                tc05_fence_after_sync();
                if (lane == 0 && alive) {
                    const uint32_t stage = smem_u32(gemm_smem) + s * L::kStageBytes;
                    const uint32_t sf_cols = tmem + L::kAccCols + s * L::kSfColsPerStage;   // [op][atom] x 4 columns
#pragma unroll
                    for (int op = 0; op < MATS + kQTerms; ++op)
#pragma unroll
                        for (int at = 0; at < 2; ++at)
                            tc05_copy_scale_atom(sf_cols + op * 8 + at * 4,
                                                 stage + (op < MATS ? L::kOffSfA + op * kQAtoms
                                                                    : L::kOffSfB + (op - MATS) * kQAtoms) + at * 512);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {                                           // K-steps of 64
                        const uint32_t idesc = tc05_idesc_mxf4(128, n_mma, (j & 1) * 2, (j & 1) * 2);
#pragma unroll
                        for (int t = 0; t < kQTerms; ++t) {
                            const uint64_t db = tc05_desc_k_sw128(stage + L::kOffB + t * kQTile + 32 * j);
#pragma unroll
                            for (int m = 0; m < MATS; ++m)
                                tc05_mma_mxf4(tmem + m * 128, tc05_desc_k_sw128(stage + m * kQTile + 32 * j), db, idesc,
                                              sf_cols + m * 8 + (j >> 1) * 4, sf_cols + (MATS + t) * 8 + (j >> 1) * 4,
                                              (kb > 0 || j > 0 || t > 0) ? 1u : 0u);
                        }
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
            const int r = tid;
            const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
            for (int c0 = 0; c0 < n_mma && alive; c0 += 16) {
                float g[16], u[16];
                tc05_ld16(trow + c0, g);
                if (MODE == 0) tc05_ld16(trow + 128 + c0, u);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int n = c0 + i;
                    if (n < n_valid) {
                        if (MODE == 0)
                            a.mid[(size_t)(slot0 + n) * a.rows + m0 + r] = (g[i] / (1.0f + __expf(-g[i]))) * u[i];
                        else
                            a.y[(size_t)(slot0 + n) * a.rows + m0 + r] = g[i] * tok_w[n];
                    }
                }
            }
        }
        tc05_fence_before_sync();
        __syncthreads();
        tc05_fence_after_sync();
    }
    __syncthreads();
    if (warp == kProducerWarps) tc05_dealloc(tmem, 512);
}

}  // namespace dsv4
