// Batched routed-expert GEMMs with BLOCK-SCALED tensor-core MMAs (tcgen05 kind::mxf4, UE8M0 scales in tensor
// memory): the MXFP4 weights go from HBM to shared memory to the tensor cores exactly as the checkpoint stores them
// (packed nibbles + E8M0 bytes) - no dequantisation instruction is executed, and a weight costs half a byte of
// shared-memory traffic instead of the four bytes the fp16 path (moe_gemm_kernel.cuh) pays.
//
// The tensor cores multiply FP4 by FP4, so the activations are given as three MXFP4 terms (moe_prep.cuh):
//   D = W * (q1 + q2 + q3) = W q1 + W q2 + W q3.
// On B200 one tcgen05.mma of M = 128 occupies the tensor pipe for about the same ~190 clocks whether N is 32 or
// 256 (measured), so the MMA count, not the flop count, decides the speed of this kernel.  The three terms are
// therefore STACKED ALONG N: the B operand of a tile holds term 1 of its tokens in rows [0, n), term 2 in [n, 2n),
// term 3 in [2n, 3n), and one MMA of N = 3n produces the three partial products in three column ranges of the
// accumulator, which the epilogue adds.  When 3n > 256 (the MMA's largest N) the third term moves to row 256 and
// gets an MMA of its own.
//
// Tiles: two blocks of 128 weight rows (two accumulators: rows m0.. of W1 and of W3 for gate/up, rows m0.. and
// m0 + 128.. of W2 for down) x up to 64 tokens; a stage covers 256 K-elements (one 128-byte swizzled row per operand row = 4 MMAs of K = 64).  Per stage
// the 16 producer warps copy with cp.async: the packed weight rows, the three packed activation terms of the
// tile's tokens, and the scale bytes re-arranged into 512-byte scale atoms; one lane of the last warp copies the
// atoms into tensor memory (tcgen05.cp) and issues the MMAs; tcgen05.commit releases the stage.  Persistent grid,
// one CTA per SM.  Producers and the MMA warp run ahead across tile boundaries: the producers start filling the
// stages of the next tile while the last MMAs of the current one are in flight, then (all 16 warps, four per lane
// quadrant of tensor memory) drain the finished accumulator and hand it back to the MMA warp through an mbarrier.
// Every wait is bounded.
#pragma once

#include "moe_gemm.cuh"

namespace dsv4 {

constexpr int kQKBlock = 256;                        // K-elements per stage
constexpr int kQTerms = 3;                           // activation terms
constexpr uint32_t kQTile = 128 * 128;               // bytes of one packed weight tile (128 rows x 128 B)
constexpr int kQTokUp = 64;                          // tokens per tile (3 x 64 = 192 accumulator columns x 2)
constexpr int kQTokDown = 64;
constexpr int kQRowsDown = 256;                      // W2 rows per down tile (two row blocks share the activation tile)

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
    static constexpr int kMats = 2;
    static constexpr int kTok = MODE == 0 ? kQTokUp : kQTokDown;
    static constexpr int kStages = 3;
    // rows of the stacked B operand: contiguous when the three terms fit one MMA, else term 3 at row 256
    static constexpr int kBRows = 3 * kTok <= 256 ? 3 * kTok : 256 + kTok;
    static constexpr int kRowGroups = (kBRows + 127) / 128;                  // scale atoms cover 128 rows
    static constexpr uint32_t kOffB = kMats * kQTile;
    static constexpr uint32_t kOffSfA = kOffB + kBRows * 128;
    static constexpr uint32_t kOffSfB = kOffSfA + kMats * 1024;              // [mat][k-atom] x 512 B
    static constexpr uint32_t kStageBytes = kOffSfB + 2 * kRowGroups * 512;  // [k-atom][row group] x 512 B
    static constexpr uint32_t kBytes = kStages * kStageBytes + 1024;
    // tensor memory: accumulators (one column per B row) first, then per stage the scale columns
    static constexpr uint32_t kAccStride = kBRows;
    static constexpr uint32_t kAccCols = kMats * kAccStride;
    static constexpr uint32_t kSfBCol = kMats * 8;                           // B scales after the A scales
    static constexpr uint32_t kSfColsPerStage = kMats * 8 + 2 * kRowGroups * 4;
    static_assert(kStageBytes % 1024 == 0, "stage size must keep tiles 1024-byte aligned");
    static_assert(kAccCols + kStages * kSfColsPerStage <= 512, "tensor memory overflow");
    static_assert(kMats * 128 + kQTerms * kTok <= kGemmProducers, "one scale row per producer thread");
    static_assert(kBytes <= 227 * 1024, "shared memory overflow");
    static_assert(kTok <= 64, "the drain handles one 16-token chunk per warp");
};

// What a tile is: expert, rows, tokens; identical in every thread of the CTA.
struct MoeQTile {
    int e, slot0, n_valid, n_mma, m0, term_row2, mats;
    bool split;
};

// tiles / offsets: the grouping kernel's prefix sums, staged in shared memory by the caller.
template <int TOK>
__device__ __forceinline__ MoeQTile moe_qtile_decode(const int* tiles, const int* offsets, int n_experts, int m_tiles,
                                                     int tile_rows, int rows, int tile) {
    int lo = 0, hi = n_experts;
    while (hi - lo > 1) {
        const int md = (lo + hi) >> 1;
        if (tiles[md] <= tile) lo = md; else hi = md;
    }
    MoeQTile t;
    t.e = lo;
    const int local = tile - tiles[lo];
    const int nt = local / m_tiles, mt = local - nt * m_tiles;
    t.slot0 = offsets[lo] + nt * TOK;
    t.n_valid = min(TOK, offsets[lo + 1] - t.slot0);
    t.n_mma = (t.n_valid + 15) & ~15;
    t.m0 = mt * tile_rows;
    t.mats = (tile_rows == 2 * kMoeTileRows && t.m0 + kMoeTileRows >= rows) ? 1 : 2;   // a last, half down tile
    t.split = 3 * t.n_mma > 256;                       // B rows (= accumulator columns) of the three terms
    t.term_row2 = t.split ? 256 : 2 * t.n_mma;
    return t;
}

template <int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1) moe_gemm_mxf4_kernel(const MoeQGemmArgs a) {
    using L = MoeQGemmLayout<MODE>;
    constexpr int S = L::kStages;
    constexpr int MATS = L::kMats;
    constexpr int TOK = L::kTok;
    constexpr int RG = L::kRowGroups;
    constexpr int kProducerWarps = kGemmProducers / 32;
    constexpr int kBChunks = (TOK * 8 + kGemmProducers - 1) / kGemmProducers;   // 16-byte chunks per thread and term
    extern __shared__ __align__(1024) uint8_t gemm_smem[];
    __shared__ __align__(8) uint64_t bar_full[S], bar_empty[S], bar_accum, bar_acc_free;
    __shared__ uint32_t tmem_holder;
    // Token tables, three deep: producers fill the table of tile N + 1 before its barrier while another warp may still
    // be draining tile N - 1 (the drain runs inside tile N's loop), so two tables are not enough when a tile has
    // few K steps (hidden <= 1536); a warp cannot get two tiles ahead of another warp's drain.
    __shared__ int tok_row[3][128];          // activation row of every token of the tile (by tile number mod 3)
    __shared__ float tok_w[3][128];          // router weight of every token (down)
    __shared__ int s_tiles[kMoeMaxExperts + 1], s_offsets[kMoeMaxExperts + 1];
    pdl_launch_dependents();

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool producer = warp < kProducerWarps;
    const int n_kb = a.K / kQKBlock;
    const int row_p = a.K >> 1, row_s = a.K >> 5;

    if (warp == kProducerWarps) tc05_alloc(smem_u32(&tmem_holder), 512);
    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(smem_u32(&bar_full[s]), kGemmProducers); mbar_init(smem_u32(&bar_empty[s]), 1); }
        mbar_init(smem_u32(&bar_accum), 1);
        mbar_init(smem_u32(&bar_acc_free), kGemmProducers);
        mbar_init_fence();
    }
    pdl_wait();
    for (int i = tid; i <= a.n_experts; i += kGemmThreads) {
        s_tiles[i] = (MODE == 0 ? a.g.tiles_up : a.g.tiles_down)[i];
        s_offsets[i] = a.g.offsets[i];
    }
    tc05_fence_before_sync();
    __syncthreads();
    tc05_fence_after_sync();
    const uint32_t tmem = tmem_holder;

    const int* tiles = s_tiles;
    const int n_tiles = tiles[a.n_experts];
    // gate/up: 128 rows of W1 and the same 128 rows of W3; down: 256 rows of W2 (the last tile may hold 128)
    const int tile_rows = MODE == 0 ? kMoeTileRows : kQRowsDown;
    const int m_tiles = (a.rows + tile_rows - 1) / tile_rows;
    uint32_t it = 0, tile_count = 0;
    bool alive = true;

    if (producer) {
        // ---- drain of a finished accumulator: warps q, q + 4, q + 8, q + 12 own lane quadrant q (rows 32 q ..)
        // and share its token chunks of 16; a token's value is the sum of its three term columns (term order)
        auto drain = [&](const MoeQTile& t, uint32_t count) {
            if (alive) alive = mbar_wait_bounded(smem_u32(&bar_accum), count & 1, 6);
            tc05_fence_after_sync();
            const int quad = warp & 3;
            const int r = quad * 32 + lane;
            const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16);
            const float* w_of = tok_w[count % 3u];
            auto hand_back = [&]() {
                // this thread's last read of the accumulator and of the token tables is done
                tc05_fence_before_sync();
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bar_acc_free)) : "memory");
            };
            // the three term columns of 16 tokens in flight together, one wait; summed in term order
            auto load_sum = [&](uint32_t col, float (&v)[16]) {
                uint32_t p0[16], p1[16], p2[16];
                tc05_ld16_issue(trow + col, p0);
                tc05_ld16_issue(trow + t.n_mma + col, p1);
                tc05_ld16_issue(trow + t.term_row2 + col, p2);
                tc05_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    v[i] = (__uint_as_float(p0[i]) + __uint_as_float(p1[i])) + __uint_as_float(p2[i]);
            };
            const int ca = (warp >> 2) * 16;                      // this warp's 16 tokens (TOK <= 64: one chunk per warp)
            const bool has_a = ca < t.n_mma && alive;
            {
                // both accumulators of this warp's 16 tokens: gate and up (SwiGLU), or two row blocks of W2
                float g[16], u[16];
                if (has_a) {
                    load_sum(ca, g);
                    if (t.mats == 2) load_sum(L::kAccStride + ca, u);
                    if (MODE == 1) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float w = ca + i < t.n_valid ? w_of[ca + i] : 0.f;
                            g[i] *= w;
                            u[i] *= w;
                        }
                    }
                }
                hand_back();
                if (has_a) {
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (ca + i < t.n_valid) {
                            if (MODE == 0) {
                                a.mid[(size_t)(t.slot0 + ca + i) * a.rows + t.m0 + r] = (g[i] / (1.0f + __expf(-g[i]))) * u[i];
                            } else {
                                float* yrow = a.y + (size_t)(t.slot0 + ca + i) * a.rows + t.m0 + r;
                                yrow[0] = g[i];
                                if (t.mats == 2) yrow[kMoeTileRows] = u[i];
                            }
                        }
                }
            }
        };

        MoeQTile prev;
        bool has_prev = false;
        const int drain_at = min(S, n_kb) - 1;        // the stage after whose issue the previous tile is drained
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tile_count) {
            const MoeQTile t = moe_qtile_decode<TOK>(tiles, s_offsets, a.n_experts, m_tiles, tile_rows, a.rows, tile);
            int* rows_of = tok_row[tile_count % 3u];
            if (tid < t.n_valid) {
                const int slot = t.slot0 + tid;
                const int pair = a.g.slot_pair[slot];
                rows_of[tid] = MODE == 0 ? pair / a.k_top : slot;
                if (MODE == 1) tok_w[tile_count % 3u][tid] = a.pair_w[pair];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kGemmProducers) : "memory");

            // what this thread copies in every stage
            // weights: chunk (row, c) of each matrix; 128 rows x 8 chunks = 1024 per matrix, 2 per thread
            const int wr[2] = {tid >> 3, (tid + kGemmProducers) >> 3};
            const int wc = tid & 7;
            const uint8_t* wsrc[MATS][2];
#pragma unroll
            for (int m = 0; m < MATS; ++m)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    wsrc[m][h] = (MODE == 0 ? (m == 0 ? a.wa_p : a.wb_p) + t.e * a.stride_p + (long long)(t.m0 + wr[h]) * row_p
                                            : a.wa_p + t.e * a.stride_p + (long long)(t.m0 + kMoeTileRows * m + wr[h]) * row_p) +
                                 wc * 16;
            // activations: chunk (token, c) of each term
            const uint8_t* bsrc[kBChunks];
            bool bok[kBChunks], bwrite[kBChunks];
#pragma unroll
            for (int h = 0; h < kBChunks; ++h) {
                bok[h] = wr[h] < t.n_valid;
                bwrite[h] = wr[h] < t.n_mma;
                bsrc[h] = a.act_q + (long long)(bok[h] ? rows_of[wr[h]] : 0) * row_p + wc * 16;
            }
            // scales: one row of 8 bytes per thread; threads [0, 128 MATS) the weight rows, then TOK per term
            const uint8_t* sfsrc = nullptr;
            uint32_t sfdst = 0;
            bool sfok = false;
            if (tid < MATS * 128) {
                const int m = tid >> 7, r = tid & 127;
                sfsrc = MODE == 0 ? (m == 0 ? a.wa_s : a.wb_s) + t.e * a.stride_s + (long long)(t.m0 + r) * row_s
                                  : a.wa_s + t.e * a.stride_s + (long long)(t.m0 + kMoeTileRows * m + r) * row_s;
                sfdst = L::kOffSfA + m * 1024 + tc05_scale_atom_offset(r, 0);
                sfok = m < t.mats;
                if (!sfok) sfsrc = nullptr;
            } else if (tid < MATS * 128 + kQTerms * TOK) {
                const int idx = tid - MATS * 128;
                const int term = idx / TOK, n = idx - term * TOK;
                if (n < t.n_mma) {
                    const int brow = (term == 2 ? t.term_row2 : term * t.n_mma) + n;
                    sfok = true;
                    sfdst = L::kOffSfB + (brow >> 7) * 512 + tc05_scale_atom_offset(brow & 127, 0);
                    if (n < t.n_valid)                                // padding rows: scale 1, data 0
                        sfsrc = a.act_s + (long long)term * a.act_rows * row_s + (long long)rows_of[n] * row_s;
                }
            }
            const uint32_t sf_atom_stride = tid < MATS * 128 ? 512u : (uint32_t)RG * 512u;   // k-atom 0 -> 1

            // Weights and activation terms go global -> shared memory with asynchronous 16-byte copies (no
            // registers in between).  Every producer thread makes the stage's "full" barrier arrive when ITS copies
            // have landed (cp.async.mbarrier.arrive), so a stage is published the moment its last byte arrives
            // while the thread is already filling the next free stage.
            for (int kb = 0; kb < n_kb; ++kb, ++it) {
                uint2 sv = make_uint2(0x7f7f7f7fu, 0x7f7f7f7fu);
                if (sfsrc) sv = __ldcg(reinterpret_cast<const uint2*>(sfsrc + (size_t)kb * 8));
                const uint32_t s = it % S;
                if (it >= (uint32_t)S && alive)
                    alive = mbar_wait_bounded(smem_u32(&bar_empty[s]), ((it / S) - 1) & 1, 4);
                const uint32_t stage = smem_u32(gemm_smem) + s * L::kStageBytes;
#pragma unroll
                for (int m = 0; m < MATS; ++m)
                    if (m < t.mats) {
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(stage + m * kQTile + tc05_sw128_offset(wr[h], wc)),
                                         "l"(wsrc[m][h] + (size_t)kb * 128) : "memory");
                    }
#pragma unroll
                for (int term = 0; term < kQTerms; ++term) {
                    const int base_row = term == 2 ? t.term_row2 : term * t.n_mma;
#pragma unroll
                    for (int h = 0; h < kBChunks; ++h)
                        if (bwrite[h])      // rows past the expert's tokens: source size 0 = zero fill
                            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(stage + L::kOffB + tc05_sw128_offset(base_row + wr[h], wc)),
                                         "l"(bsrc[h] + (long long)term * a.act_rows * row_p + (size_t)kb * 128), "r"(bok[h] ? 16 : 0) : "memory");
                }
                if (sfok) {
                    // scales 0..3 -> k-atom 0, 4..7 -> k-atom 1; the four bytes of a row are one aligned word
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(stage + sfdst), "r"(sv.x) : "memory");
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(stage + sfdst + sf_atom_stride), "r"(sv.y) : "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&bar_full[s])) : "memory");
                // the first stages of this tile are on their way: now drain the previous tile's accumulator
                if (kb == drain_at && has_prev) drain(prev, tile_count - 1);
            }
            prev = t;
            has_prev = true;
        }
        if (has_prev) drain(prev, tile_count - 1);
    } else {
        // ---- last warp: scale atoms into tensor memory, then the MMAs of the stage
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tile_count) {
            const MoeQTile t = moe_qtile_decode<TOK>(tiles, s_offsets, a.n_experts, m_tiles, tile_rows, a.rows, tile);
            const int n_first = t.split ? 2 * t.n_mma : 3 * t.n_mma;     // N of the first MMA
            const int groups = (t.term_row2 + t.n_mma + 127) >> 7;       // row groups of B scales in use
            if (tile_count > 0 && alive)                                 // previous accumulator drained?
                alive = mbar_wait_bounded(smem_u32(&bar_acc_free), (tile_count - 1) & 1, 7);
            for (int kb = 0; kb < n_kb; ++kb, ++it) {
                const uint32_t s = it % S;
                if (alive) alive = mbar_wait_bounded(smem_u32(&bar_full[s]), (it / S) & 1, 5);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // copies landed via the generic proxy
                tc05_fence_after_sync();
                if (lane == 0 && alive) {
                    const uint32_t stage = smem_u32(gemm_smem) + s * L::kStageBytes;
                    const uint32_t sfa_cols = tmem + L::kAccCols + s * L::kSfColsPerStage;  // [mat][k-atom] x 4 columns
                    const uint32_t sfb_cols = sfa_cols + L::kSfBCol;                        // [k-atom][row group] x 4
#pragma unroll
                    for (int at = 0; at < 2; ++at) {
#pragma unroll
                        for (int m = 0; m < MATS; ++m)
                            if (m < t.mats)
                                tc05_copy_scale_atom(sfa_cols + m * 8 + at * 4, stage + L::kOffSfA + m * 1024 + at * 512);
#pragma unroll
                        for (int g = 0; g < RG; ++g)
                            if (g < groups)
                                tc05_copy_scale_atom(sfb_cols + (at * RG + g) * 4, stage + L::kOffSfB + (at * RG + g) * 512);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {                                           // K-steps of 64
                        const uint32_t acc = (kb > 0 || j > 0) ? 1u : 0u;
                        const uint32_t sfb = sfb_cols + (j >> 1) * RG * 4;
                        const uint32_t idesc = tc05_idesc_mxf4(128, n_first, (j & 1) * 2, (j & 1) * 2);
                        const uint64_t db = tc05_desc_k_sw128(stage + L::kOffB + 32 * j);
#pragma unroll
                        for (int m = 0; m < MATS; ++m)
                            if (m < t.mats)
                                tc05_mma_mxf4(tmem + m * L::kAccStride, tc05_desc_k_sw128(stage + m * kQTile + 32 * j), db,
                                              idesc, sfa_cols + m * 8 + (j >> 1) * 4, sfb, acc);
                        if (t.split) {
                            const uint32_t idesc3 = tc05_idesc_mxf4(128, t.n_mma, (j & 1) * 2, (j & 1) * 2);
                            const uint64_t db3 = tc05_desc_k_sw128(stage + L::kOffB + 256 * 128 + 32 * j);
#pragma unroll
                            for (int m = 0; m < MATS; ++m)
                                if (m < t.mats) tc05_mma_mxf4(tmem + m * L::kAccStride + 256,
                                              tc05_desc_k_sw128(stage + m * kQTile + 32 * j), db3, idesc3,
                                              sfa_cols + m * 8 + (j >> 1) * 4, sfb + 8, acc);
                        }
                    }
                    tc05_commit(smem_u32(&bar_empty[s]));
                    if (kb == n_kb - 1) tc05_commit(smem_u32(&bar_accum));
                }
                __syncwarp();
            }
        }
    }
    tc05_fence_before_sync();
    __syncthreads();
    if (warp == kProducerWarps) tc05_dealloc(tmem, 512);
}

}  // namespace dsv4
