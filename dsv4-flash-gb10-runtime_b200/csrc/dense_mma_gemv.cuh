// FP8 GEMV for 2..8 tokens per pass over the weights (several passes for more) and several independent groups:
//   y[t, g*N + n] = bf16( sum_k e4m3(W[g*N + n, k]) * scale[(g*N + n)/128, k/128] * x[t, g*K + k] ).
// With a handful of tokens the per-lane fp16 dot products of dense_gemv_kernel become instruction bound (decode
// once, multiply T times, widen, reduce across lanes).  Here a warp owns a tile of 16 weight rows and feeds it to
// mma.sync.m16n8k16 (fp16 x fp16 -> fp32): the 8 columns are the tokens, so the whole token batch costs one MMA
// per 16 x 16 weights and there is no cross-lane reduction.  The products E4M3 x fp16 are exact in FP32; the
// accumulation is FP32 in a fixed order.
//   * A lane (g = lane / 4, t = lane % 4) loads 32 consecutive bytes of rows g and g + 8 per 128-element K step;
//     the K index inside an MMA is a permutation of the true one, the same for the weights and the activations.
//   * The activations of a pass's 8 tokens are staged in shared memory as fp16, 4096 K-elements at a time (once per
//     CTA when K <= 4096 and there is one group), each (token, 2048-element half) scaled by a power of two so that
//     its largest magnitude lies in [2^14, 2^15).
//   * One CTA of 16 warps per SM walks a list of work items (pass, group, 16 / ks row tiles); the weight loads run
//     kMmaDepth K steps ahead, across item boundaries.
//   * A 128 x 128 scale tile covers one K step of a row tile: acc (one K step) is folded into the running sum
//     with scale * activation scale.
//   * ks in {1, 2, 4, 8} warps share a row tile (interleaved K steps) when there are few row tiles; their partial
//     sums meet in shared memory in a fixed order.
#pragma once

#include "dense_gemv.cuh"

namespace dsv4 {

constexpr int kMmaPanel = 2048;                       // K elements one warp converts when the activations are staged
constexpr int kMmaStage = 2 * kMmaPanel;               // K elements of activations resident in shared memory
constexpr int kMmaRowBytes = kMmaStage * 2 + 16;      // fp16 row of one token; +16: tokens g and g+1 in odd banks
constexpr int kMmaThreads = 512;
constexpr int kMmaDepth = 3;                          // K steps of weights in flight per warp
constexpr int kMmaTokens = 8;

__device__ __forceinline__ void mma_f16_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct MmaWeights {
    uint4 w[4];        // row g: bytes [0,16), [16,32) of the lane's 32; row g + 8: the same
    uint32_t s;        // raw scale of the (row tile, K step)
};

// 16-byte chunk `idx` of a token's fp16 panel row sits at chunk position idx ^ (bit 3 of idx << 1): the four lanes
// t of a quarter-warp read chunks 4 t + c, which would otherwise meet in two bank groups.
__device__ __forceinline__ int mma_x_chunk(int idx) { return idx ^ (((idx >> 3) & 1) << 1); }


// Work items: item = (pass * n_groups + group) * n_tg + tg; a tile group tg is 16 >> ks_shift row tiles, each shared
// by 1 << ks_shift warps (interleaved K steps).  CTA b takes items b, b + gridDim.x, ...
template <class Sc>
__global__ void __launch_bounds__(kMmaThreads, 1) dense_mma_gemv_kernel(const DenseMultiArgs m, const int ks_shift,
                                                                       const int n_tg, const int n_items) {
    extern __shared__ __align__(16) uint8_t x_stage[];              // kMmaTokens rows of kMmaRowBytes
    __shared__ float x_scale[2][kMmaTokens];                        // per 2048-element half of the staged K range
    __shared__ float red[2][kMmaThreads / 32][128];                 // partial sums of the warps sharing a tile
    pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2;
    const int t = lane & 3;
    const DenseArgs& a = m.a;
    const int ks = 1 << ks_shift;
    const int kpart = warp & (ks - 1);
    const int tile_local = warp >> ks_shift;
    const int tiles_per_tg = (kMmaThreads / 32) >> ks_shift;
    const int tiles = a.N >> 4;
    const int nq = (a.K >> 7) >> ks_shift;                         // K steps per warp and item
    const int qpp_shift = 5 - ks_shift;                            // a warp makes 32 / ks K steps per staged range
    const int my_items = n_items > (int)blockIdx.x ? (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int total = my_items * nq;

    // ---- the load stream: kMmaDepth steps ahead of the consumer, across items
    int i_item = blockIdx.x, i_q = 0;
    const uint8_t* i_w = nullptr;        // row r0 + g of the item's tile, byte t * 32; nullptr: no tile
    const uint8_t* i_s = nullptr;        // scale tensor of the item's group
    int i_r0 = 0;
    auto load_item = [&]() {
        i_w = nullptr;
        if (i_item < n_items) {
            const int tg = i_item % n_tg;
            const int grp = (i_item / n_tg) % m.n_groups;
            const int tile = tg * tiles_per_tg + tile_local;
            if (tile < tiles) {
                i_r0 = tile << 4;
                i_w = a.w + ((long long)grp * a.N + i_r0 + g) * a.w_stride + t * 32;
                i_s = a.s + (long long)grp * (a.N >> 7) * a.s_stride;
            }
        }
    };
    auto issue = [&](MmaWeights& b) {
#pragma unroll
        for (int i = 0; i < 4; ++i) b.w[i] = make_uint4(0, 0, 0, 0);
        b.s = 0;
        if (i_w != nullptr) {
            const int k0 = (kpart + (i_q << ks_shift)) << 7;
            const uint8_t* w1 = i_w + 8 * a.w_stride;
            b.w[0] = ldg_stream_v4(i_w + k0);
            b.w[1] = ldg_stream_v4(i_w + k0 + 16);
            b.w[2] = ldg_stream_v4(w1 + k0);
            b.w[3] = ldg_stream_v4(w1 + k0 + 16);
            b.s = Sc::fetch(i_s, i_r0, k0 >> 4, a.s_stride);
        }
        if (++i_q == nq) {
            i_q = 0;
            i_item += gridDim.x;
            load_item();
        }
    };

    // ---- staging: warp w converts token (w & 7), half (w >> 3) of the 4096-element range `range` of (pass, grp)
    auto stage = [&](int pass, int grp, int range) {
        const int token = warp & 7, half = warp >> 3;
        const int k_base = range * kMmaStage + half * kMmaPanel;
        const int n_chunks = max(0, min(kMmaPanel, a.K - k_base)) >> 3;                 // 16-byte chunks of 8 values
        const int tok = pass * kMmaTokens + token;
        const bool valid = tok < m.n_tok;
        const uint4* src = reinterpret_cast<const uint4*>(a.x + (long long)grp * a.K + (long long)tok * m.x_tok + k_base);
        uint4 v[kMmaPanel / 8 / 32];
        uint32_t amax = 0;
#pragma unroll
        for (int i = 0; i < kMmaPanel / 8 / 32; ++i) {
            const int idx = lane + 32 * i;
            v[i] = make_uint4(0, 0, 0, 0);
            if (valid && idx < n_chunks) v[i] = __ldcg(src + idx);
            const uint32_t u[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) amax = max(amax, max(u[j] & 0x7fffu, (u[j] >> 16) & 0x7fffu));
        }
        amax = __reduce_max_sync(kFullMask, amax);
        const int e = min(max((int)(amax >> 7), 15), 255);                // biased exponent of the largest magnitude
        const float inv = __uint_as_float((uint32_t)(268 - e) << 23);     // 2^-(e - 127 - 14)
        uint8_t* row = x_stage + token * kMmaRowBytes;
#pragma unroll
        for (int i = 0; i < kMmaPanel / 8 / 32; ++i) {
            const int idx = lane + 32 * i;
            if (idx >= n_chunks) continue;
            const uint32_t u[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
            uint32_t h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 p = __floats2half2_rn(__uint_as_float(u[j] << 16) * inv,
                                                    __uint_as_float(u[j] & 0xffff0000u) * inv);
                h[j] = *reinterpret_cast<const uint32_t*>(&p);
            }
            *reinterpret_cast<uint4*>(row + mma_x_chunk(half * (kMmaPanel / 8) + idx) * 16) = make_uint4(h[0], h[1], h[2], h[3]);
        }
        if (lane == 0) x_scale[half][token] = __uint_as_float((uint32_t)(e - 14) << 23);
    };

    // ---- the consumer
    int c_item = blockIdx.x, c_q = 0;
    int c_pass = 0, c_grp = 0, c_r0 = 0;
    bool c_live = false;
    int st_pass = -1, st_grp = -1, st_range = -1;       // what the shared-memory activations hold
    float xs[2][2] = {{0.f, 0.f}, {0.f, 0.f}};          // activation scales of tokens 2t, 2t+1 per half
    float out[4] = {0.f, 0.f, 0.f, 0.f};
    int parity = 0;

    auto consume = [&](const MmaWeights& b) {
        if (c_q == 0) {
            const int tg = c_item % n_tg;
            const int rest = c_item / n_tg;
            c_grp = rest % m.n_groups;
            c_pass = rest / m.n_groups;
            const int tile = tg * tiles_per_tg + tile_local;
            c_live = tile < tiles;
            c_r0 = tile << 4;
        }
        if ((c_q & ((1 << qpp_shift) - 1)) == 0) {
            const int range = c_q >> qpp_shift;
            if (c_pass != st_pass || c_grp != st_grp || range != st_range) {      // uniform over the CTA
                __syncthreads();
                stage(c_pass, c_grp, range);
                __syncthreads();
                st_pass = c_pass; st_grp = c_grp; st_range = range;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    xs[h][0] = x_scale[h][2 * t];
                    xs[h][1] = x_scale[h][2 * t + 1];
                }
            }
        }
        const int it_local = (kpart + (c_q << ks_shift)) & ((kMmaStage >> 7) - 1);
        const uint8_t* xrow = x_stage + g * kMmaRowBytes;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xrow + mma_x_chunk(it_local * 16 + t * 4 + c) * 16);
            const uint4& wg = b.w[c >> 1];
            const uint4& wh = b.w[2 + (c >> 1)];
            const uint32_t word_g[2] = {(c & 1) ? wg.z : wg.x, (c & 1) ? wg.w : wg.y};
            const uint32_t word_h[2] = {(c & 1) ? wh.z : wh.x, (c & 1) ? wh.w : wh.y};
            const uint32_t xb[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                __half2 hg[2], hh[2];
                e4m3x4_to_h2x2(word_g[j], hg);
                e4m3x4_to_h2x2(word_h[j], hh);
                mma_f16_m16n8k16(acc, *reinterpret_cast<uint32_t*>(&hg[0]), *reinterpret_cast<uint32_t*>(&hh[0]),
                                 *reinterpret_cast<uint32_t*>(&hg[1]), *reinterpret_cast<uint32_t*>(&hh[1]),
                                 xb[2 * j], xb[2 * j + 1]);
            }
        }
        const float sc = Sc::value(b.s);
        const bool upper = (it_local >> 4) != 0;
        const float s0 = sc * (upper ? xs[1][0] : xs[0][0]);
        const float s1 = sc * (upper ? xs[1][1] : xs[0][1]);
        out[0] = fmaf(acc[0], s0, out[0]);
        out[1] = fmaf(acc[1], s1, out[1]);
        out[2] = fmaf(acc[2], s0, out[2]);
        out[3] = fmaf(acc[3], s1, out[3]);

        if (++c_q == nq) {                               // the item is complete: sum over the ks warps, store
            if (ks > 1) {
#pragma unroll
                for (int i = 0; i < 4; ++i) red[parity][warp][lane * 4 + i] = out[i];
                __syncthreads();
                if (kpart == 0) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float sum = out[i];
                        for (int p = 1; p < ks; ++p) sum += red[parity][warp + p][lane * 4 + i];
                        out[i] = sum;
                    }
                }
                parity ^= 1;       // the next item's partial sums go to the other half: no second barrier needed
            }
            if (c_live && kpart == 0) {
                // c0, c1: row g, tokens 2t, 2t+1; c2, c3: row g + 8
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int tok = c_pass * kMmaTokens + 2 * t + (i & 1);
                    const int row = c_r0 + g + ((i >> 1) << 3);
                    if (tok < m.n_tok)
                        a.y[(long long)c_grp * a.N + (long long)tok * m.y_tok + row] = __float2bfloat16(out[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) out[i] = 0.f;
            c_q = 0;
            c_item += gridDim.x;
        }
    };

    MmaWeights buf[kMmaDepth];
    load_item();
#pragma unroll
    for (int d = 0; d < kMmaDepth; ++d) issue(buf[d]);          // weights never depend on the previous kernel
    pdl_wait();

#pragma unroll 1
    for (int s0 = 0; s0 < total; s0 += kMmaDepth) {
#pragma unroll
        for (int d = 0; d < kMmaDepth; ++d) {
            if (s0 + d < total) {                               // uniform over the CTA
                consume(buf[d]);
                issue(buf[d]);
            }
        }
    }
}

// Needs 16-byte aligned x, weights, row strides and token strides (checked by the caller).
template <class Sc>
inline cudaError_t dense_mma_launch(const DenseMultiArgs& m, cudaStream_t stream) {
    const DenseArgs& a = m.a;
    const long long tiles = a.N >> 4;
    const long long passes = (m.n_tok + kMmaTokens - 1) / kMmaTokens;
    const int n_steps = a.K >> 7;
    const int sms = dense_sm_count();
    // warps per row tile (1 << shift): the split that keeps the SMs evenly busy, with at least 4 K steps per warp
    int best_shift = 0;
    double best_eff = -1.0;
    for (int shift = 0; shift <= 4; ++shift) {
        const int ks = 1 << shift;
        if (n_steps % ks != 0 || (shift > 0 && n_steps / ks < 4)) break;
        const long long tpg = (kMmaThreads / 32) >> shift;
        const long long items = ((tiles + tpg - 1) / tpg) * m.n_groups * passes;
        const long long rounds = (items + sms - 1) / sms;
        const double eff = (double)items / (double)(rounds * sms);
        if (eff > best_eff + 0.05) { best_eff = eff; best_shift = shift; }
    }
    const long long tpg = (kMmaThreads / 32) >> best_shift;
    const long long n_tg = (tiles + tpg - 1) / tpg;
    const long long n_items = n_tg * m.n_groups * passes;
    if (n_items > 0x7fffffffLL) return cudaErrorInvalidValue;
    static bool attr_set[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return cudaErrorInvalidDevice;
    const int smem = kMmaTokens * kMmaRowBytes;
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        const cudaError_t err = cudaFuncSetAttribute(dense_mma_gemv_kernel<Sc>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) return err;
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n_items < sms ? n_items : sms));
    cfg.blockDim = dim3(kMmaThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dense_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, dense_mma_gemv_kernel<Sc>, m, best_shift, (int)n_tg, (int)n_items);
}

}  // namespace dsv4
