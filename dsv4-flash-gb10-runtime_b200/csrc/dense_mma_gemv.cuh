// FP8 GEMV for 2..8 tokens per pass over the weights (several passes for more) and several independent groups:
//   y[t, g*N + n] = bf16( sum_k e4m3(W[g*N + n, k]) * scale[(g*N + n)/128, k/128] * x[t, g*K + k] ).
// With a handful of tokens the per-lane fp16 dot products of dense_gemv_kernel become instruction bound (decode
// once, multiply T times, widen, reduce across lanes).  Here a warp owns a tile of 16 weight rows and feeds it to
// mma.sync.m16n8k16 (fp16 x fp16 -> fp32): the 8 columns are the tokens, so the whole token batch costs one MMA
// per 16 x 16 weights and there is no cross-lane reduction.  The products E4M3 x fp16 are exact in FP32; the
// accumulation is FP32 in a fixed order.
//   * A lane (g = lane / 4, t = lane % 4) loads 32 consecutive bytes of rows g and g + 8 per 128-element K step;
//     the K index inside an MMA is a permutation of the true one, the same for the weights and the activations.
//   * The activations of the CTA's 8 tokens are staged in shared memory as fp16, one K panel of 2048 at a time,
//     each (token, panel) scaled by a power of two so that its largest magnitude lies in [2^14, 2^15).
//   * A 128 x 128 scale tile covers one K step of a row tile: acc (one K step) is folded into the running sum
//     with scale * activation scale.
//   * ks in {1, 2, 4, 8} warps share a row tile (interleaved K steps) when there are few row tiles; their partial
//     sums meet in shared memory in a fixed order.
#pragma once

#include "dense_gemv.cuh"

namespace dsv4 {

constexpr int kMmaRowBytes = kMmaPanel * 2 + 16;      // fp16 row of one token; +16: tokens g and g+1 in odd banks
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

template <class Sc>
__global__ void __launch_bounds__(kDenseThreads, 2) dense_mma_gemv_kernel(const DenseMultiArgs m, const int ks) {
    __shared__ __align__(16) uint8_t x_panel[kMmaTokens * kMmaRowBytes];
    __shared__ float x_scale[kMmaTokens];
    __shared__ float red[kDenseThreads / 32][128];
    pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int tok0 = blockIdx.z * kMmaTokens;
    const int nt = min(kMmaTokens, m.n_tok - tok0);

    DenseArgs a = m.a;
    {
        const long long grp = blockIdx.y;
        a.x += grp * a.K;
        a.w += grp * a.N * a.w_stride;
        a.s += grp * (a.N >> 7) * a.s_stride;
        a.y += grp * a.N;
    }

    const int ks_shift = 31 - __clz(ks);
    const int tiles_per_cta = (kDenseThreads / 32) >> ks_shift;
    const int tile = blockIdx.x * tiles_per_cta + (warp >> ks_shift);
    const int kpart = warp & (ks - 1);
    const bool live = tile < (a.N >> 4);
    const int r0 = tile << 4;
    const int nq = (a.K >> 7) >> ks_shift;                 // K steps of this warp; the same for every warp
    const int qpp_shift = 4 - ks_shift;                    // a warp makes 16 / ks K steps per activation panel

    const uint8_t* wrow0 = a.w + (long long)(r0 + g) * a.w_stride + t * 32;
    const uint8_t* wrow1 = wrow0 + 8 * a.w_stride;

    auto issue = [&](int q, MmaWeights& b) {
#pragma unroll
        for (int i = 0; i < 4; ++i) b.w[i] = make_uint4(0, 0, 0, 0);
        b.s = 0;
        if (live && q < nq) {
            const int k0 = (kpart + (q << ks_shift)) << 7;
            b.w[0] = ldg_stream_v4(wrow0 + k0);
            b.w[1] = ldg_stream_v4(wrow0 + k0 + 16);
            b.w[2] = ldg_stream_v4(wrow1 + k0);
            b.w[3] = ldg_stream_v4(wrow1 + k0 + 16);
            b.s = Sc::fetch(a.s, r0, k0 >> 4, a.s_stride);
        }
    };

    // warp w converts token tok0 + w: bf16 -> fp16 * 2^-e with the panel's largest magnitude in [2^14, 2^15)
    auto stage = [&](int panel) {
        const int k_base = panel * kMmaPanel;
        const int n_chunks = min(kMmaPanel, a.K - k_base) >> 3;          // 16-byte chunks of 8 values
        const bool valid = warp < nt;
        const uint4* src = reinterpret_cast<const uint4*>(a.x + (long long)(tok0 + warp) * m.x_tok + k_base);
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
        uint8_t* row = x_panel + warp * kMmaRowBytes;
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
            *reinterpret_cast<uint4*>(row + mma_x_chunk(idx) * 16) = make_uint4(h[0], h[1], h[2], h[3]);
        }
        if (lane == 0) x_scale[warp] = __uint_as_float((uint32_t)(e - 14) << 23);
    };

    float out[4] = {0.f, 0.f, 0.f, 0.f};
    float xs0 = 0.f, xs1 = 0.f;

    auto consume = [&](const MmaWeights& b, int q) {
        const int it_local = (kpart + (q << ks_shift)) & ((kMmaPanel >> 7) - 1);
        const uint8_t* xrow = x_panel + g * kMmaRowBytes;
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
        out[0] = fmaf(acc[0], sc * xs0, out[0]);
        out[1] = fmaf(acc[1], sc * xs1, out[1]);
        out[2] = fmaf(acc[2], sc * xs0, out[2]);
        out[3] = fmaf(acc[3], sc * xs1, out[3]);
    };

    MmaWeights buf[kMmaDepth];
#pragma unroll
    for (int d = 0; d < kMmaDepth; ++d) issue(d, buf[d]);      // weights never depend on the previous kernel
    pdl_wait();

#pragma unroll 1
    for (int q0 = 0; q0 < nq; q0 += kMmaDepth) {
#pragma unroll
        for (int d = 0; d < kMmaDepth; ++d) {
            const int q = q0 + d;
            if (q < nq) {                                       // uniform over the CTA
                if ((q & ((1 << qpp_shift) - 1)) == 0) {
                    __syncthreads();
                    stage(q >> qpp_shift);
                    __syncthreads();
                    xs0 = x_scale[2 * t];
                    xs1 = x_scale[2 * t + 1];
                }
                consume(buf[d], q);
                issue(q + kMmaDepth, buf[d]);
            }
        }
    }

    if (ks > 1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][lane * 4 + i] = out[i];
        __syncthreads();
        if (kpart == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float sum = out[i];
                for (int p = 1; p < ks; ++p) sum += red[warp + p][lane * 4 + i];
                out[i] = sum;
            }
        }
    }
    if (live && kpart == 0) {
        // c0, c1: row g, tokens 2t, 2t+1; c2, c3: row g + 8
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int tok = 2 * t + (i & 1);
            const int row = r0 + g + ((i >> 1) << 3);
            if (tok < nt) a.y[(long long)(tok0 + tok) * m.y_tok + row] = __float2bfloat16(out[i]);
        }
    }
}

// Needs 16-byte aligned x, weights, row strides and token strides (cudaErrorInvalidValue otherwise).
template <class Sc>
inline cudaError_t dense_mma_launch(const DenseMultiArgs& m, cudaStream_t stream) {
    const DenseArgs& a = m.a;
    const long long tiles = a.N >> 4;
    const long long passes = (m.n_tok + kMmaTokens - 1) / kMmaTokens;
    if (m.n_groups > 65535 || passes > 65535) return cudaErrorInvalidValue;
    // enough warps to fill the GPU twice: share a row tile between ks warps when there are few tiles
    const long long want = 2LL * dense_sm_count() * (kDenseThreads / 32);
    int ks = 1;
    while (ks < 8 && tiles * m.n_groups * passes * ks < want && ((a.K >> 7) % (ks * 2)) == 0) ks *= 2;
    const int tiles_per_cta = (kDenseThreads / 32) / ks;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((tiles + tiles_per_cta - 1) / tiles_per_cta), (unsigned)m.n_groups, (unsigned)passes);
    cfg.blockDim = dim3(kDenseThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dense_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, dense_mma_gemv_kernel<Sc>, m, ks);
}

}  // namespace dsv4
