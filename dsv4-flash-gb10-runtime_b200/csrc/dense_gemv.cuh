// Dense M=1 GEMV over a quantized weight matrix, shared by the MXFP4 and FP8-E4M3 libraries.
//   y[n] = bf16( sum_k W[n,k] * x[k] ),  FP32 accumulation across blocks.
// A CTA owns a contiguous range of output rows; a warp owns one 32-block slice of the reduction axis
// (1024 MXFP4 elements / 512 FP8 elements) and walks down the CTA's rows with 8 row loads in flight
// per lane and the next 8 already requested.  Per-slice partial sums meet in shared memory.
#pragma once

#include "gemv_engine.cuh"

#include <cstdio>
#include <cstdlib>
#include <utility>

namespace dsv4 {

constexpr int kDenseThreads = 256;
constexpr int kDenseRows = 8;          // rows per warp batch
constexpr int kDenseCap = 64;          // rows per CTA
constexpr int kDenseMaxSlices = 32;    // FP8 K <= 16384 -> 1024 blocks -> 32 slices

struct DenseArgs {
    const __nv_bfloat16* x;
    const uint8_t* w;
    const uint8_t* s;
    int K, N;
    long long w_stride, s_stride;      // bytes per row of W / per row of the scale tensor
    __nv_bfloat16* y;
};

// Where the scale of (row, block) lives, how it is fetched (raw 32 bits) and what it is worth.
struct Fp4Scale {   // E8M0 [N, K/32]: one byte per row per block
    __device__ static __forceinline__ uint32_t fetch(const uint8_t* s, int row, int blk, long long s_stride) {
        return ldg_stream_u8(s + (long long)row * s_stride + blk);
    }
    __device__ static __forceinline__ float value(uint32_t raw) { return e8m0_to_float(raw); }
};
struct Fp8Scale {   // E8M0 [N/128, K/128]: one byte per 128x128 tile; a block is 16 elements
    __device__ static __forceinline__ uint32_t fetch(const uint8_t* s, int row, int blk, long long s_stride) {
        return ldg_stream_u8(s + (long long)(row >> 7) * s_stride + (blk >> 3));
    }
    __device__ static __forceinline__ float value(uint32_t raw) { return e8m0_to_float(raw); }
};
struct Fp8ScaleF32 {   // FP32 [N/128, K/128], row stride in bytes
    __device__ static __forceinline__ uint32_t fetch(const uint8_t* s, int row, int blk, long long s_stride) {
        return __ldg(reinterpret_cast<const uint32_t*>(s + (long long)(row >> 7) * s_stride) + (blk >> 3));
    }
    __device__ static __forceinline__ float value(uint32_t raw) { return __uint_as_float(raw); }
};

struct DenseBatch {
    uint4 w[kDenseRows];
    uint32_t s[kDenseRows];
};

template <class Sc>
__device__ __forceinline__ void dense_issue(const DenseArgs& a, int row, int step, int row_end, int blk,
                                            bool lane_ok, DenseBatch& b) {
#pragma unroll
    for (int i = 0; i < kDenseRows; ++i) {
        const int n = row + i * step;
        b.w[i] = make_uint4(0, 0, 0, 0);
        b.s[i] = 0;
        if (n < row_end && lane_ok) {
            b.w[i] = ldg_stream_v4(a.w + (long long)n * a.w_stride + (long long)blk * 16);
            b.s[i] = Sc::fetch(a.s, n, blk, a.s_stride);
        }
    }
}

template <class Fmt, class Sc>
__device__ __forceinline__ void dense_consume(const DenseBatch& b, const ActBlock<Fmt>& xb, int lane, int local0,
                                              int step, int n_local, int ks, float (*part)[kDenseMaxSlices]) {
    float v[kDenseRows];
#pragma unroll
    for (int i = 0; i < kDenseRows; ++i) {
        v[i] = 0.f;
        if (local0 + i * step < n_local) v[i] = Fmt::dot(b.w[i], xb.h) * (Sc::value(b.s[i]) * xb.scale);
    }
    multi_reduce<kDenseRows>(v, lane);
    if (multi_reduce_owner<kDenseRows>(lane)) {
        const int local = local0 + multi_reduce_index<kDenseRows>(lane) * step;
        if (local < n_local) part[local][ks] = v[0];
    }
}

// GROUPED: blockIdx.y picks one of several independent problems stacked along the rows of W (FP8 tile scales):
// group g multiplies rows [g N, (g+1) N) with x[g K, (g+1) K) into y[g N, (g+1) N).
template <class Fmt, class Sc, bool GROUPED = false>
__global__ void __launch_bounds__(kDenseThreads, 2) dense_gemv_kernel(const DenseArgs a_in) {
    __shared__ float part[kDenseCap][kDenseMaxSlices];
    pdl_launch_dependents();
    DenseArgs a = a_in;
    if (GROUPED) {
        const long long grp = blockIdx.y;
        a.x += grp * a.K;
        a.w += grp * a.N * a.w_stride;
        a.s += grp * (a.N >> 7) * a.s_stride;
        a.y += grp * a.N;
    }

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int n_warps = blockDim.x >> 5;
    const int n_blk = a.K / Fmt::kElems;
    const int n_slices = (n_blk + 31) >> 5;
    const int n_groups = max(1, n_warps / n_slices);
    const int n_tasks = n_slices * n_groups;

    const int r_begin = (int)((long long)a.N * blockIdx.x / gridDim.x);
    const int r_end = (int)((long long)a.N * (blockIdx.x + 1) / gridDim.x);
    const int n_local = r_end - r_begin;
    const int span = kDenseRows * n_groups;

    bool waited = false;
    for (int task = warp; task < n_tasks; task += n_warps) {
        const int ks = task % n_slices;
        const int rg = task / n_slices;
        const int blk = ks * 32 + lane;
        const bool lane_ok = blk < n_blk;

        DenseBatch b0, b1;
        // weights never depend on the previous kernel in the stream: request them before waiting for it
        dense_issue<Sc>(a, r_begin + rg, n_groups, r_end, blk, lane_ok, b0);
        if (!waited) { pdl_wait(); waited = true; }

        ActBlock<Fmt> xb;
        act_block_load_bf16<Fmt>(a.x + (size_t)blk * Fmt::kElems, lane_ok, xb);

        for (int local0 = rg; local0 < n_local; local0 += 2 * span) {
            dense_issue<Sc>(a, r_begin + local0 + span, n_groups, r_end, blk, lane_ok, b1);
            dense_consume<Fmt, Sc>(b0, xb, lane, local0, n_groups, n_local, ks, part);
            dense_issue<Sc>(a, r_begin + local0 + 2 * span, n_groups, r_end, blk, lane_ok, b0);
            dense_consume<Fmt, Sc>(b1, xb, lane, local0 + span, n_groups, n_local, ks, part);
        }
    }
    if (!waited) pdl_wait();
    __syncthreads();

    for (int t = threadIdx.x; t < n_local; t += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_slices; ++s) acc += part[t][s];
        a.y[r_begin + t] = __float2bfloat16(acc);
    }
}

// Gate / up pair of a gated FFN with one token: act[n] = bf16( silu(clamp(g[n])) * clamp(u[n]) ), g = Wg x, u = Wu x,
// both rounded to bf16 first (as two separate GEMV calls would leave them).  Same streaming scheme as
// dense_gemv_kernel; a CTA owns a range of n and walks it once per matrix, so g[n] and u[n] meet in its shared memory.
// limit_g / limit_u <= 0 switch the clamp of that operand off.
constexpr int kDualCap = kDenseCap / 2;      // n per CTA

template <class Fmt, class Sc>
__global__ void __launch_bounds__(kDenseThreads, 2) dense_dual_swiglu_kernel(const DenseArgs ag, const DenseArgs au,
                                                                             float limit_g, float limit_u) {
    __shared__ float part[kDenseCap][kDenseMaxSlices];      // rows [0, kDualCap): gate, [kDualCap, 2 kDualCap): up
    pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int n_warps = blockDim.x >> 5;
    const int n_blk = ag.K / Fmt::kElems;
    const int n_slices = (n_blk + 31) >> 5;
    const int n_groups = max(1, n_warps / n_slices);
    const int n_tasks = n_slices * n_groups;

    const int r_begin = (int)((long long)ag.N * blockIdx.x / gridDim.x);
    const int r_end = (int)((long long)ag.N * (blockIdx.x + 1) / gridDim.x);
    const int n_local = r_end - r_begin;
    const int span = kDenseRows * n_groups;

    bool waited = false;
    for (int task = warp; task < n_tasks; task += n_warps) {
        const int ks = task % n_slices;
        const int rg = task / n_slices;
        const int blk = ks * 32 + lane;
        const bool lane_ok = blk < n_blk;
        ActBlock<Fmt> xb;
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            const DenseArgs& a = m == 0 ? ag : au;
            float (*pm)[kDenseMaxSlices] = part + m * kDualCap;
            DenseBatch b0, b1;
            dense_issue<Sc>(a, r_begin + rg, n_groups, r_end, blk, lane_ok, b0);
            if (!waited) { pdl_wait(); waited = true; }
            if (m == 0) act_block_load_bf16<Fmt>(a.x + (size_t)blk * Fmt::kElems, lane_ok, xb);
            for (int local0 = rg; local0 < n_local; local0 += 2 * span) {
                dense_issue<Sc>(a, r_begin + local0 + span, n_groups, r_end, blk, lane_ok, b1);
                dense_consume<Fmt, Sc>(b0, xb, lane, local0, n_groups, n_local, ks, pm);
                dense_issue<Sc>(a, r_begin + local0 + 2 * span, n_groups, r_end, blk, lane_ok, b0);
                dense_consume<Fmt, Sc>(b1, xb, lane, local0 + span, n_groups, n_local, ks, pm);
            }
        }
    }
    if (!waited) pdl_wait();
    __syncthreads();

    for (int t = threadIdx.x; t < n_local; t += blockDim.x) {
        float g = 0.f, u = 0.f;
        for (int s = 0; s < n_slices; ++s) { g += part[t][s]; u += part[kDualCap + t][s]; }
        g = __bfloat162float(__float2bfloat16(g));
        u = __bfloat162float(__float2bfloat16(u));
        if (limit_g > 0.f) g = fminf(fmaxf(g, -limit_g), limit_g);
        if (limit_u > 0.f) u = fminf(fmaxf(u, -limit_u), limit_u);
        ag.y[r_begin + t] = __float2bfloat16((g / (1.0f + expf(-g))) * u);
    }
}

// Several tokens and several independent groups in one launch (FP8 only: the attention projections):
//   y[t, g*N + n] = bf16( sum_k W[g*N + n, k] * x[t, g*K + k] ),   W [G*N, K], scales [G*N/128, K/128].
// G = 1 is a plain batched GEMV; G > 1 is the block-diagonal shape of the grouped output projection (one launch
// instead of G).  One token runs the grouped form of dense_gemv_kernel (bit-identical to the M = 1 entry); several
// tokens run dense_mma_gemv_kernel (dense_mma_gemv.cuh), which reads every weight byte once per 8 tokens.
struct DenseMultiArgs {
    DenseArgs a;                   // group 0, token 0; a.N = rows per group
    int n_groups;
    int n_tok;
    long long x_tok, y_tok;        // elements between consecutive tokens of x / y
};

// Any alignment, any stride: one warp per row, byte loads, FP32 FMA.  Only taken when a base pointer
// or a row stride is not a multiple of 16 bytes.
template <class Fmt, class Sc>
__global__ void dense_gemv_unaligned_kernel(const DenseArgs a) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= a.N) return;
    const int n_blk = a.K / Fmt::kElems;
    const uint8_t* wrow = a.w + (long long)row * a.w_stride;
    float acc = 0.f;
    for (int blk = lane; blk < n_blk; blk += 32) {
        const float sc = Sc::value(Sc::fetch(a.s, row, blk, a.s_stride));
        const __nv_bfloat16* xp = a.x + (size_t)blk * Fmt::kElems;
        float part = 0.f;
        for (int i = 0; i < 16; ++i) {
            const uint32_t byte = wrow[(size_t)blk * 16 + i];
            if (Fmt::kElems == 32) {
                const float2 f = e2m1x2_to_float2(byte);
                part = fmaf(f.x, __bfloat162float(xp[2 * i]), part);
                part = fmaf(f.y, __bfloat162float(xp[2 * i + 1]), part);
            } else {
                part = fmaf(e4m3_to_float(byte), __bfloat162float(xp[i]), part);
            }
        }
        acc = fmaf(part, sc, acc);
    }
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(kFullMask, acc, off);
    if (lane == 0) a.y[row] = __float2bfloat16(acc);
}

inline int dense_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

inline bool dense_pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = std::getenv("DSV4_B200_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// CTAs per SM that one launch asks for.  Two fill the machine (126 registers x 256 threads) and are what a large
// matrix wants.  A matrix small enough that one CTA per SM requests all of its rows up front (two batches of
// kDenseRows per warp) is bound by the launch chain instead: with one CTA per SM the next launch of the chain
// becomes resident beside this one and has its weights on the way while this one finishes (2048 x 4096 MXFP4:
// 4.3 us per call against 5.6).  DSV4_B200_DENSE_WAVES = 1 .. 4 overrides the choice.
inline int dense_waves(int n_rows, int n_blk) {
    static int forced = -1;
    if (forced < 0) {
        const char* e = std::getenv("DSV4_B200_DENSE_WAVES");
        const int w = e ? std::atoi(e) : 0;
        forced = (w >= 1 && w <= 4) ? w : 0;
    }
    if (forced > 0) return forced;
    const int n_slices = (n_blk + 31) >> 5;
    const int n_groups = (kDenseThreads / 32) / n_slices > 0 ? (kDenseThreads / 32) / n_slices : 1;
    const long long up_front = 2LL * kDenseRows * n_groups * dense_sm_count();
    return n_rows <= up_front ? 1 : 2;
}

// Launches the aligned streaming kernel when it can, the byte-wise one otherwise.
template <class Fmt, class Sc>
inline cudaError_t dense_launch(const DenseArgs& a, cudaStream_t stream) {
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; };
    if (mis(a.x) || mis(a.w) || (a.w_stride & 15) != 0) {
        const int warps = 8;
        dense_gemv_unaligned_kernel<Fmt, Sc><<<(a.N + warps - 1) / warps, warps * 32, 0, stream>>>(a);
        return cudaGetLastError();
    }
    long long grid = (long long)dense_waves(a.N, a.K / Fmt::kElems) * dense_sm_count();
    const long long need = ((long long)a.N + kDenseCap - 1) / kDenseCap;
    if (grid < need) grid = need;
    if (grid > a.N) grid = a.N;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kDenseThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dense_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, dense_gemv_kernel<Fmt, Sc>, a);
}

template <class Sc>
inline cudaError_t dense_mma_launch(const DenseMultiArgs& m, cudaStream_t stream);      // dense_mma_gemv.cuh

// Several tokens / groups: needs 16-byte aligned x, weights, row strides and token strides (cudaErrorInvalidValue
// otherwise).  One token: grid.y = groups, at most kDenseCap rows per CTA.
template <class Sc>
inline cudaError_t dense_multi_launch(const DenseMultiArgs& m, cudaStream_t stream) {
    const DenseArgs& a = m.a;
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; };
    if (mis(a.x) || mis(a.w) || (a.w_stride & 15) != 0 || (m.x_tok & 7) != 0 || m.n_groups > 65535)
        return cudaErrorInvalidValue;
    const long long need = ((long long)a.N + kDenseCap - 1) / kDenseCap;
    long long per_group = (2LL * dense_sm_count() + m.n_groups - 1) / m.n_groups;
    if (per_group < need) per_group = need;
    if (per_group > a.N) per_group = a.N;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)per_group, (unsigned)m.n_groups);
    cfg.blockDim = dim3(kDenseThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dense_pdl_enabled() ? 1 : 0;
    if (m.n_tok == 1) return cudaLaunchKernelEx(&cfg, dense_gemv_kernel<Fp8Format, Sc, true>, a);
    return dense_mma_launch<Sc>(m, stream);
}

// The gate / up pair: ag and au describe the two matrices (same K, N, x); the activation goes to ag.y.
// Needs 16-byte aligned x, weights and row strides (returns cudaErrorInvalidValue otherwise).
template <class Fmt, class Sc>
inline cudaError_t dense_dual_launch(const DenseArgs& ag, const DenseArgs& au, float limit_g, float limit_u,
                                     cudaStream_t stream) {
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; };
    if (mis(ag.x) || mis(ag.w) || mis(au.w) || (ag.w_stride & 15) != 0 || (au.w_stride & 15) != 0)
        return cudaErrorInvalidValue;
    long long grid = 2LL * dense_sm_count();
    const long long need = ((long long)ag.N + kDualCap - 1) / kDualCap;
    if (grid < need) grid = need;
    if (grid > ag.N) grid = ag.N;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kDenseThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dense_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, dense_dual_swiglu_kernel<Fmt, Sc>, ag, au, limit_g, limit_u);
}

}  // namespace dsv4
