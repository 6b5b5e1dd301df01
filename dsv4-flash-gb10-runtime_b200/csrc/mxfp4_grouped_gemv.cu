// libmxfp4_grouped_gemv.so — routed-expert MXFP4 SwiGLU FFN for one decode token on B200 (sm_100a).
//
//   out = sum_e r[e] * W2_e ( silu(W1_e x) * (W3_e x) )          e = 0 .. n_exp-1
//
// Drop-in for the entry points of the reference's kernel/mxfp4-routed/mxfp4_grouped_gemv.cu
// (:294-309 mxfp4_grouped_gemv_topk, :406-409 mxfp4_grouped_workspace_bytes): same names, argument
// order, return codes and ownership rules (caller owns all buffers, work is enqueued on the caller's
// stream, no allocation, no synchronisation).
//
// Two kernels, chained by programmatic dependent launch so that the second one is already resident
// and has its first weight tiles in flight while the first one drains:
//   gate/up kernel : every CTA owns a contiguous range of (expert, hidden-row) pairs; a warp owns a
//                    1024-element slice of the reduction axis and walks down the CTA's rows, W1 and W3
//                    row of a pair together; per-slice partial sums meet in shared memory, the CTA then
//                    writes silu(g)*u as FP32 into the workspace.
//   down kernel    : every CTA owns a contiguous range of output rows for ALL experts; a warp owns
//                    (expert, 1024-slice); the router-weighted sum over experts is taken inside the CTA
//                    in a fixed order (deterministic, no float atomics), rounded once to bf16.
#include "gemv_engine.cuh"

#include <cstdio>
#include <cstdlib>

namespace dsv4 {

constexpr int kMaxSlices = 4;        // reduction axis <= 4096 elements = 4 slices of 32 blocks
constexpr int kMaxExperts = 8;       // experts per call (the reference fixes 6)

constexpr int kGateThreads = 256;    // 8 warps
constexpr int kGatePairs = 4;        // (W1,W3) row pairs per warp batch -> 8 x 16 B loads per lane in flight
constexpr int kGateCap = 256;        // pairs per CTA held in shared memory

constexpr int kDownThreads = 384;    // 12 warps = 6 experts x 2 slices at the DSv4 shape
constexpr int kDownRows = 8;         // rows per warp batch
constexpr int kDownCap = 64;         // output rows per CTA
constexpr int kDownMaxUnits = kMaxExperts * kMaxSlices;

struct GroupedArgs {
    const __nv_bfloat16* x;
    const uint8_t* w1p; const uint8_t* w3p; const uint8_t* w2p;
    const uint8_t* w1s; const uint8_t* w3s; const uint8_t* w2s;
    const float* r;
    const int* ids;                  // nullptr: expert slot e uses bank entry e (stacked weights)
    int K, H, O, E;
    long long strideAp, strideAs, strideBp, strideBs;   // bytes per expert
    float* mid;                      // [E, H] FP32 SwiGLU intermediate (workspace)
    __nv_bfloat16* out;
};

// ------------------------------------------------------------------------------------------------
// gate/up + SwiGLU
// ------------------------------------------------------------------------------------------------

struct GateBatch {
    uint4 w1[kGatePairs];
    uint4 w3[kGatePairs];
    uint32_t s1[kGatePairs];
    uint32_t s3[kGatePairs];
};

struct PairCursor {      // next (expert slot, hidden row) this warp will request
    int q, e, h;
};

__device__ __forceinline__ void gate_issue(const GroupedArgs& a, PairCursor& c, int step, int q_end,
                                           int blk, bool lane_ok, GateBatch& b) {
#pragma unroll
    for (int i = 0; i < kGatePairs; ++i) {
        b.w1[i] = make_uint4(0, 0, 0, 0);
        b.w3[i] = make_uint4(0, 0, 0, 0);
        b.s1[i] = 0;
        b.s3[i] = 0;
        if (c.q < q_end && lane_ok) {
            const long long eid = a.ids ? a.ids[c.e] : c.e;
            const long long po = eid * a.strideAp + (long long)c.h * (a.K >> 1) + (long long)blk * 16;
            const long long so = eid * a.strideAs + (long long)c.h * (a.K >> 5) + blk;
            b.w1[i] = ldg_stream_v4(a.w1p + po);
            b.w3[i] = ldg_stream_v4(a.w3p + po);
            b.s1[i] = ldg_stream_u8(a.w1s + so);
            b.s3[i] = ldg_stream_u8(a.w3s + so);
        }
        c.q += step;
        c.h += step;
        if (c.h >= a.H) { c.h -= a.H; c.e += 1; }
    }
}

__device__ __forceinline__ void gate_consume(const GateBatch& b, const ActBlock<Fp4Format>& xb, int lane,
                                             int local0, int step, int n_local, int ks,
                                             float (*part)[kMaxSlices][2]) {
    float v[2 * kGatePairs];
#pragma unroll
    for (int i = 0; i < kGatePairs; ++i) {
        v[2 * i + 0] = 0.f;
        v[2 * i + 1] = 0.f;
        if (local0 + i * step < n_local) {   // warp-uniform: skip the arithmetic of rows past the range
            v[2 * i + 0] = Fp4Format::dot(b.w1[i], xb.h) * (e8m0_to_float(b.s1[i]) * xb.scale);
            v[2 * i + 1] = Fp4Format::dot(b.w3[i], xb.h) * (e8m0_to_float(b.s3[i]) * xb.scale);
        }
    }
    multi_reduce<2 * kGatePairs>(v, lane);
    if (multi_reduce_owner<2 * kGatePairs>(lane)) {
        const int idx = multi_reduce_index<2 * kGatePairs>(lane);
        const int local = local0 + (idx >> 1) * step;
        if (local < n_local) part[local][ks][idx & 1] = v[0];
    }
}

__global__ void __launch_bounds__(kGateThreads, 2) grouped_gate_up_kernel(const GroupedArgs a) {
    __shared__ float part[kGateCap][kMaxSlices][2];
    pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int n_warps = blockDim.x >> 5;
    const int n_blk = a.K >> 5;
    const int n_slices = (n_blk + 31) >> 5;
    const int n_groups = n_warps / n_slices;          // host guarantees >= 1
    const int ks = warp % n_slices;
    const int rg = warp / n_slices;
    const int blk = ks * 32 + lane;
    const bool lane_ok = blk < n_blk;
    const bool warp_ok = rg < n_groups;

    const long long total = (long long)a.E * a.H;
    const int q_begin = (int)(total * blockIdx.x / gridDim.x);
    const int q_end = (int)(total * (blockIdx.x + 1) / gridDim.x);
    const int n_local = q_end - q_begin;

    if (warp_ok) {
        PairCursor cur;
        cur.q = q_begin + rg;
        cur.e = cur.q / a.H;
        cur.h = cur.q - cur.e * a.H;

        GateBatch b0, b1;
        // stacked weights do not depend on the previous kernel: request them before waiting for it
        if (a.ids == nullptr) gate_issue(a, cur, n_groups, q_end, blk, lane_ok, b0);
        pdl_wait();
        if (a.ids != nullptr) gate_issue(a, cur, n_groups, q_end, blk, lane_ok, b0);

        ActBlock<Fp4Format> xb;
        act_block_load_bf16<Fp4Format>(a.x + (size_t)blk * 32, lane_ok, xb);

        const int batch_span = kGatePairs * n_groups;
        for (int local0 = rg; local0 < n_local; local0 += 2 * batch_span) {
            gate_issue(a, cur, n_groups, q_end, blk, lane_ok, b1);
            gate_consume(b0, xb, lane, local0, n_groups, n_local, ks, part);
            gate_issue(a, cur, n_groups, q_end, blk, lane_ok, b0);
            gate_consume(b1, xb, lane, local0 + batch_span, n_groups, n_local, ks, part);
        }
    } else {
        pdl_wait();
    }
    __syncthreads();

    for (int t = threadIdx.x; t < n_local; t += blockDim.x) {
        float g = 0.f, u = 0.f;
        for (int s = 0; s < n_slices; ++s) { g += part[t][s][0]; u += part[t][s][1]; }
        a.mid[q_begin + t] = (g / (1.0f + __expf(-g))) * u;
    }
}

// ------------------------------------------------------------------------------------------------
// down projection + router-weighted combine
// ------------------------------------------------------------------------------------------------

struct DownBatch {
    uint4 w[kDownRows];
    uint32_t s[kDownRows];
};

__device__ __forceinline__ void down_issue(const GroupedArgs& a, long long eid, int row, int step, int row_end,
                                           int blk, bool lane_ok, DownBatch& b) {
#pragma unroll
    for (int i = 0; i < kDownRows; ++i) {
        const int o = row + i * step;
        b.w[i] = make_uint4(0, 0, 0, 0);
        b.s[i] = 0;
        if (o < row_end && lane_ok) {
            b.w[i] = ldg_stream_v4(a.w2p + eid * a.strideBp + (long long)o * (a.H >> 1) + (long long)blk * 16);
            b.s[i] = ldg_stream_u8(a.w2s + eid * a.strideBs + (long long)o * (a.H >> 5) + blk);
        }
    }
}

__device__ __forceinline__ void down_consume(const DownBatch& b, const ActBlock<Fp4Format>& mb, int lane,
                                             int local0, int step, int n_local, int unit,
                                             float (*part)[kDownMaxUnits]) {
    float v[kDownRows];
#pragma unroll
    for (int i = 0; i < kDownRows; ++i) {
        v[i] = 0.f;
        if (local0 + i * step < n_local)
            v[i] = Fp4Format::dot(b.w[i], mb.h) * (e8m0_to_float(b.s[i]) * mb.scale);
    }
    multi_reduce<kDownRows>(v, lane);
    if (multi_reduce_owner<kDownRows>(lane)) {
        const int local = local0 + multi_reduce_index<kDownRows>(lane) * step;
        if (local < n_local) part[local][unit] = v[0];
    }
}

__global__ void __launch_bounds__(kDownThreads, 1) grouped_down_kernel(const GroupedArgs a) {
    __shared__ float part[kDownCap][kDownMaxUnits];
    pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int n_warps = blockDim.x >> 5;
    const int n_blk = a.H >> 5;
    const int n_slices = (n_blk + 31) >> 5;
    const int n_units = a.E * n_slices;                       // (expert, slice)
    const int n_groups = max(1, n_warps / n_units);           // row groups sharing a unit
    const int n_tasks = n_units * n_groups;

    const int o_begin = (int)((long long)a.O * blockIdx.x / gridDim.x);
    const int o_end = (int)((long long)a.O * (blockIdx.x + 1) / gridDim.x);
    const int n_local = o_end - o_begin;

    bool waited = false;
    for (int task = warp; task < n_tasks; task += n_warps) {
        const int unit = task % n_units;
        const int rg = task / n_units;
        const int e = unit / n_slices;
        const int ks = unit - e * n_slices;
        const int blk = ks * 32 + lane;
        const bool lane_ok = blk < n_blk;
        const int span = kDownRows * n_groups;

        DownBatch b0, b1;
        long long eid = e;
        if (!waited && a.ids == nullptr) down_issue(a, eid, o_begin + rg, n_groups, o_end, blk, lane_ok, b0);
        if (!waited) pdl_wait();
        if (a.ids != nullptr) eid = a.ids[e];
        if (waited || a.ids != nullptr) down_issue(a, eid, o_begin + rg, n_groups, o_end, blk, lane_ok, b0);
        waited = true;

        ActBlock<Fp4Format> mb;
        act_block_load_f32<Fp4Format>(a.mid + (size_t)e * a.H + (size_t)blk * 32, lane_ok, mb);

        for (int local0 = rg; local0 < n_local; local0 += 2 * span) {
            down_issue(a, eid, o_begin + local0 + span, n_groups, o_end, blk, lane_ok, b1);
            down_consume(b0, mb, lane, local0, n_groups, n_local, unit, part);
            down_issue(a, eid, o_begin + local0 + 2 * span, n_groups, o_end, blk, lane_ok, b0);
            down_consume(b1, mb, lane, local0 + span, n_groups, n_local, unit, part);
        }
    }
    if (!waited) pdl_wait();
    __syncthreads();

    for (int t = threadIdx.x; t < n_local; t += blockDim.x) {
        float acc = 0.f;
        for (int e = 0; e < a.E; ++e) {
            float y = 0.f;
            for (int s = 0; s < n_slices; ++s) y += part[t][e * n_slices + s];
            acc = fmaf(__ldcg(a.r + e), y, acc);
        }
        a.out[o_begin + t] = __float2bfloat16(acc);
    }
}

// ------------------------------------------------------------------------------------------------
// router: scores, top-k, normalised weights — on the device, no host round trip
// ------------------------------------------------------------------------------------------------
// One warp per token.  score_func 0: softmax over all experts, weights renormalised over the top-k.
// score_func 1: sqrt(softplus(logit)), w = s / (sum s + eps) * scaling (the engine's rule,
// kernel/cpp-engine-mxfp4/routed.cu:156-208).  Ties go to the lowest expert index in both.
constexpr int kRouteMaxPerLane = 32;   // up to 1024 experts

__global__ void route_topk_kernel(const float* __restrict__ logits, int n_tokens, int n_experts, int k,
                                  int score_func, float eps, float scaling,
                                  int* __restrict__ ids_out, float* __restrict__ w_out) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (token >= n_tokens) return;
    const float* row = logits + (size_t)token * n_experts;

    float s[kRouteMaxPerLane];
    const int per_lane = (n_experts + 31) >> 5;
    float row_max = -INFINITY;
#pragma unroll
    for (int i = 0; i < kRouteMaxPerLane; ++i) {
        s[i] = -INFINITY;
        if (i < per_lane) {
            const int idx = i * 32 + lane;
            if (idx < n_experts) s[i] = __ldcg(row + idx);
            row_max = fmaxf(row_max, s[i]);
        }
    }
    if (score_func == 0) {
        // softmax is monotone in the logit: select on the logits, weight by exp(logit - max); the softmax
        // denominator cancels when the weights are renormalised over the picks
        for (int off = 16; off > 0; off >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(kFullMask, row_max, off));
    } else {
#pragma unroll
        for (int i = 0; i < kRouteMaxPerLane; ++i)
            if (i < per_lane && s[i] != -INFINITY) {
                const float g = s[i];
                s[i] = sqrtf(fmaxf(g, 0.0f) + log1pf(expf(-fabsf(g))));
            }
    }

    double picked_sum = 0.0;
    float my_pick_score = 0.f;   // lane j keeps the j-th pick
    int my_pick_id = -1;
    for (int j = 0; j < k; ++j) {
        float best = -INFINITY;
        int best_idx = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kRouteMaxPerLane; ++i)
            if (i < per_lane) {
                const int idx = i * 32 + lane;
                if (s[i] > best) { best = s[i]; best_idx = idx; }   // strict: lowest index wins inside a lane
            }
        for (int off = 16; off > 0; off >>= 1) {
            const float ob = __shfl_xor_sync(kFullMask, best, off);
            const int oi = __shfl_xor_sync(kFullMask, best_idx, off);
            if (ob > best || (ob == best && oi < best_idx)) { best = ob; best_idx = oi; }
        }
        if (lane == (j & 31)) { my_pick_score = best; my_pick_id = best_idx; }
        if ((best_idx & 31) == lane) {
#pragma unroll
            for (int i = 0; i < kRouteMaxPerLane; ++i)
                if (i == (best_idx >> 5)) s[i] = -INFINITY;
        }
        const double contrib = (score_func == 0) ? exp((double)best - (double)row_max) : (double)best;
        picked_sum += contrib;
    }
    if (lane < k) {
        double w;
        if (score_func == 0) {
            w = exp((double)my_pick_score - (double)row_max) / picked_sum;   // softmax renormalised over the picks
        } else {
            w = (double)my_pick_score / (picked_sum + (double)eps) * (double)scaling;
        }
        ids_out[(size_t)token * k + lane] = my_pick_id;
        w_out[(size_t)token * k + lane] = (float)w;
    }
}

// ------------------------------------------------------------------------------------------------
// dequantisation export (test/diagnostic): MXFP4 -> bf16, byte 0xFF -> NaN as the Python reference
// ------------------------------------------------------------------------------------------------
__global__ void dequant_bf16_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scale,
                                    long long rows, int cols, __nv_bfloat16* __restrict__ out) {
    const long long n_blocks = rows * (cols >> 5);
    for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks;
         b += (long long)gridDim.x * blockDim.x) {
        const float sc = e8m0_to_float_nan(scale[b]);
        const uint8_t* src = packed + b * 16;
        __nv_bfloat16* dst = out + b * 32;
        for (int i = 0; i < 16; ++i) {
            const uint32_t byte = src[i];
            __half2 h[4];
            e2m1x8_to_h2x4(byte, h);
            const float2 f = __half22float2(h[0]);
            dst[2 * i + 0] = __float2bfloat16(f.x * sc);
            dst[2 * i + 1] = __float2bfloat16(f.y * sc);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------

static int sm_count() {
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

static bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = std::getenv("DSV4_B200_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

template <class... Params, class... Args>
static cudaError_t launch(void (*kernel)(Params...), dim3 grid, dim3 block, cudaStream_t stream, bool pdl,
                          Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

static int grouped_forward(const GroupedArgs& a, cudaStream_t stream, const char* who) {
    const int sms = sm_count();
    const bool pdl = pdl_enabled();
    {
        const long long pairs = (long long)a.E * a.H;
        long long grid = 2LL * sms;
        const long long need = (pairs + kGateCap - 1) / kGateCap;
        if (grid < need) grid = need;
        if (grid > pairs) grid = pairs;
        cudaError_t err = launch(grouped_gate_up_kernel, dim3((unsigned)grid), dim3(kGateThreads), stream, pdl, a);
        if (err != cudaSuccess) {
            std::fprintf(stderr, "%s: gate/up launch failed: %s\n", who, cudaGetErrorString(err));
            return -5;
        }
    }
    {
        long long grid = sms;
        const long long need = ((long long)a.O + kDownCap - 1) / kDownCap;
        if (grid < need) grid = need;
        if (grid > a.O) grid = a.O;
        cudaError_t err = launch(grouped_down_kernel, dim3((unsigned)grid), dim3(kDownThreads), stream, pdl, a);
        if (err != cudaSuccess) {
            std::fprintf(stderr, "%s: down launch failed: %s\n", who, cudaGetErrorString(err));
            return -6;
        }
    }
    return 0;
}

static int check_shape(const char* who, int K_in, int hidden, int out_dim) {
    if (K_in <= 0 || K_in % 32 != 0) {
        std::fprintf(stderr, "%s: K_in=%d not a positive multiple of 32\n", who, K_in);
        return -1;
    }
    if (hidden <= 0 || hidden % 32 != 0) {
        std::fprintf(stderr, "%s: hidden=%d not a positive multiple of 32\n", who, hidden);
        return -2;
    }
    if (K_in > 32 * 32 * kMaxSlices || hidden > 32 * 32 * kMaxSlices) {
        std::fprintf(stderr, "%s: K_in/hidden > %d\n", who, 32 * 32 * kMaxSlices);
        return -3;
    }
    if (out_dim <= 0) {
        std::fprintf(stderr, "%s: out_dim=%d\n", who, out_dim);
        return -8;
    }
    return 0;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace dsv4

using namespace dsv4;

// Replaces kernel/mxfp4-routed/mxfp4_grouped_gemv.cu:294-403 of the reference.
// Return codes as there: -1 K_in % 32, -2 hidden % 32, -3 K_in or hidden > 4096, -4 n_exp != 6,
// -5 / -6 launch failure.  Added: -8 null or non-16-byte-aligned pointer, or out_dim <= 0.
DSV4_API int mxfp4_grouped_gemv_topk(const __nv_bfloat16* x, const uint8_t* W1_packed, const uint8_t* W3_packed,
                                     const uint8_t* W2_packed, const uint8_t* W1_scale, const uint8_t* W3_scale,
                                     const uint8_t* W2_scale, const float* rweights, int K_in, int hidden,
                                     int out_dim, int n_exp, __nv_bfloat16* out, void* workspace,
                                     cudaStream_t stream) {
    const char* who = "mxfp4_grouped_gemv_topk";
    if (int rc = check_shape(who, K_in, hidden, out_dim)) return rc;
    if (n_exp != 6) {
        std::fprintf(stderr, "%s: n_exp=%d != 6\n", who, n_exp);
        return -4;
    }
    if (!x || !W1_packed || !W3_packed || !W2_packed || !W1_scale || !W3_scale || !W2_scale || !rweights || !out ||
        !workspace || !aligned16(x) || !aligned16(W1_packed) || !aligned16(W3_packed) || !aligned16(W2_packed) ||
        !aligned16(workspace)) {
        std::fprintf(stderr, "%s: null pointer, or x / packed weights / workspace not 16-byte aligned\n", who);
        return -8;
    }
    GroupedArgs a;
    a.x = x; a.w1p = W1_packed; a.w3p = W3_packed; a.w2p = W2_packed;
    a.w1s = W1_scale; a.w3s = W3_scale; a.w2s = W2_scale; a.r = rweights; a.ids = nullptr;
    a.K = K_in; a.H = hidden; a.O = out_dim; a.E = n_exp;
    a.strideAp = (long long)hidden * (K_in / 2); a.strideAs = (long long)hidden * (K_in / 32);
    a.strideBp = (long long)out_dim * (hidden / 2); a.strideBs = (long long)out_dim * (hidden / 32);
    a.mid = reinterpret_cast<float*>(workspace);
    a.out = out;
    return grouped_forward(a, stream, who);
}

// Replaces kernel/mxfp4-routed/mxfp4_grouped_gemv.cu:406-409.  The intermediate is kept in FP32 here
// (n_exp * hidden * 4 bytes); callers size their buffer through this query, as the reference's callers do.
DSV4_API size_t mxfp4_grouped_workspace_bytes(int n_exp, int hidden, int out_dim) {
    (void)out_dim;
    if (n_exp <= 0 || hidden <= 0) return 0;
    return (size_t)n_exp * (size_t)hidden * sizeof(float);
}

// Additive: same computation, but the experts are picked from a resident bank by index, so the caller
// no longer gathers the selected experts into contiguous scratch first.  `topk_ids` is a DEVICE array of
// n_exp bank indices (1 <= n_exp <= 8); bank tensors are [n_bank, hidden, K_in/2] etc.
DSV4_API int mxfp4_grouped_gemv_topk_ids(const __nv_bfloat16* x, const uint8_t* bank_W1_packed,
                                         const uint8_t* bank_W3_packed, const uint8_t* bank_W2_packed,
                                         const uint8_t* bank_W1_scale, const uint8_t* bank_W3_scale,
                                         const uint8_t* bank_W2_scale, const int* topk_ids, const float* rweights,
                                         int K_in, int hidden, int out_dim, int n_exp, __nv_bfloat16* out,
                                         void* workspace, cudaStream_t stream) {
    const char* who = "mxfp4_grouped_gemv_topk_ids";
    if (int rc = check_shape(who, K_in, hidden, out_dim)) return rc;
    if (n_exp < 1 || n_exp > kMaxExperts) {
        std::fprintf(stderr, "%s: n_exp=%d outside 1..%d\n", who, n_exp, kMaxExperts);
        return -4;
    }
    if (!x || !bank_W1_packed || !bank_W3_packed || !bank_W2_packed || !bank_W1_scale || !bank_W3_scale ||
        !bank_W2_scale || !topk_ids || !rweights || !out || !workspace || !aligned16(x) ||
        !aligned16(bank_W1_packed) || !aligned16(bank_W3_packed) || !aligned16(bank_W2_packed) ||
        !aligned16(workspace)) {
        std::fprintf(stderr, "%s: null pointer, or x / packed weights / workspace not 16-byte aligned\n", who);
        return -8;
    }
    GroupedArgs a;
    a.x = x; a.w1p = bank_W1_packed; a.w3p = bank_W3_packed; a.w2p = bank_W2_packed;
    a.w1s = bank_W1_scale; a.w3s = bank_W3_scale; a.w2s = bank_W2_scale; a.r = rweights; a.ids = topk_ids;
    a.K = K_in; a.H = hidden; a.O = out_dim; a.E = n_exp;
    a.strideAp = (long long)hidden * (K_in / 2); a.strideAs = (long long)hidden * (K_in / 32);
    a.strideBp = (long long)out_dim * (hidden / 2); a.strideBs = (long long)out_dim * (hidden / 32);
    a.mid = reinterpret_cast<float*>(workspace);
    a.out = out;
    return grouped_forward(a, stream, who);
}

// Additive: router scores + top-k + weights on the device (replaces the D2H copy, stream synchronise and
// host scan of kernel/cpp-engine-mxfp4/routed.cu:169-208).  logits [n_tokens, n_experts] FP32;
// score_func 0 = softmax renormalised over the top-k, 1 = sqrt-softplus with eps and scaling;
// ids_out int32 [n_tokens, k] in descending score order (ties: lowest index), w_out FP32 [n_tokens, k].
// Returns -1 for a bad shape (n_experts > 1024, k > 32 or k > n_experts), -2 null pointer, -3 launch failure.
DSV4_API int mxfp4_moe_route_topk(const float* logits, int n_tokens, int n_experts, int k, int score_func,
                                  float eps, float scaling, int* ids_out, float* w_out, cudaStream_t stream) {
    const char* who = "mxfp4_moe_route_topk";
    if (n_tokens < 0 || n_experts <= 0 || n_experts > 32 * kRouteMaxPerLane || k <= 0 || k > 32 || k > n_experts ||
        (score_func != 0 && score_func != 1)) {
        std::fprintf(stderr, "%s: bad shape tokens=%d experts=%d k=%d score_func=%d\n", who, n_tokens, n_experts, k,
                     score_func);
        return -1;
    }
    if (n_tokens == 0) return 0;
    if (!logits || !ids_out || !w_out) {
        std::fprintf(stderr, "%s: null pointer\n", who);
        return -2;
    }
    const int warps = 4;
    cudaError_t err = launch(route_topk_kernel, dim3((n_tokens + warps - 1) / warps), dim3(32 * warps), stream,
                             pdl_enabled(), logits, n_tokens, n_experts, k, score_func, eps, scaling, ids_out, w_out);
    if (err != cudaSuccess) {
        std::fprintf(stderr, "%s: launch failed: %s\n", who, cudaGetErrorString(err));
        return -3;
    }
    return 0;
}

// Additive (diagnostic): MXFP4 -> bf16 with the reference loader's semantics
// (runtime/mxfp4_loader.py:272-309; scale byte 0xFF -> NaN).  packed [rows, cols/2], scale [rows, cols/32].
DSV4_API int mxfp4_dequant_bf16(const uint8_t* packed, const uint8_t* scale, long long rows, int cols,
                                __nv_bfloat16* out, cudaStream_t stream) {
    if (rows < 0 || cols <= 0 || cols % 32 != 0) return -1;
    if (rows == 0) return 0;
    if (!packed || !scale || !out) return -2;
    const long long n_blocks = rows * (cols / 32);
    long long grid = (n_blocks + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    dequant_bf16_kernel<<<(unsigned)grid, 256, 0, stream>>>(packed, scale, rows, cols, out);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
