// libmxfp4_grouped_gemv.so — routed-expert MXFP4 SwiGLU FFN for one decode token on B200 (sm_100a).
//
//   out = sum_e r[e] * W2_e ( silu(W1_e x) * (W3_e x) )          e = 0 .. n_exp-1
//
// Drop-in for the entry points of the reference's kernel/mxfp4-routed/mxfp4_grouped_gemv.cu
// (:294-309 mxfp4_grouped_gemv_topk, :406-409 mxfp4_grouped_workspace_bytes): same names, argument
// order, return codes and ownership rules (caller owns all buffers, work is enqueued on the caller's
// stream, no allocation, no synchronisation).
//
// At the DSv4 shapes one persistent kernel does the whole call (decode_stream.cuh).  Elsewhere, and on request,
// two kernels chained by programmatic dependent launch, so that the second one can request its first weight rows
// while the first one drains:
//   gate/up kernel : a warp owns a contiguous run of (expert, hidden-row) pairs and streams the W1 and W3
//                    row of a pair whole (a lane owns up to 4 blocks of the row, the activation vector
//                    lives in its registers), reduces across lanes and writes silu(g)*u as FP32 into the
//                    workspace; no shared memory, no block barrier.
//   down kernel    : a CTA owns a contiguous range of output rows for ALL experts, a warp owns one expert;
//                    the router-weighted sum over experts is taken inside the CTA in a fixed order
//                    (deterministic, no float atomics) and rounded once to bf16.
#include "gemv_engine.cuh"
#include "stream_ring.cuh"
#include "grouped_args.cuh"
#include "router.cuh"
#include "grouped_ring.cuh"
#include "decode_stream.cuh"

#include <cstdio>
#include <cstdlib>

namespace dsv4 {

constexpr int kMaxBlocksPerLane = 4;   // reduction axis <= 4096 elements = 128 blocks = 4 per lane
constexpr int kMaxExperts = 8;         // experts per call (the reference fixes 6)

constexpr int kGateThreads = 384;      // 12 warps, one (W1,W3) row pair in flight per warp
constexpr int kDownThreads = 384;      // 12 warps = 6 experts x 2 row groups at the DSv4 shape
constexpr int kDownCap = 64;           // output rows per CTA held in shared memory
constexpr int kDownLoads = 8;          // 16-byte loads per lane per batch


// One weight row as seen by a lane: BPL 16-byte blocks and their scale bytes.
template <int BPL>
struct RowRegs {
    uint4 w[BPL];
    uint32_t s[BPL];
};

template <int BPL>
__device__ __forceinline__ void row_clear(RowRegs<BPL>& r) {
#pragma unroll
    for (int j = 0; j < BPL; ++j) { r.w[j] = make_uint4(0, 0, 0, 0); r.s[j] = 0; }
}

// wp / sp already point at this lane's first block / scale byte of the row.
template <int BPL>
__device__ __forceinline__ void row_issue(const uint8_t* wp, const uint8_t* sp, const bool (&ok)[BPL],
                                          RowRegs<BPL>& r) {
#pragma unroll
    for (int j = 0; j < BPL; ++j)
        if (ok[j]) {
            r.w[j] = ldg_stream_v4(wp + 512 * j);
            r.s[j] = ldg_stream_u8(sp + 32 * j);
        }
}

// Dot product of the lane's part of a row with the activations; each block's registers are refilled with the
// same block of a later row (at nwp / nsp) as soon as they have been consumed, so the lane always has its
// full set of loads in flight without a second register buffer.
template <int BPL>
__device__ __forceinline__ float row_dot_refill(RowRegs<BPL>& r, const LaneAct<Fp4Format, BPL>& a,
                                                const uint8_t* nwp, const uint8_t* nsp, bool more,
                                                const bool (&ok)[BPL]) {
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < BPL; ++j) {
        const float d = Fp4Format::dot(r.w[j], a.h[j]);
        const float sc = e8m0_to_float_fast(r.s[j]);
        if (more && ok[j]) {
            r.w[j] = ldg_stream_v4(nwp + 512 * j);
            r.s[j] = ldg_stream_u8(nsp + 32 * j);
        }
        acc = fmaf(d, sc, acc);
    }
    return acc * a.scale;
}

// ------------------------------------------------------------------------------------------------
// gate/up + SwiGLU: a warp owns a contiguous run of (expert slot, hidden row) pairs and streams the W1 and
// W3 row of a pair together (2 x BPL loads of 512 contiguous bytes per warp)
// ------------------------------------------------------------------------------------------------

struct GateCursor {
    const uint8_t* w1; const uint8_t* w3; const uint8_t* s1; const uint8_t* s3;   // this lane's position in pair q
    int q, h, e;
};

__device__ __forceinline__ void gate_seek(const GroupedArgs& a, GateCursor& c, int lane) {
    const long long eid = a.ids ? (long long)a.ids[c.e] : (long long)c.e;
    const long long po = eid * a.strideAp + (long long)c.h * (a.K >> 1) + lane * 16;
    const long long so = eid * a.strideAs + (long long)c.h * (a.K >> 5) + lane;
    c.w1 = a.w1p + po; c.w3 = a.w3p + po; c.s1 = a.w1s + so; c.s3 = a.w3s + so;
}

__device__ __forceinline__ void gate_advance(const GroupedArgs& a, GateCursor& c, int q_end, int lane) {
    const int row_p = a.K >> 1, row_s = a.K >> 5;
    c.q += 1;
    c.h += 1;
    c.w1 += row_p; c.w3 += row_p; c.s1 += row_s; c.s3 += row_s;
    if (c.h == a.H) {          // next expert slot: stacked experts are contiguous, a bank needs a new base
        c.h = 0;
        c.e += 1;
        if (a.ids != nullptr && c.q < q_end) gate_seek(a, c, lane);
    }
}

template <int BPL>
__global__ void __launch_bounds__(kGateThreads, 1) grouped_gate_up_kernel(const GroupedArgs a) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int n_gw = gridDim.x * (blockDim.x >> 5);
    const int n_blk = a.K >> 5;
    bool ok[BPL];
#pragma unroll
    for (int j = 0; j < BPL; ++j) ok[j] = lane + 32 * j < n_blk;

    const long long total = (long long)a.E * a.H;
    const int q_begin = (int)(total * gw / n_gw);
    const int q_end = (int)(total * (gw + 1) / n_gw);

    GateCursor cur;
    cur.q = q_begin;
    cur.e = q_begin / a.H;
    cur.h = q_begin - cur.e * a.H;
    cur.w1 = cur.w3 = cur.s1 = cur.s3 = nullptr;

    RowRegs<BPL> g, u;
    row_clear(g);
    row_clear(u);
    const bool any = q_begin < q_end;
    // stacked weights do not depend on the previous kernel in the stream: request them before waiting for it
    if (a.ids == nullptr && any) {
        gate_seek(a, cur, lane);
        row_issue<BPL>(cur.w1, cur.s1, ok, g);
        row_issue<BPL>(cur.w3, cur.s3, ok, u);
    }
    pdl_wait();
    if (a.ids != nullptr && any) {
        gate_seek(a, cur, lane);
        row_issue<BPL>(cur.w1, cur.s1, ok, g);
        row_issue<BPL>(cur.w3, cur.s3, ok, u);
    }
    LaneAct<Fp4Format, BPL> x;
    lane_act_load<Fp4Format, BPL>(a.x, lane, n_blk, x);

    for (int q = q_begin; q < q_end; ++q) {
        gate_advance(a, cur, q_end, lane);                       // cur now describes pair q + 1
        const bool more = q + 1 < q_end;
        float v[2];
        v[0] = row_dot_refill<BPL>(g, x, cur.w1, cur.s1, more, ok);
        v[1] = row_dot_refill<BPL>(u, x, cur.w3, cur.s3, more, ok);
        multi_reduce<2>(v, lane);                                // lane 0: gate sum, lane 16: up sum
        const float up = __shfl_sync(kFullMask, v[0], 16);
        if (lane == 0) a.mid[q] = swiglu_f32(v[0], up);
    }
}

// ------------------------------------------------------------------------------------------------
// down projection + router-weighted combine: a CTA owns a contiguous range of output rows for ALL experts,
// a warp owns (expert slot, row group); the sum over experts is taken in a fixed order inside the CTA
// ------------------------------------------------------------------------------------------------

template <int BPL>
__global__ void __launch_bounds__(kDownThreads, 1) grouped_down_kernel(const GroupedArgs a) {
    constexpr int RB = kDownLoads / BPL;          // rows in flight per warp
    __shared__ float part[kDownCap][kMaxExperts];
    pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int n_warps = blockDim.x >> 5;
    const int n_blk = a.H >> 5;
    bool ok[BPL];
#pragma unroll
    for (int j = 0; j < BPL; ++j) ok[j] = lane + 32 * j < n_blk;

    const int n_groups = n_warps / a.E;                       // host guarantees E <= n_warps
    const int e = warp % a.E;
    const int rg = warp / a.E;
    const int o_begin = (int)((long long)a.O * blockIdx.x / gridDim.x);
    const int o_end = (int)((long long)a.O * (blockIdx.x + 1) / gridDim.x);
    const int n_local = o_end - o_begin;
    // this warp's rows: a contiguous share of the CTA's range
    const int l_begin = (int)((long long)n_local * rg / n_groups);
    const int l_end = (rg < n_groups) ? (int)((long long)n_local * (rg + 1) / n_groups) : l_begin;
    const int row_p = a.H >> 1, row_s = a.H >> 5;
    const bool any = l_begin < l_end;

    RowRegs<BPL> b[RB];
#pragma unroll
    for (int i = 0; i < RB; ++i) row_clear(b[i]);

    const uint8_t* wp = nullptr;     // this lane's position in row l0 of the loop below
    const uint8_t* sp = nullptr;
    auto first_issue = [&]() {
        const long long eid = a.ids ? (long long)a.ids[e] : (long long)e;
        wp = a.w2p + eid * a.strideBp + (long long)(o_begin + l_begin) * row_p + lane * 16;
        sp = a.w2s + eid * a.strideBs + (long long)(o_begin + l_begin) * row_s + lane;
#pragma unroll
        for (int i = 0; i < RB; ++i)
            if (l_begin + i < l_end) row_issue<BPL>(wp + (long long)i * row_p, sp + i * row_s, ok, b[i]);
    };
    if (a.ids == nullptr && any) first_issue();
    pdl_wait();
    if (a.ids != nullptr && any) first_issue();

    if (any) {
        LaneAct<Fp4Format, BPL> m;
        lane_act_load<Fp4Format, BPL>(a.mid + (size_t)e * a.H, lane, n_blk, m);
        for (int l0 = l_begin; l0 < l_end; l0 += RB) {
            float v[RB];
#pragma unroll
            for (int i = 0; i < RB; ++i) {
                v[i] = 0.f;
                if (l0 + i < l_end)
                    v[i] = row_dot_refill<BPL>(b[i], m, wp + (long long)(RB + i) * row_p, sp + (RB + i) * row_s,
                                               l0 + RB + i < l_end, ok);
            }
            multi_reduce<RB>(v, lane);
            if (multi_reduce_owner<RB>(lane)) {
                const int l = l0 + multi_reduce_index<RB>(lane);
                if (l < l_end) part[l][e] = v[0];
            }
            wp += (long long)RB * row_p;
            sp += RB * row_s;
        }
    }
    __syncthreads();

    for (int t = threadIdx.x; t < n_local; t += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < a.E; ++k) acc = fmaf(__ldcg(a.r + k), part[t][k], acc);
        a.out[o_begin + t] = __float2bfloat16(acc);
    }
}

// ------------------------------------------------------------------------------------------------
// router: scores, top-k, normalised weights — on the device, no host round trip
// ------------------------------------------------------------------------------------------------
// One warp per token.  score_func 0: softmax over all experts, weights renormalised over the top-k.
// score_func 1: sqrt(softplus(logit)), w = s / (sum s + eps) * scaling (the engine's rule,
// kernel/cpp-engine-mxfp4/routed.cu:156-208).  Ties go to the lowest expert index in both.
template <int PL>
__global__ void route_topk_kernel(const RouteArgs r, int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (token >= n_tokens) return;
    int id;
    float w;
    route_token<PL>(r.logits + (size_t)token * r.n_experts, r.n_experts, r.k, r.score_func, r.eps, r.scaling, lane,
                    id, w);
    if (lane < r.k) {
        r.ids_out[(size_t)token * r.k + lane] = id;
        r.w_out[(size_t)token * r.k + lane] = w;
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
            const float2 f = e2m1x2_to_float2(src[i]);
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
static cudaError_t launch_smem(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               bool pdl, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <class... Params, class... Args>
static cudaError_t launch(void (*kernel)(Params...), dim3 grid, dim3 block, cudaStream_t stream, bool pdl,
                          Args&&... args) {
    return launch_smem(kernel, grid, block, 0, stream, pdl, std::forward<Args>(args)...);
}

static bool ring_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = std::getenv("DSV4_B200_RING");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// Shared-memory opt-in above 48 KB is a per-function, per-device attribute: set it once per device.
template <class Kernel>
static cudaError_t allow_smem(Kernel kernel, size_t bytes, int (&done)[64]) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (done[dev] >= (int)bytes) return cudaSuccess;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (err == cudaSuccess) done[dev] = (int)bytes;
    return err;
}

// How the single-kernel path is launched.  Its CTAs wait for one another, so all of them must be resident at once:
//   1 "coop"  cooperative launch: the runtime guarantees co-residency whatever else runs on the device;
//   3 "pdl"   programmatic stream serialisation: the next layer's CTAs are scheduled while this layer's exit,
//             which hides the launch latency; co-residency then rests on the caller running its grouped calls
//             from ONE stream per device (the reference engine's model).  Calls from several streams may leave
//             two grids half resident each; their bounded waits then give up (status 3, NaN output).
//   2 "auto"  (default) the first stream that calls on a device is launched as "pdl", every other stream as
//             "coop".  Grids of one stream never overlap each other's waits, and a cooperative grid is resident
//             as a whole, so any mix of streams makes progress: the entry points are safe from any number of
//             streams and threads, and a single decode stream keeps the faster launch.
//   0 "0"     no single kernel: the two chained kernels, which wait for nothing.
// DSV4_B200_FUSED selects the mode; dsv4_b200_set_launch_mode() overrides it at run time.
static int g_fused_mode = -1;
static int fused_mode() {
    if (g_fused_mode < 0) {
        const char* e = std::getenv("DSV4_B200_FUSED");
        int v = 2;
        if (e && e[0] == '0') v = 0;
        else if (e && e[0] == 'c') v = 1;
        else if (e && e[0] == 'p') v = 3;
        g_fused_mode = v;
    }
    return g_fused_mode;
}
// "auto": the one stream per device that is launched with programmatic stream serialisation.
static bool owns_pdl(int dev, cudaStream_t stream) {
    static void* owner[64] = {nullptr};
    static int have[64] = {0};
    void* me = reinterpret_cast<void*>(stream);
    int expected = 0;
    if (__atomic_compare_exchange_n(&have[dev], &expected, 1, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE)) {
        __atomic_store_n(&owner[dev], me, __ATOMIC_RELEASE);
        __atomic_store_n(&have[dev], 2, __ATOMIC_RELEASE);
        return true;
    }
    while (__atomic_load_n(&have[dev], __ATOMIC_ACQUIRE) != 2) { }     // another thread is writing the owner
    return __atomic_load_n(&owner[dev], __ATOMIC_ACQUIRE) == me;
}
static bool fused_enabled() { return fused_mode() != 0; }

// Poll budget of the device-side waits and the phantom producers of the give-up test (dsv4_b200_test_wait_limits).
static unsigned g_spin_limit = kSpinLimit;
static int g_phantom = 0;

// Single persistent kernel without a grid barrier (decode_stream.cuh), one CTA per SM, launched as fused_mode() says.
// Returns 1 when it cannot be used here (the caller then launches the two chained kernels).
template <int KT, int HT>
static int grouped_launch_stream(GroupedArgs a, cudaStream_t stream, const RouteArgs& rt) {
    static int done[64] = {0};
    static int usable[64] = {0};         // 1 = yes, -1 = no
    using L = StreamLayout<KT, HT>;
    auto kernel = moe_decode_stream_kernel<KT, HT>;
    constexpr int kThreads = kStreamThreads;
    int dev = 0;
    if (a.sync == nullptr || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
    if (usable[dev] == 0) {
        int coop = 0, per_sm = 0;
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
        if (allow_smem(kernel, L::kBytes, done) != cudaSuccess || !coop ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, L::kBytes) != cudaSuccess ||
            per_sm < 1) {
            cudaGetLastError();
            usable[dev] = -1;
        } else {
            usable[dev] = 1;
        }
    }
    if (usable[dev] < 0) return 1;
    long long grid = sm_count();         // one CTA per SM
    if (grid > kStreamMaxGrid) grid = kStreamMaxGrid;
    if (grid > a.O) grid = a.O;
    if (grid > HT) grid = HT;
    if ((long long)kStreamCap * grid < a.O || (long long)kStreamCapA * grid < HT || a.E > kStreamMaxExperts) return 1;
    a.spin_limit = g_spin_limit;
    a.mid8 = reinterpret_cast<unsigned long long*>(a.mid);
    a.phantom = g_phantom;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = L::kBytes;
    cfg.stream = stream;
    // a cooperative launch is not combined with programmatic stream serialisation: one or the other
    cudaLaunchAttribute attr[1];
    const int mode = fused_mode();
    if (mode == 1 || (mode == 2 && !owns_pdl(dev, stream))) {
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
    } else {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
    }
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, a, rt);
    if (err != cudaSuccess) {
        cudaGetLastError();
        usable[dev] = -1;                                            // do not try again on this device
        return 1;
    }
    return 0;
}

// Shared-memory ring path (grouped_ring.cuh).  Returns 1 when the shape is not one it serves.
template <int KT, int HT>
static int grouped_launch_ring(const GroupedArgs& a, cudaStream_t stream, const char* who, int h_shift,
                               int stages, const RouteArgs& rt) {
    static int gate_done[64] = {0}, down_done[64] = {0};
    const int sms = sm_count();
    const bool pdl = pdl_enabled();
    if (stages & 1) {
        auto kernel = gate_up_ring_kernel<KT>;
        cudaError_t err = allow_smem(kernel, GateRingLayout<KT>::kBytes, gate_done);
        const long long pairs = (long long)a.E * a.H;
        const long long grid = sms < pairs ? sms : pairs;
        if (err == cudaSuccess)
            err = launch_smem(kernel, dim3((unsigned)grid), dim3(kRingGateWarps * 32), GateRingLayout<KT>::kBytes,
                              stream, pdl, a, h_shift, rt);
        if (err != cudaSuccess) {
            std::fprintf(stderr, "%s: gate/up launch failed: %s\n", who, cudaGetErrorString(err));
            return -5;
        }
    }
    if (stages & 2) {
        GroupedArgs d = a;
        if (rt.logits != nullptr) { d.ids = rt.ids_out; d.r = rt.w_out; }    // published by the gate kernel
        auto kernel = down_ring_kernel<HT>;
        cudaError_t err = allow_smem(kernel, DownRingLayout<HT>::kBytes, down_done);
        long long grid = sms;
        const long long need = ((long long)a.O + kRingDownCap - 1) / kRingDownCap;
        if (grid < need) grid = need;
        if (grid > a.O) grid = a.O;
        if (err == cudaSuccess)
            err = launch_smem(kernel, dim3((unsigned)grid), dim3(64 * a.E), DownRingLayout<HT>::kBytes, stream, pdl, d);
        if (err != cudaSuccess) {
            std::fprintf(stderr, "%s: down launch failed: %s\n", who, cudaGetErrorString(err));
            return -6;
        }
    }
    return 0;
}

static int grouped_try_ring(const GroupedArgs& a, cudaStream_t stream, const char* who, int stages,
                            const RouteArgs& rt = RouteArgs{}) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (!ring_enabled() || a.E > kRingMaxExperts || (a.H & (a.H - 1)) != 0 || !al16(a.w1s) || !al16(a.w3s) ||
        !al16(a.w2s))
        return 1;
    int h_shift = 0;
    while ((1 << h_shift) < a.H) ++h_shift;
#define DSV4_RING(KT, HT)                                                                          \
    if (a.K == KT && a.H == HT) {                                                                  \
        if (stages == 3 && fused_enabled() && grouped_launch_stream<KT, HT>(a, stream, rt) == 0) return 0; \
        return grouped_launch_ring<KT, HT>(a, stream, who, h_shift, stages, rt);                  \
    }
    DSV4_RING(4096, 2048) DSV4_RING(4096, 1024) DSV4_RING(2048, 2048) DSV4_RING(2048, 1024)
    DSV4_RING(1024, 2048) DSV4_RING(1024, 1024)
#undef DSV4_RING
    return 1;
}

template <int BPL_A, int BPL_B>
static int grouped_launch(const GroupedArgs& a, cudaStream_t stream, const char* who, int stages) {
    const int sms = sm_count();
    const bool pdl = pdl_enabled();
    if (stages & 1) {
        const long long pairs = (long long)a.E * a.H;
        long long grid = sms;
        const long long max_grid = (pairs + (kGateThreads / 32) - 1) / (kGateThreads / 32);
        if (grid > max_grid) grid = max_grid;
        cudaError_t err = launch(grouped_gate_up_kernel<BPL_A>, dim3((unsigned)grid), dim3(kGateThreads), stream,
                                 pdl, a);
        if (err != cudaSuccess) {
            std::fprintf(stderr, "%s: gate/up launch failed: %s\n", who, cudaGetErrorString(err));
            return -5;
        }
    }
    if (stages & 2) {
        long long grid = sms;
        const long long need = ((long long)a.O + kDownCap - 1) / kDownCap;
        if (grid < need) grid = need;
        if (grid > a.O) grid = a.O;
        cudaError_t err = launch(grouped_down_kernel<BPL_B>, dim3((unsigned)grid), dim3(kDownThreads), stream, pdl, a);
        if (err != cudaSuccess) {
            std::fprintf(stderr, "%s: down launch failed: %s\n", who, cudaGetErrorString(err));
            return -6;
        }
    }
    return 0;
}

static int grouped_forward(const GroupedArgs& a, cudaStream_t stream, const char* who, int stages = 3) {
    const int ba = ((a.K >> 5) + 31) >> 5;    // 16-byte blocks per lane on the K_in axis: 1..4
    const int bb = ((a.H >> 5) + 31) >> 5;    // and on the hidden axis
    const int bpl_a = ba <= 1 ? 1 : (ba <= 2 ? 2 : 4);
    const int bpl_b = bb <= 1 ? 1 : (bb <= 2 ? 2 : 4);
    if (int rc = grouped_try_ring(a, stream, who, stages); rc != 1) return rc;
#define DSV4_CASE(A, B) if (bpl_a == A && bpl_b == B) return grouped_launch<A, B>(a, stream, who, stages);
    DSV4_CASE(1, 1) DSV4_CASE(1, 2) DSV4_CASE(1, 4)
    DSV4_CASE(2, 1) DSV4_CASE(2, 2) DSV4_CASE(2, 4)
    DSV4_CASE(4, 1) DSV4_CASE(4, 2) DSV4_CASE(4, 4)
#undef DSV4_CASE
    return -3;
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
    if (K_in > 1024 * kMaxBlocksPerLane || hidden > 1024 * kMaxBlocksPerLane) {
        std::fprintf(stderr, "%s: K_in/hidden > %d\n", who, 1024 * kMaxBlocksPerLane);
        return -3;
    }
    if (out_dim <= 0) {
        std::fprintf(stderr, "%s: out_dim=%d\n", who, out_dim);
        return -8;
    }
    return 0;
}

// Workspace layout: [n_exp * hidden * 8 bytes: the intermediate - FP32 values for the two-kernel chain, 8-byte
// {value, tag} words for the single kernel][`extra` bytes of other per-call results][64 bytes: generation word].
static uint32_t* sync_area(void* workspace, int n_exp, int hidden, size_t extra) {
    return reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(workspace) +
                                       (size_t)n_exp * (size_t)hidden * 8 + extra);
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
    a.sync = sync_area(workspace, n_exp, hidden, 0);
    return grouped_forward(a, stream, who);
}

// Replaces kernel/mxfp4-routed/mxfp4_grouped_gemv.cu:406-409.  The intermediate is kept in FP32 here
// (n_exp * hidden * 4 bytes) and is followed by the readiness flags of the single-kernel path; callers size their
// buffer through this query, as the reference's callers do.
DSV4_API size_t mxfp4_grouped_workspace_bytes(int n_exp, int hidden, int out_dim) {
    (void)out_dim;
    if (n_exp <= 0 || hidden <= 0) return 0;
    return (size_t)n_exp * (size_t)hidden * 8 + kStreamSyncBytes;
}

// Additive: same computation, but the experts are picked from a resident bank by index, so the caller
// no longer gathers the selected experts into contiguous scratch first.  `topk_ids` is a DEVICE array of
// n_exp bank indices (1 <= n_exp <= 8); bank tensors are [n_bank, hidden, K_in/2] etc.
static int grouped_ids_impl(const char* who, int stages, const __nv_bfloat16* x, const uint8_t* bank_W1_packed,
                                         const uint8_t* bank_W3_packed, const uint8_t* bank_W2_packed,
                                         const uint8_t* bank_W1_scale, const uint8_t* bank_W3_scale,
                                         const uint8_t* bank_W2_scale, const int* topk_ids, const float* rweights,
                                         int K_in, int hidden, int out_dim, int n_exp, __nv_bfloat16* out,
                                         void* workspace, cudaStream_t stream) {
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
    a.sync = sync_area(workspace, n_exp, hidden, 0);
    return grouped_forward(a, stream, who, stages);
}

DSV4_API int mxfp4_grouped_gemv_topk_ids(const __nv_bfloat16* x, const uint8_t* bank_W1_packed,
                                         const uint8_t* bank_W3_packed, const uint8_t* bank_W2_packed,
                                         const uint8_t* bank_W1_scale, const uint8_t* bank_W3_scale,
                                         const uint8_t* bank_W2_scale, const int* topk_ids, const float* rweights,
                                         int K_in, int hidden, int out_dim, int n_exp, __nv_bfloat16* out,
                                         void* workspace, cudaStream_t stream) {
    return grouped_ids_impl("mxfp4_grouped_gemv_topk_ids", 3, x, bank_W1_packed, bank_W3_packed, bank_W2_packed,
                            bank_W1_scale, bank_W3_scale, bank_W2_scale, topk_ids, rweights, K_in, hidden, out_dim,
                            n_exp, out, workspace, stream);
}

// Additive (profiling): the same call restricted to one of its two kernels, so that each can be timed alone.
// stage_mask 1 = gate/up + SwiGLU only (fills the workspace), 2 = down + combine only (reads it), 3 = both.
DSV4_API int mxfp4_grouped_gemv_topk_ids_stages(const __nv_bfloat16* x, const uint8_t* bank_W1_packed,
                                                const uint8_t* bank_W3_packed, const uint8_t* bank_W2_packed,
                                                const uint8_t* bank_W1_scale, const uint8_t* bank_W3_scale,
                                                const uint8_t* bank_W2_scale, const int* topk_ids,
                                                const float* rweights, int K_in, int hidden, int out_dim, int n_exp,
                                                __nv_bfloat16* out, void* workspace, int stage_mask,
                                                cudaStream_t stream) {
    if (stage_mask < 1 || stage_mask > 3) return -9;
    return grouped_ids_impl("mxfp4_grouped_gemv_topk_ids_stages", stage_mask, x, bank_W1_packed, bank_W3_packed,
                            bank_W2_packed, bank_W1_scale, bank_W3_scale, bank_W2_scale, topk_ids, rweights, K_in,
                            hidden, out_dim, n_exp, out, workspace, stream);
}

// Additive: router scores + top-k + weights on the device (replaces the D2H copy, stream synchronise and
// host scan of kernel/cpp-engine-mxfp4/routed.cu:169-208).  logits [n_tokens, n_experts] FP32;
// score_func 0 = softmax renormalised over the top-k, 1 = sqrt-softplus with eps and scaling;
// ids_out int32 [n_tokens, k] in descending score order (ties: lowest index), w_out FP32 [n_tokens, k].
// Returns -1 for a bad shape (n_experts > 1024, k > 32 or k > n_experts), -2 null pointer, -3 launch failure.
DSV4_API int mxfp4_moe_route_topk(const float* logits, int n_tokens, int n_experts, int k, int score_func,
                                  float eps, float scaling, int* ids_out, float* w_out, cudaStream_t stream) {
    const char* who = "mxfp4_moe_route_topk";
    if (n_tokens < 0 || n_experts <= 0 || n_experts > 1024 || k <= 0 || k > 32 || k > n_experts ||
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
    RouteArgs r;
    r.logits = logits; r.n_experts = n_experts; r.k = k; r.score_func = score_func; r.eps = eps; r.scaling = scaling;
    r.ids_out = ids_out; r.w_out = w_out;
    const dim3 grid((n_tokens + warps - 1) / warps), block(32 * warps);
    cudaError_t err = n_experts <= 256 ? launch(route_topk_kernel<8>, grid, block, stream, pdl_enabled(), r, n_tokens)
                                       : launch(route_topk_kernel<32>, grid, block, stream, pdl_enabled(), r, n_tokens);
    if (err != cudaSuccess) {
        std::fprintf(stderr, "%s: launch failed: %s\n", who, cudaGetErrorString(err));
        return -3;
    }
    return 0;
}

// Additive: one decode layer for one token in a single call: router (scores, top-k, weights) + routed-expert FFN
// over a resident bank.  logits FP32 [n_experts]; score_func / eps / scaling as in mxfp4_moe_route_topk; k experts
// per token (1..6 on the fused path, 1..8 otherwise).  At the shapes served by the shared-memory ring kernels
// (K_in in {1024, 2048, 4096}, hidden in {1024, 2048}, n_experts <= 256, k <= 6) the router runs inside the first
// kernel; otherwise a router kernel is launched first.  The picks and their weights are left in the workspace
// (see mxfp4_moe_decode_workspace_bytes) where the caller may read them after the call: int32 ids at byte offset
// k * hidden * 8, FP32 weights 32 bytes further.
DSV4_API size_t mxfp4_moe_decode_workspace_bytes(int k, int hidden, int out_dim) {
    (void)out_dim;
    if (k <= 0 || hidden <= 0) return 0;
    return (size_t)k * (size_t)hidden * 8 + 64 + kStreamSyncBytes;
}

DSV4_API int mxfp4_moe_decode_layer(const __nv_bfloat16* x, const uint8_t* bank_W1_packed,
                                    const uint8_t* bank_W3_packed, const uint8_t* bank_W2_packed,
                                    const uint8_t* bank_W1_scale, const uint8_t* bank_W3_scale,
                                    const uint8_t* bank_W2_scale, const float* logits, int n_experts, int score_func,
                                    float eps, float scaling, int K_in, int hidden, int out_dim, int k,
                                    __nv_bfloat16* out, void* workspace, cudaStream_t stream) {
    const char* who = "mxfp4_moe_decode_layer";
    if (int rc = check_shape(who, K_in, hidden, out_dim)) return rc;
    if (k < 1 || k > kMaxExperts || k > n_experts || n_experts > 1024 || (score_func != 0 && score_func != 1)) {
        std::fprintf(stderr, "%s: bad routing shape experts=%d k=%d score_func=%d\n", who, n_experts, k, score_func);
        return -4;
    }
    if (!x || !bank_W1_packed || !bank_W3_packed || !bank_W2_packed || !bank_W1_scale || !bank_W3_scale ||
        !bank_W2_scale || !logits || !out || !workspace || !aligned16(x) || !aligned16(bank_W1_packed) ||
        !aligned16(bank_W3_packed) || !aligned16(bank_W2_packed) || !aligned16(workspace)) {
        std::fprintf(stderr, "%s: null pointer, or x / packed weights / workspace not 16-byte aligned\n", who);
        return -8;
    }
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    RouteArgs rt;
    rt.logits = logits; rt.n_experts = n_experts; rt.k = k; rt.score_func = score_func; rt.eps = eps;
    rt.scaling = scaling;
    rt.ids_out = reinterpret_cast<int*>(ws + (size_t)k * hidden * 8);
    rt.w_out = reinterpret_cast<float*>(ws + (size_t)k * hidden * 8 + 32);
    GroupedArgs a;
    a.x = x; a.w1p = bank_W1_packed; a.w3p = bank_W3_packed; a.w2p = bank_W2_packed;
    a.w1s = bank_W1_scale; a.w3s = bank_W3_scale; a.w2s = bank_W2_scale;
    a.K = K_in; a.H = hidden; a.O = out_dim; a.E = k;
    a.strideAp = (long long)hidden * (K_in / 2); a.strideAs = (long long)hidden * (K_in / 32);
    a.strideBp = (long long)out_dim * (hidden / 2); a.strideBs = (long long)out_dim * (hidden / 32);
    a.mid = reinterpret_cast<float*>(workspace);
    a.out = out;
    a.sync = sync_area(workspace, k, hidden, 64);
    if (n_experts <= 256) {
        a.r = nullptr; a.ids = nullptr;                  // both come from the fused router
        if (int rc = grouped_try_ring(a, stream, who, 3, rt); rc != 1) return rc;
    }
    if (int rc = mxfp4_moe_route_topk(logits, 1, n_experts, k, score_func, eps, scaling, rt.ids_out, rt.w_out, stream))
        return rc;
    a.r = rt.w_out; a.ids = rt.ids_out;
    return grouped_forward(a, stream, who);
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

// Added (diagnostic): 0 unless a kernel of this library gave up on a bounded wait since the last call
// (1 = a gate/up row or its scales never landed, 2 = a down row or its scales, 3 = an expert's intermediate never
// became complete); the status is cleared by the call.  Synchronises the device.
DSV4_API int dsv4_b200_device_status(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) return -1;
    // (nothing else to re-arm: what the single-kernel path waits on lives in the caller's workspace and is
    // re-tagged by every launch)
    if (v != 0) cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    return v;
}

// Added (no counterpart): how the single-kernel path is launched from now on in this process.
// 0 = two chained kernels, 1 = cooperative launch, 2 = automatic (first stream of a device programmatic, the others
// cooperative; the default), 3 = programmatic stream serialisation for every stream; see fused_mode().
// Returns the previous mode, or -1 for a value outside 0..3 (nothing changes).
DSV4_API int dsv4_b200_set_launch_mode(int mode) {
    const int before = fused_mode();
    if (mode < 0 || mode > 3) return -1;
    g_fused_mode = mode;
    return before;
}

// Added (test hook, no counterpart): poll budget of the device-side waits of the single-kernel path, and a number of
// producers that never arrive.  With phantom_ctas > 0 the next calls wait for readiness flags nobody publishes, give
// up after `polls` polls (microseconds for a few thousand), record status 3 and write NaN - without a fault, a
// trap or an unbounded loop.  (0, 0) restores the defaults.  Returns -1 for negative arguments.
DSV4_API int dsv4_b200_test_wait_limits(long long polls, int phantom_ctas) {
    if (polls < 0 || phantom_ctas < 0 || phantom_ctas > 64) return -1;
    g_spin_limit = polls == 0 ? kSpinLimit : (unsigned)(polls > 0xffffffffLL ? 0xffffffffLL : polls);
    g_phantom = phantom_ctas;
    return 0;
}

// ------------------------------------------------------------------------------------------------
// Entry point that needs no workspace from the caller
// ------------------------------------------------------------------------------------------------
// Some hosts cannot hand this library a scratch buffer at call time: an engine that gave all free HBM to its
// expert bank and KV cache at start-up has nothing left to carve a workspace from, and a decode thread must not
// enter cudaMalloc because that call synchronises the whole device.  For them the SwiGLU intermediate lives in
// this fixed array inside the library image.  Every GPU that loads the library carries these 192 KB until the
// process exits.
constexpr int kStaticMaxExperts = 6;
constexpr int kStaticMaxHidden = 4096;
static __device__ __align__(256) unsigned char
    g_static_scratch[kStaticMaxExperts * kStaticMaxHidden * 8 + kStreamSyncBytes];

// Device address of g_static_scratch on the current device, or nullptr (with a message) if the runtime refuses.
// In host code the array's name is only a handle for the runtime, not an address a kernel could use, so the
// address is asked for once per device, with that device current, and remembered.
static void* static_scratch_address() {
    static void* cached[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        std::fprintf(stderr, "mxfp4_grouped_gemv_topk_static: cannot identify the current device\n");
        return nullptr;
    }
    void* p = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
    if (p != nullptr) return p;
    const cudaError_t err = cudaGetSymbolAddress(&p, g_static_scratch);
    if (err != cudaSuccess || p == nullptr) {
        std::fprintf(stderr, "mxfp4_grouped_gemv_topk_static: cudaGetSymbolAddress failed: %s\n",
                     cudaGetErrorString(err));
        return nullptr;
    }
    __atomic_store_n(&cached[dev], p, __ATOMIC_RELEASE);
    return p;
}

// The routed-expert FFN of mxfp4_grouped_gemv_topk without the workspace argument: same inputs, same output,
// same kernels, bit-identical result.  It allocates nothing and frees nothing.
//   * Limits: n_exp == 6 (as the workspace entry), hidden <= 4096; a larger hidden returns -10 with a message.
//   * The first call on each device looks up the array's device address (one cudaGetSymbolAddress); make that
//     first call before any stream capture begins on that device.
//   * All calls on a device share the one array.  Nothing in it has to be zero beforehand (the first kernel
//     overwrites every element the second one reads), but two calls whose kernels overlap on the GPU - different
//     streams, or the same stream from two threads without ordering - race on it and corrupt each other's
//     intermediate.  Serialise such calls, or use mxfp4_grouped_gemv_topk with one workspace per stream.
//   * Other return codes as mxfp4_grouped_gemv_topk; -11 if the array's address cannot be obtained.
DSV4_API int mxfp4_grouped_gemv_topk_static(const __nv_bfloat16* x, const uint8_t* W1_packed,
                                            const uint8_t* W3_packed, const uint8_t* W2_packed,
                                            const uint8_t* W1_scale, const uint8_t* W3_scale,
                                            const uint8_t* W2_scale, const float* rweights, int K_in, int hidden,
                                            int out_dim, int n_exp, __nv_bfloat16* out, cudaStream_t stream) {
    const char* who = "mxfp4_grouped_gemv_topk_static";
    // beyond what the built-in array holds: -10; a supported size but not the six experts of the workspace entry: -4
    if (hidden > kStaticMaxHidden || n_exp > kStaticMaxExperts) {
        std::fprintf(stderr, "%s: n_exp=%d hidden=%d exceed the built-in scratch (%d experts x %d)\n", who, n_exp,
                     hidden, kStaticMaxExperts, kStaticMaxHidden);
        return -10;
    }
    if (int rc = check_shape(who, K_in, hidden, out_dim)) return rc;
    if (n_exp != 6) {
        std::fprintf(stderr, "%s: n_exp=%d != 6\n", who, n_exp);
        return -4;
    }
    if (!x || !W1_packed || !W3_packed || !W2_packed || !W1_scale || !W3_scale || !W2_scale || !rweights || !out ||
        !aligned16(x) || !aligned16(W1_packed) || !aligned16(W3_packed) || !aligned16(W2_packed)) {
        std::fprintf(stderr, "%s: null pointer, or x / packed weights not 16-byte aligned\n", who);
        return -8;
    }
    void* scratch = static_scratch_address();
    if (scratch == nullptr) return -11;
    GroupedArgs a;
    a.x = x; a.w1p = W1_packed; a.w3p = W3_packed; a.w2p = W2_packed;
    a.w1s = W1_scale; a.w3s = W3_scale; a.w2s = W2_scale; a.r = rweights; a.ids = nullptr;
    a.K = K_in; a.H = hidden; a.O = out_dim; a.E = n_exp;
    a.strideAp = (long long)hidden * (K_in / 2); a.strideAs = (long long)hidden * (K_in / 32);
    a.strideBp = (long long)out_dim * (hidden / 2); a.strideBs = (long long)out_dim * (hidden / 32);
    a.mid = reinterpret_cast<float*>(scratch);
    a.out = out;
    a.sync = sync_area(scratch, n_exp, hidden, 0);
    return grouped_forward(a, stream, who);
}
