// Routed-expert decode kernels specialised for reduction lengths known at compile time (multiples of 1024),
// with the weights streamed through per-warp shared-memory rings (stream_ring.cuh).  This is the path the
// DSv4 shape (K_in 4096, hidden 2048) takes; every address inside the loops is a register plus an immediate.
//
// gate/up : 16 warps per CTA; warp w owns pairs q_begin + w, q_begin + w + 16, ... of the CTA's contiguous
//           range; a ring slot holds the W1 row, the W3 row and their two scale rows of one pair.
// down    : 2 warps per expert; warp (e, half) owns every second chunk of R output rows; a slot holds R
//           weight rows and R scale rows of one expert (contiguous in memory, so two copies per slot).
// The activation vector (x, or the SwiGLU intermediate of each expert) is converted once per CTA to fp16 with
// one power-of-two scale, parked in shared memory, and each lane keeps its blocks of it in registers.
#pragma once

#include "grouped_args.cuh"
#include "router.cuh"
#include "stream_ring.cuh"

namespace dsv4 {

constexpr int kRingGateWarps = 16;
constexpr int kRingGateStages = 3;
constexpr int kRingDownStages = 7;
constexpr int kRingDownRows = 2;
constexpr int kRingDownCap = 64;       // output rows per CTA
constexpr int kRingMaxExperts = 6;     // 2 warps per expert

#ifdef DSV4_FP32_ACCUM
// Comparison build (-DDSV4_FP32_ACCUM): 32 E2M1 weights times 32 activations with every product and every sum in
// FP32, the arithmetic of the kernels this library replaces (kernel/mxfp4-routed/mxfp4_grouped_gemv.cu:87-107 of
// the reference: fmaf over the 32 elements of a block, then the block scale).  About three times the instructions
// of the fp16 form below; the benchmark times it beside the product.
__device__ __forceinline__ float fp4_block_dot(const uint4& w, const __half2 (&x)[16]) {
    const uint32_t word[4] = {w.x, w.y, w.z, w.w};
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h[4];
        e2m1x8_to_h2x4(word[i], h);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 wf = __half22float2(h[j]);
            const float2 xf = __half22float2(x[4 * i + j]);
            acc = fmaf(wf.x, xf.x, acc);
            acc = fmaf(wf.y, xf.y, acc);
        }
    }
    return acc;
}
#else
// 32 E2M1 weights (16 bytes) times 32 activations: fp16 products (exact: an E2M1 value times a bf16-precision
// activation fits fp16's 11 significant bits) summed 16 at a time in two fp16x2 chains, then FP32.
__device__ __forceinline__ float fp4_block_dot(const uint4& w, const __half2 (&x)[16]) {
    const uint32_t word[4] = {w.x, w.y, w.z, w.w};
    __half2 acc0, acc1;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h[4];
        e2m1x8_to_h2x4(word[i], h);
        if (i == 0) {
            acc0 = __hmul2(h[0], x[0]);
            acc1 = __hmul2(h[1], x[1]);
        } else {
            acc0 = __hfma2(h[0], x[4 * i + 0], acc0);
            acc1 = __hfma2(h[1], x[4 * i + 1], acc1);
        }
        acc0 = __hfma2(h[2], x[4 * i + 2], acc0);
        acc1 = __hfma2(h[3], x[4 * i + 3], acc1);
    }
    const float2 f = __half22float2(__hadd2(acc0, acc1));
    return f.x + f.y;
}
#endif

// Largest magnitude (as float bits) of 8 consecutive values.
__device__ __forceinline__ uint32_t amax_bits8(const float (&v)[8]) {
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = max(m, __float_as_uint(v[i]) & 0x7fffffffu);
    return m;
}

// Power-of-two scale that maps a largest magnitude into [128, 256); returns the scale, sets its inverse.
__device__ __forceinline__ float fp16_scale_for(uint32_t amax_bits, float& inv) {
    int e = (int)(amax_bits >> 23) - Fp4Format::kActExp;
    e = min(max(e, 1), 253);
    inv = __uint_as_float((uint32_t)(254 - e) << 23);
    return __uint_as_float((uint32_t)e << 23);
}

// The fp16 copy of an activation vector in shared memory is stored in 16-byte chunks of 8 values; chunk c of
// 32-value block b sits at chunk slot (c + (b >> 1)) & 3 of the block, so that the eight lanes of a quarter
// warp, which read the same chunk of eight consecutive blocks, hit eight different bank groups.
__device__ __forceinline__ int swizzled_chunk(int idx8) {          // idx8: index of an 8-value chunk
    const int b = idx8 >> 2, c = idx8 & 3;
    return (b << 2) | ((c + (b >> 1)) & 3);
}

__device__ __forceinline__ void store8_as_half(__half* vec, int idx8, const float (&v)[8], float inv) {
    __half2 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i] * inv, v[2 * i + 1] * inv);
    reinterpret_cast<uint4*>(vec)[swizzled_chunk(idx8)] = *reinterpret_cast<const uint4*>(h);
}

// Lane's blocks (lane + 32 j) of an fp16 vector in shared memory -> registers.
template <int BPL>
__device__ __forceinline__ void lane_blocks_from_smem(const __half* vec, int lane, __half2 (&x)[BPL][16]) {
#pragma unroll
    for (int j = 0; j < BPL; ++j) {
        const uint4* src = reinterpret_cast<const uint4*>(vec);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint4 q = src[swizzled_chunk((lane + 32 * j) * 4 + c)];
            x[j][4 * c + 0] = *reinterpret_cast<const __half2*>(&q.x);
            x[j][4 * c + 1] = *reinterpret_cast<const __half2*>(&q.y);
            x[j][4 * c + 2] = *reinterpret_cast<const __half2*>(&q.z);
            x[j][4 * c + 3] = *reinterpret_cast<const __half2*>(&q.w);
        }
    }
}

// ------------------------------------------------------------------------------------------------ gate / up

template <int KT>
struct GateRingLayout {
    static constexpr int kBPL = KT / 1024;
    static constexpr uint32_t kRowP = KT / 2, kRowS = KT / 32;
    static constexpr uint32_t kSlot = 2 * (kRowP + kRowS);
    static constexpr uint32_t kRing = kRingGateWarps * kRingGateStages * kSlot;
    static constexpr uint32_t kVec = kRing;                          // fp16 x, KT halves
    static constexpr uint32_t kBars = kVec + KT * 2;
    static constexpr uint32_t kRed = kBars + kRingGateWarps * kRingGateStages * 8;
    static constexpr uint32_t kBytes = kRed + 32 * 4;
};

template <int KT>
__global__ void __launch_bounds__(kRingGateWarps * 32, 1) gate_up_ring_kernel(const GroupedArgs a, int h_shift,
                                                                              const RouteArgs rt) {
    using L = GateRingLayout<KT>;
    constexpr int BPL = L::kBPL;
    constexpr int S = kRingGateStages;
    constexpr int NW = kRingGateWarps;
    extern __shared__ __align__(128) uint8_t ring_smem[];
    __shared__ int expert_of_slot[8];            // bank index of expert slot e when a table is in use
    pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const bool use_table = a.ids != nullptr || rt.logits != nullptr;
    const uint32_t smem0 = smem_u32(ring_smem);
    const uint32_t ring = smem0 + warp * S * L::kSlot;
    const uint32_t bars = smem0 + L::kBars + warp * S * 8;
    __half* xh = reinterpret_cast<__half*>(ring_smem + L::kVec);
    uint32_t* red = reinterpret_cast<uint32_t*>(ring_smem + L::kRed);

    const long long total = (long long)a.E << h_shift;
    const int q_begin = (int)(total * blockIdx.x / gridDim.x);
    const int q_end = (int)(total * (blockIdx.x + 1) / gridDim.x);
    const int q0 = q_begin + warp;                                   // pair i of this warp is q0 + i * NW
    const int n_i = q0 < q_end ? (q_end - q0 + NW - 1) / NW : 0;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s) mbar_init(bars + 8 * s, 1);
    }
    mbar_init_fence();
    __syncwarp();

    // lanes 0..3 copy the W1 row, the W3 row, the W1 scales and the W3 scales of pair q into slot s
    auto issue = [&](int q, int s) {
        if (lane < 4) {
            const int e = q >> h_shift;
            const int h = q - (e << h_shift);
            const long long eid = use_table ? (long long)expert_of_slot[e] : (long long)e;
            const bool third = (lane & 1) != 0, scale = lane >= 2;
            const uint8_t* base = scale ? (third ? a.w3s : a.w1s) : (third ? a.w3p : a.w1p);
            const uint32_t bytes = scale ? L::kRowS : L::kRowP;
            const uint8_t* src = base + eid * (scale ? a.strideAs : a.strideAp) + (long long)h * bytes;
            const uint32_t dst = ring + s * L::kSlot + (scale ? 2 * L::kRowP : 0) + (third ? bytes : 0);
            const uint32_t bar = bars + 8 * s;
            if (lane == 0) mbar_arrive_expect_tx(bar, L::kSlot);
            bulk_copy_g2s(dst, src, bytes, bar);
        }
    };
    auto prologue = [&]() {
#pragma unroll
        for (int s = 0; s < S; ++s)
            if (s < n_i) issue(q0 + s * NW, s);
    };

    // stacked weights do not depend on the previous kernel in the stream: request them before waiting for it
    if (!use_table) prologue();
    pdl_wait();
    if (use_table) {
        if (rt.logits != nullptr) {
            // fused router: warp 0 of every CTA picks the experts (same result everywhere); CTA 0 publishes
            // the picks and their weights for the down kernel and the caller
            if (warp == 0) {
                int id;
                float w;
                route_token<8>(rt.logits, rt.n_experts, rt.k, rt.score_func, rt.eps, rt.scaling, lane, id, w);
                if (lane < rt.k) {
                    expert_of_slot[lane] = id;
                    if (blockIdx.x == 0) { rt.ids_out[lane] = id; rt.w_out[lane] = w; }
                }
            }
        } else if (threadIdx.x < a.E) {
            expert_of_slot[threadIdx.x] = a.ids[threadIdx.x];
        }
        __syncthreads();
        prologue();
    }

    // x -> fp16 with one scale, once per CTA
    float xs;
    {
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const bool mine = threadIdx.x * 8 < KT;                      // 512 threads x 8 covers KT <= 4096
        if (mine) load8_as_float(a.x + threadIdx.x * 8, v);
        uint32_t m = amax_bits8(v);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = max(m, __shfl_xor_sync(kFullMask, m, off));
        if (lane == 0) red[warp] = m;
        __syncthreads();
        m = 0;
#pragma unroll
        for (int w = 0; w < NW; ++w) m = max(m, red[w]);
        float inv;
        xs = fp16_scale_for(m, inv);
        if (mine) store8_as_half(xh, threadIdx.x, v, inv);
        __syncthreads();
    }
    __half2 x[BPL][16];
    lane_blocks_from_smem<BPL>(xh, lane, x);

    const uint32_t lane_w = ring + lane * 16;
    const uint32_t lane_s = ring + 2 * L::kRowP + lane;
    uint32_t parity = 0;
    bool alive = true;
    for (int i0 = 0; i0 < n_i; i0 += S, parity ^= 1) {
#pragma unroll
        for (int s = 0; s < S; ++s) {
            const int i = i0 + s;
            if (i < n_i && alive) {
                alive = mbar_wait_bounded(bars + 8 * s, parity, 1);
                float v[2] = {0.f, 0.f};
#pragma unroll
                for (int j = 0; j < BPL; ++j) {
                    const uint4 wg = lds_v4(lane_w + s * L::kSlot + 512 * j);
                    const uint4 wu = lds_v4(lane_w + s * L::kSlot + L::kRowP + 512 * j);
                    const float sg = e8m0_to_float_fast(lds_u8(lane_s + s * L::kSlot + 32 * j));
                    const float su = e8m0_to_float_fast(lds_u8(lane_s + s * L::kSlot + L::kRowS + 32 * j));
                    v[0] = fmaf(fp4_block_dot(wg, x[j]), sg, v[0]);
                    v[1] = fmaf(fp4_block_dot(wu, x[j]), su, v[1]);
                }
                multi_reduce<2>(v, lane);                            // lane 0: gate sum, lane 16: up sum
                const float up = __shfl_sync(kFullMask, v[0], 16) * xs;
                if (lane == 0 && alive) {
                    const float g = v[0] * xs;
                    a.mid[q0 + i * NW] = swiglu_f32(g, up);
                }
                __syncwarp();                                        // every lane has read the slot
                if (i + S < n_i && alive) issue(q0 + (i + S) * NW, s);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ down

template <int HT>
struct DownRingLayout {
    static constexpr int kBPL = HT / 1024;
    static constexpr uint32_t kRowP = HT / 2, kRowS = HT / 32;
    static constexpr uint32_t kSlot = kRingDownRows * (kRowP + kRowS);
    static constexpr uint32_t kRing = 2 * kRingMaxExperts * kRingDownStages * kSlot;
    static constexpr uint32_t kVec = kRing;                          // fp16 intermediates, experts x HT halves
    static constexpr uint32_t kBars = kVec + kRingMaxExperts * HT * 2;
    static constexpr uint32_t kRed = kBars + 2 * kRingMaxExperts * kRingDownStages * 8;
    static constexpr uint32_t kPart = kRed + 32 * 4;                 // [rows][experts] FP32
    static constexpr uint32_t kBytes = kPart + kRingDownCap * 8 * 4;
};

template <int HT>
__global__ void __launch_bounds__(2 * kRingMaxExperts * 32, 1) down_ring_kernel(const GroupedArgs a) {
    using L = DownRingLayout<HT>;
    constexpr int BPL = L::kBPL;
    constexpr int S = kRingDownStages;
    constexpr int R = kRingDownRows;
    extern __shared__ __align__(128) uint8_t ring_smem[];
    pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;               // blockDim.x == 64 * E
    const int e = warp >> 1;
    const int half = warp & 1;
    const uint32_t smem0 = smem_u32(ring_smem);
    const uint32_t ring = smem0 + warp * S * L::kSlot;
    const uint32_t bars = smem0 + L::kBars + warp * S * 8;
    __half* mh = reinterpret_cast<__half*>(ring_smem + L::kVec);
    uint32_t* red = reinterpret_cast<uint32_t*>(ring_smem + L::kRed);
    float (*part)[8] = reinterpret_cast<float (*)[8]>(ring_smem + L::kPart);

    const int o_begin = (int)((long long)a.O * blockIdx.x / gridDim.x);
    const int o_end = (int)((long long)a.O * (blockIdx.x + 1) / gridDim.x);
    const int n_local = o_end - o_begin;
    const int n_chunks = (n_local + R - 1) / R;
    const int n_i = half < n_chunks ? (n_chunks - half + 1) / 2 : 0;   // chunk i of this warp is half + 2 i

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s) mbar_init(bars + 8 * s, 1);
    }
    mbar_init_fence();
    __syncwarp();

    long long eid = e;
    // lane 0 copies the chunk's weight rows (contiguous in memory), lane 1 its scale rows
    auto issue = [&](int c, int s) {
        if (lane < 2) {
            const int l0 = c * R;
            const uint32_t rows = (uint32_t)min(R, n_local - l0);
            const bool scale = lane == 1;
            const uint32_t rb = scale ? L::kRowS : L::kRowP;
            const uint8_t* src = (scale ? a.w2s + eid * a.strideBs : a.w2p + eid * a.strideBp) +
                                 (long long)(o_begin + l0) * rb;
            const uint32_t dst = ring + s * L::kSlot + (scale ? R * L::kRowP : 0);
            const uint32_t bar = bars + 8 * s;
            if (lane == 0) mbar_arrive_expect_tx(bar, rows * (L::kRowP + L::kRowS));
            bulk_copy_g2s(dst, src, rows * rb, bar);
        }
    };
    auto prologue = [&]() {
#pragma unroll
        for (int s = 0; s < S; ++s)
            if (s < n_i) issue(half + 2 * s, s);
    };

    if (a.ids == nullptr) prologue();
    pdl_wait();
    if (a.ids != nullptr) { eid = a.ids[e]; prologue(); }

    // SwiGLU intermediate of this warp's expert -> fp16 with one scale per expert; the expert's two warps
    // convert half of it each
    float ms = 1.f;
    {
        // the expert's two warps (64 lanes) read the vector in coalesced 32-byte pieces: piece p of a lane covers
        // values 8 * (p * 64 + half * 32 + lane) ..., kept in registers between the two steps
        constexpr int kPieces = HT / 512;
        const float* src = a.mid + (size_t)e * HT;
        float v[kPieces][8];
        uint32_t m = 0;
#pragma unroll
        for (int p = 0; p < kPieces; ++p) {
            load8_as_float(src + 8 * (p * 64 + half * 32 + lane), v[p]);
            m = max(m, amax_bits8(v[p]));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = max(m, __shfl_xor_sync(kFullMask, m, off));
        if (lane == 0) red[warp] = m;
        __syncthreads();
        m = max(red[2 * e], red[2 * e + 1]);
        float inv;
        ms = fp16_scale_for(m, inv);
#pragma unroll
        for (int p = 0; p < kPieces; ++p) store8_as_half(mh + (size_t)e * HT, p * 64 + half * 32 + lane, v[p], inv);
        __syncthreads();
    }
    __half2 m2[BPL][16];
    lane_blocks_from_smem<BPL>(mh + (size_t)e * HT, lane, m2);

    const uint32_t lane_w = ring + lane * 16;
    const uint32_t lane_s = ring + R * L::kRowP + lane;
    uint32_t parity = 0;
    bool alive = true;
    for (int i0 = 0; i0 < n_i; i0 += S, parity ^= 1) {
#pragma unroll
        for (int s = 0; s < S; ++s) {
            const int i = i0 + s;
            if (i < n_i && alive) {
                alive = mbar_wait_bounded(bars + 8 * s, parity, 2);
                const int l0 = (half + 2 * i) * R;
                float v[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    v[r] = 0.f;
#pragma unroll
                    for (int j = 0; j < BPL; ++j) {
                        const uint4 w = lds_v4(lane_w + s * L::kSlot + r * L::kRowP + 512 * j);
                        const float sc = e8m0_to_float_fast(lds_u8(lane_s + s * L::kSlot + r * L::kRowS + 32 * j));
                        v[r] = fmaf(fp4_block_dot(w, m2[j]), sc, v[r]);
                    }
                }
                multi_reduce<R>(v, lane);
                if (multi_reduce_owner<R>(lane) && alive) {
                    const int l = l0 + multi_reduce_index<R>(lane);
                    if (l < n_local) part[l][e] = v[0] * ms;        // rows past the chunk's end hold stale bytes
                }
                __syncwarp();                                        // every lane has read the slot
                if (i + S < n_i && alive) issue(half + 2 * (i + S), s);
            }
        }
    }
    __syncthreads();

    for (int t = threadIdx.x; t < n_local; t += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < a.E; ++k) acc = fmaf(__ldcg(a.r + k), part[t][k], acc);
        a.out[o_begin + t] = __float2bfloat16(acc);
    }
}

}  // namespace dsv4
