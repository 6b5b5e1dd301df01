// One persistent kernel for the whole routed-expert decode layer of one token:
//   router (optional)  ->  gate/up + SwiGLU  ->  grid barrier  ->  down + router-weighted combine.
// It replaces the two chained kernels of grouped_ring.cuh at the same shapes; what it saves is the second launch,
// the drain between the kernels and the second set-up: while a CTA waits at the grid barrier for the other CTAs'
// SwiGLU rows, its copies of the first W2 rows are already in flight.
//
// Launched with one CTA per SM, either cooperatively (the runtime guarantees that all CTAs are resident, which is
// what makes a grid barrier legal) or with programmatic stream serialisation (the next layer's CTAs start as this
// layer's exit; legal as long as no second grid of this kernel is in flight on the device).  The barrier is a
// bounded sense-reversing one, split into arrive and wait.
//
// 16 warps per CTA.  Each warp owns a private 8.5 KB ring: two slots of one (W1 row, W3 row, 2 scale rows) pair in
// the first phase, two slots of four (W2 row, scale row) in the second (4 352 bytes per slot in both: the fixed
// cost of a task - wait, butterfly reduction, refill - is paid once per 4 KB of weights).  The second phase splits
// the CTA's (expert, output row) units evenly over the warps; a warp walks its range in tasks of up to four rows of
// one expert and reloads its blocks of the expert's fp16 intermediate from shared memory only when it crosses into
// another expert.
#pragma once

#include "grouped_ring.cuh"

namespace dsv4 {

constexpr int kFusedWarps = 16;
constexpr int kFusedStagesA = 2;
constexpr int kFusedRowsB = 4;
constexpr int kFusedCap = 64;          // output rows per CTA

// Grid barrier of the fused kernel.  Every warp arrives on its own with a fire-and-forget release increment of a counter that only grows;
// one lane per CTA waits until the counter has moved `arrivals` past the base it had when the grid started.  The
// base is kept in device memory and advanced by the last CTA to leave the kernel, off the critical path (the next
// grid reads it only after this one has completed).  Critical chain: the last warp's release increment, then one
// poll - no reset and no generation word in between.
// All CTAs of the grid must become resident without waiting for this grid to finish: one CTA per SM, and no other
// grid of this kernel in flight on the device (the cooperative launch guarantees it; the programmatic launch relies
// on the caller).  Bounded: a CTA that gives up records status 3 and carries on (its results are then garbage, the
// status says so; dsv4_b200_device_status() then also resets the three words).
__device__ unsigned int g_fused_count = 0;       // arrivals, monotonic
__device__ unsigned int g_fused_base = 0;        // value of g_fused_count before the grid in flight
__device__ unsigned int g_fused_exits = 0;       // CTAs of the grid in flight that have left

// The lane of a warp that made the warp's global writes: the release orders them before the increment.
__device__ __forceinline__ void fused_barrier_arrive() {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(&g_fused_count) : "memory");
}

// One lane per CTA; `base` was read from g_fused_base at the start of the kernel.
__device__ __forceinline__ bool fused_barrier_wait(unsigned int base, unsigned int arrivals) {
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        unsigned int now;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(now) : "l"(&g_fused_count) : "memory");
        if (now - base >= arrivals) return true;
        if (it > 256) __nanosleep(32);
    }
    atomicExch(&g_device_status, 3);
    return false;
}

// One thread per CTA at the end of the kernel: the last CTA to leave moves the base past this grid's arrivals.
__device__ __forceinline__ void fused_barrier_leave(unsigned int base, unsigned int arrivals) {
    if (atomicAdd(&g_fused_exits, 1u) == gridDim.x - 1) {
        g_fused_exits = 0;
        g_fused_base = base + arrivals;
    }
}

template <int KT, int HT>
struct FusedLayout {
    static constexpr int kBplA = KT / 1024, kBplB = HT / 1024;
    static constexpr uint32_t kRowPA = KT / 2, kRowSA = KT / 32, kSlotA = 2 * (kRowPA + kRowSA);
    static constexpr uint32_t kRowPB = HT / 2, kRowSB = HT / 32, kSlotB = kFusedRowsB * (kRowPB + kRowSB);
    static constexpr uint32_t kRingPerWarp = (kFusedStagesA * kSlotA > 2 * kSlotB) ? kFusedStagesA * kSlotA : 2 * kSlotB;
    static constexpr int kStagesA = (kRingPerWarp / kSlotA > 4) ? 4 : kRingPerWarp / kSlotA;
    static constexpr int kStagesB = (kRingPerWarp / kSlotB > 6) ? 6 : kRingPerWarp / kSlotB;
    static constexpr uint32_t kRing = kFusedWarps * kRingPerWarp;
    static constexpr uint32_t kVecBytes = (KT * 2 > kRingMaxExperts * HT * 2) ? KT * 2 : kRingMaxExperts * HT * 2;
    static constexpr uint32_t kVec = kRing;                              // fp16 x, later the fp16 intermediates
    static constexpr uint32_t kBars = kVec + kVecBytes;                  // per warp: kStagesA + kStagesB barriers
    static constexpr uint32_t kBarsPerWarp = kStagesA + kStagesB;
    static constexpr uint32_t kRed = kBars + kFusedWarps * kBarsPerWarp * 8;
    static constexpr uint32_t kPart = kRed + 64 * 4;                     // [rows][8] FP32
    static constexpr uint32_t kBytes = kPart + kFusedCap * 8 * 4;
    static_assert(kStagesA >= 2 && kStagesB >= 2, "ring too small");
};

template <int KT, int HT>
__global__ void __launch_bounds__(kFusedWarps * 32, 1) moe_decode_fused_kernel(const GroupedArgs a, int h_shift,
                                                                               const RouteArgs rt) {
    using L = FusedLayout<KT, HT>;
    constexpr int NW = kFusedWarps;
    constexpr int SA = L::kStagesA, SB = L::kStagesB, R = kFusedRowsB;
    extern __shared__ __align__(128) uint8_t ring_smem[];
    __shared__ int expert_of_slot[8];
    __shared__ float weight_of_slot[8];
    __shared__ float mid_scale[8];
    __shared__ int next_pair;                     // work queue of the first phase
    pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const bool routed = rt.logits != nullptr;
    const bool use_table = a.ids != nullptr || routed;
    const uint32_t smem0 = smem_u32(ring_smem);
    const uint32_t ring = smem0 + warp * L::kRingPerWarp;
    const uint32_t bars_a = smem0 + L::kBars + warp * L::kBarsPerWarp * 8;
    const uint32_t bars_b = bars_a + SA * 8;
    __half* vec = reinterpret_cast<__half*>(ring_smem + L::kVec);
    uint32_t* red = reinterpret_cast<uint32_t*>(ring_smem + L::kRed);
    float (*part)[8] = reinterpret_cast<float (*)[8]>(ring_smem + L::kPart);

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < SA + SB; ++s) mbar_init(bars_a + 8 * s, 1);
    }
    mbar_init_fence();
    __syncwarp();

    // ------------------------------------------------------------------ phase A: gate / up + SwiGLU
    const long long total = (long long)a.E << h_shift;
    const int q_begin = (int)(total * blockIdx.x / gridDim.x);
    const int q_end = (int)(total * (blockIdx.x + 1) / gridDim.x);
    if (threadIdx.x == 0) next_pair = q_begin;
    // work is handed out from a shared counter at the moment a ring slot is (re)filled, so that the warps of a
    // CTA finish together
    auto claim = [&](int* counter) -> int {
        int v = 0;
        if (lane == 0) v = atomicAdd(counter, 1);
        return __shfl_sync(kFullMask, v, 0);
    };

    auto issue_a = [&](int q, int s) {
        if (lane < 4) {
            const int e = q >> h_shift;
            const int h = q - (e << h_shift);
            const long long eid = use_table ? (long long)expert_of_slot[e] : (long long)e;
            const bool third = (lane & 1) != 0, scale = lane >= 2;
            const uint8_t* base = scale ? (third ? a.w3s : a.w1s) : (third ? a.w3p : a.w1p);
            const uint32_t bytes = scale ? L::kRowSA : L::kRowPA;
            const uint8_t* src = base + eid * (scale ? a.strideAs : a.strideAp) + (long long)h * bytes;
            const uint32_t dst = ring + s * L::kSlotA + (scale ? 2 * L::kRowPA : 0) + (third ? bytes : 0);
            const uint32_t bar = bars_a + 8 * s;
            if (lane == 0) mbar_arrive_expect_tx(bar, L::kSlotA);
            bulk_copy_g2s(dst, src, bytes, bar);
        }
    };
    int qa[SA];
    auto prologue_a = [&]() {
#pragma unroll
        for (int s = 0; s < SA; ++s) {
            qa[s] = claim(&next_pair);
            if (qa[s] < q_end) issue_a(qa[s], s);
        }
    };

    pdl_wait();
    // (the previous grid of this kernel, if any, has completed: its last CTA has advanced the base)
    unsigned int barrier_base = 0;
    if (lane == 0) asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(barrier_base) : "l"(&g_fused_base) : "memory");
    if (routed) {
        if (warp == 0) {
            int id;
            float w;
            route_token<8>(rt.logits, rt.n_experts, rt.k, rt.score_func, rt.eps, rt.scaling, lane, id, w);
            if (lane < rt.k) {
                expert_of_slot[lane] = id;
                weight_of_slot[lane] = w;
                if (blockIdx.x == 0) { rt.ids_out[lane] = id; rt.w_out[lane] = w; }
            }
        }
    } else if (threadIdx.x < a.E) {
        expert_of_slot[threadIdx.x] = a.ids ? a.ids[threadIdx.x] : (int)threadIdx.x;
        weight_of_slot[threadIdx.x] = __ldcg(a.r + threadIdx.x);
    }

    // x -> fp16 with one scale, once per CTA (the barrier also publishes the expert table)
    // (x is requested before the weight copies are queued: a load issued behind 20 MB of queued copies waits for them)
    float xs;
    {
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const bool mine = threadIdx.x * 8 < KT;
        if (mine) load8_as_float(a.x + threadIdx.x * 8, v);
        uint32_t m = amax_bits8(v);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = max(m, __shfl_xor_sync(kFullMask, m, off));
        if (lane == 0) red[warp] = m;
        __syncthreads();
        prologue_a();
        m = 0;
#pragma unroll
        for (int w = 0; w < NW; ++w) m = max(m, red[w]);
        float inv;
        xs = fp16_scale_for(m, inv);
        if (mine) store8_as_half(vec, threadIdx.x, v, inv);
        __syncthreads();
    }
    bool alive = true;
    {
        __half2 x[L::kBplA][16];
        lane_blocks_from_smem<L::kBplA>(vec, lane, x);
        const uint32_t lane_w = ring + lane * 16;
        const uint32_t lane_s = ring + 2 * L::kRowPA + lane;
        uint32_t parity = 0;
        for (bool any = true; any; parity ^= 1) {
            any = false;
#pragma unroll
            for (int s = 0; s < SA; ++s) {
                const int q = qa[s];
                if (q < q_end && alive) {
                    any = true;
                    alive = mbar_wait_bounded(bars_a + 8 * s, parity, 1);
                    float v[2] = {0.f, 0.f};
#pragma unroll
                    for (int j = 0; j < L::kBplA; ++j) {
                        const uint4 wg = lds_v4(lane_w + s * L::kSlotA + 512 * j);
                        const uint4 wu = lds_v4(lane_w + s * L::kSlotA + L::kRowPA + 512 * j);
                        const float sg = e8m0_to_float_fast(lds_u8(lane_s + s * L::kSlotA + 32 * j));
                        const float su = e8m0_to_float_fast(lds_u8(lane_s + s * L::kSlotA + L::kRowSA + 32 * j));
                        v[0] = fmaf(fp4_block_dot(wg, x[j]), sg, v[0]);
                        v[1] = fmaf(fp4_block_dot(wu, x[j]), su, v[1]);
                    }
                    multi_reduce<2>(v, lane);                        // lane 0: gate sum, lane 16: up sum
                    const float up = __shfl_sync(kFullMask, v[0], 16) * xs;
                    if (lane == 0 && alive) {
                        const float g = v[0] * xs;
                        a.mid[q] = (g / (1.0f + __expf(-g))) * up;
                    }
                    __syncwarp();                                    // every lane has read the slot
                    qa[s] = claim(&next_pair);
                    if (qa[s] < q_end && alive) issue_a(qa[s], s);
                }
            }
        }
    }
    // ------------------------------------------------------------------ grid barrier, first half
    // Every warp arrives on its own as soon as its SwiGLU rows are written (lane 0 wrote them); the W2 copies are
    // queued after that, and the wait for the other warps of the grid comes last.
    __shared__ int barrier_ok;
    const bool arbiter = threadIdx.x == (NW - 1) * 32;
    if (lane == 0) fused_barrier_arrive();
    __syncwarp();
    // ------------------------------------------------------------------ phase B set-up: request W2 rows, then wait
    const int o_begin = (int)((long long)a.O * blockIdx.x / gridDim.x);
    const int o_end = (int)((long long)a.O * (blockIdx.x + 1) / gridDim.x);
    const int n_local = o_end - o_begin;
    // The CTA's (expert, output row) units, expert-major, are split evenly over the warps (10.5 each at the DSv4
    // shape: every warp finishes at the same time); a warp walks its range in tasks of up to R rows of one expert.
    // A task is packed as expert << 16 | first row << 8 | rows; 0 = none.
    const int n_units = a.E * n_local;
    int u_next = (int)((long long)n_units * warp / NW);
    const int u_end = (int)((long long)n_units * (warp + 1) / NW);
    // u / n_local == (u * inv_n) >> 16: exact for u < 512 and n_local <= 64 (E <= 8, at most 64 rows per CTA)
    const uint32_t inv_n = (65536u + n_local - 1) / n_local;
    auto next_task = [&]() -> int {
        if (u_next >= u_end) return 0;
        const int e = (int)(((uint32_t)u_next * inv_n) >> 16);
        const int l0 = u_next - e * n_local;
        const int rows = min(min(R, n_local - l0), u_end - u_next);
        u_next += rows;
        return (e << 16) | (l0 << 8) | rows;
    };

    auto issue_b = [&](int t, int s) {
        if (lane < 2) {
            const int e = t >> 16, l0 = (t >> 8) & 255;
            const uint32_t rows = (uint32_t)(t & 255);
            const long long eid = (long long)expert_of_slot[e];
            const bool scale = lane == 1;
            const uint32_t rb = scale ? L::kRowSB : L::kRowPB;
            const uint8_t* src = (scale ? a.w2s + eid * a.strideBs : a.w2p + eid * a.strideBp) +
                                 (long long)(o_begin + l0) * rb;
            const uint32_t dst = ring + s * L::kSlotB + (scale ? R * L::kRowPB : 0);
            const uint32_t bar = bars_b + 8 * s;
            if (lane == 0) mbar_arrive_expect_tx(bar, rows * (L::kRowPB + L::kRowSB));
            bulk_copy_g2s(dst, src, rows * rb, bar);
        }
    };
    // No W2 row is requested before the barrier: loads issued behind queued copies (the barrier's polls, the
    // intermediate) wait for all of them.  The ring is filled once the loads of the intermediate are in flight;
    // its first rows land while the intermediate is being converted.
    int tb[SB];

    // grid barrier, second half: every SwiGLU row of every expert is written
    // (one poller per CTA: with one per warp the polls slow the arrivals down - 29 us per layer instead of 23)
    if (arbiter) barrier_ok = fused_barrier_wait(barrier_base, gridDim.x * NW) ? 1 : 0;
    __syncthreads();
    if (!barrier_ok) alive = false;

    // intermediates -> fp16, one scale per expert, once per CTA
    {
        constexpr int kPerExpert8 = HT / 8;                          // 8-value chunks per expert
        constexpr int kEntries = HT / 256;                           // warp-sized groups of chunks per expert
        constexpr int kPieces = (kRingMaxExperts * kPerExpert8 + NW * 32 - 1) / (NW * 32);
        const int n8 = a.E * kPerExpert8;
        float v[kPieces][8];
#pragma unroll
        for (int p = 0; p < kPieces; ++p) {
            const int idx8 = p * NW * 32 + threadIdx.x;
#pragma unroll
            for (int i = 0; i < 8; ++i) v[p][i] = 0.f;
            if (idx8 < n8) load8_as_float(a.mid + (size_t)idx8 * 8, v[p]);
        }
#pragma unroll
        for (int s = 0; s < SB; ++s) {                               // the W2 ring
            tb[s] = next_task();
            if (tb[s] != 0 && alive) issue_b(tb[s], s);
        }
#pragma unroll
        for (int p = 0; p < kPieces; ++p) {
            uint32_t m = amax_bits8(v[p]);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) m = max(m, __shfl_xor_sync(kFullMask, m, off));
            if (lane == 0) red[p * NW + warp] = m;                   // entry index = idx8 / 32
        }
        __syncthreads();
#pragma unroll
        for (int p = 0; p < kPieces; ++p) {
            const int idx8 = p * NW * 32 + threadIdx.x;
            if (idx8 < n8) {
                const int e = idx8 / kPerExpert8;
                uint32_t m = 0;
#pragma unroll
                for (int k = 0; k < kEntries; ++k) m = max(m, red[e * kEntries + k]);
                float inv;
                const float sc = fp16_scale_for(m, inv);
                if (idx8 - e * kPerExpert8 == 0) mid_scale[e] = sc;
                store8_as_half(vec + (size_t)e * HT, idx8 - e * kPerExpert8, v[p], inv);
            }
        }
        __syncthreads();
    }
    // ------------------------------------------------------------------ phase B: down + combine
    {
        const uint32_t lane_w = ring + lane * 16;
        const uint32_t lane_s = ring + R * L::kRowPB + lane;
        uint32_t parity = 0;
        // tasks are numbered expert-major, so a warp reloads its blocks of the intermediate only when it crosses
        // into another expert
        __half2 m2[L::kBplB][16];
        int cur_e = -1;
        for (bool any = true; any; parity ^= 1) {
            any = false;
#pragma unroll
            for (int s = 0; s < SB; ++s) {
                const int t = tb[s];
                if (t != 0 && alive) {
                    any = true;
                    const int e = t >> 16, l0 = (t >> 8) & 255, rows = t & 255;
                    if (e != cur_e) { lane_blocks_from_smem<L::kBplB>(vec + (size_t)e * HT, lane, m2); cur_e = e; }
                    alive = mbar_wait_bounded(bars_b + 8 * s, parity, 2);
                    float v[R];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        v[r] = 0.f;
#pragma unroll
                        for (int j = 0; j < L::kBplB; ++j) {
                            const uint4 w = lds_v4(lane_w + s * L::kSlotB + r * L::kRowPB + 512 * j);
                            const float sc = e8m0_to_float_fast(lds_u8(lane_s + s * L::kSlotB + r * L::kRowSB + 32 * j));
                            v[r] = fmaf(fp4_block_dot(w, m2[j]), sc, v[r]);
                        }
                    }
                    multi_reduce<R>(v, lane);
                    if (multi_reduce_owner<R>(lane) && alive) {
                        const int idx = multi_reduce_index<R>(lane);
                        if (idx < rows) part[l0 + idx][e] = v[0] * mid_scale[e];   // rows past the task hold stale bytes
                    }
                    __syncwarp();                                    // every lane has read the slot
                    tb[s] = next_task();
                    if (tb[s] != 0 && alive) issue_b(tb[s], s);
                }
            }
        }
    }
    __syncthreads();

    for (int t = threadIdx.x; t < n_local; t += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < a.E; ++k) acc = fmaf(weight_of_slot[k], part[t][k], acc);
        a.out[o_begin + t] = __float2bfloat16(acc);
    }
    if (threadIdx.x == (NW - 1) * 32) fused_barrier_leave(barrier_base, gridDim.x * NW);
}

}  // namespace dsv4
