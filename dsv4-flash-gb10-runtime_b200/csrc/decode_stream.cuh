// One persistent kernel for the whole routed-expert decode layer of one token, with no grid-wide barrier:
//   router (optional)  ->  gate/up + SwiGLU rows  ->  down rows + router-weighted combine,
// streamed as ONE queue of tasks per CTA so that the weight stream from HBM never drains between the two phases.
//
// Dependencies.  A down row of expert e needs all of that expert's SwiGLU intermediate, which every CTA of the
// grid contributes to.  There is no barrier and no flag: every intermediate value travels through the workspace as
// one 8-byte word {FP32 value, 32-bit tag}, written with a single store, where the tag names the launch and the row.
//   * every CTA owns a fixed range of hidden rows of every expert and walks them expert by expert;
//   * two service warps (the last warps of every CTA; they stream no weights) copy expert 0's 2048 tagged words
//     into shared memory (16-byte asynchronous copies through the load/store unit), then expert 1's, ...; a copy is
//     accepted when every tag in it is this launch's tag for its row (otherwise some CTA has not written its rows
//     yet and the copy is repeated); an accepted copy is converted to scaled fp16 and the CTA-local mbarrier
//     mid_ready[e] opens;
//   * the streaming warps take their tasks from the queue in order - all gate/up rows first, then the down rows
//     expert by expert - and wait on mid_ready[e] before their first down row of expert e.  By the time a CTA
//     reaches the down rows, the early experts have been complete for microseconds; only the last expert can be
//     waited for, and that wait overlaps the down rows of the experts before it.
// Nothing in the streaming warps waits for a store to be acknowledged (no fence, no release): under a saturated
// weight stream every memory round trip of an SM costs well over a microsecond.
//
// Streaming.  Each of the 14 streaming warps owns two ring slots of 4 KB and one mbarrier per slot.  A gate/up task is
// one hidden row: its W1 row and W3 row, two bulk copies (cp.async.bulk, no multicast); a down task is up to four
// consecutive W2 rows, one bulk copy.  Scale rows are not copied task by task (a bulk copy of 128 bytes costs the
// copy engine as much as one of 2 KB): the CTA's W1 / W3 scale rows of one expert arrive with two copies, its W2
// scale rows of every expert with one copy per expert.  A slot is requested again when the warp's other slot has
// landed, so every warp has one copy in flight while it works on the other slot.
//
// State.  The tagged words and a generation word live in the caller's workspace, never in the library: two calls
// with different workspaces share nothing.  The workspace may start as anything: a launch tags with generation + 1,
// and CTA 0 stores generation + 1 back when its service warps are done, so what a launch leaves behind never
// matches the next launch on that workspace; the row index is folded into the tag so that a workspace filled with
// one repeated value cannot match either.
//
// All CTAs of the grid must become resident without waiting for this grid to finish (one CTA per SM).  Every wait
// is bounded (GroupedArgs::spin_limit polls); a CTA that gives up records a status code, skips the remaining
// work, waits for its copies in flight and writes NaN to its output rows.
#pragma once

#include "grouped_ring.cuh"

namespace dsv4 {

constexpr int kStreamWarps = 14;           // streaming warps
constexpr int kServiceWarps = 2;           // warps that fetch, check and convert the intermediates
constexpr int kStreamThreads = (kStreamWarps + kServiceWarps) * 32;
constexpr int kStreamSlots = 2;            // ring slots per streaming warp
constexpr int kStreamRowsB = 4;            // down rows per task
constexpr int kStreamCap = 32;             // output rows per CTA
constexpr int kStreamCapA = 16;            // hidden rows per expert per CTA
constexpr int kStreamStages = 2;           // staging buffers for the tagged intermediates
constexpr int kStreamMaxGrid = 256;
constexpr int kStreamMaxExperts = kRingMaxExperts;
constexpr size_t kStreamSyncBytes = 64;    // generation word, behind the tagged intermediate in the workspace
constexpr int kStreamGateRows = 6;         // rows of the next expert a CTA finishes before it copies an expert

// Tag of intermediate row q in the launch of generation `want`.
__device__ __forceinline__ uint32_t stream_tag(uint32_t want, uint32_t q) { return want * 0x9E3779B1u + q; }

__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_gpu_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// 16 bytes global -> shared through the load/store unit (not the bulk-copy engine, whose queue is full of weight
// rows); L2 only.  The arrive fires when all earlier copies of this thread have landed.
__device__ __forceinline__ void ldgsts16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void ldgsts_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// x / d for x < 65536, 2 <= d < 65536, with inv = 0xffffffff / d + 1; d == 1 is handled by the caller.
__device__ __forceinline__ int div_small(int x, uint32_t inv, int d) {
    return d == 1 ? x : (int)__umulhi((uint32_t)x, inv);
}


template <int KT, int HT>
struct StreamLayout {
    static constexpr int kBplA = KT / 1024, kBplB = HT / 1024;
    static constexpr uint32_t kRowPA = KT / 2, kRowSA = KT / 32;
    static constexpr uint32_t kRowPB = HT / 2, kRowSB = HT / 32;
    static constexpr uint32_t kSlotA = 2 * kRowPA;                               // one W1 row, one W3 row
    static constexpr uint32_t kSlotB = kStreamRowsB * kRowPB;                    // up to four W2 rows (contiguous)
    static constexpr uint32_t kSlot = kSlotA > kSlotB ? kSlotA : kSlotB;
    static constexpr uint32_t kRingPerWarp = kStreamSlots * kSlot;
    static constexpr uint32_t kX = kStreamWarps * kRingPerWarp;                  // fp16 x
    static constexpr uint32_t kMid = kX + KT * 2;                                // fp16 intermediates [expert][HT]
    static constexpr uint32_t kStage = kMid + kStreamMaxExperts * HT * 2;        // three buffers of one expert's tagged words
    // scale rows are not copied task by task (a bulk copy of 128 bytes costs the copy engine as much as one of
    // 2 KB): the CTA's W1 / W3 scale rows of one expert are fetched with two copies into one of two buffers, and
    // its W2 scale rows of every expert with one copy per expert at the start
    static constexpr uint32_t kAScaleBuf = 2 * kStreamCapA * kRowSA;             // W1 rows, then W3 rows
    static constexpr uint32_t kAScale = kStage + kStreamStages * HT * 8;
    static constexpr uint32_t kBScale = kAScale + 2 * kAScaleBuf;                // [expert][row][kRowSB]
    static constexpr uint32_t kBars = kBScale + kStreamMaxExperts * kStreamCap * kRowSB;
    // barriers: per warp kStreamSlots, 8 mid_ready, 3 staging, 8 gate/up scales (one per expert), 1 down scales
    static constexpr uint32_t kPart = kBars + (kStreamWarps * kStreamSlots + 8 + kStreamStages + 8 + 1) * 8;   // [rows][8] FP32
    static constexpr uint32_t kBytes = kPart + kStreamCap * 8 * 4;
};

template <int KT, int HT>
__global__ void __launch_bounds__(kStreamThreads, 1) moe_decode_stream_kernel(const GroupedArgs a,
                                                                                       const RouteArgs rt) {
    using L = StreamLayout<KT, HT>;
    constexpr int NW = kStreamWarps, NS = kStreamSlots, R = kStreamRowsB;
    static_assert(NS == 2, "the slot bookkeeping below is written for two slots per warp");
    extern __shared__ __align__(128) uint8_t ring_smem[];
    __shared__ int expert_of_slot[8];
    __shared__ float weight_of_slot[8];
    __shared__ float mid_scale[8];
    __shared__ int done_a[8];                     // gate/up rows of expert e finished by this CTA
    __shared__ int next_task;
    __shared__ uint32_t s_want;                   // the generation this launch publishes and waits for
    __shared__ volatile int failed;
    __shared__ uint32_t red[32];
    __shared__ __align__(16) uint32_t cand_key[64];   // router: the best k of each of 8 groups of 32 experts
    __shared__ __align__(16) int cand_idx[64];
    __shared__ float pick_score[8];
    // mailbox of the service warps, three slots used round robin by attempt: {arrivals, OR of flags, largest magnitude}
    __shared__ uint32_t svc_cnt[3], svc_flags[3], svc_amax[3];
    pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const bool service = warp >= NW;
    constexpr int NSV = kServiceWarps;
    const bool routed = rt.logits != nullptr;
    const bool use_table = a.ids != nullptr || routed;
    const uint32_t smem0 = smem_u32(ring_smem);
    const uint32_t ring = smem0 + warp * L::kRingPerWarp;
    const uint32_t bars = smem0 + L::kBars + warp * NS * 8;
    const uint32_t bars_mid = smem0 + L::kBars + NW * NS * 8;
    __half* xvec = reinterpret_cast<__half*>(ring_smem + L::kX);
    __half* mvec = reinterpret_cast<__half*>(ring_smem + L::kMid);
    float (*part)[8] = reinterpret_cast<float (*)[8]>(ring_smem + L::kPart);
    uint32_t* const sync_epoch = a.sync;
    const uint32_t bars_stage = bars_mid + 8 * 8;
    const uint32_t bars_ascale = bars_stage + kStreamStages * 8;
    const uint32_t bar_bscale = bars_ascale + 8 * 8;
    const uint32_t ascale = smem0 + L::kAScale;
    const uint32_t bscale = smem0 + L::kBScale;
    const uint32_t stage = smem0 + L::kStage;

    if (warp == NW) {
        // 8 mid_ready (one arrival per service warp); 3 staging barriers (one arrival per service lane); 9 for scales
        if (lane < 8 + kStreamStages + 9) mbar_init(bars_mid + 8 * lane, lane < 8 ? NSV : (lane < 8 + kStreamStages ? NSV * 32 : 1));
        if (lane < 8) done_a[lane] = 0;
        if (lane < 3) { svc_cnt[lane] = 0; svc_flags[lane] = 0; svc_amax[lane] = 0; }
        if (lane == 0) { next_task = 0; failed = 0; }
    } else if (!service && lane == 0) {
#pragma unroll
        for (int s = 0; s < NS; ++s) mbar_init(bars + 8 * s, 1);
    }
    mbar_init_fence();

    // ---------------------------------------------------------------- this CTA's share of the two phases
    const int G = gridDim.x, cta = blockIdx.x;
    const int hb = (int)((long long)HT * cta / G), he = (int)((long long)HT * (cta + 1) / G);
    const int n_h = he - hb;                                   // hidden rows per expert (same range for every expert)
    const int n_a = a.E * n_h;                                 // gate/up tasks: expert-major, one row pair each
    const int o_begin = (int)((long long)a.O * cta / G), o_end = (int)((long long)a.O * (cta + 1) / G);
    const int n_local = o_end - o_begin;
    const int gpe = (n_local + R - 1) / R;                     // down tasks per expert: up to R rows each
    const int n_total = n_a + a.E * gpe;
    const uint32_t inv_nh = n_h > 1 ? 0xffffffffu / (uint32_t)n_h + 1u : 0u;
    const uint32_t inv_gpe = gpe > 1 ? 0xffffffffu / (uint32_t)gpe + 1u : 0u;

    // A task is described by one word: gate/up  = expert << 16 | row within the CTA's range;
    //                                 down      = expert << 16 | first local row << 8 | rows.
    auto describe = [&](int t) -> int {
        if (t < n_a) {
            const int e = div_small(t, inv_nh, n_h);
            return (e << 16) | (t - e * n_h);
        }
        const int j = t - n_a;
        const int e = div_small(j, inv_gpe, gpe);
        const int l0 = (j - e * gpe) * R;
        return (e << 16) | (l0 << 8) | min(R, n_local - l0);
    };
    auto issue = [&](int t, int d, int s) {
        const uint32_t slot = ring + s * L::kSlot;
        const uint32_t bar = bars + 8 * s;
        const int e = d >> 16;
        if (t < n_a) {
            if (lane < 2) {                                    // lane 0: the W1 row, lane 1: the W3 row
                const int h = hb + (d & 0xffff);
                const long long eid = use_table ? (long long)expert_of_slot[e] : (long long)e;
                const uint8_t* src = (lane ? a.w3p : a.w1p) + eid * a.strideAp + (long long)h * L::kRowPA;
                if (lane == 0) mbar_arrive_expect_tx(bar, L::kSlotA);
                bulk_copy_g2s(slot + lane * L::kRowPA, src, L::kRowPA, bar);
            }
        } else if (lane == 0) {                                // the task's W2 rows are contiguous: one copy
            const int l0 = (d >> 8) & 255;
            const uint32_t rows = (uint32_t)(d & 255);
            const long long eid = use_table ? (long long)expert_of_slot[e] : (long long)e;
            const uint8_t* src = a.w2p + eid * a.strideBp + (long long)(o_begin + l0) * L::kRowPB;
            mbar_arrive_expect_tx(bar, rows * L::kRowPB);
            bulk_copy_g2s(slot, src, rows * L::kRowPB, bar);
        }
    };
    // W1 and W3 scale rows of this CTA's hidden rows of expert e -> buffer e & 1 (two copies)
    auto issue_ascale = [&](int e) {
        if (lane < 2) {
            const long long eid = use_table ? (long long)expert_of_slot[e] : (long long)e;
            const uint8_t* src = (lane ? a.w3s : a.w1s) + eid * a.strideAs + (long long)hb * L::kRowSA;
            const uint32_t bar = bars_ascale + 8 * e;         // one barrier per expert, each used once per launch
            if (lane == 0) mbar_arrive_expect_tx(bar, 2u * n_h * L::kRowSA);
            bulk_copy_g2s(ascale + (e & 1) * L::kAScaleBuf + lane * (kStreamCapA * L::kRowSA), src, n_h * L::kRowSA, bar);
        }
    };
    // W2 scale rows of this CTA's output rows, every expert (one copy per expert)
    auto issue_bscale = [&]() {
        if (lane == 0) mbar_arrive_expect_tx(bar_bscale, (uint32_t)a.E * n_local * L::kRowSB);
        __syncwarp();
        if (lane < a.E) {
            const long long eid = use_table ? (long long)expert_of_slot[lane] : (long long)lane;
            const uint8_t* src = a.w2s + eid * a.strideBs + (long long)o_begin * L::kRowSB;
            bulk_copy_g2s(bscale + lane * (kStreamCap * L::kRowSB), src, n_local * L::kRowSB, bar_bscale);
        }
    };
    auto claim = [&]() -> int {
        int v = 0;
        if (lane == 0) v = atomicAdd(&next_task, 1);
        return __shfl_sync(kFullMask, v, 0);
    };

    // per-slot state of a streaming warp: the task in the slot (>= n_total: none) and its description
    int tk0 = n_total, tk1 = n_total, td0 = 0, td1 = 0;
    // the first task is claimed before the expert table is known (that needs nothing from the router) ...
    auto prologue_claim = [&]() {
        tk0 = claim();
        if (tk0 < n_total) td0 = describe(tk0);
        tk1 = -1;                                              // free: requested when slot 0 has landed
    };
    // ... and requested as soon as it is
    auto prologue = [&]() {
        if (tk0 < n_total) issue(tk0, td0, 0);
        if (warp == 0) {
            issue_ascale(0);
            if (a.E > 1) issue_ascale(1);
        }
    };

    __syncthreads();                                           // barriers and the queue are initialised
    // stacked weights do not depend on the previous kernel in the stream: request them before waiting for it
    if (!service) prologue_claim();
    if (!use_table && !service) prologue();
    // The logits may still be written by the previous kernel of the stream, so they are read after the wait; asking
    // the L2 for their lines now is harmless either way (a later write lands in the same L2) and takes the miss
    // out of the start when they are not (one 128-byte line per routing warp).
    if (routed && warp < 8 && lane == 0 && warp * 32 < rt.n_experts)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(rt.logits + warp * 32));
    pdl_wait();
    if (warp == NW + NSV - 1 && lane == 0) s_want = ld_relaxed_gpu(sync_epoch) + 1u;
    // Router, spread over the CTA (the weight stream cannot start before the picks are known, so this is the
    // critical path of the layer's start): warps 0..7 take 32 experts each, one per lane, and sort them; the best k
    // of every warp are then ranked against one another (largest score, lowest expert index on ties - the
    // reference's rule) and the k best of all enter the table.
    constexpr int kRouteWarps = 8;
    if (routed) {
        if (threadIdx.x < 8) { expert_of_slot[threadIdx.x] = 0; pick_score[threadIdx.x] = -INFINITY; }
        if (warp < kRouteWarps) {
            const int idx = warp * 32 + lane;
            uint32_t key = 0u;
            if (idx < rt.n_experts) key = route_key(route_score(__ldcg(rt.logits + idx), rt.score_func));
            // the warp's 32 (key, lane) pairs sorted by a bitonic network, best first (on equal keys the lower lane):
            // 15 compare-exchange steps, against k rounds of warp-wide arg-max with a reduction each
            unsigned long long v = ((unsigned long long)key << 32) | (unsigned)(31 - lane);
#pragma unroll
            for (int k2 = 2; k2 <= 32; k2 <<= 1)
#pragma unroll
                for (int j = k2 >> 1; j > 0; j >>= 1) {
                    const unsigned long long o = __shfl_xor_sync(kFullMask, v, j);
                    const bool descending = (lane & k2) == 0;              // (k2 == 32: every lane)
                    const bool keep_larger = ((lane & j) == 0) == descending;
                    v = keep_larger ? (v > o ? v : o) : (v < o ? v : o);
                }
            if (lane < 8) {
                const bool real = lane < rt.k && (uint32_t)(v >> 32) != 0u;
                cand_key[warp * 8 + lane] = real ? (uint32_t)(v >> 32) : 0u;
                cand_idx[warp * 8 + lane] = real ? warp * 32 + 31 - (int)(v & 31u) : 0x7fffffff;
            }
        }
    } else if (threadIdx.x < a.E) {
        expert_of_slot[threadIdx.x] = a.ids ? a.ids[threadIdx.x] : (int)threadIdx.x;
        weight_of_slot[threadIdx.x] = __ldcg(a.r + threadIdx.x);
    }

    // x -> fp16 with one scale, once per CTA (x is requested before the weight copies are queued: a load issued
    // behind queued copies waits for them)
    float xs;
    {
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const bool mine = threadIdx.x * 8 < KT;
        if (mine) load8_as_float(a.x + threadIdx.x * 8, v);
        uint32_t m = amax_bits8(v);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = max(m, __shfl_xor_sync(kFullMask, m, off));
        if (lane == 0) red[warp] = m;
        __syncthreads();                                       // candidates, s_want, the table of the unrouted entries
        if (use_table && !routed && !service) prologue();
        if (routed) {
            // rank of a candidate among all 64 entries (empty ones carry key 0): how many are better.  Eight
            // consecutive lanes share a candidate, each compares it with the eight entries of one group.
            static_assert(kStreamThreads == 512, "64 candidates x 8 lanes");
            const int c = threadIdx.x >> 3, part = threadIdx.x & 7;
            const uint32_t ck = cand_key[c];
            const int ci = cand_idx[c];
            const uint4 k0 = *reinterpret_cast<const uint4*>(cand_key + part * 8);
            const uint4 k1 = *reinterpret_cast<const uint4*>(cand_key + part * 8 + 4);
            const int4 i0 = *reinterpret_cast<const int4*>(cand_idx + part * 8);
            const int4 i1 = *reinterpret_cast<const int4*>(cand_idx + part * 8 + 4);
            const uint32_t ok[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
            const int oi[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
            int rank = 0;
#pragma unroll
            for (int q = 0; q < 8; ++q) rank += (int)(ok[q] > ck) | ((int)(ok[q] == ck) & (int)(oi[q] < ci));
            rank += __shfl_xor_sync(kFullMask, rank, 1);
            rank += __shfl_xor_sync(kFullMask, rank, 2);
            rank += __shfl_xor_sync(kFullMask, rank, 4);
            if (part == 0 && ck != 0u && rank < rt.k) { expert_of_slot[rank] = ci; pick_score[rank] = route_key_score(ck); }
        }
        m = 0;
#pragma unroll
        for (int w = 0; w < NW + NSV; ++w) m = max(m, red[w]);
        float inv;
        xs = fp16_scale_for(m, inv);
        if (mine) store8_as_half(xvec, threadIdx.x, v, inv);
        __syncthreads();                                       // the routed table, x in shared memory
        if (routed && !service) prologue();
        if (routed && warp == 0) {
            // the picks' weights (needed only by the combine at the end); a pick that does not exist (fewer than k
            // scores that are numbers) keeps expert 0 with weight 0 and is reported through the status word
            const float sc = lane < rt.k ? pick_score[lane] : -INFINITY;
            const float w = route_weight(sc, pick_score[0], rt.k, rt.score_func, rt.eps, rt.scaling, lane);
            if (lane < rt.k) {
                const bool missing = sc == -INFINITY;
                weight_of_slot[lane] = missing ? 0.f : w;
                if (missing) atomicExch(&g_device_status, 4);
                if (cta == 0) { rt.ids_out[lane] = expert_of_slot[lane]; rt.w_out[lane] = missing ? 0.f : w; }
            }
        }
    }
    const uint32_t want = s_want;
    const uint32_t spin_limit = a.spin_limit;

    if (service) {
        // ------------------------------------------------------------ the intermediates, expert by expert
        // The service warps work in lockstep (a bounded agreement through shared memory), each on its own share of an
        // expert's tagged words.  The copy of the next expert travels while this one is checked and converted.
        // A copy of expert e is requested once this CTA has finished its own rows of e and a few rows of e + 1
        // (the other CTAs are then done with e, give or take); a copy that still holds a foreign tag is repeated.
        constexpr uint32_t kStageBytes = HT * 8;
        constexpr int kChunks = HT / 64 / NSV;                 // 16-byte chunks (two tagged words) per lane
        static_assert(HT % (64 * NSV) == 0, "rows per service lane");
        const int sw = warp - NW;
        const uint32_t tag_mul = (a.phantom > 0 ? want ^ 0x5a5a5a5au : want) * 0x9E3779B1u;   // phantom: never matches
        const volatile int* progress = done_a;
        const int gate_rows = min(n_h, kStreamGateRows);
        // chunk c of this lane is chunk (sw * kChunks + c) * 32 + lane of the expert: rows 2 i, 2 i + 1 of chunk i
        const uint32_t lane_off = (uint32_t)(sw * kChunks) * 512u + lane * 16;
        const int lane_row = 2 * (sw * kChunks * 32 + lane);
        // Every service warp requests its own part of an expert (16 bytes per lane and copy, through the load/store
        // unit) and all of them wait for the landing of the whole.
        auto request = [&](int e) {
            const uint32_t dst = stage + (e % kStreamStages) * kStageBytes + lane_off;
            const uint8_t* src = reinterpret_cast<const uint8_t*>(a.mid8 + (size_t)e * HT) + lane_off;
#pragma unroll
            for (int c = 0; c < kChunks; ++c) ldgsts16(dst + c * 512, src + c * 512);
            ldgsts_arrive(bars_stage + 8 * (e % kStreamStages));
        };
        // A short pause that keeps the warp off the issue slots without the microsecond granularity of a timed sleep.
        auto pause = [&]() {
            const long long t0 = clock64();
            while (clock64() - t0 < 200) { }
        };
        auto gate_open = [&](int e) {
            return progress[e] >= n_h && (e + 1 == a.E || progress[e + 1] >= gate_rows);
        };
        // Agreement of the service warps on one attempt, through shared memory and with a bounded wait (no barrier
        // instruction: a barrier cannot give up).  Every warp adds its flags and its largest magnitude to the
        // attempt's slot, then its arrival; when all have arrived each reads the same totals.  Warp 0 clears the
        // slot of the attempt before this one (its readers all arrived here since; its next writers come two
        // attempts later, after warp 0's arrival at the next one).  Returns false if the others never arrive.
        const volatile uint32_t* v_cnt = svc_cnt;
        const volatile uint32_t* v_flags = svc_flags;
        const volatile uint32_t* v_amax = svc_amax;
        auto agree = [&](uint32_t attempt, uint32_t my_flags, uint32_t my_amax, uint32_t& flags, uint32_t& amax,
                         uint32_t& budget) -> bool {
            const uint32_t slot = attempt % 3u;
            if (lane == 0) {
                atomicOr(&svc_flags[slot], my_flags);
                atomicMax(&svc_amax[slot], my_amax);
                __threadfence_block();
                atomicAdd(&svc_cnt[slot], 1u);
            }
            bool all = false;
            while (budget > 0 && !(all = v_cnt[slot] >= (uint32_t)NSV)) { --budget; }
            flags = v_flags[slot];
            amax = v_amax[slot];
            __syncwarp();
            if (all && lane == 0 && sw == 0) {
                const uint32_t old = (attempt + 2u) % 3u;
                svc_cnt[old] = 0; svc_flags[old] = 0; svc_amax[old] = 0;
            }
            return all;
        };
        // The down scales of all experts are not needed before the down rows.  At the start every copy queues behind
        // the others in the SM's copy engine (about 25 ns each) and these would delay the first weight rows, so a
        // service warp, idle until the first expert's rows are done, requests them a microsecond or two later.
        if (sw == 0) {
            const long long t0 = clock64();
            while (clock64() - t0 < 4000) { }
            issue_bscale();
        }
        int issued = 0, finished = 0;                          // experts requested / converted
        uint32_t stage_parity = 0, attempt = 0;
        bool ok = true;
        uint32_t budget = spin_limit;                          // polls and repeated copies, per expert
        // Expert e uses staging buffer e mod kStreamStages.  The other service warps are known to be done with expert
        // e - 1 (and its buffer) once they have arrived at an agreement about expert e, so copies may run
        // kStreamStages - 1 experts ahead of the one under inspection.  When to request is decided in the agreements,
        // so that all warps request alike.
        while (finished < a.E && ok) {
            bool gave_up = false;
            if (issued == finished) {
                // nothing in flight: wait for this CTA to be far enough to expect expert `issued` complete everywhere
                // (a timed sleep: a service warp that polls in a loop takes issue slots from its scheduler's streaming warps)
                while (!gate_open(issued) && budget > 0) { --budget; __nanosleep(100); }
                gave_up = budget == 0;
                request(issued++);
            }
            const int e = finished;
            const int sb = e % kStreamStages;
            const uint32_t bar = bars_stage + 8 * sb;
            bool landed = false;
            while (budget > 0 && !(landed = mbar_try_wait(bar, (stage_parity >> sb) & 1u))) --budget;
            gave_up = gave_up || !landed;
            stage_parity ^= 1u << sb;
            const uint32_t buf = stage + sb * kStageBytes + lane_off;
            // pass 1: every tag, and the largest magnitude
            uint32_t bad = 0, m = 0;
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
                const uint4 q = lds_v4(buf + c * 512);
                const uint32_t t0 = tag_mul + (uint32_t)(e * HT + lane_row + 64 * c);
                bad |= (q.y ^ t0) | (q.w ^ (t0 + 1u));
                m = max(m, max(q.x & 0x7fffffffu, q.z & 0x7fffffffu));
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) m = max(m, __shfl_xor_sync(kFullMask, m, off));
            // flags: 1 = a foreign tag, 2 = a wait ran out, 4 / 8 = the gate of the next / next but one expert to
            // request is open
            uint32_t my_flags = (__any_sync(kFullMask, bad != 0) ? 1u : 0u) | (__any_sync(kFullMask, gave_up) ? 2u : 0u);
            if (issued < a.E && gate_open(issued)) my_flags |= (issued + 1 < a.E && gate_open(issued + 1)) ? 12u : 4u;
            uint32_t flags = 0, amax = 0;
            if (!agree(attempt, my_flags, m, flags, amax, budget) || (flags & 2u)) { ok = false; break; }
            // every warp is past expert e - 1: the buffers of the experts after e may be filled
            if ((flags & 4u) && issued < a.E && issued < e + kStreamStages) request(issued++);
            if ((flags & 8u) && issued < a.E && issued < e + kStreamStages) request(issued++);
            if (!(flags & 1u)) {
                float inv;
                const float sc = fp16_scale_for(amax, inv);
                uint8_t* dst = reinterpret_cast<uint8_t*>(mvec + (size_t)e * HT);
#pragma unroll
                for (int c = 0; c < kChunks; ++c) {
                    const uint4 q = lds_v4(buf + c * 512);
                    const int r0 = lane_row + 64 * c;          // even: the pair sits in one 8-value chunk
                    const __half2 h = __floats2half2_rn(__uint_as_float(q.x) * inv, __uint_as_float(q.z) * inv);
                    *reinterpret_cast<__half2*>(dst + swizzled_chunk(r0 >> 3) * 16 + (r0 & 7) * 2) = h;
                }
                if (lane == 0 && sw == 0) mid_scale[e] = sc;
                __syncwarp();
                if (lane == 0) mbar_arrive(bars_mid + 8 * e);
                ++finished;
                budget = spin_limit;
            } else {
                // some CTA has not written its rows of this expert yet: copy again (the other buffer is untouched)
                if (budget > 0) --budget;
                pause();
                request(e);
            }
            ++attempt;
        }
        if (!ok) {
            // gave up (all service warps together): tell the streaming warps, let the copies in flight land, open
            // every barrier
            if (lane == 0) { atomicExch(&g_device_status, 3); failed = 1; }
            __threadfence_block();
            for (int e = finished; e < issued; ++e)
                mbar_wait_limit(bars_stage + 8 * (e % kStreamStages), (stage_parity >> (e % kStreamStages)) & 1u, 0, 1u << 16);
            __syncwarp();
            if (lane == 0)
                for (int e = finished; e < a.E; ++e) mbar_arrive(bars_mid + 8 * e);
        }
        // what this launch wrote must not match the next launch on this workspace (every CTA has read the
        // generation word long ago: each tagged its rows with it)
        if (cta == 0 && sw == 0 && lane == 0) *sync_epoch = want;
    } else {
        bool alive = true;
        uint32_t parity = 0;                                   // bit s: phase parity of slot s
        int s = 0;
        // ------------------------------------------------------------ gate / up + SwiGLU rows
        {
            __half2 x[L::kBplA][16];
            lane_blocks_from_smem<L::kBplA>(xvec, lane, x);
            int cur_ea = -1;
            for (;;) {
                const int t = s ? tk1 : tk0;
                const int d = s ? td1 : td0;
                if (t >= n_a || !alive) break;
                const uint32_t slot = ring + s * L::kSlot;
                const uint32_t lane_w = slot + lane * 16;
                const int ea = d >> 16;
                const uint32_t lane_s = ascale + (ea & 1) * L::kAScaleBuf + (d & 0xffff) * L::kRowSA + lane;
                // the next task is claimed and described while this slot's rows are still on their way ...
                const bool refill = (s ? tk0 : tk1) < 0;
                int nt = 0, nd = 0;
                if (refill) {
                    nt = claim();
                    nd = nt < n_total ? describe(nt) : 0;
                }
                alive = mbar_wait_limit(bars + 8 * s, (parity >> s) & 1u, 1, spin_limit) && alive;
                parity ^= 1u << s;
                if (ea != cur_ea) {                              // the scale rows of this expert (requested long ago)
                    alive = mbar_wait_limit(bars_ascale + 8 * ea, 0, 1, spin_limit) && alive;
                    cur_ea = ea;
                }
                // ... and requested only now that this one has landed: one copy in flight per warp (the bytes in
                // flight, and with them every memory latency of the SM, stay small).
                if (refill) {
                    if (nt < n_total && alive) issue(nt, nd, s ^ 1);
                    if (s) { tk0 = nt; td0 = nd; } else { tk1 = nt; td1 = nd; }
                }
                float v[2] = {0.f, 0.f};
#pragma unroll
                for (int j = 0; j < L::kBplA; ++j) {
                    const uint4 wg = lds_v4(lane_w + 512 * j);
                    const uint4 wu = lds_v4(lane_w + L::kRowPA + 512 * j);
                    const float sg = e8m0_to_float_fast(lds_u8(lane_s + 32 * j));
                    const float su = e8m0_to_float_fast(lds_u8(lane_s + kStreamCapA * L::kRowSA + 32 * j));
                    v[0] = fmaf(fp4_block_dot(wg, x[j]), sg, v[0]);
                    v[1] = fmaf(fp4_block_dot(wu, x[j]), su, v[1]);
                }
                multi_reduce<2>(v, lane);                        // lane 0: gate sum, lane 16: up sum
                const float up = __shfl_sync(kFullMask, v[0], 16) * xs;
                __syncwarp();                                    // every lane has read the slot
                if (s) tk1 = -1; else tk0 = -1;                  // free: requested when the other slot has landed
                int rows_done = 0;
                if (lane == 0 && alive) {
                    const float g = v[0] * xs;
                    const uint32_t q = (uint32_t)(ea * HT + hb + (d & 0xffff));
                    const float mid = swiglu_f32(g, up);
                    // value and tag in one 8-byte store: a reader sees both or neither
                    st_relaxed_gpu_u64(a.mid8 + q, ((unsigned long long)stream_tag(want, q) << 32) | __float_as_uint(mid));
                    rows_done = atomicAdd(&done_a[ea], 1) + 1;   // progress: what the service warps time their copies by
                }
                // the CTA's last row of this expert: its scale buffer is free for the expert after the next
                if (__shfl_sync(kFullMask, rows_done, 0) == n_h && ea + 2 < a.E) issue_ascale(ea + 2);
                s ^= 1;
            }
        }
        // ------------------------------------------------------------ down rows + per-expert partial sums
        {
            __half2 m2[L::kBplB][16];
            int cur_e = -1;
            float cur_scale = 0.f;
            for (;;) {
                const int t = s ? tk1 : tk0;
                const int d = s ? td1 : td0;
                if (t >= n_total || !alive) break;
                const int e = d >> 16, l0 = (d >> 8) & 255, rows = d & 255;
                const uint32_t slot = ring + s * L::kSlot;
                const uint32_t lane_w = slot + lane * 16;
                const uint32_t lane_s = bscale + (e * kStreamCap + l0) * L::kRowSB + lane;
                const bool refill = (s ? tk0 : tk1) < 0;       // as above: claimed early, requested late
                int nt = 0, nd = 0;
                if (refill) {
                    nt = claim();
                    nd = nt < n_total ? describe(nt) : 0;
                }
                alive = mbar_wait_limit(bars + 8 * s, (parity >> s) & 1u, 2, spin_limit) && alive;
                parity ^= 1u << s;
                if (cur_e < 0) alive = mbar_wait_limit(bar_bscale, 0, 2, spin_limit) && alive;
                if (e != cur_e) {
                    alive = mbar_wait_limit(bars_mid + 8 * e, 0, 3, spin_limit) && !failed && alive;
                    lane_blocks_from_smem<L::kBplB>(mvec + (size_t)e * HT, lane, m2);
                    cur_scale = mid_scale[e];
                    cur_e = e;
                }
                if (refill) {
                    if (nt < n_total && alive) issue(nt, nd, s ^ 1);
                    if (s) { tk0 = nt; td0 = nd; } else { tk1 = nt; td1 = nd; }
                }
                float v[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    v[r] = 0.f;
#pragma unroll
                    for (int j = 0; j < L::kBplB; ++j) {
                        const uint4 w = lds_v4(lane_w + r * L::kRowPB + 512 * j);
                        const float sc = e8m0_to_float_fast(lds_u8(lane_s + r * L::kRowSB + 32 * j));
                        v[r] = fmaf(fp4_block_dot(w, m2[j]), sc, v[r]);
                    }
                }
                multi_reduce<R>(v, lane);
                if (multi_reduce_owner<R>(lane) && alive) {
                    const int idx = multi_reduce_index<R>(lane);
                    if (idx < rows) part[l0 + idx][e] = v[0] * cur_scale;    // rows past the task hold stale bytes
                }
                __syncwarp();                                    // every lane has read the slot
                if (s) tk1 = -1; else tk0 = -1;                  // free: requested when the other slot has landed
                s ^= 1;
            }
        }
        if (!alive) {
            // gave up somewhere: let the copies still in flight land before the CTA's shared memory is released
            if (lane == 0) failed = 1;
#pragma unroll
            for (int k = 0; k < NS; ++k) {
                const int t = s ? tk1 : tk0;
                if (t >= 0 && t < n_total) mbar_wait_limit(bars + 8 * s, (parity >> s) & 1u, 0, spin_limit);
                s ^= 1;
            }
        }
    }
    __syncthreads();

    const bool bad = failed != 0;
    for (int t = threadIdx.x; t < n_local; t += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < a.E; ++k) acc = fmaf(weight_of_slot[k], part[t][k], acc);
        a.out[o_begin + t] = bad ? __float2bfloat16(__uint_as_float(0x7fc00000u)) : __float2bfloat16(acc);
    }
}

}  // namespace dsv4
