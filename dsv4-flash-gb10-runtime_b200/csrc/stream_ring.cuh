// Per-warp shared-memory rings fed by bulk asynchronous copies (cp.async.bulk, the 1-D TMA path), used by
// the routed-expert decode kernels at the shapes where every weight row and scale row is a multiple of
// 16 bytes (reduction axis a multiple of 512).
//
// Why: the decode GEMV must keep ~50 KB of loads in flight per SM to cover HBM latency at full bandwidth, and
// a lane also has to hold a 4096-element activation vector slice (64 registers).  Loads into registers cannot
// supply that depth; bulk copies into shared memory can (up to ~200 KB per SM) and cost one issuing lane.
//
// Each warp is its own producer and consumer: it owns kStages slots and one mbarrier per slot.  Lanes 0..3
// issue the copies of a slot, lane 0 arms the barrier with the byte count, all lanes wait on the barrier's
// phase, read the slot with conflict-free 128-bit loads, __syncwarp(), and the slot is refilled at once.
// Every wait is bounded: after kSpinLimit polls the warp records an error status and stops consuming.
#pragma once

#include "gemv_engine.cuh"

namespace dsv4 {

constexpr uint32_t kSpinLimit = 1u << 22;

// Set to a non-zero code by a kernel whose bounded wait ran out; read by dsv4_b200_device_status().
__device__ int g_device_status = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Returns false (and records `code`) if the phase did not complete within the poll budget.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int code) {
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;   // try_wait itself suspends the thread for a short while
        if (it > 64) __nanosleep(64);                  // a long wait: leave the issue slots to the other warps
    }
    atomicExch(&g_device_status, code);
    return false;
}

// The same with the poll budget given at run time; code 0 records nothing.
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, int code, uint32_t limit) {
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;   // try_wait itself parks the thread for a short while
        if (it > 64) __nanosleep(64);
    }
    if (code != 0) atomicExch(&g_device_status, code);
    return false;
}

// Global -> this CTA's shared memory, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint32_t lds_u8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Lane's part of one MXFP4 row held in a ring slot: weights at `w` (row start), scale bytes at `s`.
template <int BPL>
__device__ __forceinline__ float ring_row_dot(uint32_t w, uint32_t s, int lane, const bool (&ok)[BPL],
                                              const LaneAct<Fp4Format, BPL>& a) {
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < BPL; ++j) {
        if (ok[j]) {
            const uint4 q = lds_v4(w + (lane + 32 * j) * 16);
            const float sc = e8m0_to_float_fast(lds_u8(s + lane + 32 * j));
            acc = fmaf(Fp4Format::dot(q, a.h[j]), sc, acc);
        }
    }
    return acc * a.scale;
}

}  // namespace dsv4
