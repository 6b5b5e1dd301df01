// Microbenchmark of the block-scaled tensor-core instruction the batched layer is built on: how many SM clocks one
// tcgen05.mma kind::mxf4 (M = 128, K = 64) of a given N occupies the tensor pipe, alone and with scale-atom copies
// (tcgen05.cp) between the MMAs.  One thread per CTA issues `iters` rounds of four MMAs (the four K-steps of one
// 128-byte-swizzled stage) into one accumulator, with `copies` scale-atom copies in front of every round, and the
// CTA measures the clocks until the last MMA has completed.  The operands are whatever the shared memory holds set
// to a fixed pattern: the timing does not depend on the values (measured with zeros, ones and a hash).
// This is the denominator of the batched layer's tensor roofline: FP4 peak = SMs x clock x 2 x 128 x N x 64 / clocks.
#pragma once

#include "stream_ring.cuh"
#include "tc05.cuh"

namespace dsv4 {

constexpr uint32_t kRateOperandBytes = 96 * 1024;     // A tile at 0 (16 KB), B tile at 32 KB (up to 256 rows x 128 B)
constexpr uint32_t kRateBytes = kRateOperandBytes + 4096 + 1024;

__global__ void __launch_bounds__(128) mxf4_mma_rate_kernel(int n_cols, int iters, int copies, long long* clocks) {
    extern __shared__ __align__(1024) uint8_t rate_smem[];
    __shared__ uint32_t tmem_base;
    __shared__ __align__(8) uint64_t bar;
    const int tid = threadIdx.x, warp = tid >> 5;
    for (uint32_t i = tid; i < kRateOperandBytes / 4; i += 128)
        reinterpret_cast<uint32_t*>(rate_smem)[i] = (i * 2654435761u) ^ (i << 13);
    for (uint32_t i = tid; i < 4096 / 4; i += 128) reinterpret_cast<uint32_t*>(rate_smem + kRateOperandBytes)[i] = 0x7f7f7f7fu;
    if (warp == 0) tc05_alloc(smem_u32(&tmem_base), 512);
    if (tid == 0) { mbar_init(smem_u32(&bar), 1); mbar_init_fence(); }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc05_fence_before_sync();
    __syncthreads();
    tc05_fence_after_sync();
    const uint32_t tmem = tmem_base;
    const long long t0 = clock64();
    if (tid == 0) {
        const uint32_t sa = smem_u32(rate_smem), sb = sa + 32768, sf = sa + kRateOperandBytes;
        for (int it = 0; it < iters; ++it) {
            for (int c = 0; c < copies; ++c) tc05_copy_scale_atom(tmem + 384 + 4 * c, sf + 512 * c);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                tc05_mma_mxf4(tmem, tc05_desc_k_sw128(sa + 32 * j), tc05_desc_k_sw128(sb + 32 * j),
                              tc05_idesc_mxf4(128, n_cols, (j & 1) * 2, (j & 1) * 2), tmem + 384, tmem + 388, 1);
        }
        tc05_commit(smem_u32(&bar));
    }
    mbar_wait_bounded(smem_u32(&bar), 0, 8);
    const long long t1 = clock64();
    if (tid == 0 && blockIdx.x == 0) *clocks = t1 - t0;
    tc05_fence_before_sync();
    __syncthreads();
    if (warp == 0) tc05_dealloc(tmem, 512);
}

}  // namespace dsv4
