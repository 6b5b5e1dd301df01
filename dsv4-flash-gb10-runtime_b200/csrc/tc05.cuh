// tcgen05 (5th-generation tensor core) primitives for sm_100a: tensor-memory allocation, shared-memory matrix
// descriptors for K-major 128-byte-swizzled operand tiles, the fp16 MMA, commit, and accumulator loads.
//
// Operand tile layout used throughout ("K-major, 128-byte swizzle"): a tile of R rows x 64 fp16 values; row r
// occupies bytes [128 r, 128 r + 128); inside a row the 16-byte chunk c (8 values) is stored at chunk position
// c ^ (r & 7).  Eight rows form a 1024-byte swizzle atom; the tile base is 1024-byte aligned.  One MMA consumes
// 16 values of K, i.e. 32 bytes of each row: K-step j of a tile is addressed by adding 32 j bytes to the start
// address of the descriptor.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

namespace dsv4 {

// 64-bit shared-memory matrix descriptor: start address >> 4 in bits [0,14), leading byte offset >> 4 in
// [16,30) (unused for swizzled K-major tiles, set to 1), stride byte offset >> 4 in [32,46) (distance between
// 8-row groups = 1024 bytes), descriptor version 1 in [46,48), swizzle mode in [61,64) (2 = 128 bytes).
__device__ __forceinline__ uint64_t tc05_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// 32-bit instruction descriptor of kind::f16 with fp16 A and B (K-major both), FP32 accumulator:
// accumulator format 1 (FP32) at bit 4, A / B formats 0 (fp16) at bits 7 / 10, N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ uint32_t tc05_idesc_f16(int m, int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void tc05_alloc(uint32_t smem_result_addr, uint32_t n_cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result_addr), "r"(n_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tc05_dealloc(uint32_t tmem_addr, uint32_t n_cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_addr), "r"(n_cols) : "memory");
}

__device__ __forceinline__ void tc05_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc05_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.  accumulate == 0 overwrites D.
__device__ __forceinline__ void tc05_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrive (count 1) on an mbarrier of this CTA when all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void tc05_commit(uint32_t mbar_addr) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar_addr)
                 : "memory");
}

// 16 consecutive FP32 accumulator columns of this thread's row (lane quadrant = warp index % 4).
__device__ __forceinline__ void tc05_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// The same without the wait: several loads can be in flight before one tc05_wait_ld().
__device__ __forceinline__ void tc05_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tc05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a K-major 128-byte-swizzled tile.
__device__ __forceinline__ uint32_t tc05_sw128_offset(int row, int chunk) {
    return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}

// ---------------------------------------------------------------------------------------------------------------
// Block-scaled MMA (kind::mxf4: E2M1 operands, one UE8M0 scale per 32 K-elements, scales in tensor memory)
// ---------------------------------------------------------------------------------------------------------------
// Operand tiles are K-major, 128-byte swizzled like the fp16 ones; a 128-byte row now holds 256 E2M1 values and one
// MMA consumes 64 of them (32 bytes), so K-step j still adds 32 j bytes to the descriptor's start address.
//
// Scale factors of a 128-row x 128-K-element piece (4 scale bytes per row) form a 512-byte "atom" in shared
// memory: byte (row r, scale j) at (r % 32) * 16 + (r / 32) * 4 + j.  tcgen05.cp (32x128b, warpx4) copies an atom
// into 4 tensor-memory columns (lane = r % 32 replicated in the four lane quadrants, column = r / 32, byte = j);
// an MMA with K = 64 uses two of the four bytes, selected by the scale-factor id field of the instruction
// descriptor (0: bytes 0-1, 2: bytes 2-3).

// Instruction descriptor of kind::mxf4 block-scaled: B scale id at bit 4, A / B formats 1 (E2M1) at bits 7 / 10,
// N >> 3 at bit 17, scale format 1 (UE8M0) at bit 23, M >> 4 at bit 24, A scale id at bit 29.
__device__ __forceinline__ uint32_t tc05_idesc_mxf4(int m, int n, int a_sf_id, int b_sf_id) {
    return ((uint32_t)b_sf_id << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) |
           ((uint32_t)(m >> 4) << 24) | ((uint32_t)a_sf_id << 29);
}

// Shared-memory descriptor of one scale atom: 32 rows x 16 bytes, no swizzle, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t tc05_desc_scale_atom(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)(128 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// Scale atom: shared memory -> 4 tensor-memory columns starting at `tmem_col`.  Issued by ONE thread; ordered with
// the MMAs that thread issues afterwards.
__device__ __forceinline__ void tc05_copy_scale_atom(uint32_t tmem_col, uint32_t smem_atom_addr) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col),
                 "l"(tc05_desc_scale_atom(smem_atom_addr))
                 : "memory");
}

__device__ __forceinline__ void tc05_mma_mxf4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.b32 p, %6, 0;\n"
        " tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
        : "memory");
}

// Byte offset of scale (row r, scale j of 4) inside a scale atom.
__device__ __forceinline__ uint32_t tc05_scale_atom_offset(int r, int j) {
    return (uint32_t)((r & 31) * 16 + (r >> 5) * 4 + j);
}

}  // namespace dsv4
