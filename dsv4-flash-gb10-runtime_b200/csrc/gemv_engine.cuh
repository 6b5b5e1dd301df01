// Shared device-side building blocks of the B200 (sm_100a) quantized-weight GEMV kernels.
//
// Design (decode is HBM-bound: every weight byte is read exactly once):
//   * one lane owns ONE 16-byte weight block of the reduction axis (32 E2M1 nibbles or
//     16 E4M3 bytes) and keeps the matching activation block in registers as fp16x2,
//     pre-scaled by a per-block power of two so that fp16 never overflows or flushes;
//   * a warp therefore streams 512 contiguous bytes of a weight row per 128-bit load,
//     and walks DOWN the rows of the matrix with many such loads in flight
//     (two register buffers: the next batch is requested before the current is consumed);
//   * E2M1 / E4M3 are decoded by the hardware converters (cvt.rn.f16x2.e2m1x2 /
//     cvt.rn.f16x2.e4m3x2): one instruction per two weights, no LUT traffic;
//   * products of a block are summed in four short fp16x2 chains (each E2M1 x bf16 product
//     is exact in fp16), the 32-element block sum is widened to FP32, multiplied by the
//     E8M0 scale and from there on everything (cross-block, cross-lane, cross-expert) is FP32;
//   * cross-lane sums use a multi-value butterfly (9 shuffles per 8 rows instead of 40).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cstdint>

#define DSV4_API extern "C" __attribute__((visibility("default")))

namespace dsv4 {

constexpr unsigned kFullMask = 0xffffffffu;

// ---------------------------------------------------------------------------------------------
// memory access helpers
// ---------------------------------------------------------------------------------------------

// Weights are read once: bypass L1 allocation so the activation vectors stay cached.
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t ldg_stream_u8(const uint8_t* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u8 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Programmatic dependent launch: everything before pdl_wait() may overlap the tail of the
// previous kernel in the stream; it must only touch memory that kernel does not write.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// number formats
// ---------------------------------------------------------------------------------------------

// E8M0 byte -> 2^(b-127).  Byte 0 is the FP32 subnormal 2^-127 (built from bits, never by
// exp2f, so it is exact), byte 0xFF contributes 0 like the kernels this library replaces.
__device__ __forceinline__ float e8m0_to_float(uint32_t b) {
    uint32_t bits = b << 23;
    bits = (b == 0u) ? 0x00400000u : bits;
    bits = (b == 255u) ? 0u : bits;
    return __uint_as_float(bits);
}

// Same byte with the OCP meaning of 0xFF (NaN); used by the dequantisation export only.
__device__ __forceinline__ float e8m0_to_float_nan(uint32_t b) {
    uint32_t bits = b << 23;
    bits = (b == 0u) ? 0x00400000u : bits;
    bits = (b == 255u) ? 0x7fc00000u : bits;
    return __uint_as_float(bits);
}

// Four bytes = eight E2M1 nibbles -> four fp16x2.  Byte j yields (element 2j, element 2j+1):
// the low nibble is the even element and lands in the low half.
__device__ __forceinline__ void e2m1x8_to_h2x4(uint32_t w, __half2 (&h)[4]) {
    uint32_t r0, r1, r2, r3;
    asm("{\n"
        " .reg .b8 q0, q1, q2, q3;\n"
        " mov.b32 {q0, q1, q2, q3}, %4;\n"
        " cvt.rn.f16x2.e2m1x2 %0, q0;\n"
        " cvt.rn.f16x2.e2m1x2 %1, q1;\n"
        " cvt.rn.f16x2.e2m1x2 %2, q2;\n"
        " cvt.rn.f16x2.e2m1x2 %3, q3;\n"
        "}\n"
        : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
        : "r"(w));
    h[0] = *reinterpret_cast<__half2*>(&r0);
    h[1] = *reinterpret_cast<__half2*>(&r1);
    h[2] = *reinterpret_cast<__half2*>(&r2);
    h[3] = *reinterpret_cast<__half2*>(&r3);
}

// silu(g) * u of the decode kernels, one definition for all of them (their outputs are compared bit for bit).
// The quotient uses the fast division (2 ulp): executed by the whole warp for one lane's row, the IEEE sequence was
// 0.1 us of a 20 us layer.  1 + exp(-g) is never below 1; for g below -88 it is infinite and the quotient 0.
__device__ __forceinline__ float swiglu_f32(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// One byte = two E2M1 nibbles -> (low nibble, high nibble) as floats; for the byte-at-a-time paths.
__device__ __forceinline__ float2 e2m1x2_to_float2(uint32_t byte) {
    const __half2_raw raw = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)(byte & 0xffu), __NV_E2M1);
    return __half22float2(*reinterpret_cast<const __half2*>(&raw));
}

// One E4M3 byte -> float.
__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
    const __half_raw raw = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(byte & 0xffu), __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&raw));
}

// Four E4M3 bytes -> two fp16x2 (exact: E4M3 is a subset of fp16).
__device__ __forceinline__ void e4m3x4_to_h2x2(uint32_t w, __half2 (&h)[2]) {
    uint32_t r0, r1;
    asm("{\n"
        " .reg .b16 lo, hi;\n"
        " mov.b32 {lo, hi}, %2;\n"
        " cvt.rn.f16x2.e4m3x2 %0, lo;\n"
        " cvt.rn.f16x2.e4m3x2 %1, hi;\n"
        "}\n"
        : "=r"(r0), "=r"(r1)
        : "r"(w));
    h[0] = *reinterpret_cast<__half2*>(&r0);
    h[1] = *reinterpret_cast<__half2*>(&r1);
}

// ---------------------------------------------------------------------------------------------
// weight formats: what one 16-byte lane block means
// ---------------------------------------------------------------------------------------------

struct Fp4Format {                         // MXFP4: 32 E2M1 per 16 bytes, one E8M0 per block
    static constexpr int kElems = 32;      // elements per 16-byte block
    static constexpr int kPairs = 16;      // fp16x2 activation registers per block
    // scaled |x| <= 2^8: 16 products of at most 6*256 per fp16 lane stay below 65504
    static constexpr int kActExp = 7;
    __device__ static __forceinline__ float dot(const uint4& w, const __half2 (&x)[kPairs]) {
        const uint32_t word[4] = {w.x, w.y, w.z, w.w};
        __half2 acc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h[4];
            e2m1x8_to_h2x4(word[i], h);
            acc[i] = __hmul2(h[0], x[4 * i + 0]);
            acc[i] = __hfma2(h[1], x[4 * i + 1], acc[i]);
            acc[i] = __hfma2(h[2], x[4 * i + 2], acc[i]);
            acc[i] = __hfma2(h[3], x[4 * i + 3], acc[i]);
        }
        const float2 f = __half22float2(__hadd2(__hadd2(acc[0], acc[1]), __hadd2(acc[2], acc[3])));
        return f.x + f.y;
    }
};

struct Fp8Format {                         // E4M3: 16 bytes = 16 elements
    static constexpr int kElems = 16;
    static constexpr int kPairs = 8;
    // scaled |x| < 2: 8 products of at most 448*2 per fp16 lane stay below 65504
    static constexpr int kActExp = 0;
    __device__ static __forceinline__ float dot(const uint4& w, const __half2 (&x)[kPairs]) {
        const uint32_t word[4] = {w.x, w.y, w.z, w.w};
        __half2 acc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h[2];
            e4m3x4_to_h2x2(word[i], h);
            acc[i] = __hmul2(h[0], x[2 * i + 0]);
            acc[i] = __hfma2(h[1], x[2 * i + 1], acc[i]);
        }
        const float2 f01 = __half22float2(__hadd2(acc[0], acc[1]));
        const float2 f23 = __half22float2(__hadd2(acc[2], acc[3]));
        return (f01.x + f01.y) + (f23.x + f23.y);
    }
};

// ---------------------------------------------------------------------------------------------
// lane-resident activation block
// ---------------------------------------------------------------------------------------------

template <class Fmt>
struct ActBlock {
    __half2 h[Fmt::kPairs];   // activations of this lane's block, times 1/scale, as fp16x2
    float scale;              // power of two; multiply block sums by it
};

// Scale chosen from the block's largest magnitude so that it maps into [2^kActExp, 2^(kActExp+1)).
template <class Fmt>
__device__ __forceinline__ void act_block_finish(const float (&v)[Fmt::kElems], ActBlock<Fmt>& a) {
    uint32_t amax_bits = 0;
#pragma unroll
    for (int i = 0; i < Fmt::kElems; ++i) amax_bits = max(amax_bits, __float_as_uint(v[i]) & 0x7fffffffu);
    int e = (int)(amax_bits >> 23) - Fmt::kActExp;   // biased exponent of the scale
    e = min(max(e, 1), 253);
    a.scale = __uint_as_float((uint32_t)e << 23);
    const float inv = __uint_as_float((uint32_t)(254 - e) << 23);
#pragma unroll
    for (int i = 0; i < Fmt::kPairs; ++i) a.h[i] = __floats2half2_rn(v[2 * i] * inv, v[2 * i + 1] * inv);
}

// bf16 source (the caller's activation vector); ld.cg: written by an earlier kernel.
template <class Fmt>
__device__ __forceinline__ void act_block_load_bf16(const __nv_bfloat16* src, bool valid, ActBlock<Fmt>& a) {
    float v[Fmt::kElems];
#pragma unroll
    for (int i = 0; i < Fmt::kElems / 8; ++i) {
        uint4 q = make_uint4(0, 0, 0, 0);
        if (valid) q = __ldcg(reinterpret_cast<const uint4*>(src) + i);
        const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[8 * i + 2 * j + 0] = __uint_as_float(u[j] << 16);
            v[8 * i + 2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
        }
    }
    act_block_finish<Fmt>(v, a);
}

// fp32 source (the SwiGLU intermediate in the workspace).
template <class Fmt>
__device__ __forceinline__ void act_block_load_f32(const float* src, bool valid, ActBlock<Fmt>& a) {
    float v[Fmt::kElems];
#pragma unroll
    for (int i = 0; i < Fmt::kElems / 4; ++i) {
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if (valid) q = __ldcg(reinterpret_cast<const float4*>(src) + i);
        v[4 * i + 0] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
    }
    act_block_finish<Fmt>(v, a);
}

// ---------------------------------------------------------------------------------------------
// lane-resident activations for a whole row: BPL blocks per lane, block j of the lane is block
// (lane + 32 j) of the vector, so that load j of a warp covers 512 contiguous bytes of a weight row
// ---------------------------------------------------------------------------------------------

template <class Fmt, int BPL>
struct LaneAct {
    __half2 h[BPL][Fmt::kPairs];   // activations times 1/scale, as fp16x2
    float scale;                   // one power of two for all the lane's blocks
};

__device__ __forceinline__ void load8_as_float(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 q = __ldcg(reinterpret_cast<const uint4*>(p));
    const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[2 * j + 0] = __uint_as_float(u[j] << 16);
        v[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
    }
}

__device__ __forceinline__ void load8_as_float(const float* p, float (&v)[8]) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldcg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// Elem is __nv_bfloat16 (the caller's activation vector) or float (the SwiGLU intermediate).
// Two passes over the lane's elements (largest magnitude, then convert) keep the register need small;
// the vector is at most 16 KB and sits in L2.
template <class Fmt, int BPL, class Elem>
__device__ __forceinline__ void lane_act_load(const Elem* x, int lane, int n_blk, LaneAct<Fmt, BPL>& a) {
    uint32_t amax_bits = 0;
#pragma unroll
    for (int j = 0; j < BPL; ++j) {
        const int blk = lane + 32 * j;
        if (blk < n_blk) {
#pragma unroll
            for (int c = 0; c < Fmt::kElems / 8; ++c) {
                float v[8];
                load8_as_float(x + (size_t)blk * Fmt::kElems + 8 * c, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) amax_bits = max(amax_bits, __float_as_uint(v[i]) & 0x7fffffffu);
            }
        }
    }
    int e = (int)(amax_bits >> 23) - Fmt::kActExp;   // biased exponent of the scale
    e = min(max(e, 1), 253);
    a.scale = __uint_as_float((uint32_t)e << 23);
    const float inv = __uint_as_float((uint32_t)(254 - e) << 23);
#pragma unroll
    for (int j = 0; j < BPL; ++j) {
        const int blk = lane + 32 * j;
#pragma unroll
        for (int c = 0; c < Fmt::kElems / 8; ++c) {
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (blk < n_blk) load8_as_float(x + (size_t)blk * Fmt::kElems + 8 * c, v);
#pragma unroll
            for (int i = 0; i < 4; ++i) a.h[j][4 * c + i] = __floats2half2_rn(v[2 * i] * inv, v[2 * i + 1] * inv);
        }
    }
}

// E8M0 byte -> float for the GEMV hot path: 0xFF contributes 0 (as in the kernels this library replaces);
// byte 0 gives 0 instead of 2^-127, a value no product with a bf16 activation can lift above 1e-36.
__device__ __forceinline__ float e8m0_to_float_fast(uint32_t b) {
    const uint32_t bits = b << 23;
    return __uint_as_float(b == 255u ? 0u : bits);
}

// ---------------------------------------------------------------------------------------------
// cross-lane reduction of N values at once (N in {1,2,4,8,16})
// ---------------------------------------------------------------------------------------------
// On return the sum of v[i] over the warp is in v[0] of the lanes for which
// multi_reduce_owner(lane, N) is true; that lane holds value index multi_reduce_index(lane, N).
template <int N>
__device__ __forceinline__ void multi_reduce(float (&v)[N], int lane) {
    int off = 16;
#pragma unroll
    for (int n = N; n > 1; n >>= 1, off >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float send = upper ? v[i] : v[i + n / 2];
            const float keep = upper ? v[i + n / 2] : v[i];
            v[i] = keep + __shfl_xor_sync(kFullMask, send, off);
        }
    }
#pragma unroll
    for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(kFullMask, v[0], off);
}

template <int N>
__device__ __forceinline__ bool multi_reduce_owner(int lane) {
    // the lane bits not consumed by the halving steps must be zero
    return (lane & ((32 / N) - 1)) == 0;
}

template <int N>
__device__ __forceinline__ int multi_reduce_index(int lane) {
    // halving step s (lane bit 16>>s) selected the upper half of what was left
    int idx = 0;
    int off = 16;
#pragma unroll
    for (int n = N; n > 1; n >>= 1, off >>= 1) idx += (lane & off) ? n / 2 : 0;
    return idx;
}

}  // namespace dsv4
