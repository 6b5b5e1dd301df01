// Arguments shared by the routed-expert decode kernels.
#pragma once

#include <cuda_bf16.h>
#include <cstdint>

namespace dsv4 {

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
    unsigned long long* mid8;        // single-kernel path: [E, H] {FP32 value, tag} words (same workspace as mid)
    uint32_t* sync;                  // single-kernel path: generation word (workspace tail)
    uint32_t spin_limit;             // polls after which a device-side wait gives up
    int phantom;                     // extra (never arriving) producers to wait for: test of the give-up path only
};

}  // namespace dsv4
