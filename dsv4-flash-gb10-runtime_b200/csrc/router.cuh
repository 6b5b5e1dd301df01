// Router for one token, executed by one warp: scores, top-k (descending, ties to the lowest expert index),
// normalised weights.  Shared by the stand-alone router kernel and by the decode kernel's fused prologue.
//   score_func 0: softmax over all experts; the weights are renormalised over the k picks, so the softmax
//                 denominator cancels: w_j = exp(l_j - max) / sum_picks exp(l - max).
//   score_func 1: s = sqrt(softplus(logit)), w_j = s_j / (sum_picks s + eps) * scaling.
// Selection is done on the score (for softmax: on the logit, which orders identically).  All arithmetic is
// FP32; the weights agree with a float64 evaluation to a few ulp.
#pragma once

#include "gemv_engine.cuh"

namespace dsv4 {

struct RouteArgs {
    const float* logits;   // [n_tokens, n_experts]; nullptr = no routing in this launch
    int n_experts;
    int k;
    int score_func;
    float eps;
    float scaling;
    int* ids_out;          // [n_tokens, k]
    float* w_out;          // [n_tokens, k]
};

// PL: scores held per lane (experts <= 32 * PL).  On return lane j < k holds pick j in (id, w).
template <int PL>
__device__ __forceinline__ void route_token(const float* __restrict__ row, int n_experts, int k, int score_func,
                                            float eps, float scaling, int lane, int& id, float& w) {
    float s[PL];
    float row_max = -INFINITY;
#pragma unroll
    for (int i = 0; i < PL; ++i) {
        const int idx = i * 32 + lane;
        s[i] = idx < n_experts ? __ldcg(row + idx) : -INFINITY;
        row_max = fmaxf(row_max, s[i]);
    }
    if (score_func == 0) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(kFullMask, row_max, off));
    } else {
#pragma unroll
        for (int i = 0; i < PL; ++i)
            if (s[i] != -INFINITY) {
                const float g = s[i];
                s[i] = sqrtf(fmaxf(g, 0.0f) + log1pf(expf(-fabsf(g))));
            }
    }
    float my_score = 0.f, sum = 0.f;
    id = -1;
    for (int j = 0; j < k; ++j) {
        float best = -INFINITY;
        int best_idx = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PL; ++i)
            if (s[i] > best) { best = s[i]; best_idx = i * 32 + lane; }   // strict: lowest index wins in a lane
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ob = __shfl_xor_sync(kFullMask, best, off);
            const int oi = __shfl_xor_sync(kFullMask, best_idx, off);
            if (ob > best || (ob == best && oi < best_idx)) { best = ob; best_idx = oi; }
        }
        if (lane == j) { my_score = best; id = best_idx; }
        if ((best_idx & 31) == lane) {
#pragma unroll
            for (int i = 0; i < PL; ++i)
                if (i == (best_idx >> 5)) s[i] = -INFINITY;
        }
        sum += score_func == 0 ? __expf(best - row_max) : best;
    }
    w = score_func == 0 ? __expf(my_score - row_max) / sum : my_score / (sum + eps) * scaling;
}

}  // namespace dsv4
