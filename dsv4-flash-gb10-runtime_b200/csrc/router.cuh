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

// Score of one expert from its logit (score_func 1; for softmax the logit itself orders and weighs).
__device__ __forceinline__ float route_score(float g, int score_func) {
    return score_func == 0 ? g : sqrtf(fmaxf(g, 0.0f) + log1pf(expf(-fabsf(g))));
}

// Order-preserving integer key of a score; 0 = never picked (NaN, -inf).
__device__ __forceinline__ uint32_t route_key(float s) {
    const uint32_t bits = __float_as_uint(s);
    return (s != s || s == -INFINITY) ? 0u : (bits ^ ((bits >> 31) ? 0xffffffffu : 0x80000000u));
}
__device__ __forceinline__ float route_key_score(uint32_t key) {
    return key != 0u ? __uint_as_float((key >> 31) ? (key ^ 0x80000000u) : ~key) : -INFINITY;
}

// Weight of pick `lane` (< k) from the picks' scores, by one warp: lane j holds pick j's score, `top` is the largest
// score (pick 0's).  The same sum order wherever it is called, so that the fused and the stand-alone router agree
// bit for bit.
__device__ __forceinline__ float route_weight(float my_score, float top, int k, int score_func, float eps,
                                              float scaling, int lane) {
    const float mine = lane < k ? (score_func == 0 ? __expf(my_score - top) : my_score) : 0.f;
    float sum = mine;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(kFullMask, sum, off);
    return score_func == 0 ? mine / sum : mine / (sum + eps) * scaling;
}

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
            if (s[i] != -INFINITY) s[i] = route_score(s[i], 1);
    }
    // Top-k by k rounds of warp-wide arg-max on order-preserving integer keys (redux.sync): largest score, lowest
    // expert index on ties; NaN scores are never picked.
    uint32_t key[PL];
#pragma unroll
    for (int i = 0; i < PL; ++i) key[i] = route_key(s[i]);
    float my_score = 0.f;
    id = -1;
    // the lane's best key and where it sits: recomputed only by the lane that has just given a pick away
    uint32_t best = 0;
    int best_i = 0;
#pragma unroll
    for (int i = 0; i < PL; ++i)
        if (key[i] > best) { best = key[i]; best_i = i; }                 // strict: lowest index wins in a lane
    for (int j = 0; j < k; ++j) {
        const uint32_t top = __reduce_max_sync(kFullMask, best);
        const int cand = (best == top && top != 0u) ? best_i * 32 + lane : 0x7fffffff;
        // the lane holding it: a vote; only an exact tie between lanes needs a second reduction (lowest index wins)
        const uint32_t holders = __ballot_sync(kFullMask, cand != 0x7fffffff);
        int win = 0x7fffffff;
        if (holders != 0u)
            win = (holders & (holders - 1u)) == 0u ? __shfl_sync(kFullMask, cand, __ffs(holders) - 1)
                                                   : __reduce_min_sync(kFullMask, cand);
        const uint32_t bits = (top >> 31) ? (top ^ 0x80000000u) : ~top;
        const float best_score = top != 0u ? __uint_as_float(bits) : -INFINITY;
        if (lane == j) { my_score = best_score; id = win != 0x7fffffff ? win : 0; }
        if (cand == win && win != 0x7fffffff) {
            best = 0;
#pragma unroll
            for (int i = 0; i < PL; ++i) {
                if (i == best_i) key[i] = 0u;
            }
            best_i = 0;
#pragma unroll
            for (int i = 0; i < PL; ++i)
                if (key[i] > best) { best = key[i]; best_i = i; }
        }
    }
    w = route_weight(my_score, row_max, k, score_func, eps, scaling, lane);
}

}  // namespace dsv4
