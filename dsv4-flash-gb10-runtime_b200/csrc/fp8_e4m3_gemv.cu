// libfp8_e4m3_gemv.so — FP8 E4M3 dense GEMV, M = 1, 128x128 block scales, for B200 (sm_100a).
// Drop-in for the reference's kernel/fp8-dense/fp8_e4m3_gemv.cu:132-174 (same symbol, argument order and
// return codes).  The kernel itself is in dense_gemv.cuh.
#include "dense_gemv.cuh"
#include "dense_mma_gemv.cuh"

using namespace dsv4;

// y[n] = bf16(sum_k e4m3(W[n,k]) * 2^(S[n/128,k/128]-127) * x[k]); W_fp8 [N, K] raw E4M3 bytes,
// W_scale [N/128, K/128] E8M0, row strides in bytes.
// Returns 0, or -1 (K % 128), -2 (N % 128), -3 (K > 16384), -4 (launch failure) as the reference does;
// added: -8 for a null pointer or negative sizes.  N == 0 is a no-op.
DSV4_API int fp8_e4m3_gemv_m1(const __nv_bfloat16* x, const uint8_t* W_fp8, const uint8_t* W_scale, int K, int N,
                              int64_t weight_row_stride_bytes, int64_t scale_row_stride_bytes, __nv_bfloat16* y,
                              cudaStream_t stream) {
    if (K <= 0 || K % 128 != 0) {
        std::fprintf(stderr, "fp8_e4m3_gemv_m1: K=%d not a positive multiple of 128\n", K);
        return -1;
    }
    if (N < 0 || N % 128 != 0) {
        std::fprintf(stderr, "fp8_e4m3_gemv_m1: N=%d not a multiple of 128\n", N);
        return -2;
    }
    if (K > 16384) {
        std::fprintf(stderr, "fp8_e4m3_gemv_m1: K=%d > 16384\n", K);
        return -3;
    }
    if (N == 0) return 0;
    if (!x || !W_fp8 || !W_scale || !y) {
        std::fprintf(stderr, "fp8_e4m3_gemv_m1: null pointer\n");
        return -8;
    }
    DenseArgs a;
    a.x = x; a.w = W_fp8; a.s = W_scale; a.K = K; a.N = N;
    a.w_stride = weight_row_stride_bytes; a.s_stride = scale_row_stride_bytes; a.y = y;
    const cudaError_t err = dense_launch<Fp8Format, Fp8Scale>(a, stream);
    if (err != cudaSuccess) {
        std::fprintf(stderr, "fp8_e4m3_gemv_m1 launch failed: %s\n", cudaGetErrorString(err));
        return -4;
    }
    return 0;
}

// Additive: the same GEMV with FP32 block scales (scale = amax / 448 style checkpoints) instead of E8M0 bytes.
// W_scale_f32 [N/128, K/128] FP32, its row stride in BYTES.  Same return codes as fp8_e4m3_gemv_m1, plus -8 when
// the scale pointer or stride is not 4-byte aligned.
DSV4_API int fp8_e4m3_gemv_m1_f32scale(const __nv_bfloat16* x, const uint8_t* W_fp8, const float* W_scale_f32, int K,
                                       int N, int64_t weight_row_stride_bytes, int64_t scale_row_stride_bytes,
                                       __nv_bfloat16* y, cudaStream_t stream) {
    if (K <= 0 || K % 128 != 0) return -1;
    if (N < 0 || N % 128 != 0) return -2;
    if (K > 16384) return -3;
    if (!x || !W_fp8 || !W_scale_f32 || !y || (reinterpret_cast<uintptr_t>(W_scale_f32) & 3u) ||
        (scale_row_stride_bytes & 3)) {
        std::fprintf(stderr, "fp8_e4m3_gemv_m1_f32scale: null pointer or misaligned FP32 scales\n");
        return -8;
    }
    if (N == 0) return 0;
    DenseArgs a;
    a.x = x; a.w = W_fp8; a.s = reinterpret_cast<const uint8_t*>(W_scale_f32); a.K = K; a.N = N;
    a.w_stride = weight_row_stride_bytes; a.s_stride = scale_row_stride_bytes; a.y = y;
    const cudaError_t err = dense_launch<Fp8Format, Fp8ScaleF32>(a, stream);
    if (err != cudaSuccess) {
        std::fprintf(stderr, "fp8_e4m3_gemv_m1_f32scale launch failed: %s\n", cudaGetErrorString(err));
        return -4;
    }
    return 0;
}

// Additive: the shared expert's gated FFN for one token, all FP8 (what the reference composes from three
// fp8_e4m3_gemv_m1 calls and an activation kernel: kernel/cpp-engine-mxfp4/dsv4_engine_mxfp4_wire.cu:523-556;
// Python twin runtime/dsv4_engine_mxfp4.py:399-410):
//   g = bf16(W1 x), u = bf16(W3 x), act = bf16(silu(clamp(g, limit_gate)) * clamp(u, limit_up)), out = bf16(W2 act).
// W1, W3 [hidden, K_in], W2 [out_dim, hidden] E4M3 bytes with E8M0 128x128 tile scales, rows dense (stride = row
// length).  limit_gate / limit_up <= 0 switch that clamp off: the C++ engine clamps the gate only (10, 0), the Python
// engine both (10, 10).  Two launches chained by programmatic dependent launch; `workspace` holds the activation:
// fp8_e4m3_shared_swiglu_workspace_bytes(hidden) bytes, 16-byte aligned.
// Returns 0, -1 (K_in, hidden or out_dim not a multiple of 128 or > 16384), -8 (null / misaligned pointer),
// -4 (launch failure).
DSV4_API size_t fp8_e4m3_shared_swiglu_workspace_bytes(int hidden) {
    return hidden > 0 ? (size_t)hidden * sizeof(__nv_bfloat16) : 0;
}

DSV4_API int fp8_e4m3_shared_swiglu_m1(const __nv_bfloat16* x, const uint8_t* W1_fp8, const uint8_t* W1_scale,
                                       const uint8_t* W3_fp8, const uint8_t* W3_scale, const uint8_t* W2_fp8,
                                       const uint8_t* W2_scale, int K_in, int hidden, int out_dim, float limit_gate,
                                       float limit_up, __nv_bfloat16* out, void* workspace, cudaStream_t stream) {
    auto bad = [](int v) { return v <= 0 || v % 128 != 0 || v > 16384; };
    if (bad(K_in) || bad(hidden) || bad(out_dim)) {
        std::fprintf(stderr, "fp8_e4m3_shared_swiglu_m1: unsupported shape K_in=%d hidden=%d out_dim=%d\n", K_in, hidden,
                     out_dim);
        return -1;
    }
    auto mis = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) != 0; };
    if (mis(x) || mis(W1_fp8) || mis(W3_fp8) || mis(W2_fp8) || !W1_scale || !W3_scale || !W2_scale || !out ||
        mis(workspace)) {
        std::fprintf(stderr, "fp8_e4m3_shared_swiglu_m1: null pointer or a tensor that is not 16-byte aligned\n");
        return -8;
    }
    __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(workspace);
    DenseArgs g, u, d;
    g.x = x; g.w = W1_fp8; g.s = W1_scale; g.K = K_in; g.N = hidden; g.w_stride = K_in; g.s_stride = K_in / 128; g.y = act;
    u = g; u.w = W3_fp8; u.s = W3_scale;
    d.x = act; d.w = W2_fp8; d.s = W2_scale; d.K = hidden; d.N = out_dim; d.w_stride = hidden; d.s_stride = hidden / 128;
    d.y = out;
    cudaError_t err = dense_dual_launch<Fp8Format, Fp8Scale>(g, u, limit_gate, limit_up, stream);
    if (err == cudaSuccess) err = dense_launch<Fp8Format, Fp8Scale>(d, stream);
    if (err != cudaSuccess) {
        std::fprintf(stderr, "fp8_e4m3_shared_swiglu_m1 launch failed: %s\n", cudaGetErrorString(err));
        return -4;
    }
    return 0;
}

// Additive: the FP8 GEMV for several tokens and several independent groups in one launch - what the reference
// issues as a loop of fp8_e4m3_gemv_m1 calls: one per token in the Python engine's _fp8_linear
// (runtime/dsv4_engine_mxfp4.py:310-320) and one per group for the grouped output projection wo_a
// (kernel/cpp-engine-mxfp4/dsv4_engine_mxfp4_wire.cu:484-498).
//   y[t, g*N + n] = bf16( sum_k e4m3(W[g*N + n, k]) * 2^(S[(g*N + n)/128, k/128] - 127) * x[t, g*K + k] )
// W_fp8 [n_groups*N, K], W_scale [n_groups*N/128, K/128] E8M0, row strides in bytes; x [n_tokens, >= n_groups*K],
// y [n_tokens, >= n_groups*N] bf16 with token strides in ELEMENTS.  n_groups = 1 is the batched GEMV; n_tokens = 1,
// n_groups = 8, K = 4096, N = 1024 is wo_a.  Every weight byte is read once per 8 tokens.  With one token a row of y is
// bit-identical to what fp8_e4m3_gemv_m1 returns for that group; with several tokens the sums are formed by FP32
// tensor-core MMAs (dense_mma_gemv.cuh) and agree with it to the last bf16 step.
// Returns 0, -1 (K % 128), -2 (N % 128), -3 (K > 16384), -4 (launch failure), -8 (null pointer, n_groups < 1,
// negative n_tokens, a token stride shorter than a row, or x / W / a stride that is not 16-byte aligned: this entry
// has no byte-wise path).  n_tokens == 0 or N == 0 is a no-op.
DSV4_API int fp8_e4m3_gemv_batched(const __nv_bfloat16* x, const uint8_t* W_fp8, const uint8_t* W_scale, int K, int N,
                                   int64_t weight_row_stride_bytes, int64_t scale_row_stride_bytes, int n_groups,
                                   int n_tokens, int64_t x_token_stride, int64_t y_token_stride, __nv_bfloat16* y,
                                   cudaStream_t stream) {
    if (K <= 0 || K % 128 != 0) {
        std::fprintf(stderr, "fp8_e4m3_gemv_batched: K=%d not a positive multiple of 128\n", K);
        return -1;
    }
    if (N < 0 || N % 128 != 0) {
        std::fprintf(stderr, "fp8_e4m3_gemv_batched: N=%d not a multiple of 128\n", N);
        return -2;
    }
    if (K > 16384) {
        std::fprintf(stderr, "fp8_e4m3_gemv_batched: K=%d > 16384\n", K);
        return -3;
    }
    if (n_groups < 1 || n_tokens < 0 || x_token_stride < (int64_t)n_groups * K || y_token_stride < (int64_t)n_groups * N) {
        std::fprintf(stderr, "fp8_e4m3_gemv_batched: bad group / token layout\n");
        return -8;
    }
    if (N == 0 || n_tokens == 0) return 0;
    if (!x || !W_fp8 || !W_scale || !y) {
        std::fprintf(stderr, "fp8_e4m3_gemv_batched: null pointer\n");
        return -8;
    }
    DenseMultiArgs m;
    m.a.x = x; m.a.w = W_fp8; m.a.s = W_scale; m.a.K = K; m.a.N = N;
    m.a.w_stride = weight_row_stride_bytes; m.a.s_stride = scale_row_stride_bytes; m.a.y = y;
    m.n_groups = n_groups; m.n_tok = n_tokens; m.x_tok = x_token_stride; m.y_tok = y_token_stride;
    const cudaError_t err = dense_multi_launch<Fp8Scale>(m, stream);
    if (err == cudaErrorInvalidValue) {
        (void)cudaGetLastError();
        std::fprintf(stderr, "fp8_e4m3_gemv_batched: x, W and the strides must be 16-byte aligned\n");
        return -8;
    }
    if (err != cudaSuccess) {
        std::fprintf(stderr, "fp8_e4m3_gemv_batched launch failed: %s\n", cudaGetErrorString(err));
        return -4;
    }
    return 0;
}
