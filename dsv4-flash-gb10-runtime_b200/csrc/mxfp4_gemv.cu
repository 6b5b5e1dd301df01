// libmxfp4_gemv.so — MXFP4 dense GEMV, M = 1, for B200 (sm_100a).
// Drop-in for the reference's kernel/mxfp4-dense/mxfp4_gemv.cu:131-166 (same symbol, argument order and
// return codes).  The kernel itself is in dense_gemv.cuh.
#include "dense_gemv.cuh"

using namespace dsv4;

// y[n] = bf16(sum_k W[n,k] x[k]); W_packed [N, K/2] two E2M1 per byte (low nibble = even k),
// W_scale [N, K/32] E8M0, row strides in bytes.
// Returns 0, or -1 (K not a positive multiple of 32), -2 (K > 8192), -3 (launch failure) as the reference
// does; added: -8 for a null pointer or negative N.  N == 0 is a no-op.
DSV4_API int mxfp4_gemv_m1(const __nv_bfloat16* x, const uint8_t* W_packed, const uint8_t* W_scale, int K, int N,
                           int64_t packed_row_stride_bytes, int64_t scale_row_stride_bytes, __nv_bfloat16* y,
                           cudaStream_t stream) {
    if (K <= 0 || K % 32 != 0) {
        std::fprintf(stderr, "mxfp4_gemv_m1: K=%d not a positive multiple of 32\n", K);
        return -1;
    }
    if (K > 8192) {
        std::fprintf(stderr, "mxfp4_gemv_m1: K=%d > 8192\n", K);
        return -2;
    }
    if (N == 0) return 0;
    if (N < 0 || !x || !W_packed || !W_scale || !y) {
        std::fprintf(stderr, "mxfp4_gemv_m1: null pointer or N=%d < 0\n", N);
        return -8;
    }
    DenseArgs a;
    a.x = x; a.w = W_packed; a.s = W_scale; a.K = K; a.N = N;
    a.w_stride = packed_row_stride_bytes; a.s_stride = scale_row_stride_bytes; a.y = y;
    const cudaError_t err = dense_launch<Fp4Format, Fp4Scale>(a, stream);
    if (err != cudaSuccess) {
        std::fprintf(stderr, "mxfp4_gemv_m1 launch failed: %s\n", cudaGetErrorString(err));
        return -3;
    }
    return 0;
}
