/* C ABI of the B200 (sm_100a) quantized-weight GEMV libraries.
 *
 * Three shared objects carry the file names and symbols the reference's callers load
 * (its ctypes bindings, and its C++ engine through dlsym / a global-namespace extern):
 *
 *   libmxfp4_grouped_gemv.so   mxfp4_grouped_gemv_topk, mxfp4_grouped_workspace_bytes
 *   libmxfp4_gemv.so           mxfp4_gemv_m1
 *   libfp8_e4m3_gemv.so        fp8_e4m3_gemv_m1
 *
 * Conventions, identical to the reference: every pointer is DEVICE memory owned by the caller; nothing is
 * allocated, freed or retained; work is enqueued on `stream` and the call returns without synchronising;
 * the return value is 0 on success and negative on a rejected argument or a failed launch (message on stderr);
 * outputs are fully overwritten; workspace contents are undefined afterwards and need no initialisation.  The entry
 * points keep no state of a call in the library: they are re-entrant, and calls from any number of streams and host
 * threads may overlap on a device as long as each has its own workspace (the kernels of the grouped entries wait on
 * words inside that workspace only).  `stream` is a cudaStream_t passed as void*.
 * bf16 values are passed as uint16_t bit patterns (= __nv_bfloat16).
 *
 * Alignment: x, the packed-weight bases and the workspace of the grouped entry must be 16-byte aligned
 * (cudaMalloc and torch allocations are); the dense entries take any alignment and stride (a slower
 * byte-wise kernel runs when a base or row stride is not a multiple of 16).
 */
#ifndef DSV4_B200_H
#define DSV4_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- libmxfp4_grouped_gemv.so ------------------------------------------------------------------------- */

/* Replaces kernel/mxfp4-routed/mxfp4_grouped_gemv.cu:294-403.
 * out[o] = bf16( sum_e rweights[e] * W2_e[o,:] . ( silu(W1_e x) * (W3_e x) ) ), e < n_exp, experts stacked:
 * W1/W3 packed [n_exp, hidden, K_in/2], scale [n_exp, hidden, K_in/32]; W2 packed [n_exp, out_dim, hidden/2],
 * scale [n_exp, out_dim, hidden/32].  Packed bytes hold two E2M1 values (low nibble = even index), scales are
 * E8M0 bytes (2^(b-127); 0xFF contributes 0).
 * Returns -1 K_in % 32, -2 hidden % 32, -3 K_in or hidden > 4096, -4 n_exp != 6, -5/-6 launch failure (as the
 * reference), -8 null / misaligned pointer or out_dim <= 0.
 * workspace: mxfp4_grouped_workspace_bytes() bytes (n_exp * hidden * 8 + 64 here, against the reference's
 * n_exp * hidden * 2 + out_dim * 4: callers size it through the query, as the reference's callers do). */
int mxfp4_grouped_gemv_topk(const uint16_t* x, const uint8_t* W1_packed, const uint8_t* W3_packed,
                            const uint8_t* W2_packed, const uint8_t* W1_scale, const uint8_t* W3_scale,
                            const uint8_t* W2_scale, const float* rweights, int K_in, int hidden, int out_dim,
                            int n_exp, uint16_t* out, void* workspace, void* stream);

/* Has no counterpart in the reference.  mxfp4_grouped_gemv_topk for hosts that cannot supply a workspace at call
 * time (all free HBM already given to the expert bank and KV cache, or a decode thread that must stay out of
 * cudaMalloc because it synchronises the device): the intermediate lives in a 192 KB array inside the library
 * image, present on every GPU that loads the library.  Allocates and frees nothing.  Limits: n_exp == 6,
 * hidden <= 4096 (-10 beyond that).  The first call on a device fetches the array's address: make it before any
 * stream capture on that device.  All calls on a device share the array, so calls whose kernels overlap on the GPU
 * race; serialise them or use the workspace entry.  -11 if the array's address cannot be obtained; other codes as
 * mxfp4_grouped_gemv_topk, whose result it reproduces bit for bit. */
int mxfp4_grouped_gemv_topk_static(const uint16_t* x, const uint8_t* W1_packed, const uint8_t* W3_packed,
                                   const uint8_t* W2_packed, const uint8_t* W1_scale, const uint8_t* W3_scale,
                                   const uint8_t* W2_scale, const float* rweights, int K_in, int hidden, int out_dim,
                                   int n_exp, uint16_t* out, void* stream);

/* Replaces kernel/mxfp4-routed/mxfp4_grouped_gemv.cu:406-409.  Bytes the caller must provide as `workspace`. */
size_t mxfp4_grouped_workspace_bytes(int n_exp, int hidden, int out_dim);

/* Added (no counterpart; removes the gather of kernel/cpp-engine-mxfp4/routed.cu:266-283): the same FFN with the
 * n_exp experts (1..8) picked by DEVICE index array `topk_ids` from bank tensors stacked over all experts. */
int mxfp4_grouped_gemv_topk_ids(const uint16_t* x, const uint8_t* bank_W1_packed, const uint8_t* bank_W3_packed,
                                const uint8_t* bank_W2_packed, const uint8_t* bank_W1_scale,
                                const uint8_t* bank_W3_scale, const uint8_t* bank_W2_scale, const int* topk_ids,
                                const float* rweights, int K_in, int hidden, int out_dim, int n_exp, uint16_t* out,
                                void* workspace, void* stream);

/* Added (profiling, no counterpart): the call above restricted to one of its two kernels so that each can be timed
 * alone.  stage_mask 1 = gate/up + SwiGLU (fills the workspace), 2 = down + combine (reads it), 3 = both; -9 otherwise. */
int mxfp4_grouped_gemv_topk_ids_stages(const uint16_t* x, const uint8_t* bank_W1_packed,
                                       const uint8_t* bank_W3_packed, const uint8_t* bank_W2_packed,
                                       const uint8_t* bank_W1_scale, const uint8_t* bank_W3_scale,
                                       const uint8_t* bank_W2_scale, const int* topk_ids, const float* rweights,
                                       int K_in, int hidden, int out_dim, int n_exp, uint16_t* out, void* workspace,
                                       int stage_mask, void* stream);

/* Added (replaces the host round trip of kernel/cpp-engine-mxfp4/routed.cu:156-208): router scores, top-k and
 * weights on the device.  logits FP32 [n_tokens, n_experts]; score_func 0 = softmax renormalised over the picks,
 * 1 = sqrt(softplus), w = s / (sum s + eps) * scaling; ids_out int32 [n_tokens, k] by descending score, ties to the
 * lowest index; w_out FP32 [n_tokens, k].  Returns -1 bad shape, -2 null pointer, -3 launch failure. */
int mxfp4_moe_route_topk(const float* logits, int n_tokens, int n_experts, int k, int score_func, float eps,
                         float scaling, int* ids_out, float* w_out, void* stream);

/* Added (no counterpart; the whole of kernel/cpp-engine-mxfp4/routed.cu:373-503 for one token in one call): router
 * + routed-expert FFN over a resident bank.  logits FP32 [n_experts]; k experts per token.  At K_in in {1024, 2048,
 * 4096}, hidden in {1024, 2048}, n_experts <= 256, k <= 6 the whole layer is ONE kernel launch (router inside),
 * otherwise a router kernel is launched first (3 launches).  After the call the workspace holds the picks: int32 ids
 * at byte offset k * hidden * 8, FP32 weights 32 bytes further.  `out` may be pinned host memory mapped on the device:
 * the kernel's stores are then the device-to-host transfer.  Return codes as mxfp4_grouped_gemv_topk_ids. */
int mxfp4_moe_decode_layer(const uint16_t* x, const uint8_t* bank_W1_packed, const uint8_t* bank_W3_packed,
                           const uint8_t* bank_W2_packed, const uint8_t* bank_W1_scale, const uint8_t* bank_W3_scale,
                           const uint8_t* bank_W2_scale, const float* logits, int n_experts, int score_func, float eps,
                           float scaling, int K_in, int hidden, int out_dim, int k, uint16_t* out, void* workspace,
                           void* stream);
size_t mxfp4_moe_decode_workspace_bytes(int k, int hidden, int out_dim);

/* Added (diagnostic; semantics of runtime/mxfp4_loader.py:272-309, scale 0xFF -> NaN): MXFP4 -> bf16 [rows, cols]. */
int mxfp4_dequant_bf16(const uint8_t* packed, const uint8_t* scale, long long rows, int cols, uint16_t* out,
                       void* stream);

/* Added (diagnostic, no counterpart): 0 unless a kernel of this library gave up on one of its bounded waits since
 * the last call (1 = a gate/up row never landed, 2 = a down row, 3 = an expert's intermediate never became complete),
 * or the router of mxfp4_moe_decode_layer found fewer than k pickable experts (4: NaN or -inf logits; the missing
 * picks run with weight 0, where the reference's host router aborts with -2, routed.cu:186-199);
 * clears the status.  A kernel that gives up writes NaN to its output rows, so the damage is also visible downstream.
 * Synchronises the device. */
int dsv4_b200_device_status(void);

/* Added (no counterpart): how the single-kernel path of the grouped entries is launched from now on in this process.
 * Its CTAs wait for one another's results, so all of them must be resident together:
 *   2 automatic (default): the first stream that calls on a device gets programmatic stream serialisation (the next
 *     layer's CTAs are scheduled while this layer's exit), every other stream a cooperative launch (co-residency
 *     guaranteed by the runtime) - any mix of streams makes progress;
 *   1 cooperative for every stream;  3 programmatic for every stream (only for callers with ONE stream per device);
 *   0 two chained kernels that wait for nothing.
 * The environment variable DSV4_B200_FUSED (auto | coop | pdl | 0) sets the initial mode.  Returns the previous mode,
 * -1 for another value. */
int dsv4_b200_set_launch_mode(int mode);

/* Added (test hook, no counterpart): poll budget of the device-side waits of the single-kernel path, and a number of
 * producers that never arrive (> 0: the next calls wait for data nobody writes, give up after `polls` polls, record
 * status 3 and write NaN - nothing faults or spins without a limit).  (0, 0) restores the defaults. */
int dsv4_b200_test_wait_limits(long long polls, int phantom_ctas);

/* ---- libmxfp4_gemv.so --------------------------------------------------------------------------------- */

/* Replaces kernel/mxfp4-dense/mxfp4_gemv.cu:131-166.  y[n] = bf16(sum_k W[n,k] x[k]); W_packed [N, K/2],
 * W_scale [N, K/32], row strides in bytes.  Returns -1 K % 32, -2 K > 8192, -3 launch failure (as the reference),
 * -8 null pointer or N < 0. */
int mxfp4_gemv_m1(const uint16_t* x, const uint8_t* W_packed, const uint8_t* W_scale, int K, int N,
                  int64_t packed_row_stride_bytes, int64_t scale_row_stride_bytes, uint16_t* y, void* stream);

/* ---- libfp8_e4m3_gemv.so ------------------------------------------------------------------------------ */

/* Replaces kernel/fp8-dense/fp8_e4m3_gemv.cu:132-174.  y[n] = bf16(sum_k e4m3(W[n,k]) 2^(S[n/128,k/128]-127) x[k]);
 * W_fp8 [N, K] raw E4M3, W_scale [N/128, K/128] E8M0, row strides in bytes.  Returns -1 K % 128, -2 N % 128,
 * -3 K > 16384, -4 launch failure (as the reference), -8 null pointer. */
int fp8_e4m3_gemv_m1(const uint16_t* x, const uint8_t* W_fp8, const uint8_t* W_scale, int K, int N,
                     int64_t weight_row_stride_bytes, int64_t scale_row_stride_bytes, uint16_t* y, void* stream);

/* Added: the same with FP32 tile scales [N/128, K/128] (row stride in bytes). */
int fp8_e4m3_gemv_m1_f32scale(const uint16_t* x, const uint8_t* W_fp8, const float* W_scale_f32, int K, int N,
                              int64_t weight_row_stride_bytes, int64_t scale_row_stride_bytes, uint16_t* y,
                              void* stream);

/* Added: several tokens and several independent groups in one launch - what the reference issues as a loop of
 * fp8_e4m3_gemv_m1 calls, one per token (runtime/dsv4_engine_mxfp4.py:310-320) and one per group of the grouped
 * output projection wo_a (kernel/cpp-engine-mxfp4/dsv4_engine_mxfp4_wire.cu:484-498):
 *   y[t, g*N + n] = bf16(sum_k e4m3(W[g*N + n, k]) 2^(S[(g*N + n)/128, k/128]-127) x[t, g*K + k]).
 * W_fp8 [n_groups*N, K], W_scale [n_groups*N/128, K/128] E8M0, row strides in bytes; x [n_tokens, >= n_groups*K] and
 * y [n_tokens, >= n_groups*N] bf16 with token strides in elements.  Every weight byte is read once per 8 tokens.  With
 * one token a row of y is bit-identical to fp8_e4m3_gemv_m1 for that group; with several tokens (FP32 tensor-core
 * sums) it agrees with it to the last bf16 step.  Returns -1 K % 128, -2 N % 128, -3 K > 16384,
 * -4 launch failure, -8 null pointer, n_groups < 1, n_tokens < 0, a token stride shorter than a row, or x / W /
 * a stride that is not 16-byte aligned (no byte-wise path here). */
int fp8_e4m3_gemv_batched(const uint16_t* x, const uint8_t* W_fp8, const uint8_t* W_scale, int K, int N,
                          int64_t weight_row_stride_bytes, int64_t scale_row_stride_bytes, int n_groups, int n_tokens,
                          int64_t x_token_stride, int64_t y_token_stride, uint16_t* y, void* stream);

/* Added: the shared expert's gated FFN for one token, all FP8 - what the reference composes from three
 * fp8_e4m3_gemv_m1 calls and an activation kernel (kernel/cpp-engine-mxfp4/dsv4_engine_mxfp4_wire.cu:523-556; Python
 * twin runtime/dsv4_engine_mxfp4.py:399-410): g = bf16(W1 x), u = bf16(W3 x),
 * act = bf16(silu(clamp(g, limit_gate)) * clamp(u, limit_up)), out = bf16(W2 act).  W1, W3 [hidden, K_in], W2
 * [out_dim, hidden] raw E4M3 with E8M0 128x128 tile scales, dense rows; a limit <= 0 switches that clamp off (the
 * C++ engine uses (10, 0), the Python engine (10, 10)).  workspace: fp8_e4m3_shared_swiglu_workspace_bytes(hidden)
 * bytes, 16-byte aligned like x and the weights.  Returns -1 bad shape (multiples of 128, <= 16384), -8 null or
 * misaligned pointer, -4 launch failure. */
size_t fp8_e4m3_shared_swiglu_workspace_bytes(int hidden);
int fp8_e4m3_shared_swiglu_m1(const uint16_t* x, const uint8_t* W1_fp8, const uint8_t* W1_scale, const uint8_t* W3_fp8,
                              const uint8_t* W3_scale, const uint8_t* W2_fp8, const uint8_t* W2_scale, int K_in,
                              int hidden, int out_dim, float limit_gate, float limit_up, uint16_t* out, void* workspace,
                              void* stream);

/* ---- libmxfp4_moe.so (added; no counterpart: the reference runs one token at a time) ---------------------- */

/* Routed-expert MoE layer for a batch of tokens on the tensor cores: out[t] = sum_j weights[t,j] * FFN_{ids[t,j]}(x[t]).
 * x bf16 [n_tokens, K_in]; bank tensors as in mxfp4_grouped_gemv_topk_ids; ids int32 [n_tokens, k]; weights FP32
 * [n_tokens, k]; out bf16 [n_tokens, out_dim].  A negative id marks a pair to skip (an expert-parallel caller masks
 * the experts of other ranks this way); an id >= n_experts is dropped and reported by mxfp4_moe_device_status().
 * K_in, hidden multiples of 256; out_dim multiple of 128; n_experts <= 1024.  Returns -1 bad shape, -2 null / misaligned pointer, -3 launch failure. */
int mxfp4_moe_forward(const uint16_t* x, const uint8_t* bank_W1_packed, const uint8_t* bank_W3_packed,
                      const uint8_t* bank_W2_packed, const uint8_t* bank_W1_scale, const uint8_t* bank_W3_scale,
                      const uint8_t* bank_W2_scale, const int* ids, const float* weights, int n_tokens, int n_experts,
                      int K_in, int hidden, int out_dim, int k, uint16_t* out, void* workspace, void* stream);
/* The same with the tensor-core path chosen by the caller: 1 = block-scaled MXFP4 MMAs fed with the packed weights as
 * stored, activations as three MXFP4 terms (what mxfp4_moe_forward uses unless DSV4_B200_MOE_PATH=fp16 is set);
 * 0 = fp16 MMAs with in-kernel dequantisation (exact operands). */
int mxfp4_moe_forward_path(int path, const uint16_t* x, const uint8_t* bank_W1_packed, const uint8_t* bank_W3_packed,
                           const uint8_t* bank_W2_packed, const uint8_t* bank_W1_scale, const uint8_t* bank_W3_scale,
                           const uint8_t* bank_W2_scale, const int* ids, const float* weights, int n_tokens,
                           int n_experts, int K_in, int hidden, int out_dim, int k, uint16_t* out, void* workspace,
                           void* stream);
size_t mxfp4_moe_forward_workspace_bytes(int n_tokens, int k, int K_in, int hidden, int out_dim, int n_experts);
/* 0, or the code a kernel of this library recorded since the last call (3 bad expert id, 4/5/6 a bounded wait ran
 * out); clears it.  Synchronises the device. */
int mxfp4_moe_device_status(void);
/* Microbenchmark of the instruction the batched layer is built on (no counterpart in the reference): tensor-pipe clocks
 * of one tcgen05.mma kind::mxf4 (M = 128, K = 64, N = n_cols: a multiple of 16 in 16 .. 256) with `scale_copies`
 * (0 .. 8) scale-atom copies in front of every four MMAs, one CTA per SM, `iters` rounds of four MMAs.  scratch: 8 bytes
 * of device memory; clocks_per_mma: HOST pointer.  Synchronises the stream.  FP4 peak of the device =
 * SMs x SM clock x 2 x 128 x n_cols x 64 / clocks.  Returns 0, -1 bad argument, -3 launch / execution failure. */
int mxfp4_moe_mma_rate(int n_cols, int scale_copies, int iters, void* scratch, double* clocks_per_mma, void* stream);
/* Stage timing of the block-scaled batched path (diagnostic, off by default, not thread-safe; no counterpart in the
 * reference).  mxfp4_moe_stage_timing(1) makes every later call record an event before its first kernel and after each
 * of its kernels (a timed call loses the overlap of programmatic dependent launch); it returns the previous setting.
 * mxfp4_moe_stage_times writes the microseconds of the last timed call's six stages - group, quantise x, gate/up GEMM,
 * quantise intermediate, down GEMM, combine - to us_out[0..6) (HOST pointer) after synchronising on the last event;
 * returns 0, or -1 when no timed call was made. */
int mxfp4_moe_stage_timing(int enable);
int mxfp4_moe_stage_times(float* us_out);

/* Expert parallel with the combine fused into the exchange: mxfp4_moe_forward over the gathered batch of
 * world * tokens_per_rank tokens (token t belongs to rank t / tokens_per_rank; ids index this rank's local bank, -1
 * where the expert lives on another rank); the combine kernel stores every token's partial row straight into the
 * receive buffer of its home rank (peer memory, plain stores over NVLink).  recv_ptrs: HOST array of `world` device
 * pointers, entry r = rank r's receive buffer, bf16 [world][tokens_per_rank][out_dim], mapped on this device.  After a
 * barrier over the ranks each rank calls mxfp4_moe_ep_sum on its own buffer.  Return codes as mxfp4_moe_forward. */
int mxfp4_moe_forward_ep(const uint16_t* x, const uint8_t* bank_W1_packed, const uint8_t* bank_W3_packed,
                         const uint8_t* bank_W2_packed, const uint8_t* bank_W1_scale, const uint8_t* bank_W3_scale,
                         const uint8_t* bank_W2_scale, const int* ids, const float* weights, int n_tokens, int n_experts,
                         int K_in, int hidden, int out_dim, int k, void* const* recv_ptrs, int world, int my_rank,
                         int tokens_per_rank, void* workspace, void* stream);

/* out[t] = bf16(sum of recv[r][t] over the ranks r that own one of token t's experts, ascending r).  recv bf16
 * [world][n_tokens][out_dim]; ids int32 [n_tokens, k] global expert ids of this rank's tokens; rank r owns experts
 * [r, r + 1) * experts_per_rank (the other ranks stored nothing for the token and are skipped). */
int mxfp4_moe_ep_sum(const uint16_t* recv, const int* ids, int k, int experts_per_rank, int world, int n_tokens,
                     int out_dim, uint16_t* out, void* stream);

/* Expert parallel with both sides over peer memory (no collective library on the path).  Every rank has published
 * its tokens in buffers mapped on all ranks: x bf16 [tokens_per_rank, K_in], ids int32 [tokens_per_rank, k] (global
 * expert ids), weights FP32 [tokens_per_rank, k]; x_ptrs / ids_ptrs / w_ptrs / recv_ptrs are HOST arrays of `world`
 * device pointers (entry r = rank r's buffer).  After a barrier over the ranks this call runs the rank's
 * n_experts_local experts over all world * tokens_per_rank tokens, reading each token from the rank that published
 * it and storing the partial rows into the home ranks' receive buffers as mxfp4_moe_forward_ep does; after a second
 * barrier every rank calls mxfp4_moe_ep_sum.  Block-scaled tensor-core path.  workspace:
 * mxfp4_moe_forward_ep2_workspace_bytes.  Return codes as mxfp4_moe_forward_ep. */
size_t mxfp4_moe_forward_ep2_workspace_bytes(int world, int tokens_per_rank, int k, int K_in, int hidden, int out_dim,
                                             int n_experts_local);
int mxfp4_moe_forward_ep2(void* const* x_ptrs, void* const* ids_ptrs, void* const* w_ptrs,
                          const uint8_t* bank_W1_packed, const uint8_t* bank_W3_packed, const uint8_t* bank_W2_packed,
                          const uint8_t* bank_W1_scale, const uint8_t* bank_W3_scale, const uint8_t* bank_W2_scale,
                          int tokens_per_rank, int n_experts_local, int K_in, int hidden, int out_dim, int k,
                          void* const* recv_ptrs, int world, int my_rank, void* workspace, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DSV4_B200_H */
