// libmxfp4_moe.so — routed-expert MXFP4 MoE layer for a BATCH of tokens on B200 (sm_100a): batched decode and
// prefill.  No counterpart in the reference (its path is one token at a time,
// runtime/dsv4_engine_mxfp4.py:412-422 loops tokens); the arithmetic contract is the same FFN:
//   out[t] = sum_j w[t, j] * W2_e ( silu(W1_e x_t) * (W3_e x_t) ),  e = ids[t, j].
// Pipeline on the caller's stream: pairs grouped by expert; grouped GEMM 1 (gate/up + SwiGLU) and grouped GEMM 2
// (down, router weight applied) on tcgen05 tensor cores; per-token sum in the router's order.  Two tensor-core
// paths: block-scaled MXFP4 MMAs fed with the packed weights as stored (moe_gemm_mxf4.cuh; activations as three
// MXFP4 terms; the default), and fp16 MMAs with in-kernel dequantisation (moe_gemm_kernel.cuh; exact operands).
// Nothing is allocated; all scratch lives in the caller's workspace.
#include "moe_gemm_kernel.cuh"
#include "moe_gemm_mxf4.cuh"
#include "moe_mma_rate.cuh"

#include <cstdio>
#include <cstdlib>

using namespace dsv4;

namespace {

struct Carve {
    size_t off = 0;
    size_t take(size_t bytes) { const size_t at = off; off += (bytes + 255) & ~size_t(255); return at; }
};

struct WorkspaceMap {
    size_t xh, xexp, offsets, tiles_up, tiles_down, slot_pair, pair_slot, mid, y, xq, xs, midf, mq, ms, total;
};

WorkspaceMap map_workspace(long long T, int k, int K, int H, int O, int E) {
    const long long P = T * k;
    Carve c;
    WorkspaceMap m;
    m.xh = c.take((size_t)T * K * 2);
    m.xexp = c.take((size_t)T * 4);
    m.offsets = c.take((size_t)(E + 1) * 4);
    m.tiles_up = c.take((size_t)(E + 1) * 4);
    m.tiles_down = c.take((size_t)(E + 1) * 4);
    m.slot_pair = c.take((size_t)P * 4);
    m.pair_slot = c.take((size_t)P * 4);
    m.mid = c.take((size_t)P * H * 2);
    m.y = c.take((size_t)P * O * 4);
    // block-scaled path: three MXFP4 terms of x and of the FP32 intermediate
    m.xq = c.take((size_t)3 * T * K / 2);
    m.xs = c.take((size_t)3 * T * K / 32);
    m.midf = c.take((size_t)P * H * 4);
    m.mq = c.take((size_t)3 * P * H / 2);
    m.ms = c.take((size_t)3 * P * H / 32);
    m.total = c.off;
    return m;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

template <class Kernel>
cudaError_t allow_smem(Kernel kernel, size_t bytes, int (&done)[64]) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (done[dev] >= (int)bytes) return cudaSuccess;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (err == cudaSuccess) done[dev] = (int)bytes;
    return err;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// DSV4_B200_PDL=0 switches programmatic dependent launch off (debugging).
bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = std::getenv("DSV4_B200_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// Every kernel of this library starts with griddepcontrol.launch_dependents and reads or writes global memory only
// after griddepcontrol.wait, so consecutive kernels are launched with programmatic stream serialisation: the
// next kernel's CTAs are scheduled while the previous kernel drains, and its prologue (barrier set-up, tensor
// memory allocation) overlaps the tail.
template <class... Params, class... Args>
cudaError_t launch_k(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                     Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Stage timing (diagnostic; off by default): when switched on, the block-scaled path records an event before its
// first kernel and after each of its kernels; mxfp4_moe_stage_times turns them into microseconds.  Events between
// the launches take away the overlap of programmatic dependent launch, so a timed call is slower than a normal one.
constexpr int kStageMarks = 7;      // start, group, quantise x, gate/up GEMM, quantise intermediate, down GEMM, combine
bool g_stage_timing = false;
cudaEvent_t g_stage_event[kStageMarks] = {};

void stage_mark(cudaStream_t stream, int i) {
    if (!g_stage_timing) return;
    if (!g_stage_event[i] && cudaEventCreate(&g_stage_event[i]) != cudaSuccess) return;
    cudaEventRecord(g_stage_event[i], stream);
}

}  // namespace

// Switches the stage timing of the block-scaled batched path on (1) or off (0); returns the previous setting.
// Not thread-safe; meant for one timed call on one stream at a time.
DSV4_API int mxfp4_moe_stage_timing(int enable) {
    const int before = g_stage_timing ? 1 : 0;
    g_stage_timing = enable != 0;
    return before;
}

// Microseconds of the six stages of the last timed call (group, quantise x, gate/up GEMM, quantise intermediate,
// down GEMM, combine) into us_out[0..6); synchronises on the last event.  Returns 0, -1 if no timed call was made.
DSV4_API int mxfp4_moe_stage_times(float* us_out) {
    if (!us_out) return -1;
    for (int i = 0; i < kStageMarks; ++i)
        if (!g_stage_event[i]) return -1;
    if (cudaEventSynchronize(g_stage_event[kStageMarks - 1]) != cudaSuccess) return -1;
    for (int i = 0; i + 1 < kStageMarks; ++i) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, g_stage_event[i], g_stage_event[i + 1]) != cudaSuccess) return -1;
        us_out[i] = ms * 1e3f;
    }
    return 0;
}

// Bytes of workspace mxfp4_moe_forward needs (normalised activations, grouping tables, the fp16 intermediate
// [n_tokens * k, hidden] and the FP32 per-pair outputs [n_tokens * k, out_dim]).
DSV4_API size_t mxfp4_moe_forward_workspace_bytes(int n_tokens, int k, int K_in, int hidden, int out_dim,
                                                  int n_experts) {
    if (n_tokens <= 0 || k <= 0 || K_in <= 0 || hidden <= 0 || out_dim <= 0 || n_experts <= 0) return 0;
    return map_workspace(n_tokens, k, K_in, hidden, out_dim, n_experts).total;
}

// x bf16 [n_tokens, K_in]; bank tensors stacked over n_experts as in mxfp4_grouped_gemv_topk_ids; ids int32
// [n_tokens, k] (a token lists an expert at most once; a negative id marks a pair to skip, which is how an
// expert-parallel caller masks the experts of other ranks), weights FP32 [n_tokens, k]; out bf16 [n_tokens, out_dim].
// Shapes: K_in and hidden multiples of 256, hidden and out_dim multiples of 128, n_experts <= 1024.
// Returns 0, -1 bad shape, -2 null / misaligned pointer, -3 launch failure.
static int moe_forward_impl(int path, const __nv_bfloat16* x, const uint8_t* bank_W1_packed, const uint8_t* bank_W3_packed,
                               const uint8_t* bank_W2_packed, const uint8_t* bank_W1_scale,
                               const uint8_t* bank_W3_scale, const uint8_t* bank_W2_scale, const int* ids,
                               const float* weights, int n_tokens, int n_experts, int K_in, int hidden, int out_dim,
                               int k, __nv_bfloat16* out, void* workspace, cudaStream_t stream,
                               const MoePeerOut* peer = nullptr, const MoePeerIn* peer_in = nullptr) {
    const char* who = "mxfp4_moe_forward";
    if (path != 0 && path != 1) return -1;
    if (n_tokens < 0 || k <= 0 || n_experts <= 0 || n_experts > kMoeMaxExperts || K_in <= 0 || K_in % 256 != 0 ||
        hidden <= 0 || hidden % 256 != 0 || out_dim <= 0 || out_dim % 128 != 0 || K_in > 16384 || hidden > 16384) {
        std::fprintf(stderr, "%s: unsupported shape T=%d E=%d K=%d H=%d O=%d k=%d\n", who, n_tokens, n_experts, K_in,
                     hidden, out_dim, k);
        return -1;
    }
    if (n_tokens == 0) return 0;
    if ((!x && !peer_in) || !bank_W1_packed || !bank_W3_packed || !bank_W2_packed || !bank_W1_scale || !bank_W3_scale ||
        !bank_W2_scale || !ids || !weights || (!out && !peer) || !workspace || (x && !aligned16(x)) || !aligned16(bank_W1_packed) ||
        !aligned16(bank_W3_packed) || !aligned16(bank_W2_packed) || !aligned16(bank_W1_scale) ||
        !aligned16(bank_W3_scale) || !aligned16(bank_W2_scale) || !aligned16(workspace) || (out && !aligned16(out))) {
        std::fprintf(stderr, "%s: null pointer or a tensor that is not 16-byte aligned\n", who);
        return -2;
    }
    static int up_done[64] = {0}, down_done[64] = {0};
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    const WorkspaceMap m = map_workspace(n_tokens, k, K_in, hidden, out_dim, n_experts);
    const int P = n_tokens * k;
    MoeGroups g;
    g.offsets = reinterpret_cast<int*>(ws + m.offsets);
    g.tiles_up = reinterpret_cast<int*>(ws + m.tiles_up);
    g.tiles_down = reinterpret_cast<int*>(ws + m.tiles_down);
    g.slot_pair = reinterpret_cast<int*>(ws + m.slot_pair);
    g.pair_slot = reinterpret_cast<int*>(ws + m.pair_slot);
    __half* xh = reinterpret_cast<__half*>(ws + m.xh);
    int* xexp = reinterpret_cast<int*>(ws + m.xexp);
    __half* mid = reinterpret_cast<__half*>(ws + m.mid);
    float* y = reinterpret_cast<float*>(ws + m.y);

    int* status = nullptr;
    cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_device_status);
    stage_mark(stream, 0);
    if (path == 1)
        launch_k(moe_group_kernel, dim3(1), dim3(1024), 0, stream, ids, P, n_experts, hidden / kMoeTileRows,
                 (out_dim + kQRowsDown - 1) / kQRowsDown, kQTokUp, kQTokDown, g, status);
    else
        launch_k(moe_group_kernel, dim3(1), dim3(1024), 0, stream, ids, P, n_experts, hidden / kMoeTileRows,
                 out_dim / kMoeTileRows, kMoeTileTokens, kMoeTileTokens, g, status);
    stage_mark(stream, 1);
    const int grid = sm_count();

    if (path == 1) {
        // ---- block-scaled MXFP4 tensor-core path
        static int qup_done[64] = {0}, qdown_done[64] = {0};
        uint8_t* xq = ws + m.xq; uint8_t* xs = ws + m.xs;
        uint8_t* mq = ws + m.mq; uint8_t* ms = ws + m.ms;
        float* midf = reinterpret_cast<float*>(ws + m.midf);
        const int qgrid = 4 * grid;
        // a token none of whose experts is in this bank (expert parallel: they all live on other ranks) is not read
        const int* no_rows = nullptr;
        if (peer_in)
            launch_k(moe_quantize_mxfp4x3_kernel<__nv_bfloat16, true>, dim3(qgrid), dim3(256), 0, stream, x,
                     (long long)n_tokens, K_in, xq, xs, *peer_in, no_rows, ids, k);
        else
            launch_k(moe_quantize_mxfp4x3_kernel<__nv_bfloat16, false>, dim3(qgrid), dim3(256), 0, stream, x,
                     (long long)n_tokens, K_in, xq, xs, MoePeerIn{}, no_rows, ids, k);
        stage_mark(stream, 2);
        MoeQGemmArgs qu;
        qu.wa_p = bank_W1_packed; qu.wb_p = bank_W3_packed; qu.wa_s = bank_W1_scale; qu.wb_s = bank_W3_scale;
        qu.stride_p = (long long)hidden * (K_in / 2); qu.stride_s = (long long)hidden * (K_in / 32);
        qu.rows = hidden; qu.K = K_in; qu.n_experts = n_experts; qu.k_top = k;
        qu.act_q = xq; qu.act_s = xs; qu.act_rows = n_tokens; qu.pair_w = weights; qu.g = g; qu.mid = midf; qu.y = nullptr;
        cudaError_t qerr = allow_smem(moe_gemm_mxf4_kernel<0>, MoeQGemmLayout<0>::kBytes, qup_done);
        if (qerr == cudaSuccess) {
            launch_k(moe_gemm_mxf4_kernel<0>, dim3(grid), dim3(kGemmThreads), MoeQGemmLayout<0>::kBytes, stream, qu);
            stage_mark(stream, 3);
            // only the rows that exist: the pairs of this bank's experts fill slots [0, offsets[n_experts])
            const int* used = g.offsets + n_experts;
            const int* no_ids = nullptr;
            launch_k(moe_quantize_mxfp4x3_kernel<float, false>, dim3(qgrid), dim3(256), 0, stream, midf, (long long)P,
                     hidden, mq, ms, MoePeerIn{}, used, no_ids, 0);
            stage_mark(stream, 4);
            qerr = cudaGetLastError();
        }
        MoeQGemmArgs qd = qu;
        qd.wa_p = bank_W2_packed; qd.wb_p = nullptr; qd.wa_s = bank_W2_scale; qd.wb_s = nullptr;
        qd.stride_p = (long long)out_dim * (hidden / 2); qd.stride_s = (long long)out_dim * (hidden / 32);
        qd.rows = out_dim; qd.K = hidden; qd.act_q = mq; qd.act_s = ms; qd.act_rows = P; qd.mid = nullptr; qd.y = y;
        if (qerr == cudaSuccess) qerr = allow_smem(moe_gemm_mxf4_kernel<1>, MoeQGemmLayout<1>::kBytes, qdown_done);
        if (qerr == cudaSuccess) {
            launch_k(moe_gemm_mxf4_kernel<1>, dim3(grid), dim3(kGemmThreads), MoeQGemmLayout<1>::kBytes, stream, qd);
            stage_mark(stream, 5);
            dim3 cgrid((out_dim / 4 + 127) / 128, n_tokens < 65535 ? n_tokens : 65535);
            if (peer)
                launch_k(moe_combine_peer_kernel, dim3(cgrid), dim3(128), 0, stream, y, g.pair_slot, n_tokens, k, out_dim, *peer);
            else
                launch_k(moe_combine_kernel, dim3(cgrid), dim3(128), 0, stream, y, g.pair_slot, n_tokens, k, out_dim, out);
            stage_mark(stream, 6);
            qerr = cudaGetLastError();
        }
        if (qerr != cudaSuccess) {
            std::fprintf(stderr, "%s: launch failed: %s\n", who, cudaGetErrorString(qerr));
            return -3;
        }
        return 0;
    }

    // ---- fp16 tensor-core path with in-kernel dequantisation
    launch_k(moe_token_fp16_kernel, dim3((n_tokens + 7) / 8), dim3(256), 0, stream, x, n_tokens, K_in, xh, xexp);
    MoeGemmArgs up;
    up.wa_p = bank_W1_packed; up.wb_p = bank_W3_packed; up.wa_s = bank_W1_scale; up.wb_s = bank_W3_scale;
    up.stride_p = (long long)hidden * (K_in / 2); up.stride_s = (long long)hidden * (K_in / 32);
    up.rows = hidden; up.K = K_in; up.n_experts = n_experts; up.k_top = k;
    up.act = xh; up.xexp = xexp; up.pair_w = weights; up.g = g; up.mid = mid; up.y = nullptr;
    const size_t smem_up = MoeGemmLayout<0>::bytes(K_in);
    cudaError_t err = allow_smem(moe_gemm_kernel<0>, smem_up, up_done);
    if (err == cudaSuccess) {
        launch_k(moe_gemm_kernel<0>, dim3(grid), dim3(kGemmThreads), smem_up, stream, up);
        err = cudaGetLastError();
    }
    MoeGemmArgs down = up;
    down.wa_p = bank_W2_packed; down.wb_p = nullptr; down.wa_s = bank_W2_scale; down.wb_s = nullptr;
    down.stride_p = (long long)out_dim * (hidden / 2); down.stride_s = (long long)out_dim * (hidden / 32);
    down.rows = out_dim; down.K = hidden; down.act = mid; down.mid = nullptr; down.y = y;
    const size_t smem_down = MoeGemmLayout<1>::bytes(hidden);
    if (err == cudaSuccess) err = allow_smem(moe_gemm_kernel<1>, smem_down, down_done);
    if (err == cudaSuccess) {
        launch_k(moe_gemm_kernel<1>, dim3(grid), dim3(kGemmThreads), smem_down, stream, down);
        err = cudaGetLastError();
    }
    if (err == cudaSuccess) {
        dim3 cgrid((out_dim / 4 + 127) / 128, n_tokens < 65535 ? n_tokens : 65535);
        if (peer)
            launch_k(moe_combine_peer_kernel, dim3(cgrid), dim3(128), 0, stream, y, g.pair_slot, n_tokens, k, out_dim, *peer);
        else
            launch_k(moe_combine_kernel, dim3(cgrid), dim3(128), 0, stream, y, g.pair_slot, n_tokens, k, out_dim, out);
        err = cudaGetLastError();
    }
    if (err != cudaSuccess) {
        std::fprintf(stderr, "%s: launch failed: %s\n", who, cudaGetErrorString(err));
        return -3;
    }
    return 0;
}

// Default path: block-scaled MXFP4 MMAs; DSV4_B200_MOE_PATH=fp16 in the environment selects the fp16 path.
DSV4_API int mxfp4_moe_forward(const __nv_bfloat16* x, const uint8_t* bank_W1_packed, const uint8_t* bank_W3_packed,
                               const uint8_t* bank_W2_packed, const uint8_t* bank_W1_scale,
                               const uint8_t* bank_W3_scale, const uint8_t* bank_W2_scale, const int* ids,
                               const float* weights, int n_tokens, int n_experts, int K_in, int hidden, int out_dim,
                               int k, __nv_bfloat16* out, void* workspace, cudaStream_t stream) {
    static int path = -1;
    if (path < 0) {
        const char* e = std::getenv("DSV4_B200_MOE_PATH");
        path = (e && e[0] == 'f') ? 0 : 1;
    }
    return moe_forward_impl(path, x, bank_W1_packed, bank_W3_packed, bank_W2_packed, bank_W1_scale, bank_W3_scale,
                            bank_W2_scale, ids, weights, n_tokens, n_experts, K_in, hidden, out_dim, k, out, workspace,
                            stream);
}

// The same with the tensor-core path chosen by the caller: 0 = fp16 MMAs with in-kernel dequantisation (operands
// exact), 1 = block-scaled MXFP4 MMAs (weights as stored, activations as three MXFP4 terms).
DSV4_API int mxfp4_moe_forward_path(int path, const __nv_bfloat16* x, const uint8_t* bank_W1_packed,
                                    const uint8_t* bank_W3_packed, const uint8_t* bank_W2_packed,
                                    const uint8_t* bank_W1_scale, const uint8_t* bank_W3_scale,
                                    const uint8_t* bank_W2_scale, const int* ids, const float* weights, int n_tokens,
                                    int n_experts, int K_in, int hidden, int out_dim, int k, __nv_bfloat16* out,
                                    void* workspace, cudaStream_t stream) {
    return moe_forward_impl(path, x, bank_W1_packed, bank_W3_packed, bank_W2_packed, bank_W1_scale, bank_W3_scale,
                            bank_W2_scale, ids, weights, n_tokens, n_experts, K_in, hidden, out_dim, k, out, workspace,
                            stream);
}

// 0 unless a kernel of this library gave up on a bounded wait (4 producer, 5 MMA issuer, 6 epilogue) or met an
// expert id outside the bank (3) since the last call; clears the status.  Synchronises the device.
DSV4_API int mxfp4_moe_device_status(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    return v;
}

// Expert parallel, combine fused with the exchange: the layer of mxfp4_moe_forward over the GATHERED batch of
// world * tokens_per_rank tokens (token t belongs to rank t / tokens_per_rank; ids index this rank's local bank, -1
// where the expert lives elsewhere), whose per-token sums are not written to a local output but stored by the
// combine kernel straight into the receive buffer of the token's home rank - peer memory, plain stores over NVLink,
// the transfer being the kernel's own epilogue.  recv_ptrs: HOST array of `world` device pointers, entry r the
// receive buffer of rank r, bf16 [world][tokens_per_rank][out_dim] (peer-mapped, e.g. symmetric memory); this rank
// writes slice [my_rank] of each.  After a barrier over the ranks every rank calls mxfp4_moe_ep_sum on its own
// buffer.  Return codes as mxfp4_moe_forward; -1 also for world outside 1..16 or a token count that is not
// world * tokens_per_rank.
DSV4_API int mxfp4_moe_forward_ep(const __nv_bfloat16* x, const uint8_t* bank_W1_packed, const uint8_t* bank_W3_packed,
                                  const uint8_t* bank_W2_packed, const uint8_t* bank_W1_scale,
                                  const uint8_t* bank_W3_scale, const uint8_t* bank_W2_scale, const int* ids,
                                  const float* weights, int n_tokens, int n_experts, int K_in, int hidden, int out_dim,
                                  int k, void* const* recv_ptrs, int world, int my_rank, int tokens_per_rank,
                                  void* workspace, cudaStream_t stream) {
    if (world < 1 || world > kMoeMaxRanks || my_rank < 0 || my_rank >= world || tokens_per_rank <= 0 ||
        n_tokens != world * tokens_per_rank || !recv_ptrs) {
        std::fprintf(stderr, "mxfp4_moe_forward_ep: bad rank layout world=%d rank=%d tokens_per_rank=%d n_tokens=%d\n", world,
                     my_rank, tokens_per_rank, n_tokens);
        return -1;
    }
    MoePeerOut peer = {};
    for (int r = 0; r < world; ++r) {
        if (!recv_ptrs[r] || !aligned16(recv_ptrs[r])) return -2;
        peer.recv[r] = reinterpret_cast<__nv_bfloat16*>(recv_ptrs[r]);
    }
    peer.world = world; peer.my_rank = my_rank; peer.tokens_per_rank = tokens_per_rank;
    static int path = -1;
    if (path < 0) {
        const char* e = std::getenv("DSV4_B200_MOE_PATH");
        path = (e && e[0] == 'f') ? 0 : 1;
    }
    return moe_forward_impl(path, x, bank_W1_packed, bank_W3_packed, bank_W2_packed, bank_W1_scale, bank_W3_scale,
                            bank_W2_scale, ids, weights, n_tokens, n_experts, K_in, hidden, out_dim, k, nullptr,
                            workspace, stream, &peer);
}

// out[t] = bf16(sum of recv[r][t] over the ranks r that own one of token t's experts, in ascending order): the home
// rank's side of mxfp4_moe_forward_ep, after the barrier.  recv bf16 [world][n_tokens][out_dim]; ids int32
// [n_tokens, k] GLOBAL expert ids of this rank's tokens (a rank owns experts [r, r + 1) * experts_per_rank; ranks
// without an expert of the token stored nothing and are skipped); out bf16 [n_tokens][out_dim]; out_dim a multiple
// of 4, world <= 16.  Returns 0, -1 bad shape, -2 null / misaligned pointer, -3 launch failure.
DSV4_API int mxfp4_moe_ep_sum(const __nv_bfloat16* recv, const int* ids, int k, int experts_per_rank, int world,
                              int n_tokens, int out_dim, __nv_bfloat16* out, cudaStream_t stream) {
    if (world < 1 || world > kMoeMaxRanks || n_tokens < 0 || out_dim <= 0 || out_dim % 4 != 0 || k <= 0 ||
        experts_per_rank <= 0)
        return -1;
    if (n_tokens == 0) return 0;
    if (!recv || !ids || !out || !aligned16(recv) || !aligned16(out)) return -2;
    const long long n4 = (long long)n_tokens * out_dim / 4;
    long long grid = (n4 + 255) / 256;
    if (grid > 8LL * sm_count()) grid = 8LL * sm_count();
    launch_k(moe_ep_sum_kernel, dim3((unsigned)grid), dim3(256), 0, stream, recv, ids, k, experts_per_rank, world,
             n_tokens, out_dim, out);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Expert parallel with BOTH sides over peer memory (no collective library on the path): every rank publishes its
// tokens in buffers that are mapped on all ranks (symmetric memory): x bf16 [tokens_per_rank, K_in], ids int32
// [tokens_per_rank, k] (global expert ids), weights FP32 [tokens_per_rank, k].  After a barrier over the ranks this
// call runs the rank's experts over the whole batch of world * tokens_per_rank tokens: a small kernel turns the
// published ids into this rank's view (local index, -1 for experts of other ranks), the activation quantiser reads
// every token's row from the rank that published it (plain loads over NVLink), and the combine kernel stores the
// partial rows into the home ranks' receive buffers as in mxfp4_moe_forward_ep.  x_ptrs / ids_ptrs / w_ptrs /
// recv_ptrs: HOST arrays of `world` device pointers.  Block-scaled tensor-core path only.  workspace:
// mxfp4_moe_forward_ep2_workspace_bytes.  Return codes as mxfp4_moe_forward_ep.
DSV4_API size_t mxfp4_moe_forward_ep2_workspace_bytes(int world, int tokens_per_rank, int k, int K_in, int hidden,
                                                      int out_dim, int n_experts_local) {
    if (world <= 0 || tokens_per_rank <= 0 || k <= 0) return 0;
    const long long T = (long long)world * tokens_per_rank;
    const size_t base = map_workspace(T, k, K_in, hidden, out_dim, n_experts_local).total;
    return base + 2 * (((size_t)T * k * 4 + 255) & ~size_t(255));
}

DSV4_API int mxfp4_moe_forward_ep2(void* const* x_ptrs, void* const* ids_ptrs, void* const* w_ptrs,
                                   const uint8_t* bank_W1_packed, const uint8_t* bank_W3_packed,
                                   const uint8_t* bank_W2_packed, const uint8_t* bank_W1_scale,
                                   const uint8_t* bank_W3_scale, const uint8_t* bank_W2_scale, int tokens_per_rank,
                                   int n_experts_local, int K_in, int hidden, int out_dim, int k,
                                   void* const* recv_ptrs, int world, int my_rank, void* workspace,
                                   cudaStream_t stream) {
    if (world < 1 || world > kMoeMaxRanks || my_rank < 0 || my_rank >= world || tokens_per_rank <= 0 || k <= 0 ||
        n_experts_local <= 0 || !x_ptrs || !ids_ptrs || !w_ptrs || !recv_ptrs || !workspace) {
        std::fprintf(stderr, "mxfp4_moe_forward_ep2: bad rank layout or null table\n");
        return -1;
    }
    MoePeerIn in = {};
    MoePeerOut peer = {};
    for (int r = 0; r < world; ++r) {
        if (!x_ptrs[r] || !ids_ptrs[r] || !w_ptrs[r] || !recv_ptrs[r] || !aligned16(x_ptrs[r]) || !aligned16(recv_ptrs[r]))
            return -2;
        in.x[r] = reinterpret_cast<const __nv_bfloat16*>(x_ptrs[r]);
        in.ids[r] = reinterpret_cast<const int*>(ids_ptrs[r]);
        in.w[r] = reinterpret_cast<const float*>(w_ptrs[r]);
        peer.recv[r] = reinterpret_cast<__nv_bfloat16*>(recv_ptrs[r]);
    }
    in.world = peer.world = world; in.my_rank = peer.my_rank = my_rank;
    in.tokens_per_rank = peer.tokens_per_rank = tokens_per_rank; in.experts_per_rank = n_experts_local;
    const int n_tokens = world * tokens_per_rank;
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    const size_t base = map_workspace(n_tokens, k, K_in, hidden, out_dim, n_experts_local).total;
    int* ids_local = reinterpret_cast<int*>(ws + base);
    float* w_local = reinterpret_cast<float*>(ws + base + (((size_t)n_tokens * k * 4 + 255) & ~size_t(255)));
    const int n_meta = n_tokens * k;
    launch_k(moe_ep_gather_meta_kernel, dim3((unsigned)((n_meta + 255) / 256)), dim3(256), 0, stream, in, k, ids_local,
             w_local);
    return moe_forward_impl(1, nullptr, bank_W1_packed, bank_W3_packed, bank_W2_packed, bank_W1_scale, bank_W3_scale,
                            bank_W2_scale, ids_local, w_local, n_tokens, n_experts_local, K_in, hidden, out_dim, k,
                            nullptr, workspace, stream, &peer, &in);
}

// Tensor-pipe clocks of one tcgen05.mma kind::mxf4 (M = 128, K = 64, N = n_cols: a multiple of 16 in 16 .. 256) with
// `scale_copies` (0 .. 8) scale-atom copies issued in front of every four MMAs; one CTA per SM, `iters` rounds of
// four MMAs.  clocks_per_mma: HOST pointer.  `scratch`: 8 bytes of device memory.  Synchronises the stream.
// Returns 0, -1 bad argument, -3 launch / execution failure.
DSV4_API int mxfp4_moe_mma_rate(int n_cols, int scale_copies, int iters, void* scratch, double* clocks_per_mma,
                                cudaStream_t stream) {
    if (n_cols < 16 || n_cols > 256 || n_cols % 16 != 0 || scale_copies < 0 || scale_copies > 8 || iters <= 0 ||
        iters > (1 << 20) || !scratch || !clocks_per_mma)
        return -1;
    static int done[64] = {0};
    if (allow_smem(mxf4_mma_rate_kernel, kRateBytes, done) != cudaSuccess) return -3;
    long long* dev_clocks = reinterpret_cast<long long*>(scratch);
    mxf4_mma_rate_kernel<<<sm_count(), 128, kRateBytes, stream>>>(n_cols, 8, scale_copies, dev_clocks);       // warm-up
    mxf4_mma_rate_kernel<<<sm_count(), 128, kRateBytes, stream>>>(n_cols, iters, scale_copies, dev_clocks);
    long long clocks = 0;
    if (cudaMemcpyAsync(&clocks, dev_clocks, sizeof(clocks), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess || cudaGetLastError() != cudaSuccess)
        return -3;
    *clocks_per_mma = (double)clocks / (4.0 * iters);
    return 0;
}
