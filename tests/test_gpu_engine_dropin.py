"""Drop-in proof with the REFERENCE's own caller: its routed dispatch (kernel/cpp-engine-mxfp4/routed.cu:373-503 -
router GEMV, sqrt-softplus, host top-6, 36 pack copies, call of `mxfp4_grouped_gemv_topk`), compiled unmodified into
oracle/_ref/libdsv4_routed_ref.so, runs against THIS repository's libmxfp4_grouped_gemv.so: the engine code declares
the two grouped symbols `extern "C"` (routed.cu:46-54) and finds them in the global namespace because the kernel
library was loaded RTLD_GLOBAL first, which is how the reference's tools bind them (tools/D27_baseline.py:34-38).
The reference's hot-set (hotset.cu) is replaced by a resident-bank stand-in (oracle/hotset_shim.cu)."""
import ctypes
import os
from ctypes import c_int, c_size_t, c_void_p

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

REF_LIB = os.path.join(os.path.dirname(os.path.abspath(oracle.__file__)), "_ref", "libdsv4_routed_ref.so")


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="oracle/_ref/libdsv4_routed_ref.so not built (make -C oracle)")
def test_reference_routed_dispatch_calls_the_new_library(rt, qz):
    dev = torch.device("cuda:0")
    E, K, H, k = 256, 4096, 2048, 6
    _ = rt.decode_workspace_bytes(k, H, K)           # loads libmxfp4_grouped_gemv.so with RTLD_GLOBAL
    ref = ctypes.CDLL(REF_LIB, mode=ctypes.RTLD_LOCAL)
    ref.dsv4_routed_state_alloc.restype = c_void_p
    ref.dsv4_routed_state_alloc.argtypes = [c_int, c_void_p]
    ref.dsv4_routed_state_free.argtypes = [c_void_p]
    ref.dsv4_routed_set_router_gate.argtypes = [c_void_p, c_int, c_void_p]
    ref.dsv4_routed_set_hotset.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p]
    ref.dsv4_routed_dispatch.restype = c_int
    ref.dsv4_routed_dispatch.argtypes = [c_void_p, c_int, c_void_p, c_void_p]
    ref.dsv4_routed_get_dispatch_count.restype = c_int
    ref.dsv4_routed_get_dispatch_count.argtypes = [c_void_p]
    ref.shim_set_bank.argtypes = [c_int, c_void_p, c_void_p, c_size_t, c_size_t, c_int]

    bank = qz.make_expert_bank(E, K, H, dev, seed=77, chunk=16)
    g = torch.Generator().manual_seed(78)
    gate = (torch.randn(E, K, generator=g) * 0.02).to(torch.bfloat16)
    stream = torch.cuda.current_stream(dev)
    st = ref.dsv4_routed_state_alloc(1, c_void_p(stream.cuda_stream))
    assert st
    try:
        d_gate = gate.to(dev)
        ref.dsv4_routed_set_router_gate(st, 0, c_void_p(d_gate.data_ptr()))
        # weight keys of routed.cu:67: W1 = 0, W2 = 1, W3 = 2
        for key, p, s in ((0, "w1p", "w1s"), (1, "w2p", "w2s"), (2, "w3p", "w3s")):
            ref.shim_set_bank(key, c_void_p(bank[p].data_ptr()), c_void_p(bank[s].data_ptr()),
                              bank[p][0].numel(), bank[s][0].numel(), E)
        ref.dsv4_routed_set_hotset(st, ctypes.cast(ref.shim_get_w_packed, c_void_p),
                                   ctypes.cast(ref.shim_get_w_scale, c_void_p), None)
        for step in range(3):
            x = torch.randn(K, generator=g).to(torch.bfloat16)
            d_x = x.to(dev)
            d_out = torch.full((K,), float("nan"), dtype=torch.bfloat16, device=dev)
            rc = ref.dsv4_routed_dispatch(st, 0, c_void_p(d_x.data_ptr()), c_void_p(d_out.data_ptr()))
            torch.cuda.synchronize()
            assert rc == 0 and ref.dsv4_routed_get_dispatch_count(st) == k
            # oracle: the reference's routing rule (sqrt-softplus, top-6, renormalise, x 1.5) on FP32 logits
            logits = (gate.float() @ x.float()).numpy()
            top = np.sort(logits)[::-1]
            assert top[k - 1] - top[k] > 1e-3, "seed gives a near tie at the selection boundary"
            ids, w = oracle.route_sqrt_softplus(logits[None], k)
            sel = torch.from_numpy(ids[0].astype(np.int64))
            sub = {n: v[sel.to(dev)].cpu() for n, v in bank.items()}
            want = oracle.moe_layer_ref(x[None], sub, np.arange(k)[None], w)[0]
            got = d_out.float().cpu().numpy()
            err, cos = oracle.max_abs_rel(got, want), oracle.cosine(got, want)
            assert err <= 5e-3 and cos >= 0.99999, f"step {step}: max-abs/inf {err:.3e} cosine {cos:.7f}"
            # and it was THIS library that ran: its direct entry gives the same bits on the same picks
            direct = rt.mxfp4_grouped_gemv_ids(bank, torch.from_numpy(ids[0].astype(np.int32)).to(dev), d_x,
                                               torch.from_numpy(w[0]).to(dev))
            assert np.max(np.abs(direct.float().cpu().numpy() - got)) <= 2e-2 * np.max(np.abs(want))
        assert rt.device_status() == 0
    finally:
        ref.dsv4_routed_state_free(st)


HOTSET_LIB = os.path.join(os.path.dirname(os.path.abspath(oracle.__file__)), "_ref", "libdsv4_routed_hotset_ref.so")


class HotsetStats(ctypes.Structure):         # kernel/cpp-engine-mxfp4/hotset.cu:846-854
    _fields_ = [("n_lookups", ctypes.c_uint64), ("n_hits", ctypes.c_uint64), ("n_misses", ctypes.c_uint64),
                ("last_miss_latency_us", ctypes.c_uint64), ("total_bytes_resident", ctypes.c_uint64),
                ("n_layers", c_int), ("hot_per_layer", c_int)]


@pytest.mark.skipif(not os.path.exists(HOTSET_LIB),
                    reason="oracle/_ref/libdsv4_routed_hotset_ref.so not built (make -C oracle)")
def test_reference_dispatch_with_its_real_hotset_calls_the_new_library(rt, qz, tmp_path):
    """The reference's routed dispatch AND its hot-set (kernel/cpp-engine-mxfp4/hotset.cu: hotset_init :211,
    hotset_set_consumer_stream :173, hotset_register_cold :297, hotset_prewarm_expert :498,
    hotset_get_expert_gpu_ptr :547, hotset_prefetch_batch :645), both unmodified, on this repository's library:
    one synthetic layer registered as cold host memory, 16 hot slots for 256 experts, so the pack copies
    (routed.cu:224-286) read LRU slots that miss, load and evict while the layer runs.
    The cold store is a read-only file mapping, as in the reference (its hot-set drops the source pages with
    madvise after every load, which only a file mapping survives); 256 experts share 32 distinct weight sets."""
    dev = torch.device("cuda:0")
    E, K, H, k, distinct, hot = 256, 4096, 2048, 6, 32, 16
    _ = rt.decode_workspace_bytes(k, H, K)           # loads libmxfp4_grouped_gemv.so with RTLD_GLOBAL
    ref = ctypes.CDLL(HOTSET_LIB, mode=ctypes.RTLD_LOCAL)
    ref.dsv4_routed_state_alloc.restype = c_void_p
    ref.dsv4_routed_state_alloc.argtypes = [c_int, c_void_p]
    ref.dsv4_routed_state_free.argtypes = [c_void_p]
    ref.dsv4_routed_set_router_gate.argtypes = [c_void_p, c_int, c_void_p]
    ref.dsv4_routed_set_hotset.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p]
    ref.dsv4_routed_dispatch.restype = c_int
    ref.dsv4_routed_dispatch.argtypes = [c_void_p, c_int, c_void_p, c_void_p]
    ref.hotset_init.argtypes = [c_int, c_int, c_int]
    ref.hotset_set_consumer_stream.argtypes = [c_void_p]
    ref.hotset_register_cold.argtypes = [c_int, c_int, c_int, c_void_p, c_size_t, c_void_p, c_size_t]
    ref.hotset_prewarm_expert.argtypes = [c_int, c_int]
    ref.hotset_stats.argtypes = [ctypes.POINTER(HotsetStats)]

    bank = qz.make_expert_bank(distinct, K, H, "cpu", seed=91)
    # cold store: one file per tensor kind, mapped read-only
    cold = {}
    for name, t in bank.items():
        path = tmp_path / f"{name}.bin"
        t.numpy().tofile(path)
        cold[name] = np.memmap(path, dtype=np.uint8, mode="r", shape=tuple(t.shape))
    g = torch.Generator().manual_seed(92)
    gate = (torch.randn(E, K, generator=g) * 0.02).to(torch.bfloat16)
    stream = torch.cuda.current_stream(dev)
    assert ref.hotset_init(1, E, hot) == 0
    st = None
    try:
        assert ref.hotset_set_consumer_stream(c_void_p(stream.cuda_stream)) == 0
        # weight keys of routed.cu:67: W1 = 0, W2 = 1, W3 = 2
        for e in range(E):
            for key, p, s in ((0, "w1p", "w1s"), (1, "w2p", "w2s"), (2, "w3p", "w3s")):
                pe, se = cold[p][e % distinct], cold[s][e % distinct]
                assert ref.hotset_register_cold(0, e, key, c_void_p(pe.ctypes.data), pe.nbytes,
                                                c_void_p(se.ctypes.data), se.nbytes) == 0
        for e in range(4):
            assert ref.hotset_prewarm_expert(0, e) == 0
        st = ref.dsv4_routed_state_alloc(1, c_void_p(stream.cuda_stream))
        assert st
        d_gate = gate.to(dev)
        ref.dsv4_routed_set_router_gate(st, 0, c_void_p(d_gate.data_ptr()))
        ref.dsv4_routed_set_hotset(st, ctypes.cast(ref.hotset_cb_get_w_packed, c_void_p),
                                   ctypes.cast(ref.hotset_cb_get_w_scale, c_void_p), None)
        touched = set()
        for step in range(8):                        # 8 x 6 picks over 256 experts: far more than 16 slots
            x = torch.randn(K, generator=g).to(torch.bfloat16)
            d_x = x.to(dev)
            d_out = torch.full((K,), float("nan"), dtype=torch.bfloat16, device=dev)
            rc = ref.dsv4_routed_dispatch(st, 0, c_void_p(d_x.data_ptr()), c_void_p(d_out.data_ptr()))
            torch.cuda.synchronize()
            assert rc == 0
            logits = (gate.float() @ x.float()).numpy()
            top = np.sort(logits)[::-1]
            assert top[k - 1] - top[k] > 1e-3, "seed gives a near tie at the selection boundary"
            ids, w = oracle.route_sqrt_softplus(logits[None], k)
            touched.update(int(i) for i in ids[0])
            sel = torch.from_numpy((ids[0] % distinct).astype(np.int64))
            sub = {n: v[sel] for n, v in bank.items()}
            want = oracle.moe_layer_ref(x[None], sub, np.arange(k)[None], w)[0]
            got = d_out.float().cpu().numpy()
            err, cos = oracle.max_abs_rel(got, want), oracle.cosine(got, want)
            assert err <= 5e-3 and cos >= 0.99999, f"step {step}: max-abs/inf {err:.3e} cosine {cos:.7f}"
        stats = HotsetStats()
        assert ref.hotset_stats(ctypes.byref(stats)) == 0
        assert len(touched) > hot and stats.n_misses > hot        # slots were evicted and reloaded
        assert rt.device_status() == 0
    finally:
        if st:
            ref.dsv4_routed_state_free(st)
        torch.cuda.synchronize()
        ref.hotset_destroy()
