// TEST INFRASTRUCTURE.  Stand-in for the reference's hot-set (kernel/cpp-engine-mxfp4/hotset.cu) in the drop-in test
// of its routed dispatch (kernel/cpp-engine-mxfp4/routed.cu:373-503): every expert of the layer is resident in one
// device bank, so a probe is a pointer computation and a prefetch is nothing.  It provides exactly what routed.cu
// needs from the outside: `hotset_prefetch_batch` (declared extern in routed.cu:212) and the two probe callbacks of
// its DSv4Hotset table (routed.cu:59-64), with the weight-key order of routed.cu:67 (W1 = 0, W2 = 1, W3 = 2).
// Linked together with the unmodified routed.cu into oracle/_ref/libdsv4_routed_ref.so; the grouped-GEMV symbols stay
// undefined there and are resolved at load time from whichever kernel library was loaded RTLD_GLOBAL before it.
#include <cstddef>
#include <cstdint>

namespace {
struct Bank {
    const uint8_t* packed[3];     // [n_experts, ...] stacked, by weight key
    const uint8_t* scale[3];
    size_t packed_bytes[3];       // bytes per expert
    size_t scale_bytes[3];
    int n_experts;
};
Bank g_bank = {};
}  // namespace

extern "C" int hotset_prefetch_batch(int /*layer*/, const int* /*ids*/, int /*n_ids*/) { return 0; }

// key: 0 = W1, 1 = W2, 2 = W3.
extern "C" void shim_set_bank(int key, const uint8_t* packed, const uint8_t* scale, size_t packed_bytes_per_expert,
                              size_t scale_bytes_per_expert, int n_experts) {
    if (key < 0 || key > 2) return;
    g_bank.packed[key] = packed;
    g_bank.scale[key] = scale;
    g_bank.packed_bytes[key] = packed_bytes_per_expert;
    g_bank.scale_bytes[key] = scale_bytes_per_expert;
    g_bank.n_experts = n_experts;
}

extern "C" const uint8_t* shim_get_w_packed(void* /*user*/, int /*layer*/, int expert, int key) {
    if (key < 0 || key > 2 || expert < 0 || expert >= g_bank.n_experts || !g_bank.packed[key]) return nullptr;
    return g_bank.packed[key] + (size_t)expert * g_bank.packed_bytes[key];
}

extern "C" const uint8_t* shim_get_w_scale(void* /*user*/, int /*layer*/, int expert, int key) {
    if (key < 0 || key > 2 || expert < 0 || expert >= g_bank.n_experts || !g_bank.scale[key]) return nullptr;
    return g_bank.scale[key] + (size_t)expert * g_bank.scale_bytes[key];
}
