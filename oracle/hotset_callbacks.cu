// TEST INFRASTRUCTURE.  The two probe callbacks the reference's routed dispatch expects in its DSv4Hotset table
// (kernel/cpp-engine-mxfp4/routed.cu:59-64), forwarding to the reference's REAL hot-set
// (kernel/cpp-engine-mxfp4/hotset.cu:547 hotset_get_expert_gpu_ptr).  The reference engine keeps its own pair
// `static` inside dsv4_engine_mxfp4_wire.cu:210-226, so a test that links only routed.cu + hotset.cu has to bring
// these two.  Linked with the unmodified routed.cu and hotset.cu into oracle/_ref/libdsv4_routed_hotset_ref.so.
#include <cstddef>
#include <cstdint>

// Layout of the hot-set's answer (hotset.cu:539-545); weight-key order W1 = 0, W2 = 1, W3 = 2 (routed.cu:67).
struct ExpertGpuPtrs {
    void* packed[3];
    void* scale[3];
    size_t packed_bytes[3];
    size_t scale_bytes[3];
    int hit;
};

extern "C" int hotset_get_expert_gpu_ptr(int layer, int expert_id, ExpertGpuPtrs* out);

extern "C" const uint8_t* hotset_cb_get_w_packed(void* /*user*/, int layer, int expert, int key) {
    ExpertGpuPtrs p = {};
    if (key < 0 || key > 2 || hotset_get_expert_gpu_ptr(layer, expert, &p) != 0) return nullptr;
    return static_cast<const uint8_t*>(p.packed[key]);
}

extern "C" const uint8_t* hotset_cb_get_w_scale(void* /*user*/, int layer, int expert, int key) {
    ExpertGpuPtrs p = {};
    if (key < 0 || key > 2 || hotset_get_expert_gpu_ptr(layer, expert, &p) != 0) return nullptr;
    return static_cast<const uint8_t*>(p.scale[key]);
}
