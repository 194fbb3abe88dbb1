// attn_tc.cu — placeholder while the tcgen05 kernels are brought up.
#include "internal.hpp"
namespace hc {
bool tc_supported(const AttnShape&) { return false; }
hc_status tc_prefill(hc_context*, const AttnShape&, const hc_layer_store&, const CacheView&, int,
                     const uint16_t*, int, int, const EpilogueArgs&, cudaStream_t) {
    return fail(HC_UNSUPPORTED, "tcgen05 path not built");
}
hc_status tc_make_tensor_maps(hc_kv_cache*, hc_layer_store&) { return HC_OK; }
void tc_free_tensor_maps(hc_layer_store&) {}
}  // namespace hc
