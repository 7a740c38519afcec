// Placeholder until the tcgen05 kernel lands: reports every shape as unsupported.
#include "wa_internal.cuh"
namespace wa {
size_t hsa_sm100_workspace_bytes(const wa_hsa_params *) { return 0; }
bool hsa_sm100_supported(const wa_hsa_params *, int, const wa_tensor4 *, const wa_tensor4 *) { return false; }
int hsa_sm100_launch(const wa_hsa_params *, int, const wa_tensor4 *, const wa_tensor4 *, const int32_t *,
                     const int32_t *, int, int, void *, cudaStream_t) {
    return fail(WA_ERR_UNSUPPORTED, "tcgen05 kernel not built");
}
}  // namespace wa
