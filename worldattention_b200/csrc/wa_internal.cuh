// Internal (non-ABI) declarations shared between translation units.
#pragma once
#include "wa_common.cuh"

namespace wa {

// routing (wa_routing.cu): pools x and optionally y in one launch
int pool_launch(const wa_tensor4 *x, int Lx, float *px, const wa_tensor4 *y, int Ly, float *py, int B, int H, int D,
                int block_size, cudaStream_t stream);

// optional CUDA-event bracket around the attention kernel (wa_api.cu)
void profile_mark(bool begin, cudaStream_t stream);

// tcgen05 fused HSA kernel (wa_hsa_sm100.cu)
size_t hsa_sm100_workspace_bytes(const wa_hsa_params *p);
size_t hsa_sm100_status_offset(const wa_hsa_params *p);   // int32 flag inside the tuned workspace
bool hsa_sm100_supported(const wa_hsa_params *p, int Lc, const wa_tensor4 *kc, const wa_tensor4 *vc);
int hsa_sm100_launch(const wa_hsa_params *p, int Lc, const wa_tensor4 *kc, const wa_tensor4 *vc,
                     const int32_t *index, const int32_t *num, int Nq, int Nkv, void *workspace,
                     cudaStream_t stream);

}  // namespace wa
