// placeholder: fast paths (filled in next)
#include "common.cuh"
int32_t bhd_launch_matvec_fast(bhd_ctx*, const bhd_weight*, uint64_t, const float*, float*, uint64_t, float, int,
                               cudaStream_t, bool* handled) { *handled = false; return BHD_OK; }
void bhd_weight_build_tensor_map(bhd_ctx*, bhd_weight* w) { w->tmap_ok = false; }
int32_t bhd_moe_experts_fast(bhd_ctx*, const bhd_weight*, const bhd_weight*, const bhd_weight*, const float*, uint64_t,
                             uint32_t, const int32_t*, const float*, uint32_t, uint32_t, float*, int, cudaStream_t,
                             bool* handled) { *handled = false; return BHD_OK; }
