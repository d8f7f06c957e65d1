// Tensor-core decode attention (tcgen05 block-scaled NVFP4 MMA). Placeholder until the kernel lands.
#include "pkv_common.cuh"

int pkv_attn_tc_launch(const pkv_layer_t*, const pkv_cache_t*, const void*, const int32_t*, int32_t, const int32_t*,
                       int32_t, int32_t, uint32_t, float*, float*, int64_t, int32_t*, cudaStream_t) {
    return PKV_ERR_UNSUPPORTED;
}
