// Stand-alone query absorption launch (the arithmetic lives in pkv_absorb.cuh).
#include "pkv_absorb.cuh"

int pkv_check_layer(const pkv_layer_t* L);

namespace {

using namespace pkv_absorb_impl;

__global__ void __launch_bounds__(NT) pkv_absorb_kernel(const Args P) {
    extern __shared__ __align__(16) float sm[];
    pkv_grid_wait();
    pkv_grid_launch_dependents();
    body(P, blockIdx.x, blockIdx.y, sm);
}

}  // namespace

extern "C" int64_t pkv_query_operand_bytes(int32_t W) {
    if (W <= 0 || W > PKV_MAX_WIDTH || (W % 16)) return PKV_ERR_UNSUPPORTED;
    return pkv_page_bytes(W) + 512;
}

extern "C" int pkv_absorb(const pkv_layer_t* layer, const float* q_dev, const int32_t* positions_dev,
                          const float* phasors_dev, int32_t batch, float* qabs_out_dev, uint8_t* qop_out_dev,
                          void* stream) {
    return pkv_absorb_sync(layer, q_dev, positions_dev, phasors_dev, batch, qabs_out_dev, qop_out_dev, nullptr, stream);
}

extern "C" int pkv_absorb_sync(const pkv_layer_t* layer, const float* q_dev, const int32_t* positions_dev,
                               const float* phasors_dev, int32_t batch, float* qabs_out_dev, uint8_t* qop_out_dev,
                               int32_t* qsync_dev, void* stream) {
    int st = pkv_check_layer(layer);
    if (st) return st;
    if (batch < 0) return PKV_ERR_INVALID;
    if (batch == 0) return PKV_OK;
    if (!q_dev || (!positions_dev && !phasors_dev)) return PKV_ERR_INVALID;
    if (phasors_dev && (((uintptr_t)phasors_dev) & 7u)) return PKV_ERR_INVALID;
    if (layer->head_dim / 2 > MAX_H || (layer->head_dim & 1)) return PKV_ERR_UNSUPPORTED;
    const int W = 2 * layer->R + layer->R_s, Wp = pkv_padded_width(W);
    if (qop_out_dev) {
        if (layer->n_q * PKV_QUERY_TERMS != 128) return PKV_ERR_UNSUPPORTED;   // the operand tile has 128 rows
        if (((uintptr_t)qop_out_dev) & 1023u) return PKV_ERR_INVALID;
    }
    if (batch == 0) return PKV_OK;
    if (qsync_dev && !qop_out_dev) return PKV_ERR_INVALID;          // the signal says "operand in place"
    Args P = make_args(layer, q_dev, positions_dev, phasors_dev, qabs_out_dev, qop_out_dev);
    P.qsync = qsync_dev;
    PKV_CUDA_TRY(pkv_launch_chained(pkv_absorb_kernel, dim3(batch, (layer->n_q + HG - 1) / HG), dim3(NT),
                                    smem_bytes(layer->head_dim, Wp), (cudaStream_t)stream, P));   // < 48 KB: no opt-in needed
    return PKV_OK;
}
