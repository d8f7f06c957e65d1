// Decode attention for callers that cannot allocate device memory.
//
// pkv_decode_attn needs scratch for the per-split partial results and asks its caller to own it.
// Some callers have nowhere to get it from: a host that runs inside someone else's captured or
// pre-planned memory budget, a plugin that is handed input and output tensors only, a process whose
// allocator is off limits at this point of its life. For them this file keeps the scratch in the
// library image itself, as one fixed-size array in device memory, and offers one entry point that
// uses it. The price is stated in the header: a fixed upper bound on batch * n_split, a few MB held
// on every GPU that loads the library, and no two calls in flight on one GPU at the same time.
#include "pkv_common.cuh"

int pkv_check_layer(const pkv_layer_t* L);
int pkv_check_cache(const pkv_cache_t* c);
int pkv_attn_tc_launch(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* q_dev,
                       const int32_t* page_table_dev, int32_t max_pages, const int32_t* seqlens_dev, int32_t batch,
                       int32_t n_split, uint32_t flags, float* partials_dev, float* scores_out_dev,
                       int64_t scores_stride, int32_t* status_dev, float* out_dev, cudaStream_t stream,
                       const float* q_raw_dev = nullptr, const int32_t* q_positions_dev = nullptr, int32_t* qsync_dev = nullptr);

namespace {

constexpr int NQ = 32, DH = 128;
constexpr size_t SCRATCH_FLOATS = (size_t)PKV_NOALLOC_MAX_PARTS * NQ * (DH + 2);

// The scratch itself. In host code this name is only a handle for the runtime, not an address a
// kernel could use; the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_partials[SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_scratch_ptr[MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the current device; looked up once per device. The table is
// filled without a lock: two host threads that race here look up and store the same address.
int scratch_for_current_device(float** out) {
    int dev = -1;
    PKV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return PKV_ERR_UNSUPPORTED;
    if (!g_scratch_ptr[dev]) {
        float* p = nullptr;
        PKV_CUDA_TRY(cudaGetSymbolAddress((void**)&p, g_noalloc_partials));
        if (!p) return PKV_ERR_CUDA;
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return PKV_OK;
}

}  // namespace

extern "C" int pkv_decode_attn_noalloc(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* qop_dev,
                                       const int32_t* page_table_dev, int32_t max_pages, const int32_t* seqlens_dev,
                                       int32_t batch, int32_t n_split, float* out_dev, int32_t* status_dev,
                                       void* stream) {
    int st = pkv_check_layer(layer);
    if (st) return st;
    st = pkv_check_cache(cache);
    if (st) return st;
    if (batch < 0 || n_split <= 0 || max_pages <= 0) return PKV_ERR_INVALID;
    if (batch == 0) return PKV_OK;
    if ((int64_t)batch * n_split > PKV_NOALLOC_MAX_PARTS) return PKV_ERR_UNSUPPORTED;     // beyond the built-in scratch
    if (!qop_dev || !page_table_dev || !seqlens_dev || !out_dev || !(cache->v_bits ? cache->vq_dev : cache->v_dev)) return PKV_ERR_INVALID;
    if (cache->W != 2 * layer->R + layer->R_s || cache->n_kv != layer->n_kv || cache->head_dim != layer->head_dim)
        return PKV_ERR_INVALID;
    if (layer->n_q != NQ || layer->head_dim != DH) return PKV_ERR_UNSUPPORTED;
    float* scratch = nullptr;
    st = scratch_for_current_device(&scratch);
    if (st) return st;
    // every (sequence, split) slot of the scratch is written in full by the attention kernel before
    // the merge reads it -- with its partial result, or with the neutral triple when the CTA gave up
    // (status_dev then says so) -- so nothing left over from an earlier call can leak into this one
    st = pkv_attn_tc_launch(layer, cache, qop_dev, page_table_dev, max_pages, seqlens_dev, batch, n_split, 0u, scratch,
                            nullptr, 0, status_dev, nullptr, (cudaStream_t)stream);
    if (st) return st;
    const int64_t pw = DH + 2;
    return pkv_merge(scratch, (int64_t)n_split * NQ * pw, NQ * pw, n_split, batch, NQ, DH, out_dev, nullptr, stream);
}
