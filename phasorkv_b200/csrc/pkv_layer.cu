// Layer handles for callers that have no tensor library of their own (a C or C++ host): the factors of
// phasorkv.latent.PhasorKey (phasorkv/latent.py:47-54) are uploaded once into device memory that the
// handle owns. These two calls are the only ones in the library that allocate or free device memory
// and that synchronise; Python callers keep the arrays as torch tensors and fill pkv_layer_t
// themselves. Also here: the entry points under the names a binding written against the reference's
// vocabulary would look for (quantize_nvfp4, dequant, status_read).
#include "pkv_common.cuh"

#include <cuda_bf16.h>

#include <cstdlib>
#include <vector>

int pkv_check_layer(const pkv_layer_t* L);

namespace {

struct Owned {
    pkv_layer_t layer;              // first member: a pkv_layer_t* handed out is the handle
    void* dev[9];
    int n_dev;
};

template <typename T>
cudaError_t upload(Owned* o, const T* host, size_t n, const T** out) {
    *out = nullptr;
    if (!host || n == 0) return cudaSuccess;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, n * sizeof(T));
    if (e != cudaSuccess) return e;
    o->dev[o->n_dev++] = p;
    e = cudaMemcpy(p, host, n * sizeof(T), cudaMemcpyHostToDevice);
    *out = static_cast<const T*>(p);
    return e;
}

void release(Owned* o) {
    for (int i = 0; i < o->n_dev; ++i) cudaFree(o->dev[i]);
    free(o);
}

}  // namespace

extern "C" int pkv_layer_create(const pkv_layer_host_t* h, pkv_layer_t** out) {
    if (!h || !out) return PKV_ERR_INVALID;
    *out = nullptr;
    if (!h->B_re || !h->B_im || !h->A_re || !h->A_im || !h->freq || !h->inv_freq) return PKV_ERR_INVALID;
    if (h->R <= 0 || h->R_s < 0 || h->d_model <= 0 || h->n_kv <= 0 || h->head_dim <= 0) return PKV_ERR_INVALID;
    if (h->R_s > 0 && (!h->B_s || !h->A_s || !h->slow || h->n_slow <= 0)) return PKV_ERR_INVALID;
    const int W = 2 * h->R + h->R_s, D = h->d_model;
    if (W > PKV_MAX_WIDTH) return PKV_ERR_UNSUPPORTED;
    Owned* o = static_cast<Owned*>(calloc(1, sizeof(Owned)));
    if (!o) return PKV_ERR_INVALID;
    pkv_layer_t& L = o->layer;
    L.d_model = D; L.n_q = h->n_q; L.n_kv = h->n_kv; L.head_dim = h->head_dim;
    L.R = h->R; L.R_s = h->R_s; L.n_slow = h->R_s > 0 ? h->n_slow : 0;
    L.attn_scale = h->attn_scale; L.second = h->second;
    // Bw = [Re B ; Im B ; B_s], rows of d_model floats: the layout of a latent row (phasorkv/latent.py:67-70)
    std::vector<float> bw((size_t)W * D);
    for (int r = 0; r < h->R; ++r)
        for (int k = 0; k < D; ++k) {
            bw[(size_t)r * D + k] = h->B_re[(size_t)r * D + k];
            bw[(size_t)(h->R + r) * D + k] = h->B_im[(size_t)r * D + k];
        }
    for (int r = 0; r < h->R_s; ++r)
        for (int k = 0; k < D; ++k) bw[(size_t)(2 * h->R + r) * D + k] = h->B_s[(size_t)r * D + k];
    // the same matrix as three bf16 terms whose sum is Bw to 2^-24, padded to the page width (tensor-core write)
    const int WP = pkv_padded_width(W);
    std::vector<__nv_bfloat16> bw3((size_t)3 * WP * D, __float2bfloat16(0.0f));
    for (int r = 0; r < W; ++r)
        for (int k = 0; k < D; ++k) {
            const float v = bw[(size_t)r * D + k];
            const __nv_bfloat16 hi = __float2bfloat16(v);
            const float r1 = v - __bfloat162float(hi);
            const __nv_bfloat16 mid = __float2bfloat16(r1);
            const __nv_bfloat16 lo = __float2bfloat16(r1 - __bfloat162float(mid));
            bw3[((size_t)0 * WP + r) * D + k] = hi;
            bw3[((size_t)1 * WP + r) * D + k] = mid;
            bw3[((size_t)2 * WP + r) * D + k] = lo;
        }
    cudaError_t e = cudaSuccess;
    const __nv_bfloat16* bw3_dev = nullptr;
    const size_t n_a = (size_t)h->n_kv * h->R;
    if (e == cudaSuccess) e = upload(o, bw.data(), bw.size(), &L.Bw_dev);
    if (e == cudaSuccess) e = upload(o, bw3.data(), bw3.size(), &bw3_dev);
    if (e == cudaSuccess) e = upload(o, h->A_re, n_a, &L.A_re_dev);
    if (e == cudaSuccess) e = upload(o, h->A_im, n_a, &L.A_im_dev);
    if (e == cudaSuccess) e = upload(o, h->freq, (size_t)h->R, &L.freq_dev);
    if (e == cudaSuccess) e = upload(o, h->inv_freq, (size_t)h->head_dim / 2, &L.inv_freq_dev);
    if (e == cudaSuccess && h->R_s > 0) {
        e = upload(o, h->A_s, (size_t)h->n_kv * 2 * h->n_slow * h->R_s, &L.A_s_dev);
        if (e == cudaSuccess) e = upload(o, h->slow, (size_t)h->n_slow, &L.slow_dev);
    }
    L.Bw_bf16x3_dev = bw3_dev;
    if (e != cudaSuccess) {
        g_pkv_last_cuda_error = (int)e;
        release(o);
        return PKV_ERR_CUDA;
    }
    const int st = pkv_check_layer(&L);
    if (st) { release(o); return st; }
    *out = &o->layer;
    return PKV_OK;
}

extern "C" int pkv_layer_destroy(pkv_layer_t* layer) {
    if (!layer) return PKV_OK;
    release(reinterpret_cast<Owned*>(layer));
    return PKV_OK;
}

extern "C" int pkv_quantize_nvfp4(const pkv_cache_t* cache, const float* rows_dev, const int32_t* slots_dev, int32_t n_tokens,
                                  float second, void* stream) {
    return pkv_quantize_rows(cache, rows_dev, slots_dev, n_tokens, second, stream);
}

extern "C" int pkv_dequant(const pkv_cache_t* cache, const int32_t* slots_dev, int32_t n_tokens, float second,
                           float* rows_out_dev, void* stream) {
    if (!rows_out_dev && n_tokens > 0) return PKV_ERR_INVALID;
    return pkv_cache_read(cache, slots_dev, n_tokens, second, rows_out_dev, nullptr, nullptr, stream);
}

extern "C" int pkv_status_read(const int32_t* status_dev, int32_t* status_host, void* stream) {
    if (!status_dev || !status_host) return PKV_ERR_INVALID;
    PKV_CUDA_TRY(cudaMemcpyAsync(status_host, status_dev, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    PKV_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return PKV_OK;
}
