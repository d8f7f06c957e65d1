// NVFP4 quantise-and-pack of fp32 latent rows into cache pages, V row store, and read-back.
#include "pkv_common.cuh"

#include <cstdlib>

thread_local int g_pkv_last_cuda_error = 0;

extern "C" int pkv_abi_version(void) { return 2; }

extern "C" const char* pkv_status_string(int s) {
    switch (s) {
        case PKV_OK: return "ok";
        case PKV_ERR_INVALID: return "invalid argument";
        case PKV_ERR_UNSUPPORTED: return "unsupported shape";
        case PKV_ERR_CUDA: return "CUDA runtime error";
        case PKV_ERR_ARCH: return "device is not sm_100";
        default: return "unknown status";
    }
}

extern "C" int pkv_last_cuda_error(void) { return g_pkv_last_cuda_error; }

extern "C" int pkv_device_check(void) {
    int dev = 0, major = 0;
    PKV_CUDA_TRY(cudaGetDevice(&dev));
    PKV_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    return major == 10 ? PKV_OK : PKV_ERR_ARCH;
}

extern "C" int64_t pkv_latent_page_bytes(int32_t W) {
    if (W <= 0 || W > PKV_MAX_WIDTH || (W % 16)) return PKV_ERR_UNSUPPORTED;
    return pkv_page_bytes(W);
}

extern "C" int64_t pkv_v_page_bytes(int32_t n_kv, int32_t head_dim) {
    if (n_kv <= 0 || head_dim <= 0) return PKV_ERR_INVALID;
    return (int64_t)PKV_PAGE_TOKENS * n_kv * head_dim * 2;
}

// Rounding of the E4M3 block scales: process-wide like the reference's switch, which is read once from the
// environment when phasorkv.quant is imported (phasorkv/quant.py:57). -1 = not decided yet.
static int g_scale_round_up = -1;

int pkv_scale_round_up_mode() {
    if (g_scale_round_up < 0) {
        const char* e = getenv("PHASORKV_SCALE_UP");
        g_scale_round_up = (e && e[0] == '1' && e[1] == 0) ? 1 : 0;
    }
    return g_scale_round_up;
}

extern "C" int pkv_set_scale_round_up(int32_t on) {
    g_scale_round_up = on ? 1 : 0;
    return PKV_OK;
}

int pkv_check_cache(const pkv_cache_t* c) {
    if (!c || !c->latent_dev || c->n_pages <= 0) return PKV_ERR_INVALID;
    if (c->W <= 0 || c->W > PKV_MAX_WIDTH || (c->W % 16)) return PKV_ERR_UNSUPPORTED;
    if (((uintptr_t)c->latent_dev) & 1023u) return PKV_ERR_INVALID;
    return PKV_OK;
}

// one thread per (token, 16-column block); blocks of the zero padding up to the page's row pitch
// are written as zero codes with a zero scale
__global__ void pkv_quantize_rows_kernel(uint8_t* __restrict__ latent, const float* __restrict__ rows,
                                         const int32_t* __restrict__ slots, int n_tokens, int W, int n_pages,
                                         const pkv_second second, int scale_up) {
    const int Wp = pkv_padded_width(W), RB = Wp / 2, nb = Wp / 16;
    const int page_bytes = pkv_page_bytes(W), codes_bytes = pkv_codes_bytes(W);
    long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_tokens * nb) return;
    int tok = (int)(idx / nb), j = (int)(idx % nb);
    int slot = slots[tok];
    if (slot < 0 || slot >= n_pages * PKV_PAGE_TOKENS) return;
    uint8_t* page = latent + (size_t)(slot / PKV_PAGE_TOKENS) * page_bytes;
    uint32_t row = slot % PKV_PAGE_TOKENS;
    uint2 packed = make_uint2(0u, 0u);
    uint8_t sb = 0;
    if (j * 16 < W) {
        float v[16];
        const float4* src = reinterpret_cast<const float4*>(rows + (size_t)tok * W + j * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float4 f = src[i];
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
        packed = pkv_quantize_block16(v, second.of(j), sb, scale_up != 0);
    }
    *reinterpret_cast<uint2*>(page + pkv_code_offset(row, j * 8, RB)) = packed;
    page[codes_bytes + pkv_scale_offset(row, j)] = sb;
}

static int quantize_rows_impl(const pkv_cache_t* cache, const float* rows_dev, const int32_t* slots_dev, int32_t n_tokens,
                              float second, const float* second_blocks_dev, void* stream);

extern "C" int pkv_quantize_rows(const pkv_cache_t* cache, const float* rows_dev, const int32_t* slots_dev,
                                 int32_t n_tokens, float second, void* stream) {
    if (!(second > 0.0f)) return PKV_ERR_INVALID;
    return quantize_rows_impl(cache, rows_dev, slots_dev, n_tokens, second, nullptr, stream);
}

extern "C" int pkv_quantize_rows_tiered(const pkv_cache_t* cache, const float* rows_dev, const int32_t* slots_dev,
                                        int32_t n_tokens, const float* second_blocks_dev, void* stream) {
    if (!second_blocks_dev) return PKV_ERR_INVALID;
    return quantize_rows_impl(cache, rows_dev, slots_dev, n_tokens, 1.0f, second_blocks_dev, stream);
}

static int quantize_rows_impl(const pkv_cache_t* cache, const float* rows_dev, const int32_t* slots_dev, int32_t n_tokens,
                              float second, const float* second_blocks_dev, void* stream) {
    int st = pkv_check_cache(cache);
    if (st) return st;
    if (n_tokens < 0) return PKV_ERR_INVALID;
    if (n_tokens == 0) return PKV_OK;                      // nothing to do: buffers may be empty (NULL)
    if (!rows_dev || !slots_dev || (((uintptr_t)rows_dev) & 15u)) return PKV_ERR_INVALID;
    long n = (long)n_tokens * (pkv_padded_width(cache->W) / 16);
    pkv_quantize_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        cache->latent_dev, rows_dev, slots_dev, n_tokens, cache->W, cache->n_pages, pkv_second{second, second_blocks_dev},
        pkv_scale_round_up_mode());
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

// V rows: 16-byte vectors, one thread each
__global__ void pkv_v_write_kernel(uint4* __restrict__ vpool, const uint4* __restrict__ v,
                                   const int32_t* __restrict__ slots, int n_tokens, int vec_per_row, int n_kv, int n_pages) {
    long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_tokens * vec_per_row) return;
    int tok = (int)(idx / vec_per_row), c = (int)(idx % vec_per_row);
    int slot = slots[tok];
    if (slot < 0 || slot >= n_pages * PKV_PAGE_TOKENS) return;
    vpool[pkv_v_vec_index(slot, c, n_kv, vec_per_row / n_kv)] = v[(size_t)tok * vec_per_row + c];
}

extern "C" int pkv_v_write(const pkv_cache_t* cache, const void* v_dev, const int32_t* slots_dev,
                           int32_t n_tokens, void* stream) {
    if (!cache || !cache->v_dev || n_tokens < 0) return PKV_ERR_INVALID;
    if (n_tokens == 0) return PKV_OK;
    if (!v_dev || !slots_dev) return PKV_ERR_INVALID;
    int row_bytes = cache->n_kv * cache->head_dim * 2;
    if (row_bytes <= 0 || (cache->head_dim % 8) || (((uintptr_t)v_dev | (uintptr_t)cache->v_dev) & 15u))
        return PKV_ERR_INVALID;
    if (n_tokens == 0) return PKV_OK;
    long n = (long)n_tokens * (row_bytes / 16);
    pkv_v_write_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (uint4*)cache->v_dev, (const uint4*)v_dev, slots_dev, n_tokens, row_bytes / 16, cache->n_kv, cache->n_pages);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

// one thread per (token, 16-column block) of the true width W
__global__ void pkv_cache_read_kernel(const uint8_t* __restrict__ latent, const int32_t* __restrict__ slots,
                                      int n_tokens, int W, int n_pages, const pkv_second second, float* __restrict__ rows_out,
                                      uint8_t* __restrict__ codes_out, uint8_t* __restrict__ scales_out) {
    const int RB = pkv_row_bytes(W), nb = W / 16;
    const int page_bytes = pkv_page_bytes(W), codes_bytes = pkv_codes_bytes(W);
    long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_tokens * nb) return;
    int tok = (int)(idx / nb), j = (int)(idx % nb);
    int slot = slots[tok];
    if (slot < 0 || slot >= n_pages * PKV_PAGE_TOKENS) return;
    const uint8_t* page = latent + (size_t)(slot / PKV_PAGE_TOKENS) * page_bytes;
    uint32_t row = slot % PKV_PAGE_TOKENS;
    uint2 packed = *reinterpret_cast<const uint2*>(page + pkv_code_offset(row, j * 8, RB));
    uint8_t sb = page[codes_bytes + pkv_scale_offset(row, j)];
    if (codes_out) *reinterpret_cast<uint2*>(codes_out + (size_t)tok * (W / 2) + j * 8) = packed;
    if (scales_out) scales_out[(size_t)tok * nb + j] = sb;
    if (rows_out) {
        float scale = __fmul_rn(pkv_e4m3_to_float(sb), second.of(j));
        float* dst = rows_out + (size_t)tok * W + j * 16;
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[i] = __fmul_rn(pkv_e2m1_value((packed.x >> (4 * i)) & 15u), scale);
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[8 + i] = __fmul_rn(pkv_e2m1_value((packed.y >> (4 * i)) & 15u), scale);
    }
}

static int cache_read_impl(const pkv_cache_t* cache, const int32_t* slots_dev, int32_t n_tokens, pkv_second second,
                           float* rows_out_dev, uint8_t* codes_out_dev, uint8_t* scales_out_dev, void* stream);

extern "C" int pkv_cache_read(const pkv_cache_t* cache, const int32_t* slots_dev, int32_t n_tokens, float second,
                              float* rows_out_dev, uint8_t* codes_out_dev, uint8_t* scales_out_dev, void* stream) {
    return cache_read_impl(cache, slots_dev, n_tokens, pkv_second{second, nullptr}, rows_out_dev, codes_out_dev, scales_out_dev, stream);
}

extern "C" int pkv_cache_read_tiered(const pkv_cache_t* cache, const int32_t* slots_dev, int32_t n_tokens,
                                     const float* second_blocks_dev, float* rows_out_dev, uint8_t* codes_out_dev,
                                     uint8_t* scales_out_dev, void* stream) {
    if (!second_blocks_dev) return PKV_ERR_INVALID;
    return cache_read_impl(cache, slots_dev, n_tokens, pkv_second{1.0f, second_blocks_dev}, rows_out_dev, codes_out_dev, scales_out_dev,
                           stream);
}

static int cache_read_impl(const pkv_cache_t* cache, const int32_t* slots_dev, int32_t n_tokens, pkv_second second,
                           float* rows_out_dev, uint8_t* codes_out_dev, uint8_t* scales_out_dev, void* stream) {
    int st = pkv_check_cache(cache);
    if (st) return st;
    if (n_tokens < 0) return PKV_ERR_INVALID;
    if (n_tokens == 0) return PKV_OK;
    if (!slots_dev) return PKV_ERR_INVALID;
    if (codes_out_dev && (((uintptr_t)codes_out_dev) & 7u)) return PKV_ERR_INVALID;
    long n = (long)n_tokens * (cache->W / 16);
    pkv_cache_read_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        cache->latent_dev, slots_dev, n_tokens, cache->W, cache->n_pages, second, rows_out_dev, codes_out_dev,
        scales_out_dev);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}
