// Quantised V pages: every (token, kv head) value row of head_dim reals is stored as E2M1 codes with one bf16
// scale -- the per-token low-bit tier of the reference (phasorkv/kernels/nvfp4.py:58-67, quantize_per_token:
// 3 bits = integers -4 .. 3, scale = bf16(max(amax, 1e-5) / 3), round half to even; 2 bits = levels +-0.5,
// +-1.5, scale = bf16(max(amax, 1e-5) / 1.5)), four bits of storage per code as in its "nib" cache layout
// (phasorkv/kernels/latent_attn.py:207-212).
//
// Pool layout (pkv_cache_t::vq_dev): a page is n_kv * 66 rows of 128 bytes,
//   rows g * 64 .. g * 64 + 63 : the codes of kv head g, 64 bytes per token (two per byte, even dim in the low
//                                nibble); the 16-byte chunk c of token r sits at chunk position c ^ ((r >> 1) & 3)
//                                of the token's 64 bytes, so that 8 consecutive tokens read the same chunk without
//                                a shared-memory bank conflict
//   rows n_kv * 64 ..          : the bf16 scales, 128 per kv head (256 bytes), heads in order
// The attention kernel copies a code tile (64 rows) and the scale block of its 8 kv heads (16 rows) to shared
// memory as they are.
#include "pkv_common.cuh"
#include "pkv_vq.cuh"

int pkv_check_cache(const pkv_cache_t* c);

namespace {

// one warp per (token, kv head) row of 128 values; lane l holds dims 4l .. 4l+3
__global__ void __launch_bounds__(256) pkv_vq_write_kernel(const uint2* __restrict__ v_rows, const int32_t* __restrict__ slots, int n_tokens,
                                                           int n_kv, int n_pages, int bits, uint8_t* __restrict__ pool) {
    pkv_grid_wait();
    pkv_grid_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long row = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= (long)n_tokens * n_kv) return;
    const int tok = (int)(row / n_kv), g = (int)(row % n_kv);
    const int slot = slots[tok];
    if (slot < 0 || slot >= n_pages * PKV_PAGE_TOKENS) return;
    pkv_vq_store_row(v_rows[row * 32 + lane], lane, slot, g, n_kv, bits, pool);
}

// read-back in the reference's form: dequantised rows, unpacked codes, scale bit patterns
__global__ void __launch_bounds__(256) pkv_vq_read_kernel(const uint8_t* __restrict__ pool, const int32_t* __restrict__ slots, int n_tokens,
                                                          int n_kv, int n_pages, float* __restrict__ rows_out,
                                                          uint8_t* __restrict__ codes_out, uint16_t* __restrict__ scales_out) {
    const int lane = threadIdx.x & 31;
    const long row = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= (long)n_tokens * n_kv) return;
    const int tok = (int)(row / n_kv), g = (int)(row % n_kv);
    const int slot = slots[tok];
    if (slot < 0 || slot >= n_pages * PKV_PAGE_TOKENS) return;
    const uint8_t* page = pool + (size_t)(slot / PKV_PAGE_TOKENS) * n_kv * PKV_VQ_TILE_BYTES;
    const uint8_t* tile = page + (size_t)g * 8192;
    const uint32_t r = slot % PKV_PAGE_TOKENS;
    const uint32_t chunk = (lane >> 3) ^ ((r >> 1) & 3u);
    const uint32_t packed = *reinterpret_cast<const uint16_t*>(tile + r * 64 + chunk * 16 + (lane & 7) * 2);
    const uint16_t sbits = *reinterpret_cast<const uint16_t*>(page + (size_t)n_kv * 8192 + g * 256 + r * 2);
    const float s = pkv_bf16_bits_to_float(sbits);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t code = (packed >> (4 * i)) & 15u;
        if (rows_out) rows_out[row * 128 + lane * 4 + i] = __fmul_rn(pkv_e2m1_value(code), s);
        if (codes_out) codes_out[row * 128 + lane * 4 + i] = (uint8_t)code;
    }
    if (scales_out && lane == 0) scales_out[row] = sbits;
}

int check_vq(const pkv_cache_t* c) {
    int st = pkv_check_cache(c);
    if (st) return st;
    if (!c->vq_dev || (((uintptr_t)c->vq_dev) & 127u)) return PKV_ERR_INVALID;
    if (c->head_dim != 128) return PKV_ERR_UNSUPPORTED;
    if (c->v_bits != 2 && c->v_bits != 3) return PKV_ERR_INVALID;
    return PKV_OK;
}

}  // namespace

extern "C" int64_t pkv_vq_page_bytes(int32_t n_kv, int32_t head_dim) {
    if (n_kv <= 0 || head_dim != 128) return PKV_ERR_UNSUPPORTED;
    return (int64_t)n_kv * PKV_VQ_TILE_BYTES;
}

extern "C" int pkv_vq_write(const pkv_cache_t* cache, const void* v_dev, const int32_t* slots_dev, int32_t n_tokens, void* stream) {
    int st = check_vq(cache);
    if (st) return st;
    if (n_tokens < 0) return PKV_ERR_INVALID;
    if (n_tokens == 0) return PKV_OK;
    if (!v_dev || !slots_dev || (((uintptr_t)v_dev) & 7u)) return PKV_ERR_INVALID;
    const long rows = (long)n_tokens * cache->n_kv;
    PKV_CUDA_TRY(pkv_launch_chained(pkv_vq_write_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, (cudaStream_t)stream,
                                    (const uint2*)v_dev, slots_dev, n_tokens, cache->n_kv, cache->n_pages, cache->v_bits,
                                    (uint8_t*)cache->vq_dev));
    return PKV_OK;
}

extern "C" int pkv_vq_read(const pkv_cache_t* cache, const int32_t* slots_dev, int32_t n_tokens, float* rows_out_dev,
                           uint8_t* codes_out_dev, uint16_t* scales_out_dev, void* stream) {
    int st = check_vq(cache);
    if (st) return st;
    if (n_tokens < 0) return PKV_ERR_INVALID;
    if (n_tokens == 0) return PKV_OK;
    if (!slots_dev) return PKV_ERR_INVALID;
    const long rows = (long)n_tokens * cache->n_kv;
    pkv_vq_read_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)cache->vq_dev, slots_dev, n_tokens, cache->n_kv, cache->n_pages, rows_out_dev, codes_out_dev, scales_out_dev);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}
