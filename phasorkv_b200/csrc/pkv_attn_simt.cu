// Decode attention on the latent cache, CUDA-core version: the correctness scaffold next to the
// tensor-core kernel. Split-T flash decoding: a CTA owns one (sequence, token split), dequantises
// 32-token tiles of the latent, scores all query heads against them, keeps a running base-2
// softmax and accumulates P.V from the bf16 V pages. Also the log-sum-exp merge kernel.
#include "pkv_common.cuh"
#include "pkv_merge.cuh"

int pkv_check_layer(const pkv_layer_t* L);
int pkv_check_cache(const pkv_cache_t* c);
int pkv_attn_tc_launch(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* q_dev,
                       const int32_t* page_table_dev, int32_t max_pages, const int32_t* seqlens_dev, int32_t batch,
                       int32_t n_split, uint32_t flags, float* partials_dev, float* scores_out_dev,
                       int64_t scores_stride, int32_t* status_dev, float* out_dev, cudaStream_t stream,
                       const float* q_raw_dev = nullptr, const int32_t* q_positions_dev = nullptr, int32_t* qsync_dev = nullptr);

namespace {

using pkv_merge_impl::MG;
using pkv_merge_impl::MergeSmem;
using pkv_merge_impl::merge_row;

constexpr int NT = 256;
constexpr int TT = 32;          // tokens per tile
constexpr int NQ = 32;          // query heads
constexpr int DH = 128;         // head_dim

template <int WP>
struct SimtSmem {
    static constexpr int CP = WP + 4;                       // pitch of the dequantised tile
    static constexpr int floats = NQ * WP + TT * CP + NQ * TT + 3 * NQ;
    static constexpr int bytes = floats * 4;
};

template <int WP, int REP>
__global__ void __launch_bounds__(NT) pkv_attn_simt_kernel(
    const float* __restrict__ q, const uint8_t* __restrict__ latent, const uint16_t* __restrict__ vpool,
    const int32_t* __restrict__ page_table, int max_pages, const int32_t* __restrict__ seqlens, int n_split,
    int n_pages_pool, int W, float second, float logit_scale, uint32_t flags, float* __restrict__ partials,
    float* __restrict__ scores_out, long scores_stride) {
    extern __shared__ __align__(16) float sm[];
    constexpr int CP = SimtSmem<WP>::CP, NB = WP / 16, RB = WP / 2;
    constexpr int EPT = 16 / REP;                           // V elements per thread
    float* qs = sm;                                         // [NQ][WP]
    float* cs = qs + NQ * WP;                               // [TT][CP]
    float* ps = cs + TT * CP;                               // [NQ][TT]
    float* m_s = ps + NQ * TT;                              // [NQ] running max (base-2 logits)
    float* l_s = m_s + NQ;                                  // [NQ] running sum
    float* corr_s = l_s + NQ;                               // [NQ] rescale of this tile

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int split = blockIdx.x, b = blockIdx.y;
    const int T = seqlens[b];
    const int npages = min((T + PKV_PAGE_TOKENS - 1) / PKV_PAGE_TOKENS, max_pages);
    const int pps = (npages + n_split - 1) / n_split;
    const int p_lo = split * pps, p_hi = min(npages, p_lo + pps);
    const int page_bytes = pkv_page_bytes(W), codes_bytes = pkv_codes_bytes(W);
    const bool with_v = !(flags & PKV_ATTN_SCORES_ONLY);
    const int n_kv = NQ / REP;

    for (int i = tid; i < NQ * WP; i += NT) {
        int h = i / WP, c = i % WP;
        qs[i] = c < W ? q[((size_t)b * NQ + h) * W + c] : 0.0f;
    }
    if (tid < NQ) { m_s[tid] = -INFINITY; l_s[tid] = 0.0f; }
    float acc[REP][EPT];
#pragma unroll
    for (int r = 0; r < REP; ++r)
#pragma unroll
        for (int e = 0; e < EPT; ++e) acc[r][e] = 0.0f;
    const int elem0 = tid * EPT;                            // first V element of this thread in a token row
    const int g = elem0 / DH;                               // its kv head
    __syncthreads();

    for (int page = p_lo; page < p_hi; ++page) {
        int pidx = page_table[(size_t)b * max_pages + page];
        if (pidx < 0 || pidx >= n_pages_pool) continue;     // out-of-range entry: skipped, never dereferenced
        const uint8_t* pg = latent + (size_t)pidx * page_bytes;
        for (int sub = 0; sub < PKV_PAGE_TOKENS / TT; ++sub) {
            const int t0 = page * PKV_PAGE_TOKENS + sub * TT;
            if (t0 >= T) break;
            // ---- dequantise the tile
            {
                int t = tid >> 3, part = tid & 7;
                uint32_t row = sub * TT + t;
#pragma unroll
                for (int jj = 0; jj < NB / 8; ++jj) {
                    int j = part * (NB / 8) + jj;
                    uint2 packed = *reinterpret_cast<const uint2*>(pg + pkv_code_offset(row, j * 8, RB));
                    float scale = __fmul_rn(pkv_e4m3_to_float(pg[codes_bytes + pkv_scale_offset(row, j)]), second);
                    float* dst = cs + t * CP + j * 16;
#pragma unroll
                    for (int i = 0; i < 8; ++i) dst[i] = __fmul_rn(pkv_e2m1_value((packed.x >> (4 * i)) & 15u), scale);
#pragma unroll
                    for (int i = 0; i < 8; ++i) dst[8 + i] = __fmul_rn(pkv_e2m1_value((packed.y >> (4 * i)) & 15u), scale);
                }
            }
            __syncthreads();
            // ---- scores of 4 heads per warp, one token per lane; online softmax statistics
            {
                float s[4] = {0.f, 0.f, 0.f, 0.f};
                const float* crow = cs + lane * CP;
                const float* q0 = qs + (warp * 4) * WP;
#pragma unroll 4
                for (int k = 0; k < WP; k += 4) {
                    float4 c = *reinterpret_cast<const float4*>(crow + k);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float4 qv = *reinterpret_cast<const float4*>(q0 + i * WP + k);
                        s[i] = fmaf(c.x, qv.x, s[i]); s[i] = fmaf(c.y, qv.y, s[i]);
                        s[i] = fmaf(c.z, qv.z, s[i]); s[i] = fmaf(c.w, qv.w, s[i]);
                    }
                }
                const bool valid = t0 + lane < T;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int h = warp * 4 + i;
                    if (scores_out && valid) scores_out[((size_t)b * NQ + h) * scores_stride + t0 + lane] = s[i];
                    float s2 = valid ? s[i] * logit_scale : -INFINITY;
                    float mx = s2;
#pragma unroll
                    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                    const float m_old = m_s[h];
                    const float m_new = fmaxf(m_old, mx);
                    const float p = valid ? exp2f(s2 - m_new) : 0.0f;
                    float sum = p;
#pragma unroll
                    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                    const float corr = exp2f(m_old - m_new);        // 0 on the first tile (m_old = -inf)
                    ps[h * TT + lane] = p;
                    __syncwarp();
                    if (lane == 0) { m_s[h] = m_new; l_s[h] = l_s[h] * corr + sum; corr_s[h] = corr; }
                }
            }
            __syncthreads();
            // ---- P.V: this thread owns EPT consecutive V elements of kv head g and its REP query heads
            if (with_v) {
#pragma unroll
                for (int r = 0; r < REP; ++r) {
                    const float c = corr_s[g * REP + r];
#pragma unroll
                    for (int e = 0; e < EPT; ++e) acc[r][e] *= c;
                }
                const uint16_t* vrow = vpool + (((size_t)pidx * n_kv + g) * PKV_PAGE_TOKENS + sub * TT) * DH + elem0 % DH;
                const int nt = min(TT, T - t0);
#pragma unroll 4
                for (int t = 0; t < nt; ++t) {
                    float v[EPT];
                    if constexpr (EPT == 2) {
                        uint32_t u = *reinterpret_cast<const uint32_t*>(vrow + (size_t)t * DH);
                        v[0] = pkv_bf16_bits_to_float(u & 0xffffu); v[1] = pkv_bf16_bits_to_float(u >> 16);
                    } else {
#pragma unroll
                        for (int e4 = 0; e4 < EPT / 4; ++e4) {
                            uint2 u = *reinterpret_cast<const uint2*>(vrow + (size_t)t * DH + e4 * 4);
                            v[e4 * 4 + 0] = pkv_bf16_bits_to_float(u.x & 0xffffu); v[e4 * 4 + 1] = pkv_bf16_bits_to_float(u.x >> 16);
                            v[e4 * 4 + 2] = pkv_bf16_bits_to_float(u.y & 0xffffu); v[e4 * 4 + 3] = pkv_bf16_bits_to_float(u.y >> 16);
                        }
                    }
#pragma unroll
                    for (int r = 0; r < REP; ++r) {
                        const float p = ps[(g * REP + r) * TT + t];
#pragma unroll
                        for (int e = 0; e < EPT; ++e) acc[r][e] = fmaf(p, v[e], acc[r][e]);
                    }
                }
            }
            __syncthreads();
        }
    }
    // ---- partial triple of this split: o[DH], m, l per head
    float* part = partials + ((size_t)b * n_split + split) * NQ * (DH + 2);
    const int d0 = elem0 % DH;
#pragma unroll
    for (int r = 0; r < REP; ++r)
#pragma unroll
        for (int e = 0; e < EPT; ++e) part[(g * REP + r) * (DH + 2) + d0 + e] = with_v ? acc[r][e] : 0.0f;
    if (tid < NQ) {
        part[tid * (DH + 2) + DH] = m_s[tid];
        part[tid * (DH + 2) + DH + 1] = l_s[tid];
    }
}

// One CTA per (sequence, head): the merge of pkv_merge.cuh, then the normalised and / or packed store.
__global__ void __launch_bounds__(MG * 128) pkv_merge_kernel(const float* __restrict__ parts, long stride_b, long stride_p,
                                                             int n_parts, int n_q, int head_dim, int batch,
                                                             const float* __restrict__ exact, float* __restrict__ out,
                                                             float* __restrict__ packed_out) {
    __shared__ MergeSmem S;
    const int tid = threadIdx.x, d = tid & 127, g = tid >> 7;
    const int b = blockIdx.x / n_q, h = blockIdx.x % n_q;
    const int PW = head_dim + 2;
    pkv_grid_launch_dependents();
    pkv_grid_wait();
    float a0, a1, M, den;
    merge_row(parts + (size_t)b * stride_b + (size_t)h * PW, stride_p, n_parts, head_dim, S, a0, a1, M, den,
              exact ? exact + ((size_t)b * n_q + h) * PW : nullptr);
    if (g == 0) {
        const size_t row = (size_t)b * n_q + h;
        if (d < head_dim) {
            if (out) out[row * head_dim + d] = den > 0.0f ? a0 / den : 0.0f;
            if (packed_out) packed_out[row * PW + d] = a0;
        }
        if (d + 128 < head_dim) {
            if (out) out[row * head_dim + d + 128] = den > 0.0f ? a1 / den : 0.0f;
            if (packed_out) packed_out[row * PW + d + 128] = a1;
        }
        if (packed_out && d == 0) {
            packed_out[row * PW + head_dim] = M;
            packed_out[row * PW + head_dim + 1] = den;
        }
    }
}

template <int WP, int REP>
int launch_simt(const pkv_layer_t* L, const pkv_cache_t* C, const float* q, const int32_t* pt, int max_pages,
                const int32_t* seqlens, int batch, int n_split, uint32_t flags, float* partials, float* scores,
                long scores_stride, cudaStream_t st) {
    auto kern = pkv_attn_simt_kernel<WP, REP>;
    constexpr int smem = SimtSmem<WP>::bytes;
    PKV_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    float logit_scale = PKV_LOG2E / sqrtf((float)L->head_dim);
    kern<<<dim3(n_split, batch), NT, smem, st>>>(q, C->latent_dev, (const uint16_t*)C->v_dev, pt, max_pages, seqlens,
                                                  n_split, C->n_pages, C->W, L->second, logit_scale, flags, partials,
                                                  scores, scores_stride);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

}  // namespace

extern "C" int pkv_decode_attn(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* q_dev,
                               const int32_t* page_table_dev, int32_t max_pages, const int32_t* seqlens_dev,
                               int32_t batch, int32_t n_split, uint32_t flags, float* partials_dev,
                               float* scores_out_dev, int64_t scores_stride, int32_t* status_dev, float* out_dev,
                               void* stream) {
    return pkv_decode_attn_sync(layer, cache, q_dev, nullptr, page_table_dev, max_pages, seqlens_dev, batch, n_split, flags,
                                partials_dev, scores_out_dev, scores_stride, status_dev, out_dev, stream);
}

extern "C" int pkv_decode_attn_sync(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* q_dev, int32_t* qsync_dev,
                                    const int32_t* page_table_dev, int32_t max_pages, const int32_t* seqlens_dev,
                                    int32_t batch, int32_t n_split, uint32_t flags, float* partials_dev,
                                    float* scores_out_dev, int64_t scores_stride, int32_t* status_dev, float* out_dev,
                                    void* stream) {
    int st = pkv_check_layer(layer);
    if (st) return st;
    st = pkv_check_cache(cache);
    if (st) return st;
    if (batch == 0) return PKV_OK;
    if (!q_dev || !page_table_dev || !seqlens_dev || !partials_dev) return PKV_ERR_INVALID;
    if (batch < 0 || n_split <= 0 || max_pages <= 0 || n_split > 65535 || batch > 65535) return PKV_ERR_INVALID;
    if (cache->W != 2 * layer->R + layer->R_s || cache->n_kv != layer->n_kv || cache->head_dim != layer->head_dim)
        return PKV_ERR_INVALID;
    if (layer->n_q != NQ || layer->head_dim != DH) return PKV_ERR_UNSUPPORTED;
    const bool with_v = !(flags & PKV_ATTN_SCORES_ONLY);
    if (with_v && !(cache->v_bits ? cache->vq_dev : cache->v_dev)) return PKV_ERR_INVALID;
    if (with_v && cache->v_bits && (flags & PKV_ATTN_SIMT)) return PKV_ERR_UNSUPPORTED;   // quantised V pages: tensor-core kernel only
    if (batch == 0) return PKV_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (!(flags & PKV_ATTN_SIMT))
        return pkv_attn_tc_launch(layer, cache, q_dev, page_table_dev, max_pages, seqlens_dev, batch, n_split, flags,
                                  partials_dev, scores_out_dev, scores_stride, status_dev, out_dev, s, nullptr, nullptr, qsync_dev);
    if (qsync_dev) return PKV_ERR_INVALID;                 // the CUDA-core kernel waits for the whole launch before it
    if (((uintptr_t)q_dev) & 15u) return PKV_ERR_INVALID;
    const int rep = layer->n_q / layer->n_kv;
    const bool wide = pkv_padded_width(cache->W) == 256;
    int rc = PKV_ERR_UNSUPPORTED;
#define PKV_SIMT_CASE(R_)                                                                                          \
    case R_:                                                                                                       \
        rc = wide ? launch_simt<256, R_>(layer, cache, (const float*)q_dev, page_table_dev, max_pages, seqlens_dev, \
                                           batch, n_split, flags, partials_dev, scores_out_dev, scores_stride, s)  \
                    : launch_simt<128, R_>(layer, cache, (const float*)q_dev, page_table_dev, max_pages, seqlens_dev, \
                                           batch, n_split, flags, partials_dev, scores_out_dev, scores_stride, s); \
        break;
    switch (rep) {
        PKV_SIMT_CASE(1)
        PKV_SIMT_CASE(2)
        PKV_SIMT_CASE(4)
        PKV_SIMT_CASE(8)
        default: break;
    }
#undef PKV_SIMT_CASE
    if (rc == PKV_OK && out_dev) {                         // the CUDA-core kernel merges with a second launch
        const int64_t pw = DH + 2;
        const bool packed = (flags & PKV_ATTN_PACKED_OUT) != 0;
        rc = pkv_merge(partials_dev, (int64_t)n_split * NQ * pw, NQ * pw, n_split, batch, NQ, DH, packed ? nullptr : out_dev,
                       packed ? out_dev : nullptr, stream);
    }
    return rc;
}

extern "C" int pkv_decode_attn_q(const pkv_layer_t* layer, const pkv_cache_t* cache, const float* q_dev,
                                 const int32_t* query_positions_dev, const int32_t* page_table_dev, int32_t max_pages,
                                 const int32_t* seqlens_dev, int32_t batch, int32_t n_split, uint32_t flags,
                                 float* partials_dev, float* scores_out_dev, int64_t scores_stride, int32_t* status_dev,
                                 float* out_dev, void* stream) {
    int st = pkv_check_layer(layer);
    if (st) return st;
    st = pkv_check_cache(cache);
    if (st) return st;
    if (batch == 0) return PKV_OK;
    if (!q_dev || !query_positions_dev || !page_table_dev || !seqlens_dev || !partials_dev) return PKV_ERR_INVALID;
    if (batch < 0 || n_split <= 0 || max_pages <= 0 || n_split > 65535 || batch > 65535) return PKV_ERR_INVALID;
    if (cache->W != 2 * layer->R + layer->R_s || cache->n_kv != layer->n_kv || cache->head_dim != layer->head_dim)
        return PKV_ERR_INVALID;
    if (layer->n_q != NQ || layer->head_dim != DH) return PKV_ERR_UNSUPPORTED;
    if (flags & PKV_ATTN_SIMT) return PKV_ERR_UNSUPPORTED;             // the CUDA-core kernel takes the fp32 absorbed query
    if (!(flags & PKV_ATTN_SCORES_ONLY) && (cache->v_bits || !cache->v_dev)) return cache->v_bits ? PKV_ERR_UNSUPPORTED : PKV_ERR_INVALID;
    return pkv_attn_tc_launch(layer, cache, nullptr, page_table_dev, max_pages, seqlens_dev, batch, n_split, flags, partials_dev,
                              scores_out_dev, scores_stride, status_dev, out_dev, (cudaStream_t)stream, q_dev,
                              query_positions_dev);
}

extern "C" int pkv_merge_exact(const float* parts_dev, int64_t stride_b, int64_t stride_p, int32_t n_parts, int32_t batch,
                               int32_t n_q, int32_t head_dim, const float* exact_dev, float* out_dev, float* packed_out_dev,
                               void* stream) {
    if (!parts_dev || n_parts <= 0 || batch < 0 || n_q <= 0 || head_dim <= 0 || head_dim > 256) return PKV_ERR_INVALID;
    if (n_parts + (exact_dev ? 1 : 0) > pkv_merge_impl::MAX_PARTS) return PKV_ERR_UNSUPPORTED;
    if ((head_dim & 1) || (stride_b & 1) || (stride_p & 1) || (((uintptr_t)parts_dev) & 7u)) return PKV_ERR_INVALID;   // (m, l) is read as one 8-byte pair
    if (((uintptr_t)exact_dev) & 7u) return PKV_ERR_INVALID;
    if (!out_dev && !packed_out_dev) return PKV_ERR_INVALID;
    if (batch == 0) return PKV_OK;
    PKV_CUDA_TRY(pkv_launch_chained(pkv_merge_kernel, dim3(batch * n_q), dim3(MG * 128), 0, (cudaStream_t)stream,
                                    parts_dev, (long)stride_b, (long)stride_p, n_parts, n_q, head_dim, batch, exact_dev, out_dev,
                                    packed_out_dev));
    return PKV_OK;
}

extern "C" int pkv_merge(const float* parts_dev, int64_t stride_b, int64_t stride_p, int32_t n_parts, int32_t batch,
                         int32_t n_q, int32_t head_dim, float* out_dev, float* packed_out_dev, void* stream) {
    return pkv_merge_exact(parts_dev, stride_b, stride_p, n_parts, batch, n_q, head_dim, nullptr, out_dev, packed_out_dev, stream);
}
