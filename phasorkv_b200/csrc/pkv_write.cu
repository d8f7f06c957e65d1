// Fused cache write: latent projection (fp32 FMA), phasor rotation, NVFP4 quantisation, paged store.
//
// One CTA owns 64 tokens and the whole latent row of each, because the rotation pairs column k with
// column R + k and the quantiser needs 16 consecutive columns of a row.
#include "pkv_common.cuh"

int pkv_check_cache(const pkv_cache_t* c);

namespace {

constexpr int TM = 64;        // tokens per CTA
constexpr int KC = 16;        // d_model slice per main-loop step
constexpr int NT = 256;       // threads

template <int WP>
struct WriteSmem {
    static constexpr int main_floats = KC * TM + KC * WP;
    static constexpr int epi_floats = TM * (WP + 1);
    static constexpr int bytes = 4 * (main_floats > epi_floats ? main_floats : epi_floats);
};

template <int WP, typename XT>
__global__ void __launch_bounds__(NT) pkv_cache_write_kernel(
    const float* __restrict__ Bw, const XT* __restrict__ x, const int32_t* __restrict__ positions,
    const float2* __restrict__ phasors, int h2, const int32_t* __restrict__ slots, int n_tokens, int D, int W, int R, const int32_t* __restrict__ freq,
    const double* __restrict__ inv_freq, float attn_scale, float second, uint8_t* __restrict__ latent, int n_pages,
    float* __restrict__ latent_out) {
    extern __shared__ __align__(16) float smem[];
    float* Xs = smem;                   // [KC][TM]
    float* Bs = smem + KC * TM;         // [KC][WP]
    constexpr int CG = WP / 64;         // column groups of 4 per thread
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int tok0 = blockIdx.x * TM;

    float acc[4][4 * CG];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4 * CG; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < D; k0 += KC) {
        // x tile, transposed into Xs[k][token]; tokens past the end read as zero
        {
            int t = tid >> 2, kq = (tid & 3) * 4;
            int tok = tok0 + t;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (tok < n_tokens) {
                const XT* src = x + (size_t)tok * D + k0 + kq;
                if constexpr (sizeof(XT) == 4) {
                    float4 f = *reinterpret_cast<const float4*>(src);
                    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                } else {
                    uint2 u = *reinterpret_cast<const uint2*>(src);
                    v[0] = pkv_bf16_bits_to_float(u.x & 0xffffu); v[1] = pkv_bf16_bits_to_float(u.x >> 16);
                    v[2] = pkv_bf16_bits_to_float(u.y & 0xffffu); v[3] = pkv_bf16_bits_to_float(u.y >> 16);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) Xs[(kq + i) * TM + t] = v[i];
        }
        // factor tile Bs[k][col]; columns past W are zero padding
        for (int c = tid; c < WP; c += NT) {
            float4 f[4];
            if (c < W) {
                const float4* src = reinterpret_cast<const float4*>(Bw + (size_t)c * D + k0);
#pragma unroll
                for (int i = 0; i < 4; ++i) f[i] = src[i];
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) f[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                Bs[(4 * i + 0) * WP + c] = f[i].x; Bs[(4 * i + 1) * WP + c] = f[i].y;
                Bs[(4 * i + 2) * WP + c] = f[i].z; Bs[(4 * i + 3) * WP + c] = f[i].w;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < KC; ++k) {
            float4 xv = *reinterpret_cast<const float4*>(Xs + k * TM + ty * 4);
            float xr[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int g = 0; g < CG; ++g) {
                float4 bv = *reinterpret_cast<const float4*>(Bs + k * WP + g * 64 + tx * 4);
                float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][g * 4 + j] = fmaf(xr[i], br[j], acc[i][g * 4 + j]);
            }
        }
        __syncthreads();
    }

    // ---- epilogue: tile to shared memory as Ls[token][WP + 1]
    float* Ls = smem;
    constexpr int LP = WP + 1;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int g = 0; g < CG; ++g)
#pragma unroll
            for (int j = 0; j < 4; ++j) Ls[(ty * 4 + i) * LP + g * 64 + tx * 4 + j] = acc[i][g * 4 + j];
    __syncthreads();

    // rotation of (column k, column R + k) by attn_scale * e^{i * position * inv_freq[freq[k]]};
    // the angle is formed and reduced in double, the phasor rounded to fp32, the product taken in fp32
    for (int idx = tid; idx < TM * R; idx += NT) {
        int t = idx % TM, k = idx / TM;
        int tok = tok0 + t;
        if (tok >= n_tokens) continue;
        float pr, pi;
        if (phasors) {
            float2 p = phasors[(size_t)tok * h2 + freq[k]];
            pr = p.x; pi = p.y;
        } else {
            double sn, cs;
            sincos((double)positions[tok] * inv_freq[freq[k]], &sn, &cs);
            pr = (float)((double)attn_scale * cs); pi = (float)((double)attn_scale * sn);
        }
        float a = Ls[t * LP + k], b = Ls[t * LP + R + k];
        Ls[t * LP + k] = __fsub_rn(__fmul_rn(a, pr), __fmul_rn(b, pi));
        Ls[t * LP + R + k] = __fadd_rn(__fmul_rn(a, pi), __fmul_rn(b, pr));
    }
    __syncthreads();

    if (latent_out) {
        for (int idx = tid; idx < TM * W; idx += NT) {
            int t = idx / W, c = idx % W;
            if (tok0 + t < n_tokens) latent_out[(size_t)(tok0 + t) * W + c] = Ls[t * LP + c];
        }
    }

    if (!latent) return;
    // quantise: one (token, 16-column block) per thread step, tokens along the lanes
    constexpr int RB = WP / 2, NB = WP / 16;
    const int page_bytes = pkv_page_bytes(W), codes_bytes = pkv_codes_bytes(W);
    for (int idx = tid; idx < TM * NB; idx += NT) {
        int t = idx % TM, j = idx / TM;
        int tok = tok0 + t;
        if (tok >= n_tokens) continue;
        int slot = slots[tok];
        if (slot < 0 || slot >= n_pages * PKV_PAGE_TOKENS) continue;
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = Ls[t * LP + j * 16 + i];
        uint8_t sb;
        uint2 packed = pkv_quantize_block16(v, second, sb);
        uint8_t* page = latent + (size_t)(slot / PKV_PAGE_TOKENS) * page_bytes;
        uint32_t row = slot % PKV_PAGE_TOKENS;
        *reinterpret_cast<uint2*>(page + pkv_code_offset(row, j * 8, RB)) = packed;
        page[codes_bytes + pkv_scale_offset(row, j)] = sb;
    }
}

template <int WP, typename XT>
int launch_write(const pkv_layer_t* L, const pkv_cache_t* C, const void* x, const int32_t* pos, const float* ph,
                 const int32_t* slots, int n, float* latent_out, cudaStream_t st) {
    auto kern = pkv_cache_write_kernel<WP, XT>;
    constexpr int smem = WriteSmem<WP>::bytes;
    PKV_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<(n + TM - 1) / TM, NT, smem, st>>>(L->Bw_dev, (const XT*)x, pos, (const float2*)ph, L->head_dim / 2, slots, n,
                                                 L->d_model, 2 * L->R + L->R_s, L->R, L->freq_dev, L->inv_freq_dev,
                                                 L->attn_scale, L->second, C ? C->latent_dev : nullptr,
                                                 C ? C->n_pages : 0, latent_out);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

// ------------------------------------------------------------------------------------------------
// Decode-time write (a handful of tokens): the projection is spread over Wp/8 CTAs so that the
// factor matrix streams through many SMs, raw rows go to caller-provided scratch, and a second
// kernel rotates, quantises and stores them.
// ------------------------------------------------------------------------------------------------
constexpr int SM_TOK = 16;      // tokens per pass of the small projection
constexpr int SM_KC = 1024;     // d_model slice staged in shared memory

template <typename XT>
__global__ void __launch_bounds__(256) pkv_project_small_kernel(const float* __restrict__ Bw, const XT* __restrict__ x,
                                                                int n_tokens, int D, int W, int WP,
                                                                float* __restrict__ raw) {
    extern __shared__ __align__(16) float xs[];            // [SM_TOK][SM_KC]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * 8 + warp;
    for (int t0 = 0; t0 < n_tokens; t0 += SM_TOK) {
        const int nt = min(SM_TOK, n_tokens - t0);
        float acc[SM_TOK];
#pragma unroll
        for (int t = 0; t < SM_TOK; ++t) acc[t] = 0.0f;
        for (int k0 = 0; k0 < D; k0 += SM_KC) {
            const int kc = min(SM_KC, D - k0);
            __syncthreads();
            for (int i = threadIdx.x; i < SM_TOK * (kc / 4); i += 256) {
                int t = i / (kc / 4), k4 = i % (kc / 4);
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (t < nt) {
                    const XT* src = x + (size_t)(t0 + t) * D + k0 + k4 * 4;
                    if constexpr (sizeof(XT) == 4) {
                        v = *reinterpret_cast<const float4*>(src);
                    } else {
                        uint2 u = *reinterpret_cast<const uint2*>(src);
                        v = make_float4(pkv_bf16_bits_to_float(u.x & 0xffffu), pkv_bf16_bits_to_float(u.x >> 16),
                                        pkv_bf16_bits_to_float(u.y & 0xffffu), pkv_bf16_bits_to_float(u.y >> 16));
                    }
                }
                *reinterpret_cast<float4*>(xs + t * SM_KC + k4 * 4) = v;
            }
            __syncthreads();
            if (c < W) {
                for (int k = lane * 4; k < kc; k += 128) {
                    float4 b = *reinterpret_cast<const float4*>(Bw + (size_t)c * D + k0 + k);
#pragma unroll
                    for (int t = 0; t < SM_TOK; ++t) {
                        float4 xv = *reinterpret_cast<const float4*>(xs + t * SM_KC + k);
                        acc[t] = fmaf(xv.x, b.x, acc[t]); acc[t] = fmaf(xv.y, b.y, acc[t]);
                        acc[t] = fmaf(xv.z, b.z, acc[t]); acc[t] = fmaf(xv.w, b.w, acc[t]);
                    }
                }
            }
        }
#pragma unroll
        for (int t = 0; t < SM_TOK; ++t) {
            float v = acc[t];
#pragma unroll
            for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && t < nt && c < WP) raw[(size_t)(t0 + t) * WP + c] = c < W ? v : 0.0f;
        }
    }
}

// one CTA per token: rotate the complex pairs of its raw row, quantise, store
__global__ void __launch_bounds__(256) pkv_rotate_store_kernel(
    const float* __restrict__ raw, const int32_t* __restrict__ positions, const float2* __restrict__ phasors, int h2,
    const int32_t* __restrict__ slots, int W, int WP, int R, const int32_t* __restrict__ freq,
    const double* __restrict__ inv_freq, float attn_scale, float second, uint8_t* __restrict__ latent, int n_pages,
    float* __restrict__ latent_out) {
    __shared__ float row[PKV_MAX_WIDTH];
    const int tok = blockIdx.x, tid = threadIdx.x;
    for (int c = tid; c < WP; c += 256) row[c] = raw[(size_t)tok * WP + c];
    __syncthreads();
    float re = 0.f, im = 0.f;
    if (tid < R) {
        float pr, pi;
        if (phasors) {
            float2 p = phasors[(size_t)tok * h2 + freq[tid]];
            pr = p.x; pi = p.y;
        } else {
            double sn, cs;
            sincos((double)positions[tok] * inv_freq[freq[tid]], &sn, &cs);
            pr = (float)((double)attn_scale * cs); pi = (float)((double)attn_scale * sn);
        }
        float a = row[tid], b = row[R + tid];
        re = __fsub_rn(__fmul_rn(a, pr), __fmul_rn(b, pi));
        im = __fadd_rn(__fmul_rn(a, pi), __fmul_rn(b, pr));
    }
    __syncthreads();
    if (tid < R) { row[tid] = re; row[R + tid] = im; }
    __syncthreads();
    if (latent_out)
        for (int c = tid; c < W; c += 256) latent_out[(size_t)tok * W + c] = row[c];
    if (!latent) return;
    const int slot = slots[tok];
    if (slot < 0 || slot >= n_pages * PKV_PAGE_TOKENS) return;
    const int NB = WP / 16, RB = WP / 2;
    if (tid < NB) {
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = row[tid * 16 + i];
        uint8_t sb;
        uint2 packed = pkv_quantize_block16(v, second, sb);
        uint8_t* page = latent + (size_t)(slot / PKV_PAGE_TOKENS) * pkv_page_bytes(W);
        uint32_t r = slot % PKV_PAGE_TOKENS;
        *reinterpret_cast<uint2*>(page + pkv_code_offset(r, tid * 8, RB)) = packed;
        page[pkv_codes_bytes(W) + pkv_scale_offset(r, tid)] = sb;
    }
}

template <typename XT>
int launch_write_small(const pkv_layer_t* L, const pkv_cache_t* C, const void* x, const int32_t* pos, const float* ph,
                       const int32_t* slots, int n, float* latent_out, float* scratch, cudaStream_t st) {
    const int W = 2 * L->R + L->R_s, WP = pkv_padded_width(W);
    auto kern = pkv_project_small_kernel<XT>;
    constexpr int smem = SM_TOK * SM_KC * 4;
    PKV_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<WP / 8, 256, smem, st>>>(L->Bw_dev, (const XT*)x, n, L->d_model, W, WP, scratch);
    PKV_LAUNCH_CHECK();
    pkv_rotate_store_kernel<<<n, 256, 0, st>>>(scratch, pos, (const float2*)ph, L->head_dim / 2, slots, W, WP, L->R,
                                               L->freq_dev, L->inv_freq_dev, L->attn_scale, L->second,
                                               C ? C->latent_dev : nullptr, C ? C->n_pages : 0, latent_out);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

}  // namespace

int pkv_check_layer(const pkv_layer_t* L) {
    if (!L || !L->Bw_dev || !L->A_re_dev || !L->A_im_dev || !L->freq_dev || !L->inv_freq_dev) return PKV_ERR_INVALID;
    if (L->R <= 0 || L->R_s < 0 || L->n_slow < 0 || L->n_q <= 0 || L->n_kv <= 0 || L->head_dim <= 0) return PKV_ERR_INVALID;
    if (L->R_s > 0 && (!L->A_s_dev || !L->slow_dev || L->n_slow <= 0)) return PKV_ERR_INVALID;
    if (L->n_q % L->n_kv) return PKV_ERR_INVALID;
    int W = 2 * L->R + L->R_s;
    if (W > PKV_MAX_WIDTH) return PKV_ERR_UNSUPPORTED;       // a cache additionally needs W % 16 == 0
    if (L->d_model <= 0 || (L->d_model % 16)) return PKV_ERR_UNSUPPORTED;
    if (!(L->second > 0.0f)) return PKV_ERR_INVALID;
    return PKV_OK;
}

extern "C" int pkv_cache_write(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* x_dev, int32_t x_dtype,
                               const int32_t* positions_dev, const float* phasors_dev, const int32_t* slots_dev,
                               int32_t n_tokens, float* latent_out_dev, float* scratch_dev, void* stream) {
    int st = pkv_check_layer(layer);
    if (st) return st;
    const int W = 2 * layer->R + layer->R_s;
    if (n_tokens == 0) return PKV_OK;
    if (cache) {
        st = pkv_check_cache(cache);
        if (st) return st;
        if (cache->W != W || !slots_dev) return PKV_ERR_INVALID;
    } else if (!latent_out_dev) {
        return PKV_ERR_INVALID;
    }
    if (!x_dev || (!positions_dev && !phasors_dev) || n_tokens < 0) return PKV_ERR_INVALID;
    if (phasors_dev && (((uintptr_t)phasors_dev) & 7u)) return PKV_ERR_INVALID;
    if ((((uintptr_t)x_dev) | ((uintptr_t)layer->Bw_dev)) & 15u) return PKV_ERR_INVALID;
    if (x_dtype != PKV_F32 && x_dtype != PKV_BF16) return PKV_ERR_INVALID;
    if (n_tokens == 0) return PKV_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (scratch_dev && n_tokens <= PKV_SMALL_WRITE_TOKENS) {
        if ((((uintptr_t)scratch_dev) & 15u) || (layer->d_model % 4)) return PKV_ERR_INVALID;
        return x_dtype == PKV_F32 ? launch_write_small<float>(layer, cache, x_dev, positions_dev, phasors_dev, slots_dev,
                                                              n_tokens, latent_out_dev, scratch_dev, s)
                                  : launch_write_small<uint16_t>(layer, cache, x_dev, positions_dev, phasors_dev,
                                                                 slots_dev, n_tokens, latent_out_dev, scratch_dev, s);
    }
    if (pkv_padded_width(W) == 128) {
        return x_dtype == PKV_F32
                   ? launch_write<128, float>(layer, cache, x_dev, positions_dev, phasors_dev, slots_dev, n_tokens, latent_out_dev, s)
                   : launch_write<128, uint16_t>(layer, cache, x_dev, positions_dev, phasors_dev, slots_dev, n_tokens, latent_out_dev, s);
    }
    return x_dtype == PKV_F32
               ? launch_write<256, float>(layer, cache, x_dev, positions_dev, phasors_dev, slots_dev, n_tokens, latent_out_dev, s)
               : launch_write<256, uint16_t>(layer, cache, x_dev, positions_dev, phasors_dev, slots_dev, n_tokens, latent_out_dev, s);
}
