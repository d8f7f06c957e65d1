// Fused cache write: latent projection (fp32 FMA), phasor rotation, NVFP4 quantisation, paged store.
//
// One CTA owns 64 tokens and the whole latent row of each, because the rotation pairs column k with
// column R + k and the quantiser needs 16 consecutive columns of a row.
#include "pkv_common.cuh"

int pkv_check_cache(const pkv_cache_t* c);
bool pkv_write_tc_usable(const pkv_layer_t* L, int32_t x_dtype, const void* x_dev);
int pkv_write_tc_launch(const pkv_layer_t* L, const pkv_cache_t* C, const void* x_dev, const int32_t* pos, const float* ph,
                        const int32_t* slots, int n, float* latent_out, int32_t* status, cudaStream_t st);

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
    const double* __restrict__ inv_freq, float attn_scale, const pkv_second second, int scale_up, uint8_t* __restrict__ latent, int n_pages,
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
        uint2 packed = pkv_quantize_block16(v, second.of(j), sb, scale_up != 0);
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
                                                 L->attn_scale, pkv_second_of(L), pkv_scale_round_up_mode(), C ? C->latent_dev : nullptr,
                                                 C ? C->n_pages : 0, latent_out);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

// ------------------------------------------------------------------------------------------------
// Decode-time write (a handful of tokens). The factor matrix (W x D fp32, 4 MB for a Llama-3.1-8B layer)
// has to stream through many SMs to be fast, so the projection is cut both by latent column (tiles of
// 16) and by d_model (slices of 512): CTA (ct, ks) writes the partial dot products of its slice to
// caller scratch [ks][token][WP]; a second kernel, one CTA per token, adds the slices, rotates,
// quantises and stores the latent row, and copies the token's V row.
// ------------------------------------------------------------------------------------------------
constexpr int SM_TOK = 16;      // tokens per pass
constexpr int SM_COL = 16;      // latent columns per CTA
constexpr int SM_KC = 512;      // d_model slice per CTA
constexpr int SM_BP = SM_KC + 4;   // pitch of the factor tile: 16-byte reads of 8 consecutive rows hit distinct banks

template <typename XT>
__global__ void __launch_bounds__(256) pkv_project_small_kernel(const float* __restrict__ Bw, const XT* __restrict__ x,
                                                                int n_tokens, int D, int W, int WP,
                                                                float* __restrict__ raw) {
    extern __shared__ __align__(16) float sm[];
    float* xs = sm;                         // [SM_TOK][SM_KC]
    float* bs = sm + SM_TOK * SM_KC;        // [SM_COL][SM_BP]
    const int tid = threadIdx.x;
    const int c0 = blockIdx.x * SM_COL, ks = blockIdx.y, k0 = ks * SM_KC;
    const int kc = min(SM_KC, D - k0);
    pkv_grid_launch_dependents();
    pkv_grid_wait();                                     // x may be the output of the kernel before
    constexpr int NV = SM_COL * (SM_KC / 4) / 256;          // 16-byte vectors per thread and tile (8)
    auto load_x = [&](int t0, float4 (&xv)[NV]) {
#pragma unroll
        for (int n = 0; n < NV; ++n) {
            const int i = tid + n * 256, tt = i / (SM_KC / 4), k4 = i % (SM_KC / 4);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t0 + tt < n_tokens && k4 * 4 < kc) {
                const XT* src = x + (size_t)(t0 + tt) * D + k0 + k4 * 4;
                if constexpr (sizeof(XT) == 4) {
                    v = *reinterpret_cast<const float4*>(src);
                } else {
                    uint2 u = *reinterpret_cast<const uint2*>(src);
                    v = make_float4(pkv_bf16_bits_to_float(u.x & 0xffffu), pkv_bf16_bits_to_float(u.x >> 16),
                                    pkv_bf16_bits_to_float(u.y & 0xffffu), pkv_bf16_bits_to_float(u.y >> 16));
                }
            }
            xv[n] = v;
        }
    };
    // factor tile and the first token tile: all 16 loads of a thread are issued before any is used
    {
        float4 bv[NV], xv[NV];
#pragma unroll
        for (int n = 0; n < NV; ++n) {
            const int i = tid + n * 256, cc = i / (SM_KC / 4), k4 = i % (SM_KC / 4);
            bv[n] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c0 + cc < W && k4 * 4 < kc) bv[n] = *reinterpret_cast<const float4*>(Bw + (size_t)(c0 + cc) * D + k0 + k4 * 4);
        }
        load_x(0, xv);
#pragma unroll
        for (int n = 0; n < NV; ++n) {
            const int i = tid + n * 256;
            *reinterpret_cast<float4*>(bs + (i / (SM_KC / 4)) * SM_BP + (i % (SM_KC / 4)) * 4) = bv[n];
            *reinterpret_cast<float4*>(xs + (i / (SM_KC / 4)) * SM_KC + (i % (SM_KC / 4)) * 4) = xv[n];
        }
    }
    const int t = tid >> 4, c = tid & 15;
    for (int t0 = 0; t0 < n_tokens; t0 += SM_TOK) {
        if (t0 > 0) {
            float4 xv[NV];
            load_x(t0, xv);
            __syncthreads();
#pragma unroll
            for (int n = 0; n < NV; ++n) {
                const int i = tid + n * 256;
                *reinterpret_cast<float4*>(xs + (i / (SM_KC / 4)) * SM_KC + (i % (SM_KC / 4)) * 4) = xv[n];
            }
        }
        __syncthreads();
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        const float* xr = xs + t * SM_KC;
        const float* br = bs + c * SM_BP;
#pragma unroll 8
        for (int k = 0; k < SM_KC; k += 4) {
            float4 xv = *reinterpret_cast<const float4*>(xr + k);
            float4 bv = *reinterpret_cast<const float4*>(br + k);
            a0 = fmaf(xv.x, bv.x, a0); a1 = fmaf(xv.y, bv.y, a1); a2 = fmaf(xv.z, bv.z, a2); a3 = fmaf(xv.w, bv.w, a3);
        }
        if (t0 + t < n_tokens) raw[((size_t)ks * n_tokens + t0 + t) * WP + c0 + c] = (a0 + a1) + (a2 + a3);
    }
}

// one CTA per token: add the d_model slices, rotate the complex pairs, quantise, store; V row too
__global__ void __launch_bounds__(256) pkv_rotate_store_kernel(
    const float* __restrict__ raw, int n_slices, int n_tokens, const int32_t* __restrict__ positions,
    const float2* __restrict__ phasors, int h2, const int32_t* __restrict__ slots, int W, int WP, int R,
    const int32_t* __restrict__ freq, const double* __restrict__ inv_freq, float attn_scale, const pkv_second second, int scale_up,
    uint8_t* __restrict__ latent, int n_pages, float* __restrict__ latent_out, const uint4* __restrict__ v_rows,
    uint4* __restrict__ v_pool, int v_vecs, int n_kv) {
    __shared__ float row[PKV_MAX_WIDTH];
    const int tok = blockIdx.x, tid = threadIdx.x;
    pkv_grid_launch_dependents();
    pkv_grid_wait();
    // the slice loads are issued first; the phasor (double-precision sincos) is computed while they fly
    float a = 0.0f;
    if (tid < WP) {
#pragma unroll 8
        for (int s = 0; s < n_slices; ++s) a += __ldcg(raw + ((size_t)s * n_tokens + tok) * WP + tid);
    }
    float pr = 1.0f, pi = 0.0f;
    if (tid < R) {
        if (phasors) {
            float2 p = phasors[(size_t)tok * h2 + freq[tid]];
            pr = p.x; pi = p.y;
        } else {
            double sn, cs;
            sincos((double)positions[tok] * inv_freq[freq[tid]], &sn, &cs);
            pr = (float)((double)attn_scale * cs); pi = (float)((double)attn_scale * sn);
        }
    }
    if (tid < WP) row[tid] = a;                  // WP <= 256 = blockDim
    __syncthreads();
    float re = 0.f, im = 0.f;
    if (tid < R) {
        float x0 = row[tid], x1 = row[R + tid];
        re = __fsub_rn(__fmul_rn(x0, pr), __fmul_rn(x1, pi));
        im = __fadd_rn(__fmul_rn(x0, pi), __fmul_rn(x1, pr));
    }
    __syncthreads();
    if (tid < R) { row[tid] = re; row[R + tid] = im; }
    __syncthreads();
    if (latent_out)
        for (int c = tid; c < W; c += 256) latent_out[(size_t)tok * W + c] = row[c];
    if (!latent) return;
    const int slot = slots[tok];
    if (slot < 0 || slot >= n_pages * PKV_PAGE_TOKENS) return;
    if (v_rows)
        for (int i = tid; i < v_vecs; i += 256) v_pool[pkv_v_vec_index(slot, i, n_kv, v_vecs / n_kv)] = v_rows[(size_t)tok * v_vecs + i];
    const int NB = WP / 16, RB = WP / 2;
    if (tid < NB) {
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = row[tid * 16 + i];
        uint8_t sb;
        uint2 packed = pkv_quantize_block16(v, second.of(tid), sb, scale_up != 0);
        uint8_t* page = latent + (size_t)(slot / PKV_PAGE_TOKENS) * pkv_page_bytes(W);
        uint32_t r = slot % PKV_PAGE_TOKENS;
        *reinterpret_cast<uint2*>(page + pkv_code_offset(r, tid * 8, RB)) = packed;
        page[pkv_codes_bytes(W) + pkv_scale_offset(r, tid)] = sb;
    }
}

template <typename XT>
int launch_write_small(const pkv_layer_t* L, const pkv_cache_t* C, const void* x, const int32_t* pos, const float* ph,
                       const int32_t* slots, int n, float* latent_out, float* scratch, const void* v_rows,
                       cudaStream_t st) {
    const int W = 2 * L->R + L->R_s, WP = pkv_padded_width(W);
    const int n_slices = (L->d_model + SM_KC - 1) / SM_KC;
    auto kern = pkv_project_small_kernel<XT>;
    constexpr int smem = (SM_TOK * SM_KC + SM_COL * SM_BP) * 4;
    static pkv_attr_flags attr;                          // per instantiation and device
    PKV_CUDA_TRY(pkv_set_max_smem(kern, smem, attr));
    PKV_CUDA_TRY(pkv_launch_chained(kern, dim3(WP / SM_COL, n_slices), dim3(256), smem, st, L->Bw_dev, (const XT*)x, n,
                                    L->d_model, W, WP, scratch));
    const bool with_v = C && C->v_dev && v_rows;
    PKV_CUDA_TRY(pkv_launch_chained(pkv_rotate_store_kernel, dim3(n), dim3(256), 0, st, scratch, n_slices, n, pos,
                                    (const float2*)ph, L->head_dim / 2, slots, W, WP, L->R, L->freq_dev, L->inv_freq_dev,
                                    L->attn_scale, pkv_second_of(L), pkv_scale_round_up_mode(), C ? C->latent_dev : nullptr, C ? C->n_pages : 0, latent_out,
                                    with_v ? (const uint4*)v_rows : nullptr, with_v ? (uint4*)C->v_dev : nullptr,
                                    with_v ? C->n_kv * C->head_dim * 2 / 16 : 0, with_v ? C->n_kv : 1));
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
                               int32_t n_tokens, float* latent_out_dev, float* scratch_dev, const void* v_rows_dev,
                               int32_t* status_dev, void* stream) {
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
                                                              n_tokens, latent_out_dev, scratch_dev, v_rows_dev, s)
                                  : launch_write_small<uint16_t>(layer, cache, x_dev, positions_dev, phasors_dev,
                                                                 slots_dev, n_tokens, latent_out_dev, scratch_dev,
                                                                 v_rows_dev, s);
    }
    if (v_rows_dev && cache && cache->v_dev) {
        int vst = pkv_v_write(cache, v_rows_dev, slots_dev, n_tokens, stream);
        if (vst) return vst;
    }
    if (pkv_write_tc_usable(layer, x_dtype, x_dev))
        return pkv_write_tc_launch(layer, cache, x_dev, positions_dev, phasors_dev, slots_dev, n_tokens, latent_out_dev,
                                   status_dev, s);
    if (pkv_padded_width(W) == 128) {
        return x_dtype == PKV_F32
                   ? launch_write<128, float>(layer, cache, x_dev, positions_dev, phasors_dev, slots_dev, n_tokens, latent_out_dev, s)
                   : launch_write<128, uint16_t>(layer, cache, x_dev, positions_dev, phasors_dev, slots_dev, n_tokens, latent_out_dev, s);
    }
    return x_dtype == PKV_F32
               ? launch_write<256, float>(layer, cache, x_dev, positions_dev, phasors_dev, slots_dev, n_tokens, latent_out_dev, s)
               : launch_write<256, uint16_t>(layer, cache, x_dev, positions_dev, phasors_dev, slots_dev, n_tokens, latent_out_dev, s);
}

extern "C" int64_t pkv_write_scratch_floats(int32_t n_tokens, int32_t d_model) {
    if (n_tokens < 0 || d_model <= 0) return PKV_ERR_INVALID;
    return (int64_t)n_tokens * PKV_MAX_WIDTH * ((d_model + 511) / 512);
}
