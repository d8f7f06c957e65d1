// Query absorption: q'_k = conj(A[g, k]) * zq_{freq[k]} * e^{i theta m}, slow block unrotated, and the
// NVFP4 residual expansion of the absorbed query that the tensor-core attention kernel consumes.
#include "pkv_common.cuh"

#include <cuda_fp4.h>

int pkv_check_layer(const pkv_layer_t* L);

namespace {

// NVFP4 quantisation of the QUERY operand. Unlike the cache (which must reproduce the reference's
// rounding bit for bit) this format is private to the library: any rounding is admissible because the
// next residual term is formed from the value actually stored. So: reciprocal instead of division and
// the hardware float -> E2M1 conversion (round to nearest even, saturating).
__device__ __forceinline__ uint2 quantize_query_block16(float (&res)[16], float second, float inv_second, uint8_t& sb) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(res[i]));
    sb = pkv_float_to_e4m3(fminf(amax * (1.0f / 6.0f) * inv_second, 448.0f));
    const float scale = pkv_e4m3_to_float(sb) * second;
    const float inv = scale > 0.0f ? __frcp_rn(scale) : 0.0f;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t byte = (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(res[2 * i] * inv, res[2 * i + 1] * inv), __NV_E2M1,
                                                                 cudaRoundNearest);
        w[i >> 2] |= byte << (8 * (i & 3));
        res[2 * i] = fmaf(-pkv_e2m1_value(byte & 15u), scale, res[2 * i]);
        res[2 * i + 1] = fmaf(-pkv_e2m1_value((byte >> 4) & 15u), scale, res[2 * i + 1]);
    }
    return make_uint2(w[0], w[1]);
}

constexpr int MAX_H = 128;     // head_dim / 2 limit
constexpr int NT = 256;
constexpr int HG = 8;          // query heads per CTA

// One CTA per (sequence, group of 8 query heads).
//   stage 1: phasors of the query position (double angle, as the cache write does)
//   stage 2: zq = (q[j] + i q[j + h]) * phasor, complex product in fp32
//   stage 3: absorbed rows [Re q' | Im q' | slow] to shared memory (and to qabs_out)
//   stage 4: PKV_QUERY_TERMS rounds of "quantise the residual to NVFP4", one tensor scale per head row
__global__ void __launch_bounds__(NT) pkv_absorb_kernel(
    const float* __restrict__ q, const int32_t* __restrict__ positions, const float2* __restrict__ phasors, int n_q,
    int n_kv, int head_dim, int R, int R_s, int n_slow, const float* __restrict__ A_re, const float* __restrict__ A_im,
    const float* __restrict__ A_s, const int32_t* __restrict__ freq, const int32_t* __restrict__ slow,
    const double* __restrict__ inv_freq, float attn_scale, float* __restrict__ qabs_out, uint8_t* __restrict__ qop_out,
    long qop_bytes) {
    extern __shared__ __align__(16) float sm[];
    const int h2 = head_dim / 2, W = 2 * R + R_s, Wp = pkv_padded_width(W);
    float2* ph = reinterpret_cast<float2*>(sm);                    // [h2]
    float2* zq = ph + MAX_H;                                       // [HG][h2]
    float* row = reinterpret_cast<float*>(zq + HG * h2);           // [HG][Wp]
    unsigned* amax_bits = reinterpret_cast<unsigned*>(row + HG * Wp);    // [HG]
    const int b = blockIdx.x, h0 = blockIdx.y * HG, tid = threadIdx.x;
    const int nh = min(HG, n_q - h0);
    const float* qb = q + ((size_t)b * n_q + h0) * head_dim;
    pkv_grid_wait();
    pkv_grid_launch_dependents();

    // start the global loads of the query and of this thread's factor column before the trigonometry
    constexpr int QPF = 4;                                          // (head, frequency) pairs per thread, head_dim <= 256
    float qre[QPF], qim[QPF];
#pragma unroll
    for (int n = 0; n < QPF; ++n) {
        const int i = tid + n * NT;
        qre[n] = qim[n] = 0.0f;
        if (i < nh * h2) { qre[n] = qb[(i / h2) * head_dim + i % h2]; qim[n] = qb[(i / h2) * head_dim + i % h2 + h2]; }
    }
    const int rep = n_q / n_kv;
    float a_re[HG], a_im[HG];
    int my_f = 0;
    {
        const int c = tid;
#pragma unroll
        for (int h = 0; h < HG; ++h) a_re[h] = a_im[h] = 0.0f;
        if (c < 2 * R && c < Wp) {
            const int k = c < R ? c : c - R;
            my_f = freq[k];
#pragma unroll
            for (int h = 0; h < HG; ++h)
                if (h < nh) { a_re[h] = A_re[((h0 + h) / rep) * R + k]; a_im[h] = A_im[((h0 + h) / rep) * R + k]; }
        }
    }
    for (int j = tid; j < h2; j += NT) {
        if (phasors) {
            ph[j] = phasors[(size_t)b * h2 + j];
        } else {
            double sn, cs;
            sincos((double)positions[b] * inv_freq[j], &sn, &cs);
            ph[j] = make_float2((float)((double)attn_scale * cs), (float)((double)attn_scale * sn));
        }
    }
    __syncthreads();
#pragma unroll
    for (int n = 0; n < QPF; ++n) {
        const int i = tid + n * NT;
        if (i < nh * h2) {
            const float a = qre[n], c = qim[n];
            const float2 p = ph[i % h2];
            zq[i] = make_float2(__fsub_rn(__fmul_rn(a, p.x), __fmul_rn(c, p.y)),
                                __fadd_rn(__fmul_rn(a, p.y), __fmul_rn(c, p.x)));
        }
    }
    __syncthreads();
    // thread -> column, loop over the heads of the group: the factor loads of a column are shared by the
    // heads of one kv head and independent across iterations
    for (int c = tid; c < Wp; c += NT) {
        if (c < 2 * R) {
            const int f = my_f;                                     // c == tid here: Wp <= NT
#pragma unroll
            for (int h = 0; h < HG; ++h) {
                if (h >= nh) break;
                const float ar = a_re[h], ai = a_im[h];
                const float2 z = zq[h * h2 + f];
                // conj(A) * z = (ar*zr + ai*zi) + i (ar*zi - ai*zr)
                const float v = c < R ? __fadd_rn(__fmul_rn(ar, z.x), __fmul_rn(ai, z.y))
                                      : __fsub_rn(__fmul_rn(ar, z.y), __fmul_rn(ai, z.x));
                row[h * Wp + c] = v;
                if (qabs_out) qabs_out[((size_t)b * n_q + h0 + h) * W + c] = v;
            }
        } else {
            for (int h = 0; h < nh; ++h) {
                float v = 0.0f;
                if (c < W) {
                    const int r = c - 2 * R, g = (h0 + h) / rep;
                    for (int s = 0; s < 2 * n_slow; ++s) {
                        int col = s < n_slow ? slow[s] : slow[s - n_slow] + h2;
                        v = fmaf(qb[h * head_dim + col], A_s[((size_t)g * 2 * n_slow + s) * R_s + r], v);
                    }
                    if (qabs_out) qabs_out[((size_t)b * n_q + h0 + h) * W + c] = v;
                }
                row[h * Wp + c] = v;
            }
        }
    }
    if (!qop_out) return;
    // ---- operand: row n = term * n_q + head of a 128-row tile in the cache-page layout
    const int NB = Wp / 16, RB = Wp / 2;
    // layout: a 128-row tile (row = term * 32 + head) exactly like a cache page (swizzled codes, then the E4M3
    // block scales in scale-factor order) | 32 fp32 tensor scales, one per head, shared by its residual terms
    const int codes_bytes = pkv_codes_bytes(W), page_bytes = pkv_page_bytes(W);
    uint8_t* blob = qop_out + (size_t)b * qop_bytes;
    float* row_scale = reinterpret_cast<float*>(blob + page_bytes);
    const bool live = tid < nh * NB;                  // <= 8 * 16 threads
    const int h = live ? tid / NB : 0, j = live ? tid % NB : 0;
    float res[16];
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 16; ++i) res[i] = live ? row[h * Wp + j * 16 + i] : 0.0f;
    // one tensor scale per head row, shared by its residual terms: the terms then differ only in their
    // E4M3 block scales and can be summed by the tensor core
    if (tid < HG) amax_bits[tid] = 0u;
    __syncthreads();
    {
        float am = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) am = fmaxf(am, fabsf(res[i]));
        if (live) atomicMax(&amax_bits[h], __float_as_uint(am));      // non-negative floats order as integers
    }
    __syncthreads();
    if (live) {
        const float second = fmaxf(__uint_as_float(amax_bits[h]), 1e-30f) * (1.0f / (448.0f * 6.0f));
        const float inv_second = __frcp_rn(second);
        for (int term = 0; term < PKV_QUERY_TERMS; ++term) {
            uint8_t sb;
            const uint2 packed = quantize_query_block16(res, second, inv_second, sb);
            const uint32_t n = term * n_q + h0 + h;
            *reinterpret_cast<uint2*>(blob + pkv_code_offset(n, j * 8, RB)) = packed;
            blob[codes_bytes + pkv_scale_offset(n, j)] = sb;
            if (j == 0 && term == 0) row_scale[h0 + h] = second;
        }
    }
}

}  // namespace

extern "C" int64_t pkv_query_operand_bytes(int32_t W) {
    if (W <= 0 || W > PKV_MAX_WIDTH || (W % 16)) return PKV_ERR_UNSUPPORTED;
    return pkv_page_bytes(W) + 512;
}

extern "C" int pkv_absorb(const pkv_layer_t* layer, const float* q_dev, const int32_t* positions_dev,
                          const float* phasors_dev, int32_t batch, float* qabs_out_dev, uint8_t* qop_out_dev,
                          void* stream) {
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
    size_t smem = sizeof(float2) * (MAX_H + (size_t)HG * (layer->head_dim / 2)) + sizeof(float) * (size_t)HG * Wp +
                  sizeof(unsigned) * HG;                                   // < 48 KB: no opt-in needed
    PKV_CUDA_TRY(pkv_launch_chained(pkv_absorb_kernel, dim3(batch, (layer->n_q + HG - 1) / HG), dim3(NT), smem,
                                    (cudaStream_t)stream, q_dev, positions_dev, (const float2*)phasors_dev, layer->n_q,
                                    layer->n_kv, layer->head_dim, layer->R, layer->R_s, layer->n_slow, layer->A_re_dev,
                                    layer->A_im_dev, layer->A_s_dev, layer->freq_dev, layer->slow_dev, layer->inv_freq_dev,
                                    layer->attn_scale, qabs_out_dev, qop_out_dev, (long)pkv_query_operand_bytes(W)));
    return PKV_OK;
}
