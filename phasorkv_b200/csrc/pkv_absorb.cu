// Query absorption: q'_k = conj(A[g, k]) * zq_{freq[k]} * e^{i theta m}, slow block unrotated, and the
// NVFP4 residual expansion of the absorbed query that the tensor-core attention kernel consumes.
#include "pkv_common.cuh"

int pkv_check_layer(const pkv_layer_t* L);

namespace {

constexpr int MAX_H = 128;     // head_dim / 2 limit
constexpr int NT = 512;

// One CTA per sequence.
//   stage 1: phasors of the query position (double angle, as the cache write does)
//   stage 2: zq = (q[j] + i q[j + h]) * phasor, complex product in fp32
//   stage 3: absorbed row [Re q' | Im q' | slow] to shared memory (and to qabs_out)
//   stage 4: PKV_QUERY_TERMS rounds of "quantise the residual to NVFP4 with a per-row tensor scale"
__global__ void __launch_bounds__(NT) pkv_absorb_kernel(
    const float* __restrict__ q, const int32_t* __restrict__ positions, const float2* __restrict__ phasors, int n_q, int n_kv, int head_dim, int R,
    int R_s, int n_slow, const float* __restrict__ A_re, const float* __restrict__ A_im,
    const float* __restrict__ A_s, const int32_t* __restrict__ freq, const int32_t* __restrict__ slow,
    const double* __restrict__ inv_freq, float attn_scale, float* __restrict__ qabs_out, uint8_t* __restrict__ qop_out,
    long qop_bytes) {
    extern __shared__ __align__(16) float sm[];
    const int h2 = head_dim / 2, W = 2 * R + R_s, Wp = pkv_padded_width(W);
    float2* ph = reinterpret_cast<float2*>(sm);                    // [h2]
    float2* zq = ph + MAX_H;                                       // [n_q][h2]
    float* row = reinterpret_cast<float*>(zq + n_q * h2);          // [n_q][Wp]
    unsigned* amax_bits = reinterpret_cast<unsigned*>(row + n_q * Wp);   // [n_q]
    const int b = blockIdx.x, tid = threadIdx.x;
    const float* qb = q + (size_t)b * n_q * head_dim;

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
    for (int i = tid; i < n_q * h2; i += NT) {
        int h = i / h2, j = i % h2;
        float a = qb[h * head_dim + j], c = qb[h * head_dim + j + h2];
        float2 p = ph[j];
        zq[i] = make_float2(__fsub_rn(__fmul_rn(a, p.x), __fmul_rn(c, p.y)),
                            __fadd_rn(__fmul_rn(a, p.y), __fmul_rn(c, p.x)));
    }
    __syncthreads();
    const int rep = n_q / n_kv;
    for (int i = tid; i < n_q * Wp; i += NT) {
        int h = i / Wp, c = i % Wp, g = h / rep;
        float v = 0.0f;
        if (c < 2 * R) {
            int k = c < R ? c : c - R;
            float ar = A_re[g * R + k], ai = A_im[g * R + k];
            float2 z = zq[h * h2 + freq[k]];
            // conj(A) * z = (ar*zr + ai*zi) + i (ar*zi - ai*zr)
            v = c < R ? __fadd_rn(__fmul_rn(ar, z.x), __fmul_rn(ai, z.y))
                      : __fsub_rn(__fmul_rn(ar, z.y), __fmul_rn(ai, z.x));
        } else if (c < W) {
            int r = c - 2 * R;
            for (int s = 0; s < 2 * n_slow; ++s) {
                int col = s < n_slow ? slow[s] : slow[s - n_slow] + h2;
                v = fmaf(qb[h * head_dim + col], A_s[((size_t)g * 2 * n_slow + s) * R_s + r], v);
            }
        }
        row[i] = v;
        if (qabs_out && c < W) qabs_out[((size_t)b * n_q + h) * W + c] = v;
    }
    if (!qop_out) return;
    // ---- operand: row n = term * n_q + h of a 128-row tile in the cache-page layout
    const int NB = Wp / 16, RB = Wp / 2;
    const int codes_bytes = pkv_codes_bytes(W), page_bytes = pkv_page_bytes(W);
    uint8_t* blob = qop_out + (size_t)b * qop_bytes;
    float* row_scale = reinterpret_cast<float*>(blob + page_bytes);
    const int n_blk = n_q * NB;                       // <= 32 * 16 = NT
    const bool live = tid < n_blk;
    const int h = live ? tid / NB : 0, j = live ? tid % NB : 0;
    float res[16];
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 16; ++i) res[i] = live ? row[h * Wp + j * 16 + i] : 0.0f;
    for (int term = 0; term < PKV_QUERY_TERMS; ++term) {
        if (tid < n_q) amax_bits[tid] = 0u;
        __syncthreads();
        float am = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) am = fmaxf(am, fabsf(res[i]));
        if (live) atomicMax(&amax_bits[h], __float_as_uint(am));      // non-negative floats order as integers
        __syncthreads();
        if (live) {
            float second = __fdiv_rn(fmaxf(__uint_as_float(amax_bits[h]), 1e-30f), 448.0f * 6.0f);
            uint8_t sb;
            uint2 packed = pkv_quantize_block16(res, second, sb);
            float scale = __fmul_rn(pkv_e4m3_to_float(sb), second);
#pragma unroll
            for (int i = 0; i < 8; ++i) res[i] = fmaf(-pkv_e2m1_value((packed.x >> (4 * i)) & 15u), scale, res[i]);
#pragma unroll
            for (int i = 0; i < 8; ++i) res[8 + i] = fmaf(-pkv_e2m1_value((packed.y >> (4 * i)) & 15u), scale, res[8 + i]);
            uint32_t n = term * n_q + h;
            *reinterpret_cast<uint2*>(blob + pkv_code_offset(n, j * 8, RB)) = packed;
            blob[codes_bytes + pkv_scale_offset(n, j)] = sb;
            if (j == 0) row_scale[n] = second;
        }
        __syncthreads();
    }
}

}  // namespace

extern "C" int64_t pkv_query_operand_bytes(int32_t W) {
    if (W <= 0 || W > PKV_MAX_WIDTH || (W % 16)) return PKV_ERR_UNSUPPORTED;
    return pkv_page_bytes(W) + 128 * 4;
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
    size_t smem = sizeof(float2) * (MAX_H + (size_t)layer->n_q * (layer->head_dim / 2)) +
                  sizeof(float) * (size_t)layer->n_q * Wp + sizeof(unsigned) * layer->n_q;
    if (smem > 200 * 1024) return PKV_ERR_UNSUPPORTED;
    PKV_CUDA_TRY(cudaFuncSetAttribute(pkv_absorb_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    pkv_absorb_kernel<<<batch, NT, smem, (cudaStream_t)stream>>>(
        q_dev, positions_dev, (const float2*)phasors_dev, layer->n_q, layer->n_kv, layer->head_dim, layer->R, layer->R_s, layer->n_slow,
        layer->A_re_dev, layer->A_im_dev, layer->A_s_dev, layer->freq_dev, layer->slow_dev, layer->inv_freq_dev,
        layer->attn_scale, qabs_out_dev, qop_out_dev, (long)pkv_query_operand_bytes(W));
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}
