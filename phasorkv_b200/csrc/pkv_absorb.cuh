// Query absorption as a device function, so that both the stand-alone kernel and the fused decode-step
// prologue run the same arithmetic: q'_k = conj(A[g, k]) * zq_{freq[k]} * e^{i theta m}, slow block
// unrotated, and the NVFP4 residual expansion of the absorbed query that the tensor-core attention
// kernel consumes.
#pragma once
#include "pkv_common.cuh"

#include <cuda_fp4.h>

namespace pkv_absorb_impl {

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

struct Args {
    const float* q;                 // [batch][n_q][head_dim]
    const int32_t* positions;       // [batch] or null with `phasors`
    const float2* phasors;          // [batch][head_dim / 2] or null
    int n_q, n_kv, head_dim, R, R_s, n_slow;
    const float *A_re, *A_im, *A_s;
    const int32_t *freq, *slow;
    const double* inv_freq;
    float attn_scale;
    float* qabs_out;                // [batch][n_q][W] or null
    uint8_t* qop_out;               // operand blobs or null
    long qop_bytes;
    const float* second_blocks;     // tiers: tensor scale of each 16-column block of the cache, or null
    float inv_second;               // 1 / the layer's tensor scale
    int32_t* qsync;                 // [2 * batch] or null: qsync[b] counts the head groups of sequence b whose operand rows are in place
};

inline Args make_args(const pkv_layer_t* L, const float* q, const int32_t* positions, const float* phasors, float* qabs_out,
                      uint8_t* qop_out) {
    Args P;
    P.q = q; P.positions = positions; P.phasors = reinterpret_cast<const float2*>(phasors);
    P.n_q = L->n_q; P.n_kv = L->n_kv; P.head_dim = L->head_dim; P.R = L->R; P.R_s = L->R_s; P.n_slow = L->n_slow;
    P.A_re = L->A_re_dev; P.A_im = L->A_im_dev; P.A_s = L->A_s_dev;
    P.freq = L->freq_dev; P.slow = L->slow_dev; P.inv_freq = L->inv_freq_dev;
    P.attn_scale = L->attn_scale;
    P.qabs_out = qabs_out; P.qop_out = qop_out;
    P.qop_bytes = pkv_page_bytes(2 * L->R + L->R_s) + 512;
    P.second_blocks = L->second_blocks_dev;
    P.inv_second = L->second > 0.0f ? 1.0f / L->second : 1.0f;
    P.qsync = nullptr;
    return P;
}

__host__ __device__ inline size_t smem_bytes(int head_dim, int Wp) {
    return sizeof(float2) * (MAX_H + (size_t)HG * (head_dim / 2)) + sizeof(float) * (size_t)HG * Wp + sizeof(unsigned) * HG;
}

// One CTA of NT threads per (sequence b, group hg of 8 query heads); `sm` = smem_bytes() of shared memory.
//   stage 1: phasors of the query position (double angle, as the cache write does)
//   stage 2: zq = (q[j] + i q[j + h]) * phasor, complex product in fp32
//   stage 3: absorbed rows [Re q' | Im q' | slow] to shared memory (and to qabs_out)
//   stage 4: PKV_QUERY_TERMS rounds of "quantise the residual to NVFP4", one tensor scale per head row
__device__ __forceinline__ void body(const Args& P, int b, int hg, float* sm) {
    const float* __restrict__ q = P.q;
    const int32_t* __restrict__ positions = P.positions;
    const float2* __restrict__ phasors = P.phasors;
    const int n_q = P.n_q, n_kv = P.n_kv, head_dim = P.head_dim, R = P.R, R_s = P.R_s, n_slow = P.n_slow;
    const float* __restrict__ A_re = P.A_re;
    const float* __restrict__ A_im = P.A_im;
    const float* __restrict__ A_s = P.A_s;
    const int32_t* __restrict__ freq = P.freq;
    const int32_t* __restrict__ slow = P.slow;
    const double* __restrict__ inv_freq = P.inv_freq;
    const float attn_scale = P.attn_scale;
    // tiers: the cache's block j is in units of second_blocks[j] while the decode kernels apply the layer's one scale,
    // so the query's columns of block j carry the ratio
    const float* __restrict__ tiers = P.second_blocks;
    const float inv_second = P.inv_second;
    float* __restrict__ qabs_out = P.qabs_out;
    uint8_t* __restrict__ qop_out = P.qop_out;
    const long qop_bytes = P.qop_bytes;
    const int h2 = head_dim / 2, W = 2 * R + R_s, Wp = pkv_padded_width(W);
    float2* ph = reinterpret_cast<float2*>(sm);                    // [h2]
    float2* zq = ph + MAX_H;                                       // [HG][h2]
    float* row = reinterpret_cast<float*>(zq + HG * h2);           // [HG][Wp]
    unsigned* amax_bits = reinterpret_cast<unsigned*>(row + HG * Wp);    // [HG]
    const int h0 = hg * HG, tid = threadIdx.x;
    const int nh = min(HG, n_q - h0);
    const float* qb = q + ((size_t)b * n_q + h0) * head_dim;

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
                float v = c < R ? __fadd_rn(__fmul_rn(ar, z.x), __fmul_rn(ai, z.y))
                                : __fsub_rn(__fmul_rn(ar, z.y), __fmul_rn(ai, z.x));
                if (tiers) v *= tiers[c >> 4] * inv_second;
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
                    if (tiers) v *= tiers[c >> 4] * inv_second;
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
    // Operand-ready signal for an attention launch that polls instead of waiting for this whole grid: the rows
    // of this head group are made visible device-wide, then the sequence's counter goes up by one.
    if (P.qsync) {
        __threadfence();
        __syncthreads();
        if (tid == 0) atomicAdd(P.qsync + b, 1);
    }
}


// The same arithmetic for ALL 32 query heads of one sequence by a group of 128 threads, the operand tile
// written to SHARED memory: the attention kernel absorbs its own query instead of reading the blob a
// separate launch left in global memory. Thread (h = tid / 4, quarter = tid % 4) owns a quarter of head
// h's row in registers. `blob` = the kernel's query-operand region, `scratch` = TILE_SCRATCH_FLOATS floats
// of shared memory free until the call returns. The 128 threads meet on named barrier 1. Every operation
// is the one `body` makes, in the same order per value: the operand bytes are identical.
constexpr int TILE_THREADS = 128;
constexpr int TILE_QP = 132;                                   // pitch of a query row in shared memory (bank spread)
constexpr int TILE_SCRATCH_FLOATS = 2 * MAX_H + 32 * TILE_QP;

__device__ __forceinline__ void tile_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int WP>
__device__ __forceinline__ void body_tile(const Args& P, int b, uint8_t* blob, float* scratch, int tid) {
    constexpr int NBT = WP / 64;                               // 16-column blocks per thread
    const int head_dim = P.head_dim, h2 = head_dim / 2, R = P.R, R_s = P.R_s, n_slow = P.n_slow;
    const int W = 2 * R + R_s, n_q = P.n_q;
    float2* ph = reinterpret_cast<float2*>(scratch);           // [h2]
    float* qs = scratch + 2 * MAX_H;                           // [n_q][TILE_QP] raw (pre-RoPE) query
    const float* qb = P.q + (size_t)b * n_q * head_dim;
    // query rows first (the loads fly while the phasors are formed)
    const int n4 = n_q * head_dim / 4;
    constexpr int QV = 8;                                      // 16-byte loads per thread: 32 heads x 128 dims
    float4 qv[QV];
#pragma unroll
    for (int n = 0; n < QV; ++n) {
        const int i = tid + n * TILE_THREADS;
        qv[n] = i < n4 ? *reinterpret_cast<const float4*>(qb + (size_t)i * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int j = tid; j < h2; j += TILE_THREADS) {
        double sn, cs;
        sincos((double)P.positions[b] * P.inv_freq[j], &sn, &cs);
        ph[j] = make_float2((float)((double)P.attn_scale * cs), (float)((double)P.attn_scale * sn));
    }
#pragma unroll
    for (int n = 0; n < QV; ++n) {
        const int i = tid + n * TILE_THREADS;
        if (i < n4) {
            const int e = i * 4, hh = e / head_dim, col = e % head_dim;
            float* dst = qs + hh * TILE_QP + col;
            dst[0] = qv[n].x; dst[1] = qv[n].y; dst[2] = qv[n].z; dst[3] = qv[n].w;
        }
    }
    tile_barrier();
    const int h = tid >> 2, quarter = tid & 3, g = h / (n_q / P.n_kv);
    const float* qh = qs + h * TILE_QP;
    float res[NBT][16];
    float am = 0.0f;
#pragma unroll
    for (int blk = 0; blk < NBT; ++blk) {
        // all global loads of the block first (frequency index and factor of each column are independent
        // loads: one memory latency per block, not one per column), then the arithmetic
        int fk[16];
        float ar[16], ai[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {                       // unconditional (index clamped): straight-line code, loads in flight together
            const int c = (quarter * NBT + blk) * 16 + i;
            const int k = min(c < R ? c : c - R, R - 1);
            fk[i] = P.freq[k];
            ar[i] = P.A_re[g * R + k];
            ai[i] = P.A_im[g * R + k];
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int c = (quarter * NBT + blk) * 16 + i;
            float v = 0.0f;
            if (c < 2 * R) {
                const int f = fk[i];
                const float a = qh[f], cc = qh[f + h2];
                const float2 p = ph[f];
                const float zx = __fsub_rn(__fmul_rn(a, p.x), __fmul_rn(cc, p.y));
                const float zy = __fadd_rn(__fmul_rn(a, p.y), __fmul_rn(cc, p.x));
                // conj(A) * z = (ar*zr + ai*zi) + i (ar*zi - ai*zr)
                v = c < R ? __fadd_rn(__fmul_rn(ar[i], zx), __fmul_rn(ai[i], zy)) : __fsub_rn(__fmul_rn(ar[i], zy), __fmul_rn(ai[i], zx));
            } else if (c < W) {
                const int r = c - 2 * R;
                for (int s = 0; s < 2 * n_slow; ++s) {
                    const int col = s < n_slow ? P.slow[s] : P.slow[s - n_slow] + h2;
                    v = fmaf(qh[col], P.A_s[((size_t)g * 2 * n_slow + s) * R_s + r], v);
                }
            }
            if (P.second_blocks && c < W) v *= P.second_blocks[c >> 4] * P.inv_second;
            res[blk][i] = v;
            am = fmaxf(am, fabsf(v));
        }
    }
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));        // the four threads of a head are neighbours in a warp
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
    const float second = fmaxf(am, 1e-30f) * (1.0f / (448.0f * 6.0f));
    const float inv_second = __frcp_rn(second);
    constexpr int RB = WP / 2, CODES = PKV_PAGE_TOKENS * RB, PAGE = CODES + (WP / 64) * 512;
    for (int term = 0; term < PKV_QUERY_TERMS; ++term) {
        const uint32_t n = term * n_q + h;
#pragma unroll
        for (int blk = 0; blk < NBT; ++blk) {
            const int j = quarter * NBT + blk;
            uint8_t sb;
            const uint2 packed = quantize_query_block16(res[blk], second, inv_second, sb);
            *reinterpret_cast<uint2*>(blob + pkv_code_offset(n, j * 8, RB)) = packed;
            blob[CODES + pkv_scale_offset(n, j)] = sb;
        }
    }
    if (quarter == 0) reinterpret_cast<float*>(blob + PAGE)[h] = second;
}

}  // namespace pkv_absorb_impl
