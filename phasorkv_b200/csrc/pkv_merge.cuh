// Log-sum-exp merge of split partials by one warp: M = max m_p, w_p = 2^(m_p - M),
// O = sum w_p o_p / sum w_p l_p  (the combine of a split-K flash decode).
#pragma once

#include "pkv_common.cuh"

// base points at the (o[head_dim], m, l) triple of partial 0 for one (sequence, head); partial p sits
// stride_p floats further. Loads bypass L1 (the partials may have been written by other SMs of the
// same launch). head_dim <= 256. All 32 lanes of the warp call this together.
__device__ __forceinline__ void pkv_merge_warp(const float* __restrict__ base, long stride_p, int n_parts, int head_dim,
                                               int lane, float* __restrict__ out, float* __restrict__ packed) {
    float M = -INFINITY;
    for (int p = lane; p < n_parts; p += 32) M = fmaxf(M, __ldcg(base + (size_t)p * stride_p + head_dim));
#pragma unroll
    for (int o = 16; o; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float den = 0.0f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    const int nd = (head_dim + 31) / 32;
    if (M > -INFINITY) {
        for (int p0 = 0; p0 < n_parts; p0 += 32) {
            const int p = p0 + lane;
            float w = 0.0f;
            if (p < n_parts) {
                const float* pp = base + (size_t)p * stride_p;
                w = exp2f(__ldcg(pp + head_dim) - M);        // a split that saw no token has m = -inf, w = 0
                den = fmaf(w, __ldcg(pp + head_dim + 1), den);
            }
            const int np = min(32, n_parts - p0);
#pragma unroll 4
            for (int pi = 0; pi < np; ++pi) {
                const float wp = __shfl_sync(0xffffffffu, w, pi);
                const float* pp = base + (size_t)(p0 + pi) * stride_p;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (i < nd && lane + 32 * i < head_dim) acc[i] = fmaf(wp, __ldcg(pp + lane + 32 * i), acc[i]);
            }
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = lane + 32 * i;
        if (i < nd && d < head_dim) {
            if (out) out[d] = den > 0.0f ? acc[i] / den : 0.0f;
            if (packed) packed[d] = acc[i];
        }
    }
    if (packed && lane == 0) {
        packed[head_dim] = M;
        packed[head_dim + 1] = den;
    }
}
