// Log-sum-exp merge of split-T partials (o[d], m, l) of ONE (sequence, head) row by one CTA of
// MG * 128 threads: M = max m, w = 2^(m - M), sums of w o and w l -- the split combine of
// phasorkv/kernels/dense_attn.py:72-74. Shared by the stand-alone merge launch and by the merge that
// is fused with the NVLink exchange of the token-sharded decode.
//
// The work is pure latency (a few hundred KB at most), so every load is issued before anything is
// consumed: thread p fetches the (m, l) pair of partial p, thread (g, d) fetches output dim d of the
// partials g, g + MG, ... into registers; only then are the maxima reduced, the weights formed and the
// register values scaled and added (across the MG groups through shared memory).
#pragma once
#include "pkv_common.cuh"

namespace pkv_merge_impl {

constexpr int MG = 4;                       // partial groups per CTA
constexpr int REG_PARTS = 16;               // partials per thread held in registers in one pass
constexpr int MAX_PARTS = MG * 128;         // one (m, l) pair per thread

struct MergeSmem {
    float w[MAX_PARTS];
    float red[MG][256];
    float wred[MG * 4];
    float M, den;
};

// Called by all MG * 128 threads. `base` = partial 0 of the row, partial p at base + p * stride_p,
// layout [head_dim values | m | l]; `extra`, if not null, is one more partial of the same layout (the
// exact-token side path) merged as partial number n_parts. On return every thread holds M and the
// denominator; the threads with tid < 128 hold the weighted sums of dims tid (a0) and tid + 128 (a1),
// relative to M.
__device__ __forceinline__ void merge_row(const float* __restrict__ base, long stride_p, int n_parts, int head_dim,
                                          MergeSmem& S, float& a0, float& a1, float& M_out, float& den_out,
                                          const float* __restrict__ extra = nullptr) {
    const int tid = threadIdx.x, d = tid & 127, g = tid >> 7;
    const int n_own = n_parts;
    if (extra) ++n_parts;
    auto part_ptr = [&](int p) -> const float* { return p < n_own ? base + (size_t)p * stride_p : extra; };
    // ---- all loads first
    float2 ml = make_float2(-INFINITY, 0.0f);
    if (tid < n_parts) ml = __ldcg(reinterpret_cast<const float2*>(part_ptr(tid) + head_dim));
    float o0[REG_PARTS], o1[REG_PARTS];
#pragma unroll
    for (int k = 0; k < REG_PARTS; ++k) {
        const int p = g + k * MG;
        o0[k] = (p < n_parts && d < head_dim) ? __ldcg(part_ptr(p) + d) : 0.0f;
        o1[k] = (p < n_parts && d + 128 < head_dim) ? __ldcg(part_ptr(p) + d + 128) : 0.0f;
    }
    // ---- maximum over the partials, weights, denominator
    float M = ml.x;
#pragma unroll
    for (int o = 16; o; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if ((tid & 31) == 0) S.wred[tid >> 5] = M;
    __syncthreads();
    if (tid == 0) {
        float mm = -INFINITY;
        for (int i = 0; i < MG * 4; ++i) mm = fmaxf(mm, S.wred[i]);
        S.M = mm;
    }
    __syncthreads();
    M = S.M;
    const float w = (tid < n_parts && M > -INFINITY) ? exp2f(ml.x - M) : 0.0f;     // a split that saw no token: m = -inf, w = 0
    if (tid < n_parts) S.w[tid] = w;
    float lw = w * ml.y;
#pragma unroll
    for (int o = 16; o; o >>= 1) lw += __shfl_xor_sync(0xffffffffu, lw, o);
    __syncthreads();                         // everyone has read wred / M
    if ((tid & 31) == 0) S.wred[tid >> 5] = lw;
    __syncthreads();
    if (tid == 0) {
        float dd = 0.0f;
        for (int i = 0; i < MG * 4; ++i) dd += S.wred[i];
        S.den = dd;
    }
    // ---- weighted sums: registers first, further partials (more than MG * REG_PARTS) straight from memory
    float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
    for (int k = 0; k < REG_PARTS; ++k) {
        const int p = g + k * MG;
        if (p < n_parts) { acc0 = fmaf(S.w[p], o0[k], acc0); acc1 = fmaf(S.w[p], o1[k], acc1); }
    }
#pragma unroll 4
    for (int p = g + REG_PARTS * MG; p < n_parts; p += MG) {
        const float* pp = part_ptr(p);
        if (d < head_dim) acc0 = fmaf(S.w[p], __ldcg(pp + d), acc0);
        if (d + 128 < head_dim) acc1 = fmaf(S.w[p], __ldcg(pp + d + 128), acc1);
    }
    S.red[g][d] = acc0;
    S.red[g][d + 128] = acc1;
    __syncthreads();
    a0 = a1 = 0.0f;
    if (g == 0) {
#pragma unroll
        for (int k = 0; k < MG; ++k) { a0 += S.red[k][d]; a1 += S.red[k][d + 128]; }
    }
    M_out = S.M;
    den_out = S.den;
}

}  // namespace pkv_merge_impl
