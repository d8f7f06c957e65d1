// Exact-token side path: a handful of tokens per sequence (attention sinks and the recent window) whose
// keys are kept as rotated bf16 rows instead of latent rows take part in the same softmax as the
// latent tokens (phasorkv/kernels/latent_attn.py:448-495, 548-596: `exact = (k, v)` bf16
// [B, n_kv, E, d], k after RoPE). Here they contribute ONE more partial triple (o, m, l) per
// (sequence, head), in the convention of the split-T partials, and the merge adds it to the splits.
//
// One CTA per (sequence, kv head), 128 threads:
//   1. the REP query heads of the kv head are rotated to the query position (angle in double, the
//      phasor of pkv_absorb: scale * e^{i theta m}, rotate-half pairing of rope.py:12-15),
//   2. thread e forms the logits of exact token e for the REP heads (fp32 dot products),
//   3. base-2 softmax statistics per head, then thread d accumulates o[d] = sum_e p_e v[e][d].
#include "pkv_common.cuh"

int pkv_check_layer(const pkv_layer_t* L);

namespace {

constexpr int NT = 128;
constexpr int MAX_REP = 8, MAX_E = 512, MAX_D = 128;

__global__ void __launch_bounds__(NT) pkv_exact_partial_kernel(
    const float* __restrict__ q, const int32_t* __restrict__ positions, const double* __restrict__ inv_freq,
    float attn_scale, const int32_t* __restrict__ slow, int n_slow, const uint16_t* __restrict__ k_exact, const uint16_t* __restrict__ v_exact,
    const int32_t* __restrict__ n_exact, int e_max, int n_q, int n_kv, int head_dim, float logit_scale,
    float* __restrict__ out) {
    __shared__ float qr[MAX_REP][MAX_D];
    __shared__ float p_s[MAX_REP][MAX_E];
    __shared__ float red[MAX_REP][NT / 32];
    __shared__ float m_s[MAX_REP], l_s[MAX_REP];
    const int b = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rep = n_q / n_kv, h2 = head_dim / 2, PW = head_dim + 2;
    pkv_grid_launch_dependents();
    pkv_grid_wait();
    const int E = n_exact ? min(max(n_exact[b], 0), e_max) : e_max;
    // ---- 1. rotated query heads
    for (int j = tid; j < h2; j += NT) {
        double sn, cs;
        sincos((double)positions[b] * inv_freq[j], &sn, &cs);
        float pr = (float)((double)attn_scale * cs), pi = (float)((double)attn_scale * sn);
        for (int s = 0; s < n_slow; ++s)              // band layouts: these frequencies are scored without rotation
            if (slow[s] == j) { pr = attn_scale; pi = 0.0f; }
        for (int r = 0; r < rep; ++r) {
            const float* qh = q + ((size_t)b * n_q + g * rep + r) * head_dim;
            const float a = qh[j], c = qh[j + h2];
            qr[r][j] = __fsub_rn(__fmul_rn(a, pr), __fmul_rn(c, pi));
            qr[r][j + h2] = __fadd_rn(__fmul_rn(a, pi), __fmul_rn(c, pr));
        }
    }
    __syncthreads();
    // ---- 2. logits in base-2 units
    const uint16_t* kb = k_exact + ((size_t)b * n_kv + g) * e_max * head_dim;
    const uint16_t* vb = v_exact + ((size_t)b * n_kv + g) * e_max * head_dim;
    float mx[MAX_REP];
#pragma unroll
    for (int r = 0; r < MAX_REP; ++r) mx[r] = -INFINITY;
    for (int e = tid; e < E; e += NT) {
        float acc[MAX_REP];
#pragma unroll
        for (int r = 0; r < MAX_REP; ++r) acc[r] = 0.0f;
        const uint4* kr = reinterpret_cast<const uint4*>(kb + (size_t)e * head_dim);
        for (int d8 = 0; d8 < head_dim / 8; ++d8) {
            const uint4 u = kr[d8];
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float k0 = pkv_bf16_bits_to_float(w[i] & 0xffffu), k1 = pkv_bf16_bits_to_float(w[i] >> 16);
#pragma unroll
                for (int r = 0; r < MAX_REP; ++r)
                    if (r < rep) acc[r] = fmaf(k1, qr[r][d8 * 8 + 2 * i + 1], fmaf(k0, qr[r][d8 * 8 + 2 * i], acc[r]));
            }
        }
#pragma unroll
        for (int r = 0; r < MAX_REP; ++r)
            if (r < rep) { const float s = acc[r] * logit_scale; p_s[r][e] = s; mx[r] = fmaxf(mx[r], s); }
    }
    // ---- 3. maxima, weights, sums
#pragma unroll
    for (int r = 0; r < MAX_REP; ++r) {
#pragma unroll
        for (int o = 16; o; o >>= 1) mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], o));
        if (lane == 0) red[r][warp] = mx[r];
    }
    __syncthreads();
    if (tid < rep) {
        float m = -INFINITY;
        for (int w = 0; w < NT / 32; ++w) m = fmaxf(m, red[tid][w]);
        m_s[tid] = m;
    }
    __syncthreads();
    float ls[MAX_REP];
#pragma unroll
    for (int r = 0; r < MAX_REP; ++r) ls[r] = 0.0f;
    for (int e = tid; e < E; e += NT) {
#pragma unroll
        for (int r = 0; r < MAX_REP; ++r)
            if (r < rep) { const float p = exp2f(p_s[r][e] - m_s[r]); p_s[r][e] = p; ls[r] += p; }
    }
    __syncthreads();                                  // red is reused; every p is in place
#pragma unroll
    for (int r = 0; r < MAX_REP; ++r) {
#pragma unroll
        for (int o = 16; o; o >>= 1) ls[r] += __shfl_xor_sync(0xffffffffu, ls[r], o);
        if (lane == 0) red[r][warp] = ls[r];
    }
    __syncthreads();
    if (tid < rep) {
        float l = 0.0f;
        for (int w = 0; w < NT / 32; ++w) l += red[tid][w];
        l_s[tid] = l;
    }
    // ---- o[d] = sum_e p_e v[e][d], thread d
    for (int d = tid; d < head_dim; d += NT) {
        float acc[MAX_REP];
#pragma unroll
        for (int r = 0; r < MAX_REP; ++r) acc[r] = 0.0f;
        for (int e = 0; e < E; ++e) {
            const float v = pkv_bf16_bits_to_float(vb[(size_t)e * head_dim + d]);
#pragma unroll
            for (int r = 0; r < MAX_REP; ++r)
                if (r < rep) acc[r] = fmaf(p_s[r][e], v, acc[r]);
        }
#pragma unroll
        for (int r = 0; r < MAX_REP; ++r)
            if (r < rep) out[((size_t)b * n_q + g * rep + r) * PW + d] = acc[r];
    }
    __syncthreads();
    if (tid < rep) {                                  // no exact token: the neutral triple (m = -inf, l = 0, o = 0)
        out[((size_t)b * n_q + g * rep + tid) * PW + head_dim] = m_s[tid];
        out[((size_t)b * n_q + g * rep + tid) * PW + head_dim + 1] = l_s[tid];
    }
}

}  // namespace

extern "C" int pkv_exact_partial(const pkv_layer_t* layer, const float* q_dev, const int32_t* positions_dev,
                                 const void* k_exact_dev, const void* v_exact_dev, const int32_t* n_exact_dev,
                                 int32_t e_max, int32_t batch, float* exact_out_dev, void* stream) {
    int st = pkv_check_layer(layer);
    if (st) return st;
    if (batch < 0 || e_max < 0) return PKV_ERR_INVALID;
    if (batch == 0) return PKV_OK;
    if (!q_dev || !positions_dev || !exact_out_dev || (e_max > 0 && (!k_exact_dev || !v_exact_dev))) return PKV_ERR_INVALID;
    if ((((uintptr_t)k_exact_dev) | ((uintptr_t)v_exact_dev)) & 15u) return PKV_ERR_INVALID;
    const int rep = layer->n_q / layer->n_kv;
    if (rep > MAX_REP || e_max > MAX_E || layer->head_dim > MAX_D || (layer->head_dim % 8)) return PKV_ERR_UNSUPPORTED;
    const float logit_scale = PKV_LOG2E / sqrtf((float)layer->head_dim);
    PKV_CUDA_TRY(pkv_launch_chained(pkv_exact_partial_kernel, dim3(batch, layer->n_kv), dim3(NT), 0, (cudaStream_t)stream, q_dev,
                                    positions_dev, layer->inv_freq_dev, layer->attn_scale, layer->R_s > 0 ? layer->slow_dev : nullptr,
                                    layer->R_s > 0 ? layer->n_slow : 0, (const uint16_t*)k_exact_dev,
                                    (const uint16_t*)v_exact_dev, n_exact_dev, e_max, layer->n_q, layer->n_kv, layer->head_dim,
                                    logit_scale, exact_out_dev));
    return PKV_OK;
}
