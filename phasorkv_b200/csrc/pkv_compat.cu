// The reference's three PhasorKey calls in the precision of their arguments, without quantisation:
//   pkv_scores_exact     PhasorKey.scores  (phasorkv/latent.py:85-88)   q_abs @ cache^T, fp32 or fp64
//   pkv_write_rows_f64   PhasorKey.write   (phasorkv/latent.py:61-70)   for fp64 x ("fp64 if given fp64")
//   pkv_absorb_rows_f64  PhasorKey.absorb  (phasorkv/latent.py:72-83)   for fp64 q
// These are the calls existing host code and the reference's exactness statement (2e-15 against rebuilt
// keys, README.md:75-77) are written against. They are not on the decode path -- that one streams the
// NVFP4 cache through the tensor cores -- so they are plain CUDA-core kernels: a tiled X . Y^T product and
// two elementwise kernels.
#include "pkv_common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

// C[m, n] = sum_k X[m, k] * Y[n, k]; 256 threads, a 4 x 4 block of C per thread
template <typename T>
__global__ void __launch_bounds__(256) pkv_gemm_nt_kernel(const T* __restrict__ X, const T* __restrict__ Y, T* __restrict__ C,
                                                          int M, int N, int K, long ldx, long ldy, long ldc) {
    __shared__ T xs[BK][BM + 1], ys[BK][BN + 1];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    T acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = tid; i < BM * BK; i += 256) {
            const int r = i / BK, k = i % BK;
            xs[k][r] = (m0 + r < M && k0 + k < K) ? X[(size_t)(m0 + r) * ldx + k0 + k] : T(0);
            ys[k][r] = (n0 + r < N && k0 + k < K) ? Y[(size_t)(n0 + r) * ldy + k0 + k] : T(0);
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            T a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = xs[k][ty * 4 + i]; b[i] = ys[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) C[(size_t)m * ldc + n] = acc[i][j];
        }
}

template <typename T>
int gemm_nt(const T* X, const T* Y, T* C, int M, int N, int K, long ldx, long ldy, long ldc, cudaStream_t st) {
    if (M == 0 || N == 0) return PKV_OK;
    pkv_gemm_nt_kernel<T><<<dim3((N + BN - 1) / BN, (M + BM - 1) / BM), 256, 0, st>>>(X, Y, C, M, N, K, ldx, ldy, ldc);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

// rows [n, W] hold x . [Re B | Im B | B_s]^T; columns k and R + k become the complex product with the
// phasor of frequency freq[k] (the slow columns stay as they are)
__global__ void pkv_rotate_rows_f64_kernel(double* __restrict__ rows, const double2* __restrict__ ph, const int32_t* __restrict__ freq,
                                           int n, int W, int R, int h) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)n * R) return;
    const int t = (int)(i / R), k = (int)(i % R);
    const double2 p = ph[(size_t)t * h + freq[k]];
    double* row = rows + (size_t)t * W;
    const double a = row[k], b = row[R + k];
    row[k] = a * p.x - b * p.y;
    row[R + k] = a * p.y + b * p.x;
}

// one thread per (query position, head, output column)
__global__ void pkv_absorb_rows_f64_kernel(const double* __restrict__ A_re, const double* __restrict__ A_im,
                                           const double* __restrict__ A_s, const int32_t* __restrict__ freq,
                                           const int32_t* __restrict__ slow, int n_q, int n_kv, int d, int R, int R_s, int n_slow,
                                           const double* __restrict__ q, const double2* __restrict__ ph, int Tq,
                                           double* __restrict__ out) {
    const int W = 2 * R + R_s, h = d / 2;
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)Tq * n_q * (R + R_s)) return;
    const int c = (int)(i % (R + R_s)), head = (int)((i / (R + R_s)) % n_q), t = (int)(i / ((long)(R + R_s) * n_q));
    const int g = head / (n_q / n_kv);
    const double* qr = q + ((size_t)t * n_q + head) * d;
    double* o = out + ((size_t)t * n_q + head) * W;
    if (c < R) {
        const int j = freq[c];
        const double2 p = ph[(size_t)t * h + j];
        const double zr = qr[j] * p.x - qr[j + h] * p.y, zi = qr[j] * p.y + qr[j + h] * p.x;      // zq * phasor
        const double ar = A_re[(size_t)g * R + c], ai = -A_im[(size_t)g * R + c];                 // conj(A)
        o[c] = ar * zr - ai * zi;
        o[R + c] = ar * zi + ai * zr;
    } else {
        const int r = c - R;
        double acc = 0.0;
        for (int s = 0; s < 2 * n_slow; ++s) {
            const double qs = s < n_slow ? qr[slow[s]] : qr[slow[s - n_slow] + h];                // unrotated
            acc += qs * A_s[((size_t)g * 2 * n_slow + s) * R_s + r];
        }
        o[2 * R + r] = acc;
    }
}

}  // namespace

extern "C" int pkv_scores_exact(const void* q_abs_dev, const void* rows_dev, int32_t n_query_rows, int32_t n_tokens, int32_t W,
                                int32_t dtype, void* out_dev, void* stream) {
    if (n_query_rows < 0 || n_tokens < 0 || W <= 0) return PKV_ERR_INVALID;
    if (n_query_rows == 0 || n_tokens == 0) return PKV_OK;
    if (!q_abs_dev || !rows_dev || !out_dev) return PKV_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == PKV_F32)
        return gemm_nt<float>((const float*)q_abs_dev, (const float*)rows_dev, (float*)out_dev, n_query_rows, n_tokens, W, W, W,
                              n_tokens, st);
    if (dtype == PKV_F64)
        return gemm_nt<double>((const double*)q_abs_dev, (const double*)rows_dev, (double*)out_dev, n_query_rows, n_tokens, W, W, W,
                               n_tokens, st);
    return PKV_ERR_INVALID;
}

extern "C" int pkv_write_rows_f64(const double* Bw_dev, const int32_t* freq_dev, int32_t d_model, int32_t R, int32_t R_s,
                                  int32_t half_dim, const double* x_dev, const double* phasors_dev, int32_t n_tokens,
                                  double* rows_out_dev, void* stream) {
    if (d_model <= 0 || R < 0 || R_s < 0 || 2 * R + R_s <= 0 || half_dim <= 0 || n_tokens < 0) return PKV_ERR_INVALID;
    if (n_tokens == 0) return PKV_OK;
    if (!Bw_dev || !x_dev || !rows_out_dev || (R && (!freq_dev || !phasors_dev))) return PKV_ERR_INVALID;
    if (((uintptr_t)phasors_dev) & 15u) return PKV_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    const int W = 2 * R + R_s;
    int rc = gemm_nt<double>(x_dev, Bw_dev, rows_out_dev, n_tokens, W, d_model, d_model, d_model, W, st);
    if (rc || !R) return rc;
    const long n = (long)n_tokens * R;
    pkv_rotate_rows_f64_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(rows_out_dev, (const double2*)phasors_dev, freq_dev,
                                                                           n_tokens, W, R, half_dim);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

extern "C" int pkv_absorb_rows_f64(const double* A_re_dev, const double* A_im_dev, const double* A_s_dev, const int32_t* freq_dev,
                                   const int32_t* slow_dev, int32_t n_q, int32_t n_kv, int32_t head_dim, int32_t R, int32_t R_s,
                                   int32_t n_slow, const double* q_dev, const double* phasors_dev, int32_t n_positions,
                                   double* out_dev, void* stream) {
    if (n_q <= 0 || n_kv <= 0 || n_q % n_kv || head_dim <= 0 || (head_dim & 1) || R < 0 || R_s < 0 || n_positions < 0)
        return PKV_ERR_INVALID;
    if (n_positions == 0 || R + R_s == 0) return PKV_OK;
    if (!q_dev || !out_dev || (R && (!A_re_dev || !A_im_dev || !freq_dev || !phasors_dev))) return PKV_ERR_INVALID;
    if (R_s && (!A_s_dev || !slow_dev || n_slow <= 0)) return PKV_ERR_INVALID;
    if (((uintptr_t)phasors_dev) & 15u) return PKV_ERR_INVALID;
    const long n = (long)n_positions * n_q * (R + R_s);
    pkv_absorb_rows_f64_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        A_re_dev, A_im_dev, A_s_dev, freq_dev, slow_dev, n_q, n_kv, head_dim, R, R_s, n_slow, q_dev, (const double2*)phasors_dev,
        n_positions, out_dev);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}
