// Token-sharded decode: exchange of the per-rank partial triples over NVLink and their merge, in one
// kernel. Every rank holds, in memory its peers can address, a gather buffer of 8-byte words
// [2 slots][world][rows][d+2]: the low half of a word is a float of a triple (o[d], m, l), the high
// half the number (epoch) of the exchange it belongs to. CTA c of rank r
//   1. stores its rows of the local merged triple, each value together with the current epoch in one
//      8-byte peer store, into slot s of EVERY rank's buffer (plain stores through NVSwitch; no
//      multicast, no TMA). A word is valid the moment its epoch half matches, so neither a fence nor
//      a separate flag round trip is needed: the exchange costs one NVLink latency,
//   2. merges the `world` triples of its rows straight from its own buffer, each thread spinning
//      (bounded; a give-up is recorded in `status` and the CTA returns) on exactly the words it needs:
//      M = max m, w = 2^(m - M), O = sum w o / sum w l, the split combine of
//      phasorkv/kernels/dense_attn.py:72-74 applied across ranks.
// CTAs depend only on the same-numbered CTA of the peers. Slots alternate with the epoch, which each
// CTA keeps in device memory, so the kernel can be replayed from a CUDA graph; a rank can be at most
// one exchange ahead of any peer (it needs that peer's words to finish), which two slots cover.
#include "pkv_common.cuh"
#include "pkv_merge.cuh"

namespace {

constexpr int NT = 256;
constexpr int MAX_WORLD = 16;
constexpr uint32_t POLL_LIMIT = 1u << 22;      // polls of a few hundred ns: about a second, then give up

__device__ __forceinline__ void st_word(uint2* p, float v, uint32_t epoch) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(epoch) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const uint2* p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
// Gather and merge of rows r0 .. r0 + nrow - 1: all words this CTA needs, [source][row][d+2], are polled into
// shared memory `got`. Every thread keeps a batch of independent loads in flight and re-reads only the
// words whose epoch is not there yet. Called by all NTH threads of the CTA.
template <int NTH>
__device__ __forceinline__ void gather_merge(const pkv_exchange_t& X, int c, int r0, int nrow, uint32_t epoch, size_t slot_off,
                                             size_t rank_words, float* got, int* fail_s, float* __restrict__ out,
                                             int32_t* __restrict__ status) {
    const int tid = threadIdx.x, PW = X.head_dim + 2;
    constexpr int NT = NTH;
    const uint2* mine = reinterpret_cast<const uint2*>(X.peer_data_dev[X.rank]) + slot_off;
    volatile int* fail = fail_s;
    const int row_words = nrow * PW, total = X.world * row_words;
    constexpr int BATCH = 8;
    for (int base = 0; base < total; base += NT * BATCH) {
        uint2 v[BATCH];
        const uint2* p[BATCH];
        unsigned pending = 0;
#pragma unroll
        for (int k = 0; k < BATCH; ++k) {
            const int i = base + k * NT + tid;
            p[k] = nullptr;
            if (i < total) {
                p[k] = mine + (size_t)(i / row_words) * rank_words + (size_t)r0 * PW + i % row_words;
                v[k] = ld_word(p[k]);
                pending |= 1u << k;
            }
        }
        for (uint32_t it = 0; pending && it < POLL_LIMIT; ++it) {
#pragma unroll
            for (int k = 0; k < BATCH; ++k) {
                if (!(pending & (1u << k))) continue;
                if (v[k].y == epoch) {
                    got[base + k * NT + tid] = __uint_as_float(v[k].x);
                    pending &= ~(1u << k);
                } else {
                    v[k] = ld_word(p[k]);
                }
            }
            if (pending && (it & 255u) == 255u) {
                if (*fail) break;
                __nanosleep(100);
            }
        }
        if (pending) *fail = 1;
    }
    __syncthreads();
    if (!*fail) {
        for (int e = tid; e < nrow * X.head_dim; e += NT) {
            const int rr = e / X.head_dim, d = e % X.head_dim;
            float M = -INFINITY;
            for (int s = 0; s < X.world; ++s) M = fmaxf(M, got[s * row_words + rr * PW + X.head_dim]);
            float num = 0.0f, den = 0.0f;
            for (int s = 0; s < X.world; ++s) {
                const float* g = got + s * row_words + rr * PW;
                const float w = M > -INFINITY ? exp2f(g[X.head_dim] - M) : 0.0f;   // a rank without a token of this sequence: m = -inf
                num = fmaf(w, g[d], num);
                den = fmaf(w, g[X.head_dim + 1], den);
            }
            out[(size_t)(r0 + rr) * X.head_dim + d] = den > 0.0f ? num / den : 0.0f;
        }
    }
    __syncthreads();
    if (*fail) {                                   // epoch not advanced: the exchange did not happen
        if (tid == 0 && status) { atomicExch(&status[0], 3); atomicExch(&status[1], c); }
        return;
    }
    if (tid == 0) X.epoch_dev[c] = epoch;
}

__global__ void __launch_bounds__(NT) pkv_exchange_merge_kernel(pkv_exchange_t X, const float* __restrict__ packed,
                                                                float* __restrict__ out, uint32_t phases,
                                                                int32_t* __restrict__ status) {
    __shared__ uint32_t epoch_s;
    __shared__ int fail_s;
    const int tid = threadIdx.x, c = blockIdx.x;
    const int rows = X.batch * X.n_q, PW = X.head_dim + 2;
    const int rows_per = (rows + X.n_cta - 1) / X.n_cta;
    const int r0 = c * rows_per, r1 = min(rows, r0 + rows_per);
    const int nrow = max(0, r1 - r0);
    pkv_grid_launch_dependents();
    pkv_grid_wait();                               // the attention launch before this one has written `packed`
    if (tid == 0) { epoch_s = X.epoch_dev[c] + 1u; fail_s = 0; }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    const size_t rank_words = (size_t)rows * PW;                        // one rank's triple
    const size_t slot_off = (size_t)(epoch & 1u) * X.world * rank_words;

    if (phases & PKV_EXCHANGE_PUSH) {
        const float* src = packed + (size_t)r0 * PW;
        const int n = nrow * PW;
        for (int i = tid; i < n; i += NT) {
            const float v = src[i];
            for (int dst = 0; dst < X.world; ++dst)
                st_word(reinterpret_cast<uint2*>(X.peer_data_dev[dst]) + slot_off + X.rank * rank_words + (size_t)r0 * PW + i, v, epoch);
        }
    }
    if (!(phases & PKV_EXCHANGE_MERGE)) return;

    extern __shared__ float got[];                  // [world][nrow][PW]
    gather_merge<NT>(X, c, r0, nrow, epoch, slot_off, rank_words, got, &fail_s, out, status);
}

// The merge of a row's split-T partials (pkv_merge.cuh) and its exchange in one launch: CTA = one
// (sequence, head) row, MG * 128 threads. The row's local triple never goes through global memory: it is
// pushed to the peers straight from the registers that hold it.
constexpr int NTM = pkv_merge_impl::MG * 128;

__global__ void __launch_bounds__(NTM) pkv_merge_exchange_kernel(pkv_exchange_t X, const float* __restrict__ parts, long stride_b,
                                                                 long stride_p, int n_parts, float* __restrict__ out,
                                                                 int32_t* __restrict__ status) {
    __shared__ pkv_merge_impl::MergeSmem S;
    __shared__ float got[MAX_WORLD * (128 + 2)];
    __shared__ uint32_t epoch_s;
    __shared__ int fail_s;
    const int tid = threadIdx.x, c = blockIdx.x;     // c = row = b * n_q + h
    const int PW = X.head_dim + 2;
    pkv_grid_launch_dependents();
    pkv_grid_wait();                               // the attention launch before this one has written the partials
    if (tid == 0) { epoch_s = X.epoch_dev[c] + 1u; fail_s = 0; }
    float a0, a1, M, den;
    pkv_merge_impl::merge_row(parts + (size_t)(c / X.n_q) * stride_b + (size_t)(c % X.n_q) * PW, stride_p, n_parts, X.head_dim,
                              S, a0, a1, M, den);    // has block-wide barriers: epoch_s is visible afterwards
    const uint32_t epoch = epoch_s;
    const size_t rank_words = (size_t)X.batch * X.n_q * PW;
    const size_t slot_off = (size_t)(epoch & 1u) * X.world * rank_words;
    if (tid < PW) {                                // head_dim <= 128: thread d holds dim d, threads d, d+1 beyond push m and l
        const float v = tid < X.head_dim ? a0 : (tid == X.head_dim ? M : den);
        for (int dst = 0; dst < X.world; ++dst)
            st_word(reinterpret_cast<uint2*>(X.peer_data_dev[dst]) + slot_off + X.rank * rank_words + (size_t)c * PW + tid, v, epoch);
    }
    gather_merge<NTM>(X, c, c, 1, epoch, slot_off, rank_words, got, &fail_s, out, status);
}

}  // namespace

extern "C" int pkv_exchange_merge(const pkv_exchange_t* x, const float* packed_dev, float* out_dev, uint32_t phases,
                                  int32_t* status_dev, void* stream) {
    if (!x || !x->peer_data_dev || !x->epoch_dev) return PKV_ERR_INVALID;
    if (x->world <= 0 || x->world > MAX_WORLD || x->rank < 0 || x->rank >= x->world) return PKV_ERR_INVALID;
    if (x->batch <= 0 || x->n_q <= 0 || x->head_dim <= 0 || (x->head_dim & 1) || x->n_cta <= 0) return PKV_ERR_INVALID;
    const int rows = x->batch * x->n_q;
    const size_t smem = (size_t)((rows + x->n_cta - 1) / x->n_cta) * x->world * (x->head_dim + 2) * sizeof(float);
    if (smem > 48 * 1024) return PKV_ERR_UNSUPPORTED;                      // use more CTAs (fewer rows each)
    if (!(phases & (PKV_EXCHANGE_PUSH | PKV_EXCHANGE_MERGE))) return PKV_ERR_INVALID;
    if ((phases & PKV_EXCHANGE_PUSH) && !packed_dev) return PKV_ERR_INVALID;
    if ((phases & PKV_EXCHANGE_MERGE) && !out_dev) return PKV_ERR_INVALID;
    PKV_CUDA_TRY(pkv_launch_chained(pkv_exchange_merge_kernel, dim3(x->n_cta), dim3(NT), smem, (cudaStream_t)stream, *x,
                                    packed_dev, out_dev, phases, status_dev));
    return PKV_OK;
}

extern "C" int pkv_merge_exchange(const pkv_exchange_t* x, const float* parts_dev, int64_t stride_b, int64_t stride_p,
                                  int32_t n_parts, float* out_dev, int32_t* status_dev, void* stream) {
    if (!x || !x->peer_data_dev || !x->epoch_dev || !parts_dev || !out_dev) return PKV_ERR_INVALID;
    if (x->world <= 0 || x->world > MAX_WORLD || x->rank < 0 || x->rank >= x->world) return PKV_ERR_INVALID;
    if (x->batch <= 0 || x->n_q <= 0 || x->head_dim <= 0 || (x->head_dim & 1)) return PKV_ERR_INVALID;
    if (x->head_dim > 128) return PKV_ERR_UNSUPPORTED;
    if (x->n_cta != x->batch * x->n_q) return PKV_ERR_INVALID;             // one CTA (and one epoch counter) per row
    if (n_parts <= 0 || (stride_b & 1) || (stride_p & 1) || (((uintptr_t)parts_dev) & 7u)) return PKV_ERR_INVALID;
    if (n_parts > pkv_merge_impl::MAX_PARTS) return PKV_ERR_UNSUPPORTED;
    PKV_CUDA_TRY(pkv_launch_chained(pkv_merge_exchange_kernel, dim3(x->n_cta), dim3(NTM), 0, (cudaStream_t)stream, *x, parts_dev,
                                    (long)stride_b, (long)stride_p, n_parts, out_dev, status_dev));
    return PKV_OK;
}
