// Decode-step prologue in ONE launch: the cache write of the newest token of every sequence
// (phasorkv/latent.py: PhasorKey.write + the NVFP4 store) and the absorption of the step's queries
// (PhasorKey.absorb). Both only depend on the layer input, so they run side by side as two roles of
// one grid instead of three launches in a row.
//
// Write role. The factor matrix (W x D fp32, 4 MB for a Llama-3.1-8B layer) has to stream through many
// SMs, so the projection is cut by latent column AND by d_model. A thread-block cluster of 8 CTAs owns
// one column tile -- 16 complex pairs, i.e. the 16 Re columns and the 16 Im columns that rotate
// together and that form two whole NVFP4 blocks -- and CTA r of the cluster owns the r-th eighth of
// d_model. Each CTA leaves its partial dot products in its own shared memory; after one cluster
// barrier CTA r adds the eight partials of tokens 2r and 2r+1 through distributed shared memory,
// rotates, quantises and stores them. No scratch in global memory, no second launch. (The partial sums of a
// slice are added in another order than in the two-launch path of pkv_write.cu: the two may differ in the last
// bit of a latent value.)
//
// Absorb role: the grid rows behind the column tiles run pkv_absorb_impl::body unchanged.
#include "pkv_absorb.cuh"
#include "pkv_vq.cuh"

#include <cooperative_groups.h>

int pkv_check_layer(const pkv_layer_t* L);
int pkv_check_cache(const pkv_cache_t* c);

namespace {

namespace cg = cooperative_groups;

constexpr int CL = 8;             // CTAs per cluster = d_model slices of one column tile
constexpr int PT = 16;            // tokens per pass
constexpr int PC = 16;            // complex pairs per column tile (Re block + Im block), or plain columns
constexpr int KC = 512;           // d_model chunk staged in shared memory
constexpr int BP = KC + 4;        // pitch of the factor tile: 16-byte reads of 8 consecutive rows hit distinct banks
constexpr int MAX_CH = 4;         // chunks per slice: d_model <= CL * MAX_CH * KC = 16384
constexpr int NT = 256;
constexpr int TPR = PT / CL;      // tokens of a pass that each CTA of the cluster finishes

constexpr int XS_FLOATS = PT * KC, BS_FLOATS = 2 * PC * BP, PART_FLOATS = MAX_CH * 2 * PT * PC, SUM_FLOATS = TPR * 2 * PC;
constexpr size_t WRITE_SMEM = sizeof(float) * (XS_FLOATS + BS_FLOATS + PART_FLOATS + SUM_FLOATS);

struct WriteArgs {
    const float* Bw;              // [W][D]
    const void* x;                // [n_tokens][D] fp32 or bf16
    int n_tokens, D, W, WP, R;
    const int32_t* positions;     // [n_tokens]
    const int32_t* slots;         // [n_tokens]
    const int32_t* freq;          // [R]
    const double* inv_freq;
    float attn_scale;
    pkv_second second;            // tensor scale: per layer, or per 16-column block (tiers)
    int scale_up;                 // block scales rounded up (pkv_set_scale_round_up)
    uint8_t* latent;
    int n_pages;
    float* latent_out;            // [n_tokens][W] or null
    const uint4* v_rows;          // [n_tokens][v_vecs] or null
    uint4* v_pool;
    uint8_t* vq_pool;             // quantised V pages instead (v_bits = 3 or 2): the rows are quantised here
    int v_bits;
    int v_vecs, n_kv;
    int n_tiles;                  // grid rows of the write role: R / 16 pair tiles, then (WP - 2R) / 16 plain tiles
};

template <typename XT>
__device__ __forceinline__ float4 load_x4(const XT* src) {
    if constexpr (sizeof(XT) == 4) {
        return *reinterpret_cast<const float4*>(src);
    } else {
        const uint2 u = *reinterpret_cast<const uint2*>(src);
        return make_float4(pkv_bf16_bits_to_float(u.x & 0xffffu), pkv_bf16_bits_to_float(u.x >> 16),
                           pkv_bf16_bits_to_float(u.y & 0xffffu), pkv_bf16_bits_to_float(u.y >> 16));
    }
}

// The projection of a pass is register-tiled: a thread owns one pair column, PTS tokens and one slice of the
// chunk's k range, so that a factor value read from shared memory feeds PTS multiply-adds (6 reads of 16 bytes per
// 32 multiply-adds; one token per thread needs 3 per 8 and is bound by shared-memory bandwidth: 12.1 us per launch
// at 16 tokens against 7.1 us at 4). TG = token groups of a pass: 1 (at most PTS tokens: a token-sharded sequence
// set, a batch of a few sequences; 16 k slices) or 4 (16 tokens, 4 k slices). The k slices are added in ascending
// order.
constexpr int PTS = 4;

template <typename XT, int TG>
__device__ __forceinline__ void write_role(const WriteArgs& A, float* sm) {
    cg::cluster_group cluster = cg::this_cluster();
    const int tid = threadIdx.x;
    const int ks = blockIdx.x;                                    // rank in the cluster (grid.x == CL)
    const int ct = blockIdx.y;
    const int R = A.R, D = A.D, W = A.W, n_tokens = A.n_tokens;
    const bool pair = ct < R / PC;
    const int colA = pair ? ct * PC : 2 * R + (ct - R / PC) * PC;       // Re block (or the plain block)
    const int colB = R + ct * PC;                                       // Im block of a pair tile
    const int DS = D / CL, k_lo = ks * DS, n_ch = (DS + KC - 1) / KC;
    float* xs = sm;                           // [PT][KC]
    float* bs = xs + XS_FLOATS;               // [2 * PC][BP]
    float* part = bs + BS_FLOATS;             // [MAX_CH][2][PT][PC]: this CTA's partial sums, read by the whole cluster
    float* sums = part + PART_FLOATS;         // [TPR][2][PC]
    const XT* x = reinterpret_cast<const XT*>(A.x);
    const int t = tid >> 4, c = tid & 15;
    constexpr int NVB = 2 * PC * (KC / 4) / NT;     // 16-byte vectors per thread: factor tile (16)
    constexpr int PTT = TG * PTS;                   // tokens of a pass that are worked on
    constexpr int NVX = PTT * (KC / 4) / NT;        // ... and token tile (8; 2 with one token group)

    for (int t0 = 0; t0 < n_tokens; t0 += PT) {
        const int my_tok = t0 + ks * TPR + (tid >> 4);              // for tid < TPR * PC: the token this thread rotates
        float pr = 1.0f, pi = 0.0f;
        for (int ch = 0; ch < n_ch; ++ch) {
            const int k0 = k_lo + ch * KC, kc = min(KC, DS - ch * KC);
            const bool load_b = n_ch > 1 || t0 == 0;                // a single chunk stays in shared memory across passes
            float4 bv[NVB], xv[NVX];
            if (load_b) {
#pragma unroll
                for (int n = 0; n < NVB; ++n) {
                    const int i = tid + n * NT, rr = i / (KC / 4), k4 = i % (KC / 4);
                    const int col = rr < PC ? colA + rr : colB + rr - PC;
                    bv[n] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if ((rr < PC || pair) && col < W && k4 * 4 < kc)
                        bv[n] = *reinterpret_cast<const float4*>(A.Bw + (size_t)col * D + k0 + k4 * 4);
                }
            }
#pragma unroll
            for (int n = 0; n < NVX; ++n) {
                const int i = tid + n * NT, tt = i / (KC / 4), k4 = i % (KC / 4);
                xv[n] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (t0 + tt < n_tokens && k4 * 4 < kc) xv[n] = load_x4<XT>(x + (size_t)(t0 + tt) * D + k0 + k4 * 4);
            }
            (void)t;
            if (ch == 0) {
                // while the tiles are in flight: the V rows of this CTA's tokens, and the phasors it will need
                if (ct == 0 && A.v_rows && A.vq_pool) {              // a warp per (token, kv head) row
                    for (int r = tid >> 5; r < TPR * A.n_kv; r += NT / 32) {
                        const int tok = t0 + ks * TPR + r / A.n_kv;
                        if (tok >= n_tokens) break;
                        const int slot = A.slots[tok];
                        if (slot < 0 || slot >= A.n_pages * PKV_PAGE_TOKENS) continue;
                        const uint2 u = reinterpret_cast<const uint2*>(A.v_rows)[((size_t)tok * A.n_kv + r % A.n_kv) * 32 + (tid & 31)];
                        pkv_vq_store_row(u, tid & 31, slot, r % A.n_kv, A.n_kv, A.v_bits, A.vq_pool);
                    }
                } else if (ct == 0 && A.v_rows) {
                    for (int i = tid; i < TPR * A.v_vecs; i += NT) {
                        const int tok = t0 + ks * TPR + i / A.v_vecs;
                        if (tok >= n_tokens) break;
                        const int slot = A.slots[tok];
                        if (slot < 0 || slot >= A.n_pages * PKV_PAGE_TOKENS) continue;
                        A.v_pool[pkv_v_vec_index(slot, i % A.v_vecs, A.n_kv, A.v_vecs / A.n_kv)] = A.v_rows[(size_t)tok * A.v_vecs + i % A.v_vecs];
                    }
                }
                if (pair && tid < TPR * PC && my_tok < n_tokens) {
                    double sn, cs;
                    sincos((double)A.positions[my_tok] * A.inv_freq[A.freq[ct * PC + c]], &sn, &cs);
                    pr = (float)((double)A.attn_scale * cs);
                    pi = (float)((double)A.attn_scale * sn);
                }
            }
            if (ch > 0 || t0 > 0) __syncthreads();                  // the tiles of the chunk before are no longer read
            if (load_b) {
#pragma unroll
                for (int n = 0; n < NVB; ++n) {
                    const int i = tid + n * NT;
                    *reinterpret_cast<float4*>(bs + (i / (KC / 4)) * BP + (i % (KC / 4)) * 4) = bv[n];
                }
            }
#pragma unroll
            for (int n = 0; n < NVX; ++n) {
                const int i = tid + n * NT;
                *reinterpret_cast<float4*>(xs + (i / (KC / 4)) * KC + (i % (KC / 4)) * 4) = xv[n];
            }
            __syncthreads();
            {
                // thread = (pair column c2, token group tgi, k slice kq of KC / KQ values)
                constexpr int KQ = 16 / TG, KS = KC / KQ;
                const int c2 = tid & 15, tgi = (tid >> 4) % TG, kq = (tid >> 4) / TG;
                float re[PTS][4], im[PTS][4];
#pragma unroll
                for (int tt = 0; tt < PTS; ++tt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) re[tt][e] = im[tt][e] = 0.0f;
                const float* ar = bs + c2 * BP + kq * KS;
                const float* br = bs + (PC + c2) * BP + kq * KS;
                const float* xr = xs + tgi * PTS * KC + kq * KS;
#pragma unroll 4
                for (int k = 0; k < KS; k += 4) {
                    const float4 av = *reinterpret_cast<const float4*>(ar + k);
                    const float4 bq = pair ? *reinterpret_cast<const float4*>(br + k) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int tt = 0; tt < PTS; ++tt) {
                        const float4 xq = *reinterpret_cast<const float4*>(xr + tt * KC + k);
                        re[tt][0] = fmaf(xq.x, av.x, re[tt][0]); re[tt][1] = fmaf(xq.y, av.y, re[tt][1]);
                        re[tt][2] = fmaf(xq.z, av.z, re[tt][2]); re[tt][3] = fmaf(xq.w, av.w, re[tt][3]);
                        im[tt][0] = fmaf(xq.x, bq.x, im[tt][0]); im[tt][1] = fmaf(xq.y, bq.y, im[tt][1]);
                        im[tt][2] = fmaf(xq.z, bq.z, im[tt][2]); im[tt][3] = fmaf(xq.w, bq.w, im[tt][3]);
                    }
                }
                __syncthreads();                                    // every thread is done with the token tile: it becomes the exchange area
                float* red = xs;                                    // [KQ k slices][PTT tokens][2][PC]
#pragma unroll
                for (int tt = 0; tt < PTS; ++tt) {
                    red[((kq * PTT + tgi * PTS + tt) * 2 + 0) * PC + c2] = (re[tt][0] + re[tt][1]) + (re[tt][2] + re[tt][3]);
                    red[((kq * PTT + tgi * PTS + tt) * 2 + 1) * PC + c2] = (im[tt][0] + im[tt][1]) + (im[tt][2] + im[tt][3]);
                }
                __syncthreads();
                for (int idx = tid; idx < PTT * 2 * PC; idx += NT) {
                    const int tt = idx >> 5, half = (idx >> 4) & 1, cc = idx & 15;
                    float v = 0.0f;
#pragma unroll
                    for (int q = 0; q < KQ; ++q) v += red[((q * PTT + tt) * 2 + half) * PC + cc];
                    part[((ch * 2 + half) * PT + tt) * PC + cc] = v;
                }
            }                                                       // (the next chunk's first barrier protects `red`)
        }
        cluster.sync();                                             // every partial of the pass is in place

        // ---- this CTA finishes tokens ks * TPR .. + TPR - 1 of the pass
        if (tid < TPR * 2 * PC) {
            const int tl = tid >> 5, half = (tid >> 4) & 1;
            const int row = ks * TPR + tl;
            float pv[CL][MAX_CH];
#pragma unroll
            for (int s = 0; s < CL; ++s) {
                const float* rp = cluster.map_shared_rank(part, s);
#pragma unroll
                for (int ch = 0; ch < MAX_CH; ++ch) pv[s][ch] = ch < n_ch ? rp[((ch * 2 + half) * PT + row) * PC + c] : 0.0f;
            }
            float v = 0.0f;                                         // slices in ascending d_model order
#pragma unroll
            for (int s = 0; s < CL; ++s)
#pragma unroll
                for (int ch = 0; ch < MAX_CH; ++ch)
                    if (ch < n_ch) v += pv[s][ch];
            sums[(tl * 2 + half) * PC + c] = v;
        }
        __syncthreads();
        if (pair && tid < TPR * PC) {
            const int tl = tid >> 4;
            const float x0 = sums[(tl * 2) * PC + c], x1 = sums[(tl * 2 + 1) * PC + c];
            sums[(tl * 2) * PC + c] = __fsub_rn(__fmul_rn(x0, pr), __fmul_rn(x1, pi));
            sums[(tl * 2 + 1) * PC + c] = __fadd_rn(__fmul_rn(x0, pi), __fmul_rn(x1, pr));
        }
        __syncthreads();
        if (tid < TPR * 2 * PC) {
            const int tl = tid >> 5, half = (tid >> 4) & 1;
            const int tok = t0 + ks * TPR + tl, col = half ? colB + c : colA + c;
            if (A.latent_out && tok < n_tokens && (pair || !half) && col < W) A.latent_out[(size_t)tok * W + col] = sums[(tl * 2 + half) * PC + c];
        }
        if (tid < TPR * 2) {
            const int tl = tid >> 1, half = tid & 1;
            const int tok = t0 + ks * TPR + tl;
            if (A.latent && tok < n_tokens && (pair || !half)) {
                const int slot = A.slots[tok];
                if (slot >= 0 && slot < A.n_pages * PKV_PAGE_TOKENS) {
                    float v[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = sums[(tl * 2 + half) * PC + i];
                    uint8_t sb;
                    const int j = (half ? colB : colA) / 16, RB = A.WP / 2;
                    const uint2 packed = pkv_quantize_block16(v, A.second.of(j), sb, A.scale_up != 0);
                    uint8_t* page = A.latent + (size_t)(slot / PKV_PAGE_TOKENS) * pkv_page_bytes(W);
                    const uint32_t r = slot % PKV_PAGE_TOKENS;
                    *reinterpret_cast<uint2*>(page + pkv_code_offset(r, j * 8, RB)) = packed;
                    page[pkv_codes_bytes(W) + pkv_scale_offset(r, j)] = sb;
                }
            }
        }
        cluster.sync();             // nobody reads this CTA's partials any more: next pass, or exit
    }
}

template <typename XT, int TG>
__global__ void __launch_bounds__(NT) pkv_step_prologue_kernel(const WriteArgs Wa, const pkv_absorb_impl::Args Aa, int batch) {
    extern __shared__ __align__(16) float sm[];
    // Wait first, trigger second (as pkv_absorb does): the attention kernel behind this one streams cache
    // pages before its own wait, which is only safe if every launch up to this kernel's predecessor -- a
    // chunk write of the same cache, for instance -- has completed by the time it starts.
    pkv_grid_wait();                                     // x and q may be the output of the kernel before
    pkv_grid_launch_dependents();
    if ((int)blockIdx.y >= Wa.n_tiles) {
        const int n_hg = (Aa.n_q + pkv_absorb_impl::HG - 1) / pkv_absorb_impl::HG;
        const int a = ((int)blockIdx.y - Wa.n_tiles) * CL + (int)blockIdx.x;
        if (a < batch * n_hg) pkv_absorb_impl::body(Aa, a / n_hg, a % n_hg, sm);
        return;
    }
    write_role<XT, TG>(Wa, sm);
}

template <typename XT, int TG>
cudaError_t launch_prologue(const WriteArgs& Wa, const pkv_absorb_impl::Args& Aa, int batch, size_t smem, cudaStream_t st) {
    auto kern = pkv_step_prologue_kernel<XT, TG>;
    static pkv_attr_flags smem_set;                      // per instantiation and device
    {
        cudaError_t e = pkv_set_max_smem(kern, (int)smem, smem_set);
        if (e != cudaSuccess) return e;
    }
    const int n_hg = (Aa.n_q + pkv_absorb_impl::HG - 1) / pkv_absorb_impl::HG;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(CL, Wa.n_tiles + (batch * n_hg + CL - 1) / CL);
    cfg.blockDim = dim3(NT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = CL;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kern, Wa, Aa, batch);
}

}  // namespace

extern "C" int pkv_decode_prologue(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* x_dev, int32_t x_dtype,
                                   const int32_t* write_positions_dev, const int32_t* slots_dev, const void* v_rows_dev,
                                   const float* q_dev, const int32_t* query_positions_dev, int32_t batch,
                                   float* latent_out_dev, float* scratch_dev, float* qabs_out_dev, uint8_t* qop_out_dev,
                                   int32_t* status_dev, void* stream) {
    return pkv_decode_prologue_sync(layer, cache, x_dev, x_dtype, write_positions_dev, slots_dev, v_rows_dev, q_dev,
                                    query_positions_dev, batch, latent_out_dev, scratch_dev, qabs_out_dev, qop_out_dev, nullptr,
                                    status_dev, stream);
}

extern "C" int pkv_decode_prologue_sync(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* x_dev, int32_t x_dtype,
                                        const int32_t* write_positions_dev, const int32_t* slots_dev, const void* v_rows_dev,
                                        const float* q_dev, const int32_t* query_positions_dev, int32_t batch,
                                        float* latent_out_dev, float* scratch_dev, float* qabs_out_dev, uint8_t* qop_out_dev,
                                        int32_t* qsync_dev, int32_t* status_dev, void* stream) {
    int st = pkv_check_layer(layer);
    if (st) return st;
    if (batch < 0) return PKV_ERR_INVALID;
    if (batch == 0) return PKV_OK;
    if (!cache || !x_dev || !write_positions_dev || !slots_dev || (q_dev && !query_positions_dev)) return PKV_ERR_INVALID;
    st = pkv_check_cache(cache);
    if (st) return st;
    const int W = 2 * layer->R + layer->R_s, WP = pkv_padded_width(W), D = layer->d_model;
    if (cache->W != W) return PKV_ERR_INVALID;
    if (x_dtype != PKV_F32 && x_dtype != PKV_BF16) return PKV_ERR_INVALID;
    const bool fused = batch <= PKV_SMALL_WRITE_TOKENS && layer->R % PC == 0 && D % (CL * 4) == 0 && D / CL <= MAX_CH * KC &&
                       !((((uintptr_t)x_dev) | ((uintptr_t)layer->Bw_dev)) & 15u) &&
                       layer->head_dim / 2 <= pkv_absorb_impl::MAX_H && !(layer->head_dim & 1) &&
                       (!qop_out_dev || (layer->n_q * PKV_QUERY_TERMS == 128 && !(((uintptr_t)qop_out_dev) & 1023u)));
    if (!fused) {                                        // same results from the separate launches
        if (cache->v_bits && v_rows_dev) {               // quantised V pages have their own writer
            st = pkv_vq_write(cache, v_rows_dev, slots_dev, batch, stream);
            if (st) return st;
        }
        st = pkv_cache_write(layer, cache, x_dev, x_dtype, write_positions_dev, nullptr, slots_dev, batch, latent_out_dev,
                             scratch_dev, cache->v_bits ? nullptr : v_rows_dev, status_dev, stream);
        if (st || !q_dev) return st;
        return pkv_absorb_sync(layer, q_dev, query_positions_dev, nullptr, batch, qabs_out_dev, qop_out_dev, qsync_dev, stream);
    }
    WriteArgs Wa;
    Wa.Bw = layer->Bw_dev; Wa.x = x_dev; Wa.n_tokens = batch; Wa.D = D; Wa.W = W; Wa.WP = WP; Wa.R = layer->R;
    Wa.positions = write_positions_dev; Wa.slots = slots_dev; Wa.freq = layer->freq_dev; Wa.inv_freq = layer->inv_freq_dev;
    Wa.attn_scale = layer->attn_scale; Wa.second = pkv_second_of(layer); Wa.scale_up = pkv_scale_round_up_mode();
    Wa.latent = cache->latent_dev; Wa.n_pages = cache->n_pages; Wa.latent_out = latent_out_dev;
    const bool with_vq = cache->v_bits != 0 && cache->vq_dev && v_rows_dev && cache->head_dim == 128;
    const bool with_v = (cache->v_dev && v_rows_dev && !cache->v_bits) || with_vq;
    Wa.v_rows = with_v ? reinterpret_cast<const uint4*>(v_rows_dev) : nullptr;
    Wa.v_pool = with_v && !with_vq ? reinterpret_cast<uint4*>(cache->v_dev) : nullptr;
    Wa.vq_pool = with_vq ? reinterpret_cast<uint8_t*>(cache->vq_dev) : nullptr;
    Wa.v_bits = cache->v_bits;
    Wa.v_vecs = with_v ? cache->n_kv * cache->head_dim * 2 / 16 : 0;
    Wa.n_kv = cache->n_kv;
    Wa.n_tiles = layer->R / PC + (WP - 2 * layer->R) / PC;
    if (qsync_dev && !(q_dev && qop_out_dev)) return PKV_ERR_INVALID;
    pkv_absorb_impl::Args Aa = pkv_absorb_impl::make_args(layer, q_dev, query_positions_dev, nullptr, qabs_out_dev, qop_out_dev);
    Aa.qsync = qsync_dev;
    size_t smem = WRITE_SMEM;
    const size_t absorb_smem = pkv_absorb_impl::smem_bytes(layer->head_dim, WP);
    if (absorb_smem > smem) smem = absorb_smem;
    const int absorb_batch = q_dev ? batch : 0;                      // no queries: the write role alone
    const cudaStream_t cst = (cudaStream_t)stream;
    cudaError_t le;
    if (batch <= PTS)                                                 // a few tokens: one token group, 16 k slices
        le = x_dtype == PKV_F32 ? launch_prologue<float, 1>(Wa, Aa, absorb_batch, smem, cst)
                                : launch_prologue<uint16_t, 1>(Wa, Aa, absorb_batch, smem, cst);
    else
        le = x_dtype == PKV_F32 ? launch_prologue<float, 4>(Wa, Aa, absorb_batch, smem, cst)
                                : launch_prologue<uint16_t, 4>(Wa, Aa, absorb_batch, smem, cst);
    PKV_CUDA_TRY(le);
    return PKV_OK;
}
