// Fused cache write on tensor cores (prefill / chunk write of bf16 hidden states).
//
//   latent[t, :] = x[t, :] . Bw^T   as tcgen05.mma kind::f16 with fp32 accumulation in tensor memory.
// x is bf16 and therefore exact; the fp32 factor matrix enters as the sum of three bf16 matrices
// (hi + mid + lo, exact to 2^-24 relative), i.e. three passes over the same x tile that accumulate in
// the same 128 x W accumulator. A tile is 128 tokens and the whole latent row of each; a CTA takes the tiles
// blockIdx.x, blockIdx.x + gridDim.x, ... (the grid is at most one CTA per SM) and keeps two accumulators in tensor
// memory, so that the epilogue of a tile runs under the MMAs of the next one:
//   warp 0     producer: TMA tensor loads of the x tile [128 tokens x KT] and of the three factor
//              tiles [W x KT] per KT-wide slice of d_model, through a ring of shared-memory stages
//   warp 1     MMA issuer
//   warps 2-15, once an accumulator is complete (warps 0 and 1 join them when the CTA has one tile): the epilogue.
//              A warp reads the tensor-memory lanes of its quarter (warp % 4: 32 tokens, one per lane) and takes
//              *units* from a counter of that quarter: a unit is the 16 real columns 16u .. 16u+15 with their 16
//              imaginary partners R + 16u .., i.e. two whole NVFP4 blocks, or one block of the unrotated rest.
//              Rotation by the token's phasors, NVFP4 quantisation with the reference's rounding and the store
//              into the token's cache page all happen in registers, straight from tensor memory. (R not a
//              multiple of 16: a real block and its partners do not line up; then a CTA has one tile and four
//              warps take a token row each through shared memory, which the stages no longer need.)
// Every wait is bounded; a give-up is recorded in `status` and the roles unwind.
#include "pkv_common.cuh"
#include "pkv_tcgen05.cuh"

#include <cudaTypedefs.h>

namespace {

using namespace pkv;

constexpr int TM_TOK = 128;                  // tokens per CTA
constexpr int NTHREADS = 16 * 32;
constexpr int NST_MAX = 4;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

// d_model slice per stage. What bounds the main loop is how long a slice takes to arrive, so a CTA keeps all of its
// shared memory in flight; at W = 256 four slices of 32 (64-byte rows, 64-byte swizzle) do that better than two of
// 64 (measured 77 against 86 us for 16384 tokens), at W = 128 three slices of 64 (128-byte rows and swizzle) beat
// seven of 32 (46 against 53 us: a slice of 32 is only 0.2 us of MMA work).
template <int WP>
struct WCfg {
    static constexpr int KT = WP == 256 ? 32 : 64;
    static constexpr uint64_t SWZ = KT == 64 ? SWZ_128B : SWZ_64B;
    static constexpr int SBO = 8 * KT * 2;                         // 8 rows of a swizzle atom
    static constexpr int X_TILE = TM_TOK * KT * 2;
    static constexpr int B_TILE = WP * KT * 2;                     // one bf16 term of the factor slice
    static constexpr int STAGE = X_TILE + 3 * B_TILE;
    static constexpr int FIT = (232448 - 1024) / STAGE;
    static constexpr int NST = FIT > NST_MAX ? NST_MAX : FIT;
    static constexpr int ROWS = TM_TOK * (WP + 1) * 4;              // epilogue rows (R % 16 != 0), reusing the stages
    static constexpr int BODY = NST * STAGE > ROWS ? NST * STAGE : ROWS;
    static constexpr int SMEM = BODY + 256;
    static_assert(STAGE % 1024 == 0 && NST >= 2 && SMEM <= 232448, "stages");
};

struct WExtra {
    uint64_t full[NST_MAX], empty[NST_MAX];
    uint64_t acc_full[2], acc_empty[2];      // accumulator b complete (MMA issuer -> epilogue) / read out (14 epilogue warps -> MMA issuer)
    int next_unit[2][4];                     // epilogue units handed out, per accumulator and lane quarter
    uint32_t tmem_base;
    volatile int abort_flag;
};
constexpr int EPI_WARPS = NTHREADS / 32 - 2;

// store one quantised block of a token row
template <int WP>
__device__ __forceinline__ void store_block(uint8_t* page, uint32_t pr_row, int j, int codes_bytes, const float (&v)[16], float second,
                                            bool round_up) {
    uint8_t sb;
    const uint2 packed = pkv_quantize_block16(v, second, sb, round_up);
    *reinterpret_cast<uint2*>(page + pkv_code_offset(pr_row, j * 8, WP / 2)) = packed;
    page[codes_bytes + pkv_scale_offset(pr_row, j)] = sb;
}

__device__ __forceinline__ bool wwait(uint64_t* bar, uint32_t parity, WExtra* X, int32_t* status, int where) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && X->abort_flag) return false;
    }
    X->abort_flag = 1;
    if (status) { atomicExch(&status[0], 1); atomicExch(&status[1], where); }
    return false;
}

template <int WP>
__global__ void __launch_bounds__(NTHREADS, 1) pkv_cache_write_tc_kernel(
    const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap bmap, int n_tokens, int n_tiles, int D, int W, int R,
    const int32_t* __restrict__ positions, const float2* __restrict__ phasors, int h2, const int32_t* __restrict__ slots,
    const int32_t* __restrict__ freq, const double* __restrict__ inv_freq, float attn_scale, const pkv_second second, int scale_up,
    uint8_t* __restrict__ latent, int n_pages, float* __restrict__ latent_out, int32_t* __restrict__ status) {
    using C = WCfg<WP>;
    extern __shared__ __align__(1024) uint8_t smem[];
    WExtra* X = reinterpret_cast<WExtra*>(smem + C::BODY);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int KT = C::KT, X_TILE = C::X_TILE;
    const int n_kt = D / KT;
    const int my_tiles = ((int)blockIdx.x < n_tiles) ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    pkv_grid_launch_dependents();
    if (tid == 0) {
        for (int s = 0; s < NST_MAX; ++s) { mbar_init(&X->full[s], 1); mbar_init(&X->empty[s], 1); }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&X->acc_full[b], 1);
            mbar_init(&X->acc_empty[b], EPI_WARPS);
            for (int q = 0; q < 4; ++q) X->next_unit[b][q] = 0;
        }
        X->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(&X->tmem_base, 2 * WP);         // two accumulators of WP columns
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = X->tmem_base;
    const uint32_t sbase = smem_u32(smem);
    pkv_grid_wait();                               // x may be the output of the kernel before

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&xmap);
            tma_prefetch_desc(&bmap);
            int c = 0;                                                             // slices asked for so far, over all tiles
            bool ok = true;
            for (int it = 0; it < my_tiles && ok; ++it) {
                const int tok0 = ((int)blockIdx.x + it * (int)gridDim.x) * TM_TOK;
                for (int kt = 0; kt < n_kt; ++kt, ++c) {
                    const int s = c % C::NST;
                    if (c >= C::NST && !wwait(&X->empty[s], ((c / C::NST) - 1) & 1, X, status, 60)) { ok = false; break; }
                    uint8_t* st = smem + s * C::STAGE;
                    mbar_arrive_expect_tx(&X->full[s], C::STAGE);
                    tma_load_2d(st, &xmap, kt * KT, tok0, &X->full[s]);           // rows past n_tokens arrive as zeros
                    for (int t = 0; t < 3; ++t) tma_load_2d(st + X_TILE + t * C::B_TILE, &bmap, kt * KT, t * WP, &X->full[s]);
                }
            }
            if (X->abort_flag)                                                     // let copies in flight land before leaving
                for (int k = max(0, c - C::NST); k < c; ++k) mbar_wait(&X->full[k % C::NST], (k / C::NST) & 1, 1u << 16);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(TM_TOK, WP, false, false);
            bool ok = true;
            int c = 0;
            for (int it = 0; it < my_tiles && ok; ++it) {
                const int b = it & 1;
                if (it >= 2) {                                                     // accumulator b has been read out (tile it - 2)
                    ok = wwait(&X->acc_empty[b], ((it >> 1) - 1) & 1, X, status, 63);
                    if (!ok) break;
                    for (int q = 0; q < 4; ++q) X->next_unit[b][q] = 0;
                    __threadfence_block();
                    tc_fence_after_sync();
                }
                for (int kt = 0; kt < n_kt && ok; ++kt, ++c) {
                    const int s = c % C::NST;
                    ok = wwait(&X->full[s], (c / C::NST) & 1, X, status, 61);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t xa = sbase + s * C::STAGE;
#pragma unroll
                    for (int t = 0; t < 3; ++t)
#pragma unroll
                        for (int k = 0; k < KT / 16; ++k)
                            mma_bf16(tb + b * WP, smem_desc(xa + k * 32, 0, C::SBO, C::SWZ),
                                     smem_desc(xa + X_TILE + t * C::B_TILE + k * 32, 0, C::SBO, C::SWZ), idesc, (kt | t | k) != 0);
                    tc_commit(&X->empty[s]);
                }
                if (ok) tc_commit(&X->acc_full[b]);
            }
        }
    }
    __syncwarp();

    // ================================================================== epilogue
    // warps 2 .. 15 take every tile of the CTA; warps 0 and 1, done with their own loops by then, help when the CTA has
    // a single tile (with several, a wait for the last tile alone could not tell its barrier phase from an earlier one)
    const int it_first = warp >= 2 ? 0 : (my_tiles == 1 ? 0 : my_tiles);
    for (int it = it_first; it < my_tiles; ++it) {
        const int acc = it & 1;
        const int tok0 = ((int)blockIdx.x + it * (int)gridDim.x) * TM_TOK;
        const int quad = warp & 3;
        const int rowi = quad * 32 + lane;
        const int tok = tok0 + rowi;
        const bool ok = __all_sync(0xffffffffu, wwait(&X->acc_full[acc], (it >> 1) & 1, X, status, 62));
        if (!ok) break;
        const uint32_t tl = tb + acc * WP + ((uint32_t)(quad * 32) << 16);
        const bool live = ok && tok < n_tokens;
        const int slot = live && latent ? slots[tok] : -1;
        const bool paged = slot >= 0 && slot < n_pages * PKV_PAGE_TOKENS;
        uint8_t* page = paged ? latent + (size_t)(slot / PKV_PAGE_TOKENS) * pkv_page_bytes(W) : nullptr;
        const uint32_t pr_row = paged ? slot % PKV_PAGE_TOKENS : 0;
        const int codes_bytes = pkv_codes_bytes(W);
        constexpr int NB = WP / 16;
        if (ok) tc_fence_after_sync();
        if (ok && (R & 15) == 0) {
            // units: R / 16 rotated pairs of blocks (u, R / 16 + u), then the blocks behind 2R one by one
            const int n_pair = R >> 4, n_unit = n_pair + (NB - 2 * n_pair);
            const double pos = live && !phasors ? (double)positions[tok] : 0.0;
            for (;;) {
                int u = 0;
                if (lane == 0) u = atomicAdd(&X->next_unit[acc][quad], 1);
                u = __shfl_sync(0xffffffffu, u, 0);
                if (u >= n_unit) break;
                if (u < n_pair) {
                    uint32_t ra[16], rb[16];
                    tmem_ld16(tl + 16 * u, ra);                         // whole warp: tensor-memory loads are warp-wide
                    tmem_ld16(tl + R + 16 * u, rb);
                    tmem_ld_wait();
                    if (live) {
                        float re[16], im[16];
                        int f_prev = -1;
                        float pr = 1.0f, pi = 0.0f;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int f = freq[16 * u + i];
                            if (f != f_prev) {                         // attn_scale * e^{i * position * inv_freq[f]}
                                if (phasors) {
                                    const float2 p = phasors[(size_t)tok * h2 + f];
                                    pr = p.x; pi = p.y;
                                } else {
                                    double sn, cs;
                                    sincos(pos * inv_freq[f], &sn, &cs);
                                    pr = (float)((double)attn_scale * cs); pi = (float)((double)attn_scale * sn);
                                }
                                f_prev = f;
                            }
                            const float a = __uint_as_float(ra[i]), b = __uint_as_float(rb[i]);
                            re[i] = __fsub_rn(__fmul_rn(a, pr), __fmul_rn(b, pi));
                            im[i] = __fadd_rn(__fmul_rn(a, pi), __fmul_rn(b, pr));
                        }
                        if (latent_out) {
                            float4* o = reinterpret_cast<float4*>(latent_out + (size_t)tok * W + 16 * u);
                            float4* o2 = reinterpret_cast<float4*>(latent_out + (size_t)tok * W + R + 16 * u);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                o[i] = make_float4(re[4 * i], re[4 * i + 1], re[4 * i + 2], re[4 * i + 3]);
                                o2[i] = make_float4(im[4 * i], im[4 * i + 1], im[4 * i + 2], im[4 * i + 3]);
                            }
                        }
                        if (paged) {
                            store_block<WP>(page, pr_row, u, codes_bytes, re, second.of(u), scale_up != 0);
                            store_block<WP>(page, pr_row, n_pair + u, codes_bytes, im, second.of(n_pair + u), scale_up != 0);
                        }
                    }
                } else {
                    const int j = 2 * n_pair + (u - n_pair);
                    uint32_t ra[16];
                    tmem_ld16(tl + 16 * j, ra);
                    tmem_ld_wait();
                    if (live) {
                        float v[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(ra[i]);
                        if (latent_out && 16 * j < W) {                // W is a multiple of 16: a block is all row or all padding
                            float4* o = reinterpret_cast<float4*>(latent_out + (size_t)tok * W + 16 * j);
#pragma unroll
                            for (int i = 0; i < 4; ++i) o[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                        }
                        if (paged) store_block<WP>(page, pr_row, j, codes_bytes, v, second.of(j), scale_up != 0);
                    }
                }
            }
        } else if (ok && warp >= 2 && warp < 6) {
            // real blocks and their imaginary partners do not line up: a thread takes a whole token row through shared
            // memory (the CTA has this one tile: the launch makes the grid as large as the tile count)
            float* row = reinterpret_cast<float*>(smem) + (size_t)rowi * (WP + 1);     // the stages are idle now
#pragma unroll 1
            for (int c0 = 0; c0 < WP; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tl + c0, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) row[c0 + i] = __uint_as_float(r[i]);
            }
            if (live) {
                const double pos = phasors ? 0.0 : (double)positions[tok];
                int f_prev = -1;
                float pr = 1.0f, pi = 0.0f;
                for (int k = 0; k < R; ++k) {
                    const int f = freq[k];
                    if (f != f_prev) {
                        if (phasors) {
                            const float2 p = phasors[(size_t)tok * h2 + f];
                            pr = p.x; pi = p.y;
                        } else {
                            double sn, cs;
                            sincos(pos * inv_freq[f], &sn, &cs);
                            pr = (float)((double)attn_scale * cs); pi = (float)((double)attn_scale * sn);
                        }
                        f_prev = f;
                    }
                    const float a = row[k], b = row[R + k];
                    row[k] = __fsub_rn(__fmul_rn(a, pr), __fmul_rn(b, pi));
                    row[R + k] = __fadd_rn(__fmul_rn(a, pi), __fmul_rn(b, pr));
                }
                if (latent_out)
                    for (int c = 0; c < W; ++c) latent_out[(size_t)tok * W + c] = row[c];
                if (paged) {
#pragma unroll 1
                    for (int j = 0; j < NB; ++j) {
                        float v[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = row[j * 16 + i];
                        store_block<WP>(page, pr_row, j, codes_bytes, v, second.of(j), scale_up != 0);
                    }
                }
            }
        }
        // this warp has read what it needs of the accumulator: the issuer may reuse it for the tile after next
        tc_fence_before_sync();
        __syncwarp();
        if (warp >= 2 && lane == 0) mbar_arrive(&X->acc_empty[acc]);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tb, 2 * WP);
}

PFN_cuTensorMapEncodeTiled_v12000 g_encode_w = nullptr;

int encode_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
    if (!g_encode_w) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        PKV_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return PKV_ERR_CUDA;
        g_encode_w = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {box_cols, box_rows};                  // a box row is one swizzle row: 64 or 128 bytes
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode_w(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { g_pkv_last_cuda_error = (int)r; return PKV_ERR_CUDA; }
    return PKV_OK;
}

template <int WP>
int launch_write_tc(const CUtensorMap& xmap, const CUtensorMap& bmap, const pkv_layer_t* L, const pkv_cache_t* C,
                    const int32_t* pos, const float* ph, const int32_t* slots, int n, float* latent_out, int32_t* status,
                    cudaStream_t st) {
    auto kern = pkv_cache_write_tc_kernel<WP>;
    constexpr int smem = WCfg<WP>::SMEM;
    static pkv_attr_flags attr;                          // per instantiation and device
    PKV_CUDA_TRY(pkv_set_max_smem(kern, smem, attr));
    // one CTA per SM at most, each taking every gridDim-th tile; a layer whose real and imaginary blocks do not line up
    // needs the stages for its epilogue and gets a CTA per tile
    const int n_tiles = (n + TM_TOK - 1) / TM_TOK;
    int grid = n_tiles;
    if ((L->R & 15) == 0) {
        int dev = 0, sms = 0;
        PKV_CUDA_TRY(cudaGetDevice(&dev));
        PKV_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (sms > 0 && grid > sms) grid = sms;
    }
    PKV_CUDA_TRY(pkv_launch_chained(kern, dim3(grid), dim3(NTHREADS), smem, st, xmap, bmap, n, n_tiles, L->d_model,
                                    2 * L->R + L->R_s, L->R, pos, (const float2*)ph, L->head_dim / 2, slots, L->freq_dev,
                                    L->inv_freq_dev, L->attn_scale, pkv_second_of(L), pkv_scale_round_up_mode(),
                                    C ? C->latent_dev : nullptr, C ? C->n_pages : 0, latent_out, status));
    return PKV_OK;
}

}  // namespace

// bf16 x, three-term bf16 factors present, d_model a multiple of 64: the tensor-core write can run
bool pkv_write_tc_usable(const pkv_layer_t* L, int32_t x_dtype, const void* x_dev) {
    return x_dtype == PKV_BF16 && L->Bw_bf16x3_dev && (L->d_model % 64) == 0 && !(((uintptr_t)x_dev) & 15u) &&
           !(((uintptr_t)L->Bw_bf16x3_dev) & 15u);
}

int pkv_write_tc_launch(const pkv_layer_t* L, const pkv_cache_t* C, const void* x_dev, const int32_t* pos, const float* ph,
                        const int32_t* slots, int n, float* latent_out, int32_t* status, cudaStream_t st) {
    const int W = 2 * L->R + L->R_s, WP = pkv_padded_width(W);
    CUtensorMap xmap, bmap;
    const uint32_t kt = WP == 128 ? WCfg<128>::KT : WCfg<256>::KT;
    int rc = encode_2d_bf16(&xmap, x_dev, (uint64_t)n, (uint64_t)L->d_model, TM_TOK, kt);
    if (rc) return rc;
    rc = encode_2d_bf16(&bmap, L->Bw_bf16x3_dev, (uint64_t)3 * WP, (uint64_t)L->d_model, (uint32_t)WP, kt);
    if (rc) return rc;
    return WP == 128 ? launch_write_tc<128>(xmap, bmap, L, C, pos, ph, slots, n, latent_out, status, st)
                     : launch_write_tc<256>(xmap, bmap, L, C, pos, ph, slots, n, latent_out, status, st);
}
