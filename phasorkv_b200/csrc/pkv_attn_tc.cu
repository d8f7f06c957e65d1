// Decode attention on the NVFP4 latent cache with 5th-generation tensor cores.
//
// One CTA = one (sequence, token split). Seven warps, each with one job:
//   warp 0     K producer : bulk-copies latent pages (codes + scales, already in operand layout) to smem
//   warp 1     V producer : TMA tensor loads of the bf16 V page, one kv head (128 tokens x 128 dims) per stage
//   warp 2     MMA issuer : S = C . Q'^T as block-scaled NVFP4 tcgen05.mma (tokens on M = 128, the 32 query
//                           heads on N; the four NVFP4 residual terms of the query are four passes over
//                           the same cache tile that accumulate in TMEM), scale factors copied
//                           smem -> TMEM with tcgen05.cp; O^T += V^T . P^T as bf16 tcgen05.mma per kv head
//   warps 3-6  softmax    : one token row (TMEM lane) per thread; online base-2 softmax whose reference
//                           maximum only moves when a tile exceeds it by 2^8, P to smem as bf16, and the
//                           rare rescale of the O accumulators in TMEM
// Stages are handed over through mbarriers; every wait is bounded and a give-up is recorded in
// `status` while all roles unwind, free TMEM and return.
#include "pkv_common.cuh"
#include "pkv_tcgen05.cuh"

#include <cudaTypedefs.h>
#include <cstdlib>

int pkv_check_layer(const pkv_layer_t* L);

namespace {

using namespace pkv;

constexpr int NQ = 32, DH = 128;
constexpr int NK_STAGES = 2, NV_STAGES = 4;
constexpr int NK_MAX = 8;              // K stages in scores-only mode (they take over the idle V stages)
constexpr int V_STAGE_BYTES = PKV_PAGE_TOKENS * DH * 2;        // one kv head of one page
constexpr int P_BYTES = 2 * PKV_PAGE_TOKENS * NQ * 2;          // softmax weights of a page as hi + lo bf16 (2^-17 relative)
constexpr int NTHREADS = 7 * 32;
constexpr float RESCALE_THRESHOLD = 8.0f;                      // in base-2 logits
constexpr uint32_t WAIT_LIMIT = 1u << 22;

// tensor memory columns
constexpr int NSB = 4;                // score buffers: pages whose S = C.Q'^T may be in flight between MMA and softmax
constexpr uint32_t TM_S = 0;          // NSB x 32 : scores (tokens x heads)
constexpr uint32_t TM_O = 128;        // n_kv x 32 : O^T accumulators, 16 columns for the hi and 16 for the lo weights
constexpr uint32_t TM_SFA = 384;      // NSB x 16 : cache scale factors, one set per score buffer
constexpr uint32_t TM_SFB = 448;      // 4 x 16 : query scale factors, a 4-column group per (residual term, K step)
constexpr uint32_t TM_COLS = 512;

template <int WP>
struct Cfg {
    static constexpr int RB = WP / 2;                          // code bytes per row
    static constexpr int KB = WP / 64;                         // K = 64 MMA steps
    static constexpr int CODES = PKV_PAGE_TOKENS * RB;
    static constexpr int PAGE = CODES + KB * 512;
    static constexpr int SFQ = PKV_QUERY_TERMS * KB * 512;     // query scale blocks, one per (term, K step)
    static constexpr int QBLOB = CODES + SFQ + 512;
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = ((QBLOB + 1023) / 1024) * 1024;
    static constexpr int V_OFF = K_OFF + NK_STAGES * PAGE;
    static constexpr int P_OFF = V_OFF + NV_STAGES * V_STAGE_BYTES;
    static constexpr int X_OFF = P_OFF + 2 * P_BYTES;          // barriers and small arrays
    static constexpr int SMEM = X_OFF + 2048;
    static constexpr uint64_t SWZ = RB == 128 ? SWZ_128B : SWZ_64B;
    static constexpr uint32_t SBO = 8 * RB;
};

struct Extra {                       // lives at X_OFF
    uint64_t q_full, k_full[NK_MAX], k_empty[NK_MAX], v_full[NV_STAGES], v_empty[NV_STAGES];
    uint64_t s_full[NSB], s_empty[NSB], p_full[2], pv_done[2];
    uint64_t sm_bar;                 // rendezvous of the 128 softmax threads (bounded, unlike bar.sync)
    uint32_t tmem_base;
    volatile int abort_flag;
    float wmax[2][4][NQ];
    int wflag[2][4];
    float lsum[4][NQ];
};

__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, const uint32_t (&r)[4]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                 "r"(r[3]) : "memory");
}

// order-preserving map float -> uint so that an integer warp reduction gives the float maximum
__device__ __forceinline__ uint32_t f2ord(float f) { uint32_t b = __float_as_uint(f); return b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u); }
__device__ __forceinline__ float ord2f(uint32_t u) { return __uint_as_float(u ^ ((u >> 31) ? 0x80000000u : 0xFFFFFFFFu)); }

// bounded wait that also gives up when another role has already given up
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, Extra* X, int32_t* status, int where) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && X->abort_flag) return false;
    }
    X->abort_flag = 1;
    if (status) { atomicExch(&status[0], 1); atomicExch(&status[1], where); }
    return false;
}

template <int WP, int REP>
__global__ void __launch_bounds__(NTHREADS, 1) pkv_attn_tc_kernel(
    const __grid_constant__ CUtensorMap vmap, const uint8_t* __restrict__ qop, long qop_stride,
    const uint8_t* __restrict__ latent, const int32_t* __restrict__ page_table, int max_pages,
    const int32_t* __restrict__ seqlens, int n_split, int n_pages_pool, float col_scale, float inv_logit_scale,
    uint32_t flags, float* __restrict__ partials, float* __restrict__ scores_out, long scores_stride,
    int32_t* __restrict__ status) {
    using C = Cfg<WP>;
    constexpr int NKV = NQ / REP;                 // kv heads
    constexpr int G16 = 16 / REP;                 // kv heads per 16-head group of P rows
    extern __shared__ __align__(1024) uint8_t smem[];
    Extra* X = reinterpret_cast<Extra*>(smem + C::X_OFF);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, b = blockIdx.y;
    pkv_grid_launch_dependents();

    // ---- prologue that touches no global memory: barriers, tensor memory
    if (tid == 0) {
        mbar_init(&X->q_full, 1);
        for (int s = 0; s < NK_MAX; ++s) { mbar_init(&X->k_full[s], 1); mbar_init(&X->k_empty[s], 1); }
        for (int s = 0; s < NV_STAGES; ++s) { mbar_init(&X->v_full[s], 1); mbar_init(&X->v_empty[s], 1); }
        for (int s = 0; s < NSB; ++s) { mbar_init(&X->s_full[s], 1); mbar_init(&X->s_empty[s], 128); }
        for (int s = 0; s < 2; ++s) { mbar_init(&X->p_full[s], 128); mbar_init(&X->pv_done[s], 1); }
        mbar_init(&X->sm_bar, 128);
        X->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 2) tmem_alloc(&X->tmem_base, TM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = X->tmem_base;
    const uint32_t sbase = smem_u32(smem);

    // Normally everything waits here for the kernel launched before this one. With PKV_ATTN_EARLY_STREAM the
    // caller vouches that that kernel only produces the query operand (it is pkv_absorb): the cache, the
    // page table and the lengths are then already final, the producers start streaming pages at once and
    // only the load of the query operand waits.
    const bool early = (flags & PKV_ATTN_EARLY_STREAM) != 0;
    if (!early) pkv_grid_wait();

    const int T = seqlens[b];
    const int npages = min((T + PKV_PAGE_TOKENS - 1) / PKV_PAGE_TOKENS, max_pages);
    const int pps = (npages + n_split - 1) / n_split;
    const int p_lo = split * pps, p_hi = min(npages, p_lo + pps);
    const int P = p_hi - p_lo;
    const bool with_v = !(flags & PKV_ATTN_SCORES_ONLY);
    const int nks = with_v ? NK_STAGES : NK_MAX;      // without V its stages hold more latent pages in flight
    float* part = partials + ((size_t)b * n_split + split) * NQ * (DH + 2);

    if (P <= 0) {                                  // this split has no token: the neutral partial
        for (int i = tid; i < NQ * (DH + 2); i += NTHREADS) {
            int c = i % (DH + 2);
            part[i] = c == DH ? -INFINITY : 0.0f;
        }
        tc_fence_before_sync();
        __syncthreads();
        if (warp == 2) tmem_dealloc(tb, TM_COLS);
        return;
    }

    if (warp == 0) {
        // ================================================================== K producer
        if (lane == 0) {
            int issued = 0;
            bool q_sent = false;
            for (int i = 0; i <= P; ++i) {
                if (!q_sent && (!early || i == min(P, nks))) {       // early mode: first fill the latent stages
                    if (early) pkv_grid_wait();
                    mbar_arrive_expect_tx(&X->q_full, C::QBLOB);
                    bulk_g2s(smem + C::Q_OFF, qop + (size_t)b * qop_stride, C::QBLOB, &X->q_full);
                    q_sent = true;
                }
                if (i == P) break;
                const int s = i % nks;
                if (i >= nks && !wait_or_abort(&X->k_empty[s], ((i / nks) - 1) & 1, X, status, 10)) break;
                int pidx = page_table[(size_t)b * max_pages + p_lo + i];
                if (pidx < 0 || pidx >= n_pages_pool) {              // never dereference a bad page index
                    X->abort_flag = 1;
                    if (status) { atomicExch(&status[0], 2); atomicExch(&status[1], p_lo + i); }
                    break;
                }
                mbar_arrive_expect_tx(&X->k_full[s], C::PAGE);
                bulk_g2s(smem + C::K_OFF + s * C::PAGE, latent + (size_t)pidx * C::PAGE, C::PAGE, &X->k_full[s]);
                issued = i + 1;
            }
            if (X->abort_flag) {                                     // let copies in flight land before leaving
                mbar_wait(&X->q_full, 0, 1u << 16);
                for (int i = max(0, issued - nks); i < issued; ++i)
                    mbar_wait(&X->k_full[i % nks], (i / nks) & 1, 1u << 16);
            }
        }
    } else if (warp == 1) {
        // ================================================================== V producer
        if (lane == 0 && with_v) {
            tma_prefetch_desc(&vmap);
            int issued = 0;
            bool ok = true;
            for (int i = 0; i < P && ok; ++i) {
                int pidx = page_table[(size_t)b * max_pages + p_lo + i];
                if (pidx < 0 || pidx >= n_pages_pool) break;         // the K producer reports it
                for (int g = 0; g < NKV; ++g) {
                    const int j = i * NKV + g, s = j % NV_STAGES;
                    if (j >= NV_STAGES && !wait_or_abort(&X->v_empty[s], ((j / NV_STAGES) - 1) & 1, X, status, 20)) { ok = false; break; }
                    uint8_t* dst = smem + C::V_OFF + s * V_STAGE_BYTES;
                    mbar_arrive_expect_tx(&X->v_full[s], V_STAGE_BYTES);
                    tma_load_2d(dst, &vmap, g * DH, pidx * PKV_PAGE_TOKENS, &X->v_full[s]);
                    tma_load_2d(dst + V_STAGE_BYTES / 2, &vmap, g * DH + 64, pidx * PKV_PAGE_TOKENS, &X->v_full[s]);
                    issued = j + 1;
                }
            }
            if (X->abort_flag)
                for (int j = max(0, issued - NV_STAGES); j < issued; ++j)
                    mbar_wait(&X->v_full[j % NV_STAGES], (j / NV_STAGES) & 1, 1u << 16);
        }
    } else if (warp == 2) {
        // ================================================================== MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_nvfp4(128, NQ);
            constexpr uint32_t idesc_o = idesc_bf16(128, 32, true, false);
            bool ok = wait_or_abort(&X->q_full, 0, X, status, 30);
            if (ok) {
                tc_fence_after_sync();
                for (int blk = 0; blk < PKV_QUERY_TERMS * C::KB; ++blk)
                    tmem_cp_32x128b_warpx4(tb + TM_SFB + 4 * blk,
                                           smem_desc(sbase + C::Q_OFF + C::CODES + blk * 512, 0, 128, SWZ_NONE));
            }
            auto do_pv = [&](int i) -> bool {
                const int pb = i & 1;
                if (!wait_or_abort(&X->p_full[pb], (i >> 1) & 1, X, status, 31)) return false;
                tc_fence_after_sync();
                for (int g = 0; g < NKV; ++g) {
                    const int j = i * NKV + g, s = j % NV_STAGES;
                    if (!wait_or_abort(&X->v_full[s], (j / NV_STAGES) & 1, X, status, 32)) return false;
                    tc_fence_after_sync();
                    const uint32_t va = sbase + C::V_OFF + s * V_STAGE_BYTES;
                    // B operand: 32 rows = the hi weights of this kv head's 16-head group, then their lo parts
                    const uint32_t pa = sbase + C::P_OFF + pb * P_BYTES + (g / G16) * 512;
#pragma unroll
                    for (int k = 0; k < PKV_PAGE_TOKENS / 16; ++k)
                        mma_bf16(tb + TM_O + 32 * g, smem_desc(va + k * 2048, V_STAGE_BYTES / 2, 1024, SWZ_128B),
                                 smem_desc(pa + k * 2048, 1024, 128, SWZ_NONE), idesc_o, !(i == 0 && k == 0));
                    tc_commit(&X->v_empty[s]);
                }
                tc_commit(&X->pv_done[pb]);
                return true;
            };
            for (int i = 0; i < P && ok; ++i) {
                const int s = i % nks, buf = i % NSB;
                ok = wait_or_abort(&X->k_full[s], (i / nks) & 1, X, status, 33);
                if (ok && i >= NSB) ok = wait_or_abort(&X->s_empty[buf], ((i / NSB) - 1) & 1, X, status, 34);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t ka = sbase + C::K_OFF + s * C::PAGE;
                for (int k = 0; k < C::KB; ++k)
                    tmem_cp_32x128b_warpx4(tb + TM_SFA + 16 * buf + 4 * k, smem_desc(ka + C::CODES + k * 512, 0, 128, SWZ_NONE));
                // the four residual terms of the query (rows 32 t .. 32 t + 31 of its tile) all accumulate into
                // the same 32 columns: the tensor core adds them up, the tile of cache codes is reused as is
                for (int t = 0; t < PKV_QUERY_TERMS; ++t)
                    for (int k = 0; k < C::KB; ++k)
                        mma_nvfp4(tb + TM_S + 32 * buf, smem_desc(ka + k * 32, 0, C::SBO, C::SWZ),
                                  smem_desc(sbase + C::Q_OFF + t * NQ * C::RB + k * 32, 0, C::SBO, C::SWZ), idesc_s,
                                  tb + TM_SFA + 16 * buf + 4 * k, tb + TM_SFB + 4 * (t * C::KB + k), (t | k) != 0);
                tc_commit(&X->k_empty[s]);
                tc_commit(&X->s_full[buf]);
                if (with_v && i >= 1) ok = do_pv(i - 1);
            }
            if (ok && with_v) do_pv(P - 1);
        }
    } else {
        // ================================================================== softmax (128 threads, one token row each)
        const int quad = warp & 3;                          // TMEM lane quadrant this warp may access
        const int row = quad * 32 + lane;
        const uint32_t tl = tb + ((uint32_t)(quad * 32) << 16);
        const float* rs = reinterpret_cast<const float*>(smem + C::Q_OFF + C::CODES + C::SFQ);     // [head] tensor scale of the query operand
        // waits are made warp-uniform: the warp-collective instructions below need all 32 lanes
        auto wait_all = [&](uint64_t* bar, uint32_t parity, int where) -> bool {
            return __all_sync(0xffffffffu, wait_or_abort(bar, parity, X, status, where));
        };
        int sync_phase = 0;
        auto softmax_sync = [&]() -> bool {                 // all 128 softmax threads meet here
            mbar_arrive(&X->sm_bar);
            return wait_all(&X->sm_bar, (sync_phase++) & 1, 45);
        };
        // Per head (all kept in registers, identical in every thread that shares statistics): the
        // column scale that turns the MMA result into a base-2 logit, the reference maximum, and
        // this thread's share of the sum of 2^(s - m).
        float cs[NQ], m[NQ], l[NQ];
        bool ok = wait_all(&X->q_full, 0, 40);
#pragma unroll
        for (int h = 0; h < NQ; ++h) { cs[h] = ok ? rs[h] * col_scale : 0.0f; m[h] = -INFINITY; l[h] = 0.0f; }
        for (int i = 0; i < P && ok; ++i) {
            const int sb = i % NSB;                         // score buffer
            const int buf = i & 1;                          // P buffer and exchange slots
            ok = wait_all(&X->s_full[sb], (i / NSB) & 1, 41);
            if (!ok) break;
            tc_fence_after_sync();
            float s[NQ];
            {
                uint32_t r[32];
                tmem_ld32(tl + TM_S + 32 * sb, r);
                tmem_ld_wait();
                tc_fence_before_sync();
                mbar_arrive(&X->s_empty[sb]);               // the MMA warp may overwrite this S buffer
#pragma unroll
                for (int h = 0; h < NQ; ++h) s[h] = __uint_as_float(r[h]) * cs[h];
            }
            const int token = (p_lo + i) * PKV_PAGE_TOKENS + row;
            const bool valid = token < T;
            if (scores_out && valid) {
#pragma unroll
                for (int h = 0; h < NQ; ++h) scores_out[((size_t)b * NQ + h) * scores_stride + token] = s[h] * inv_logit_scale;
            }
            // ---- does any head of any row outgrow its reference maximum by more than the threshold?
            float exc = -INFINITY;
#pragma unroll
            for (int h = 0; h < NQ; ++h) {
                if (!valid) s[h] = -INFINITY;
                exc = fmaxf(exc, s[h] - m[h]);              // +inf while the head has no reference yet
            }
            bool grow = __any_sync(0xffffffffu, exc > RESCALE_THRESHOLD);
            if (with_v) {                                   // P.V needs one reference per head for all 128 rows
                if (lane == 0) X->wflag[buf][quad] = grow ? 1 : 0;
                ok = softmax_sync();
                if (!ok) break;
                grow = (X->wflag[buf][0] | X->wflag[buf][1] | X->wflag[buf][2] | X->wflag[buf][3]) != 0;
            }                                               // scores only: every warp keeps its own statistics
            if (grow) {
                // exact tile maximum per head: warp reduction, then (with V) across the four warps
                float wm = -INFINITY;
#pragma unroll
                for (int h = 0; h < NQ; ++h) {
                    const uint32_t red = __reduce_max_sync(0xffffffffu, f2ord(s[h]));
                    if (lane == h) wm = ord2f(red);
                }
                float tm = wm;
                if (with_v) {
                    X->wmax[buf][quad][lane] = wm;
                    ok = softmax_sync();
                    if (!ok) break;
                    tm = fmaxf(fmaxf(X->wmax[buf][0][lane], X->wmax[buf][1][lane]),
                               fmaxf(X->wmax[buf][2][lane], X->wmax[buf][3][lane]));
                    if (i > 0) {                            // the accumulators must be at rest before they are rescaled
                        ok = wait_all(&X->pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1, 42);
                        if (!ok) break;
                        tc_fence_after_sync();
                    }
                }
                float corr[NQ];
#pragma unroll
                for (int h = 0; h < NQ; ++h) {
                    const float m_new = fmaxf(m[h], __shfl_sync(0xffffffffu, tm, h));
                    corr[h] = m[h] > -INFINITY ? exp2f(m[h] - m_new) : 1.0f;     // nothing accumulated yet: leave as is
                    m[h] = m_new;
                    l[h] *= corr[h];
                }
                if (with_v && i > 0) {
#pragma unroll
                    for (int g = 0; g < NKV; ++g) {
                        // REP query heads of kv head g: columns (g % G16) * REP .. + REP - 1 of its 16
                        const uint32_t a = tl + TM_O + 32 * g + (g % G16) * REP;
#pragma unroll
                        for (int half = 0; half < 2; ++half)                     // hi columns, then lo columns
#pragma unroll
                            for (int c0 = 0; c0 < REP; c0 += 4) {
                                uint32_t r[4];
                                tmem_ld4(a + 16 * half + c0, r);
                                tmem_ld_wait();
#pragma unroll
                                for (int c = 0; c < 4; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * corr[g * REP + c0 + c]);
                                tmem_st4(a + 16 * half + c0, r);
                            }
                    }
                    tmem_st_wait();
                    tc_fence_before_sync();
                }
            }
            // ---- probabilities relative to the reference maximum; row sums stay per thread
            if (with_v && i >= 2) {
                ok = wait_all(&X->pv_done[buf], ((i >> 1) - 1) & 1, 43);      // P buffer free again
                if (!ok) break;
            }
            // weights of token `row`, head h: 8-token group (row / 8) of 1024 bytes = per 16-head group
            // [hi heads 0-7 | hi 8-15 | lo 0-7 | lo 8-15] x (8 heads x 16 bytes), token (row % 8) inside the 16 bytes
            uint8_t* pbuf = smem + C::P_OFF + buf * P_BYTES + (row >> 3) * 1024 + (row & 7) * 2;
#pragma unroll
            for (int h = 0; h < NQ; ++h) {
                float p = exp2f(s[h] - (m[h] > -INFINITY ? m[h] : 0.0f));             // exp2(-inf) = 0 for masked rows
                if (with_v) {
                    // the weight goes to the tensor core as hi + lo bf16; the row sum is taken over exactly
                    // that value, so numerator and denominator of softmax . V carry the same rounding
                    const __nv_bfloat16 hi = __float2bfloat16(p);
                    const __nv_bfloat16 lo = __float2bfloat16(p - __bfloat162float(hi));
                    uint8_t* dst = pbuf + (h >> 4) * 512 + ((h >> 3) & 1) * 128 + (h & 7) * 16;
                    *reinterpret_cast<__nv_bfloat16*>(dst) = hi;
                    *reinterpret_cast<__nv_bfloat16*>(dst + 256) = lo;
                    p = __bfloat162float(hi) + __bfloat162float(lo);
                }
                l[h] += p;
            }
            if (with_v) {
                fence_proxy_async_smem();                   // generic-proxy writes -> visible to the tensor core
                mbar_arrive(&X->p_full[buf]);
            }
        }
        // ---- epilogue: O^T back from TMEM, row sums reduced over the 128 token rows
        if (ok && with_v) ok = wait_all(&X->pv_done[(P - 1) & 1], ((P - 1) >> 1) & 1, 44);
        if (ok) {
            tc_fence_after_sync();
            if (with_v) {
#pragma unroll
                for (int g = 0; g < NKV; ++g) {
#pragma unroll
                    for (int c0 = 0; c0 < REP; c0 += 4) {
                        uint32_t r[4], r2[4];
                        tmem_ld4(tl + TM_O + 32 * g + (g % G16) * REP + c0, r);
                        tmem_ld4(tl + TM_O + 32 * g + 16 + (g % G16) * REP + c0, r2);
                        tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            part[(g * REP + c0 + c) * (DH + 2) + row] = __uint_as_float(r[c]) + __uint_as_float(r2[c]);
                    }
                }
            } else {
                for (int h = 0; h < NQ; ++h) part[h * (DH + 2) + row] = 0.0f;
            }
            float lw = 0.0f, mw = -INFINITY;
#pragma unroll
            for (int h = 0; h < NQ; ++h) {
                float v = l[h];
#pragma unroll
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == h) { lw = v; mw = m[h]; }
            }
            X->lsum[quad][lane] = lw;
            X->wmax[0][quad][lane] = mw;                    // per warp in scores-only mode, identical otherwise
            if (softmax_sync() && quad == 0) {
                float M = -INFINITY, lt = 0.0f;
#pragma unroll
                for (int w = 0; w < 4; ++w) M = fmaxf(M, X->wmax[0][w][lane]);
#pragma unroll
                for (int w = 0; w < 4; ++w)
                    if (X->wmax[0][w][lane] > -INFINITY) lt = fmaf(X->lsum[w][lane], exp2f(X->wmax[0][w][lane] - M), lt);
                part[lane * (DH + 2) + DH] = M;
                part[lane * (DH + 2) + DH + 1] = lt;
            }
        }
    }
    // ---- teardown: everyone meets, tensor memory goes back
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tb, TM_COLS);
}

// ------------------------------------------------------------------------------------------------ host
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

int encode_v_map(CUtensorMap* map, const pkv_cache_t* C) {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        PKV_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return PKV_ERR_CUDA;
        g_encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    }
    // V pool as a 2-D bf16 tensor [n_pages * 128 tokens, n_kv * head_dim]; box = 64 dims x 128 tokens, 128-byte swizzle
    cuuint64_t dims[2] = {(cuuint64_t)C->n_kv * C->head_dim, (cuuint64_t)C->n_pages * PKV_PAGE_TOKENS};
    cuuint64_t strides[1] = {(cuuint64_t)C->n_kv * C->head_dim * 2};
    cuuint32_t box[2] = {64, PKV_PAGE_TOKENS};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C->v_dev, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { g_pkv_last_cuda_error = (int)r; return PKV_ERR_CUDA; }
    return PKV_OK;
}

template <int WP, int REP>
int launch_tc(const CUtensorMap& vmap, const pkv_layer_t* L, const pkv_cache_t* C, const uint8_t* qop, const int32_t* pt,
              int max_pages, const int32_t* seqlens, int batch, int n_split, uint32_t flags, float* partials, float* scores,
              long scores_stride, int32_t* status, cudaStream_t st) {
    auto kern = pkv_attn_tc_kernel<WP, REP>;
    constexpr int smem = Cfg<WP>::SMEM;
    static bool attr_done = false;                                  // once per instantiation
    if (!attr_done) {
        PKV_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_done = true;
    }
    const float logit_scale = PKV_LOG2E / sqrtf((float)L->head_dim);
    PKV_CUDA_TRY(pkv_launch_chained(kern, dim3(n_split, batch), dim3(NTHREADS), smem, st, vmap, qop, (long)Cfg<WP>::QBLOB,
                                    C->latent_dev, pt, max_pages, seqlens, n_split, C->n_pages, L->second * logit_scale,
                                    1.0f / logit_scale, flags, partials, scores, scores_stride, status));
    return PKV_OK;
}

}  // namespace

int pkv_attn_tc_launch(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* q_dev,
                       const int32_t* page_table_dev, int32_t max_pages, const int32_t* seqlens_dev, int32_t batch,
                       int32_t n_split, uint32_t flags, float* partials_dev, float* scores_out_dev,
                       int64_t scores_stride, int32_t* status_dev, float* out_dev, cudaStream_t stream) {
    const int rep = layer->n_q / layer->n_kv;
    if (rep != 4 && rep != 8) return PKV_ERR_UNSUPPORTED;          // P.V on tensor cores needs >= 4 query heads per kv head
    if (((uintptr_t)q_dev) & 15u) return PKV_ERR_INVALID;
    const bool with_v = !(flags & PKV_ATTN_SCORES_ONLY);
    CUtensorMap vmap;
    memset(&vmap, 0, sizeof(vmap));
    if (with_v) {
        if (((uintptr_t)cache->v_dev) & 15u) return PKV_ERR_INVALID;
        int st = encode_v_map(&vmap, cache);
        if (st) return st;
    }
    const bool wide = pkv_padded_width(cache->W) == 256;
    const uint8_t* qop = (const uint8_t*)q_dev;
    int rc;
#define PKV_TC_CASE(WP_, R_)                                                                                         \
    rc = launch_tc<WP_, R_>(vmap, layer, cache, qop, page_table_dev, max_pages, seqlens_dev, batch, n_split, flags, \
                            partials_dev, scores_out_dev, scores_stride, status_dev, stream)
    if (rep == 4) { if (wide) PKV_TC_CASE(256, 4); else PKV_TC_CASE(128, 4); }
    else { if (wide) PKV_TC_CASE(256, 8); else PKV_TC_CASE(128, 8); }
#undef PKV_TC_CASE
    if (rc == PKV_OK && out_dev) {                  // the merge of the splits: a second, latency-tuned launch
        const int64_t pw = DH + 2;
        const bool packed = (flags & PKV_ATTN_PACKED_OUT) != 0;
        rc = pkv_merge(partials_dev, (int64_t)n_split * NQ * pw, NQ * pw, n_split, batch, NQ, DH, packed ? nullptr : out_dev,
                       packed ? out_dev : nullptr, stream);
    }
    return rc;
}
