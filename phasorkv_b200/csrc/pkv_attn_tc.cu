// Decode attention on the NVFP4 latent cache with 5th-generation tensor cores.
//
// One CTA = one (sequence, token split) -- and, with one query head per kv head, one group of 8 heads.
// Seven warps, each with one job:
//   warp 0     K producer : TMA tiles of whole latent pages (codes + scales, already in operand layout);
//                           the page table is fetched 32 entries at a time by the warp
//   warp 1     V producer : TMA tensor loads of the bf16 V page, one kv head (128 tokens x 128 dims) per stage
//   warp 2     MMA issuer : S = C . Q'^T as block-scaled NVFP4 tcgen05.mma, tokens on M = 128 and on N = 128
//                           the 32 query heads x the four NVFP4 residual terms of the query (one operand
//                           tile, one pass per K step of 64), scale factors copied smem -> TMEM with
//                           tcgen05.cp; O^T += V^T . P^T as bf16 tcgen05.mma per kv head (N = 16: hi and lo
//                           halves of the weights of 8 heads)
//   warps 3-6  softmax    : one token row (TMEM lane) per thread; adds the four term columns of a head; online
//                           base-2 softmax whose reference maximum only moves when a tile exceeds it by 2^8,
//                           P to smem as hi + lo bf16, and the rare rescale of the O accumulators in TMEM
// Scores-only launches (no V) are a separate instantiation with 20 warps: warps 1-3 issue the MMAs (page i belongs to
// issuer and score buffer i % 3) and warps 4-19 are four softmax groups that split the heads of every page. Quantised V
// pages (per-token low-bit codes) have a third instantiation with 21 warps: converter warps turn code tiles into E4M3
// operands, P.V runs as kind::f8f6f4 with the token scales folded into the weights. A further instantiation absorbs
// raw queries itself (pkv_absorb_impl::body_tile) instead of loading the operand.
// Stages are handed over through mbarriers; every wait is bounded and a give-up is recorded in
// `status` while all roles unwind, free TMEM and return.
#include "pkv_absorb.cuh"
#include "pkv_common.cuh"
#include "pkv_tcgen05.cuh"

#include <cudaTypedefs.h>
#include <cstdlib>

int pkv_check_layer(const pkv_layer_t* L);

namespace {

using namespace pkv;

constexpr int NQ = 32, DH = 128;
constexpr int NK_STAGES = 2, NV_STAGES = 4;
// Quantised V pages: the codes of a (page, kv head) tile land in a ring of NVR raw stages; four converter warps turn
// each into an E4M3 operand tile (every E2M1 level is an exact E4M3 number), of which NVS_Q stages are kept. The
// per-token scales of a page (one 2 KB block for the CTA's 8 kv heads) have a ring of their own: the softmax folds
// them into the weights (E5M2, whose exponent range takes any scale), so that P.V runs as kind::f8f6f4 MMAs
// (K = 32) on exact V operands.
constexpr int NVR = 8, NVS_Q = 4;                              // a whole page of codes in flight: the raw ring is what hides HBM latency
constexpr int RAW_BYTES = PKV_PAGE_TOKENS * 64;                // codes of one tile
constexpr int VQ_STAGE_BYTES = PKV_PAGE_TOKENS * DH;           // the tile as E4M3: one 128-byte row per token
constexpr int VQ_SCALE_BYTES = 8 * PKV_PAGE_TOKENS * 2;        // bf16 scales of 8 kv heads x 128 tokens
constexpr int VQ_TERMS = 4;                                    // weights: p * scale as E5M2 terms (2^-11 of the value, any scale
                                                               // whose product with p stays inside half precision)
constexpr int NK_MAX = 8;              // K stages in scores-only mode (they take over the idle V stages)
constexpr int NV_BARS = NVS_Q > NV_STAGES ? NVS_Q : NV_STAGES;    // barrier pairs of the V operand stages, whichever instantiation has more
constexpr int V_STAGE_BYTES = PKV_PAGE_TOKENS * DH * 2;        // one kv head of one page
constexpr int P_BYTES = 2 * PKV_PAGE_TOKENS * NQ * 2;          // softmax weights of a page as hi + lo bf16 (2^-17 relative)
constexpr int NTHREADS = 7 * 32;              // with V: producers, MMA issuer, one softmax group
constexpr int NTHREADS_SCORES = 20 * 32;      // scores only: K producer, three MMA issuers (page i: issuer and score buffer i % 3), four
                                              // softmax groups that split the heads of every page
constexpr int NTHREADS_VQ = 21 * 32;          // quantised V: warps 0, 1 producers, 2 scores issuer, 3 and 20 P.V issuers (odd / even kv heads),
                                              // 4-11 softmax (two groups that split the kv heads), 12-19 converters (two per tile). Each
                                              // role's chain of dependent instructions is what bounds a page, so the roles are spread
                                              // over as many warps as the layout allows
template <bool WV, bool VQ> constexpr int n_threads() { return VQ ? NTHREADS_VQ : (WV ? NTHREADS : NTHREADS_SCORES); }
constexpr float RESCALE_THRESHOLD = 8.0f;                      // in base-2 logits
constexpr uint32_t WAIT_LIMIT = 1u << 19;     // probes of a bounded wait (a probe may itself block for microseconds): a second or two, then give up

// tensor memory columns
// Score buffers (pages in flight between MMA and softmax): two; three in scores-only mode, where buffer = page % 3 =
// issuer, so that a buffer's barriers are waited for by one issuer, phase after phase (a barrier whose phases are
// waited for by two threads in turn could be seen a whole phase early by the one that runs ahead).
constexpr int NSB_V = 2, NSB_S = 3;
constexpr uint32_t TM_S = 0;          // NSB x 128 : scores, tokens x (4 residual terms x 32 heads)
constexpr uint32_t TM_O = 256;        // with V only (then NSB = 2): n_kv x 16 O^T accumulators, 8 hi + 8 lo weight columns
constexpr uint32_t TM_SFA = 384;      // NSB x 16 : cache scale factors, one set per score buffer
constexpr uint32_t TM_SFB = 432;      // 16 per MMA issuer (three in scores-only mode): query scale factors, a 4-column group per K step
constexpr uint32_t TM_L = 464;        // quantised V: 32 columns of row sums (lane = token row, column = head), the softmax threads' own scratch
constexpr uint32_t TM_COLS = 512;

template <int WP, bool VQ = false>
struct Cfg {
    static constexpr int NVS = VQ ? NVS_Q : NV_STAGES;           // V operand stages
    static_assert(NVS <= NV_BARS, "every operand stage has its barrier pair");
    static constexpr int VSB = VQ ? VQ_STAGE_BYTES : V_STAGE_BYTES;
    static constexpr int RB = WP / 2;                          // code bytes per row
    static constexpr int KB = WP / 64;                         // K = 64 MMA steps
    static constexpr int CODES = PKV_PAGE_TOKENS * RB;
    static constexpr int PAGE = CODES + KB * 512;
    static constexpr int QBLOB = PAGE + 512;                   // query operand: a 128-row tile like a page + 32 head scales
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = ((QBLOB + 1023) / 1024) * 1024;
    static constexpr int V_OFF = K_OFF + NK_STAGES * PAGE;
    static constexpr int R_OFF = V_OFF + NVS * VSB;              // raw tiles of quantised V pages
    static constexpr int SC_OFF = R_OFF + (VQ ? NVR * RAW_BYTES : 0);      // their scale blocks, two pages
    static constexpr int P_OFF = SC_OFF + (VQ ? 2 * VQ_SCALE_BYTES : 0);
    static constexpr int X_OFF = P_OFF + 2 * P_BYTES;          // barriers and small arrays
    static constexpr int SMEM = X_OFF + 6144;
    static constexpr uint64_t SWZ = RB == 128 ? SWZ_128B : SWZ_64B;
    static constexpr uint32_t SBO = 8 * RB;
};

struct Extra {                       // lives at X_OFF
    uint64_t q_full, k_full[NK_MAX], k_empty[NK_MAX], v_full[NV_BARS], v_empty[NV_BARS];
    uint64_t s_full[NSB_S], s_empty[NSB_S], p_full[2], pv_done[2];
    uint64_t vr_full[NVR], vr_empty[NVR];                        // raw tiles of quantised V pages
    // Quantised V: the operand stages are filled by four converter warps and drained by two MMA issuers (tiles of
    // even / odd kv heads). A parity wait only tells neighbouring phases apart, so a barrier must be waited for by
    // one thread (or warps in lockstep), phase after phase, never every other phase: tile j uses operand stage j % 4 (an
    // even number: a stage always serves the same issuer) and raw stage j % 8, both always with the converter pair j % 4.
    uint64_t sc_full[2], sc_empty[2];                            // scale blocks of quantised V pages
#ifdef PKV_WAITPROF
    unsigned long long waited[64];
#endif
    uint64_t sm_bar;                 // rendezvous of the 128 softmax threads (bounded, unlike bar.sync)
    uint32_t tmem_base;
    volatile int abort_flag;
    float wmax[2][4][NQ];
    int wflag[2][8];
    float lsum[NSB_S][4][NQ];        // [0][warp quarter][head] (the leading index is left from groups that split the pages)
    float mfin[NSB_S][4][NQ];
};

constexpr int X_BYTES = 6144;
static_assert(sizeof(Extra) <= X_BYTES, "barriers and exchange arrays must fit behind the stages");
static_assert(Cfg<256, true>::SMEM <= 232448 && Cfg<256, false>::SMEM <= 232448, "shared memory of one CTA");
static_assert(Cfg<256, true>::V_OFF % 1024 == 0 && VQ_STAGE_BYTES % 1024 == 0, "swizzled operand stages start on 1024 bytes");

// order-preserving map float -> uint so that an integer warp reduction gives the float maximum
__device__ __forceinline__ uint32_t f2ord(float f) { uint32_t b = __float_as_uint(f); return b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u); }
__device__ __forceinline__ float ord2f(uint32_t u) { return __uint_as_float(u ^ ((u >> 31) ? 0x80000000u : 0xFFFFFFFFu)); }

// bounded wait that also gives up when another role has already given up
// 2^x by the special-function unit alone (2 ulp; results below 2^-126 become 0): the weights of a softmax need no more,
// and exp2f() wraps the same instruction in a range reduction of its own
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Build with -DPKV_WAITPROF to turn `scores_out` into a table of 64 counters per CTA: the cycles lane 0 of each
// warp spent in the wait with code `where` (entry 0: the CTA's cycles from entry to exit). The role that waits
// least is the one that bounds the kernel. A development aid; the library is never shipped with it.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, Extra* X, int32_t* status, int where) {
#ifdef PKV_WAITPROF
    const long long t0 = clock64();
    struct Tally {
        Extra* X; int where; long long t0;
        __device__ ~Tally() { if ((threadIdx.x & 31) == 0) atomicAdd(&X->waited[where & 63], (unsigned long long)(clock64() - t0)); }
    } tally{X, where, t0};
#endif
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && X->abort_flag) return false;
    }
    X->abort_flag = 1;
    if (status) { atomicExch(&status[0], 1); atomicExch(&status[1], where); }
    return false;
}


// Build with -DPKV_TIMELINE to turn `scores_out` into a table of time stamps, 16 per CTA (clock64 unless noted):
// 0 entry, 1 entry (globaltimer ns), 2 set-up done, 3 lengths known, 4 first page asked for, 5 query asked for,
// 6 last page asked for, 7 query there, 8 first page there, 9 last scores committed, 10 first scores seen,
// 11 last page reduced, 12 partial written, 13 all roles done, 14 exit (globaltimer ns), 15 SM id.
// A development aid for the fixed cost of a launch; the library is never shipped with it.
#ifdef PKV_WAITPROF
#define PKV_WPM(slot) do { const long long n_ = clock64(); if ((threadIdx.x & 31) == 0) atomicAdd(&X->waited[slot], (unsigned long long)(n_ - wp_t)); wp_t = n_; } while (0)
#else
#define PKV_WPM(slot) do { } while (0)
#endif
#ifdef PKV_TIMELINE
#define PKV_TL(slot) do { tl_buf[slot] = clock64(); } while (0)
__device__ __forceinline__ long long pkv_globaltimer() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#else
#define PKV_TL(slot) do { } while (0)
#endif

template <int WP, int REP, bool WV, bool INLQ, bool VQ>
__global__ void __launch_bounds__(n_threads<WV, VQ>(), 1) pkv_attn_tc_kernel(
    const __grid_constant__ CUtensorMap vmap, const __grid_constant__ CUtensorMap kmap,
    const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap smap,
    const int32_t* __restrict__ page_table, int max_pages,
    const int32_t* __restrict__ seqlens, int n_split, int n_pages_pool, float col_scale, float inv_logit_scale,
    uint32_t flags, float* __restrict__ partials, float* __restrict__ scores_out, long scores_stride,
    int32_t* __restrict__ status, const pkv_absorb_impl::Args qa) {
    using C = Cfg<WP, VQ>;
    static_assert(!VQ || WV, "quantised V pages only matter when V is read");
    // qa.q set: the kernel absorbs the raw queries itself (softmax group 0, pkv_absorb_impl::body_tile) instead
    // of loading the operand a pkv_absorb launch left in global memory
    constexpr bool inline_q = INLQ;                  // a separate instantiation: the plain kernels do not carry this code
    // A CTA handles at most 8 kv heads (their O^T accumulators take 16 tensor-memory columns each). With
    // grouped queries (REP = 4 or 8) that is the whole layer; with one query head per kv head (REP = 1, 32
    // kv heads) blockIdx.z selects a group of 8 heads: the scores of all 32 heads are formed (the latent is
    // 1 % of the bytes), softmax and P.V run for the group's 8.
    constexpr int NKV = NQ / REP > 8 ? 8 : NQ / REP;      // kv heads per CTA
    constexpr int HPC = NKV * REP;                         // query heads per CTA
    constexpr int PGS = (HPC / 8) * 256;                   // bytes of P per 8-token group: per 8 heads [hi 128 | lo 128]
    // quantised V: the weights of kv head g are NPV operand rows (row = term * REP + head of the group; VQ_TERMS E5M2
    // residual terms of p * scale, further rows zero), MN-major: a token's 16 rows of an MN group are 16 contiguous
    // bytes, tokens 16 bytes apart, the second MN group (REP = 8) 2 KB on
    constexpr int NPV = REP == 8 ? 32 : 16;
    static_assert(!VQ || (VQ_TERMS == 4 && VQ_TERMS * REP <= NPV), "weight rows of a kv head");
    constexpr int PG8 = PKV_PAGE_TOKENS * NPV;             // bytes of one kv head's weights of a page
    constexpr int VQ_TILE_ROWS = RAW_BYTES / 128, VQ_PAGE_ROWS = (NQ / REP) * (PKV_VQ_TILE_BYTES / 128);
    const int h_base = (WV ? (int)blockIdx.z : 0) * HPC, g_base = (WV ? (int)blockIdx.z : 0) * NKV;
    static_assert(WV || HPC == NQ, "scores-only launches use a grouped-query instantiation");
    extern __shared__ __align__(1024) uint8_t smem[];
    Extra* X = reinterpret_cast<Extra*>(smem + C::X_OFF);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, b = blockIdx.y;
#ifdef PKV_TIMELINE
    long long* tl_buf = reinterpret_cast<long long*>(scores_out) + ((size_t)(blockIdx.z * gridDim.y + b) * gridDim.x + split) * 16;
    scores_out = nullptr;
    if (tid == 0) { PKV_TL(0); tl_buf[1] = pkv_globaltimer(); uint32_t sm; asm volatile("mov.u32 %0, %%smid;" : "=r"(sm)); tl_buf[15] = sm; }
#endif
#ifdef PKV_WAITPROF
    unsigned long long* wp_buf = reinterpret_cast<unsigned long long*>(scores_out) + ((size_t)(blockIdx.z * gridDim.y + b) * gridDim.x + split) * 64;
    scores_out = nullptr;
    const long long wp_t0 = clock64();
#endif
    pkv_grid_launch_dependents();

    // ---- prologue that touches no global memory: barriers, tensor memory
    if (warp == 0) {                                 // lane s initialises entry s of every barrier array (62 barriers: ~0.3 us for one thread)
        if (lane == 0) {
#ifdef PKV_WAITPROF
            for (int k = 0; k < 64; ++k) X->waited[k] = 0;
#endif
            mbar_init(&X->q_full, inline_q ? pkv_absorb_impl::TILE_THREADS : 1);
            mbar_init(&X->sm_bar, WV ? (VQ ? 256 : 128) : 512);
            X->abort_flag = 0;
        }
        static_assert(NK_MAX <= 32 && NV_BARS <= 32 && NVR <= 32 && NSB_S <= 32, "a lane per barrier of an array");
        if (lane < NK_MAX) { mbar_init(&X->k_full[lane], 1); mbar_init(&X->k_empty[lane], 1); }
        // quantised V: two converter warps per tile, 256 softmax threads, two P.V issuers
        if (lane < NV_BARS) { mbar_init(&X->v_full[lane], VQ ? 2 : 1); mbar_init(&X->v_empty[lane], 1); }
        if (lane < NVR) { mbar_init(&X->vr_full[lane], 1); mbar_init(&X->vr_empty[lane], 2); }
        if (lane < 2) {
            mbar_init(&X->sc_full[lane], 1); mbar_init(&X->sc_empty[lane], 256);
            mbar_init(&X->p_full[lane], VQ ? 256 : 128); mbar_init(&X->pv_done[lane], VQ ? 2 : 1);
        }
        if (lane < NSB_S) { mbar_init(&X->s_full[lane], 1); mbar_init(&X->s_empty[lane], WV ? (VQ ? 256 : 128) : 512); }
        fence_barrier_init();
    }
    if (warp == 2) tmem_alloc(&X->tmem_base, TM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = X->tmem_base;
    const uint32_t sbase = smem_u32(smem);
    if (tid == 0) PKV_TL(2);

    // Normally everything waits here for the kernel launched before this one. With PKV_ATTN_EARLY_STREAM the
    // caller vouches that that kernel only produces the query operand (it is pkv_absorb): the cache, the
    // page table and the lengths are then already final, the producers start streaming pages at once and
    // only the load of the query operand waits.
    // PKV_ATTN_TAIL_WRITTEN on top: that kernel also writes rows of the LAST page of a sequence (the newest
    // token: pkv_decode_prologue), so the last page is only fetched after the wait.
    const bool early = (flags & PKV_ATTN_EARLY_STREAM) != 0;
    const bool tail_written = (flags & PKV_ATTN_TAIL_WRITTEN) != 0;
    if (!early) pkv_grid_wait();

    const int T = seqlens[b];
    if (tid == 0) PKV_TL(3);
    const int npages = min((T + PKV_PAGE_TOKENS - 1) / PKV_PAGE_TOKENS, max_pages);
    const int pps = (npages + n_split - 1) / n_split;
    const int p_lo = split * pps, p_hi = min(npages, p_lo + pps);
    const int P = p_hi - p_lo;
    constexpr bool with_v = WV;                      // scores-only launches are a separate instantiation
    constexpr int SG = 1;                            // softmax groups that split the pages (none does any more)
    constexpr int NSB = WV ? NSB_V : NSB_S;
    constexpr int nks = WV ? NK_STAGES : NK_MAX;      // without V its stages hold more latent pages in flight
    float* part = partials + ((size_t)b * n_split + split) * NQ * (DH + 2);

    // Operand-ready counters (qa.qsync, the qsync_dev of pkv_decode_attn_sync): every CTA of a sequence, when it no longer
    // needs the operand, counts itself in qsync[batch + b]; the last one clears both counters for the next use.
    auto operand_released = [&]() {
        if (qa.qsync && tid == 0) {
            const int n_cta = (int)(gridDim.x * gridDim.z), nb = (int)gridDim.y;
            if (atomicAdd(qa.qsync + nb + b, 1) == n_cta - 1) {
                qa.qsync[b] = 0;
                qa.qsync[nb + b] = 0;
                __threadfence();
            }
        }
    };
    if (P <= 0) {                                  // this split has no token: the neutral partial
        operand_released();
        if (early) pkv_grid_wait();                // the partials may still be read by the launches before (see the epilogue)
        for (int i = tid; i < NQ * (DH + 2); i += blockDim.x) {
            int c = i % (DH + 2);
            part[i] = c == DH ? -INFINITY : 0.0f;
        }
        tc_fence_before_sync();
        __syncthreads();
        if (warp == 2) tmem_dealloc(tb, TM_COLS);
        return;
    }

    constexpr int W_SM = (VQ || !WV) ? 4 : 3;         // first softmax warp
    if (warp == 0) {
        // ================================================================== K producer
        // The page indices are fetched 32 at a time by the whole warp (one coalesced load, one round trip per
        // 32 pages) and handed to lane 0 by shuffle: a dependent global load per page would cap the producer
        // at one page per memory latency.
        if (lane == 0) { tma_prefetch_desc(&kmap); tma_prefetch_desc(&qmap); }
        // A lane's chain of wait, arm and copy costs ~0.4 - 0.7 us per page: as much as a page lasts in scores-only mode.
        // So lane s takes the pages of stage s (page i, stage i % nks) and the lanes work side by side, one sweep of
        // nks pages after the other; lane 0 also fetches the query operand -- at once, or in early mode after the first
        // sweep, so that the stages fill while the launch before this one still runs.
        static_assert(32 % nks == 0, "a sweep of pages lies inside one fetch of 32 page indices");
        int issued = -1;                                             // the lane's own last page
        bool q_sent = inline_q, stop = false, waited = !early;
        auto send_query = [&]() {                                    // lane 0
            if (qa.qsync && early) {
                // the launch before signals each sequence's operand as soon as it is in place (it may
                // still be busy with other work, e.g. the cache write of the newest token): poll
                // the counter instead of waiting for that whole grid
                const int need = (NQ + pkv_absorb_impl::HG - 1) / pkv_absorb_impl::HG;
                bool there = false;
                for (uint32_t it = 0; it < WAIT_LIMIT && !there; ++it) {    // about half a second, then give up
                    int v;
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(qa.qsync + b) : "memory");
                    there = v >= need;
                    if (!there) {
                        if ((it & 63u) == 63u && X->abort_flag) break;
                        __nanosleep(40);
                    }
                }
                if (!there) {
                    if (!X->abort_flag && status) { atomicExch(&status[0], 1); atomicExch(&status[1], 11); }
                    X->abort_flag = 1;
                    stop = true;
                }
                asm volatile("fence.proxy.async;" ::: "memory");    // the operand was written by ordinary stores, the tile load reads it
            } else if (!waited) { pkv_grid_wait(); waited = true; }
            if (!stop) {
                mbar_arrive_expect_tx(&X->q_full, C::QBLOB);
                tma_load_2d(smem + C::Q_OFF, &qmap, 0, b * (C::QBLOB / 128), &X->q_full);
                PKV_TL(5);
            }
            q_sent = true;
        };
        // (the first page indices are asked for before anything else: their round trip is the longest wait of the start-up)
        int mine = lane < P ? page_table[(size_t)b * max_pages + p_lo + lane] : 0;
        if (lane == 0 && !q_sent && !early) send_query();
        stop = __shfl_sync(0xffffffffu, stop ? 1 : 0, 0) != 0;
        for (int base = 0; base < P && !stop; base += 32) {
            if (base > 0) mine = base + lane < P ? page_table[(size_t)b * max_pages + p_lo + base + lane] : 0;
            for (int r0 = 0; r0 < 32 && base + r0 < P && !stop; r0 += nks) {
                const int i = base + r0 + lane;                      // this lane's page of the sweep
                const int pidx = __shfl_sync(0xffffffffu, mine, (r0 + lane) & 31);
                if (lane < nks && i < P) {
                    // a page that the launch before this one still writes (the newest token's) waits for that launch
                    if (!waited && tail_written && p_lo + i == npages - 1) { pkv_grid_wait(); waited = true; }
                    if (i >= nks && !wait_or_abort(&X->k_empty[lane], ((i / nks) - 1) & 1, X, status, 10)) {
                        stop = true;
                    } else if (pidx < 0 || pidx >= n_pages_pool) {   // never dereference a bad page index
                        X->abort_flag = 1;
                        if (status) { atomicExch(&status[0], 2); atomicExch(&status[1], p_lo + i); }
                        stop = true;
                    } else {
                        mbar_arrive_expect_tx(&X->k_full[lane], C::PAGE);
                        // one tensor tile of PAGE/128 rows x 128 bytes (plain bulk copies of this size were
                        // measured at ~16 GB/s per SM, tiled loads are not limited that way)
                        tma_load_2d(smem + C::K_OFF + lane * C::PAGE, &kmap, 0, pidx * (C::PAGE / 128), &X->k_full[lane]);
                        issued = i;
                        if (i == 0) PKV_TL(4);
                        if (i == P - 1) PKV_TL(6);
                    }
                }
                if (lane == 0 && !q_sent && !stop) send_query();     // early mode: the first sweep of pages is on its way
                stop = __any_sync(0xffffffffu, stop);
            }
        }
        if (lane == 0 && !q_sent && !stop) send_query();             // (no page at all)
        if (X->abort_flag) {                                         // let copies in flight land before leaving
            if (lane == 0 && q_sent && !inline_q) mbar_wait(&X->q_full, 0, 1u << 16);
            if (lane < nks && issued >= 0) mbar_wait(&X->k_full[lane], (issued / nks) & 1, 1u << 16);
        }
    } else if (warp == 1 && WV) {
        // ================================================================== V producer
        {
            if (lane == 0) { tma_prefetch_desc(&vmap); if (VQ) tma_prefetch_desc(&smap); }
            int issued = 0;
            bool stop = false, waited = !(early && tail_written);
            for (int base = 0; base < P && !stop; base += 32) {
                const int mine = base + lane < P ? page_table[(size_t)b * max_pages + p_lo + base + lane] : 0;
                for (int jj = 0; jj < 32 && base + jj < P && !stop; ++jj) {
                    const int i = base + jj;
                    const int pidx = __shfl_sync(0xffffffffu, mine, jj);
                    if constexpr (VQ) {
                        // Quantised pages: a lane's chain of wait, arm and copy takes ~0.4 us per tile, too long for eight tiles
                        // of a page that lasts 2 us. Lanes 0 .. 7 therefore work side by side, lane s on the tiles of raw
                        // stage s (tile j = page * NKV + kv head, stage j % 8), lane 8 on the page's scale block.
                        static_assert(NVR == 8 && (NKV == 4 || NKV == 8), "a lane per raw stage");
                        if (pidx < 0 || pidx >= n_pages_pool) {
                            stop = true;                             // the K producer reports it
                        } else {
                            if (!waited && p_lo + i == npages - 1) { pkv_grid_wait(); waited = true; }
                            if (lane == NVR) {                       // 8 kv heads x 128 bf16
                                const int ss = i & 1;
                                if (i >= 2 && !wait_or_abort(&X->sc_empty[ss], ((i >> 1) - 1) & 1, X, status, 22)) stop = true;
                                if (!stop) {
                                    mbar_arrive_expect_tx(&X->sc_full[ss], VQ_SCALE_BYTES);
                                    tma_load_2d(smem + C::SC_OFF + ss * VQ_SCALE_BYTES, &smap, 0,
                                                pidx * VQ_PAGE_ROWS + (NQ / REP) * VQ_TILE_ROWS + g_base * 2, &X->sc_full[ss]);
                                    issued = i + 1;
                                }
                            } else if (lane < NVR) {
                                for (int g = 0; g < NKV && !stop; ++g) {
                                    const int j = i * NKV + g;                     // the codes of (page, kv head) as stored
                                    if (j % NVR != lane) continue;
                                    if (j >= NVR && !wait_or_abort(&X->vr_empty[lane], ((j / NVR) - 1) & 1, X, status, 21)) { stop = true; break; }
                                    mbar_arrive_expect_tx(&X->vr_full[lane], RAW_BYTES);
                                    tma_load_2d(smem + C::R_OFF + lane * RAW_BYTES, &vmap, 0, pidx * VQ_PAGE_ROWS + (g_base + g) * VQ_TILE_ROWS,
                                                &X->vr_full[lane]);
                                    issued = j + 1;
                                }
                            }
                        }
                        stop = __any_sync(0xffffffffu, stop);
                        continue;
                    }
                    if (lane == 0) {
                        if (pidx < 0 || pidx >= n_pages_pool) {
                            stop = true;                             // the K producer reports it
                        } else {
                            if (!waited && p_lo + i == npages - 1) { pkv_grid_wait(); waited = true; }
                            for (int g = 0; g < NKV; ++g) {
                                const int j = i * NKV + g, s = j % NV_STAGES;
                                if (j >= NV_STAGES && !wait_or_abort(&X->v_empty[s], ((j / NV_STAGES) - 1) & 1, X, status, 20)) { stop = true; break; }
                                uint8_t* dst = smem + C::V_OFF + s * V_STAGE_BYTES;
                                mbar_arrive_expect_tx(&X->v_full[s], V_STAGE_BYTES);
                                tma_load_2d(dst, &vmap, 0, (pidx * (NQ / REP) + g_base + g) * PKV_PAGE_TOKENS, &X->v_full[s]);
                                tma_load_2d(dst + V_STAGE_BYTES / 2, &vmap, 64, (pidx * (NQ / REP) + g_base + g) * PKV_PAGE_TOKENS, &X->v_full[s]);
                                issued = j + 1;
                            }
                        }
                    }
                    stop = __shfl_sync(0xffffffffu, stop ? 1 : 0, 0) != 0;
                }
            }
            if (X->abort_flag) {                                     // let copies in flight land before leaving
                if constexpr (VQ) {
                    // `issued` is the lane's own: one past its last tile (lanes 0 .. 7), one past its last page (lane 8)
                    if (lane < NVR && issued > 0) mbar_wait(&X->vr_full[lane], ((issued - 1) / NVR) & 1, 1u << 16);
                    if (lane == NVR)
                        for (int j = max(0, issued - 2); j < issued; ++j) mbar_wait(&X->sc_full[j & 1], (j >> 1) & 1, 1u << 16);
                } else if (lane == 0) {
                    for (int j = max(0, issued - NV_STAGES); j < issued; ++j)
                        mbar_wait(&X->v_full[j % NV_STAGES], (j / NV_STAGES) & 1, 1u << 16);
                }
            }
        }
    } else if (warp == 2 || warp == 1 || ((VQ || !WV) && warp == 3) || (VQ && warp == 20)) {
        // ================================================================== MMA issuer
        // One thread issues every tcgen05 instruction of its pages; what bounds it is the latency of its own
        // instruction chain (two satisfied barrier waits, 4 + 4 tcgen05 issues of ~75 cycles, two commits:
        // ~1600 cycles per page). With V that is a fifth of a page's HBM time. Without V the issuer's chain is what a page
        // costs, so there are three: warp 2 takes the pages 0, 3, 6 .., warp 1 (which the V stream leaves idle) 1, 4, 7 ..,
        // warp 3 the rest, each with a score buffer of its own; all softmax groups read every buffer (a part of the heads each).
        // With quantised V a page's bytes last a third as long, and the issue chains become the longest link: warp 2 then
        // issues the scores alone (a P.V issuer that waits for a converted tile must not hold up the next page's scores:
        // 116 -> 109 us per layer), warp 20 the P.V of the even kv heads, warp 3 of the odd ones.
        constexpr int PV_STEP = VQ ? 2 : 1;
        if (lane == 0) {
            const int first = WV ? 0 : (warp == 2 ? 0 : (warp == 1 ? 1 : 2));
            constexpr int STEP = WV ? 1 : NSB_S;
            const uint32_t sfb_tm = tb + TM_SFB + 16u * (uint32_t)first;
            constexpr uint32_t idesc_s = idesc_nvfp4(128, PKV_QUERY_TERMS * NQ);
            constexpr uint32_t idesc_o = VQ ? idesc_f8(128, NPV, true, true, 0u, 1u) : idesc_bf16(128, 16, true, false);   // V: E4M3, weights: E5M2
            // quantised V: warp 2 issues the scores only, so that a P.V issuer waiting for a converted tile never holds up
            // the scores of the next page; warp 20 takes the P.V of the even kv heads, warp 3 of the odd ones
            const bool pv_only = VQ && (warp == 3 || warp == 20);
            bool ok = pv_only || wait_or_abort(&X->q_full, 0, X, status, 30);
            if (warp == 2) PKV_TL(7);
            if (ok && !pv_only) {
                tc_fence_after_sync();
                for (int k = 0; k < C::KB; ++k)
                    tmem_cp_32x128b_warpx4(sfb_tm + 4 * k, smem_desc(sbase + C::Q_OFF + C::CODES + k * 512, 0, 128, SWZ_NONE));
            }
            const uint64_t q_desc = smem_desc(sbase + C::Q_OFF, 0, C::SBO, C::SWZ);
            auto do_pv = [&](int i) -> bool {
                const int pb = i & 1;
                if (!wait_or_abort(&X->p_full[pb], (i >> 1) & 1, X, status, 31)) return false;
                tc_fence_after_sync();
                for (int g = (VQ && warp == 3) ? 1 : 0; g < NKV; g += PV_STEP) {
                    const int j = i * NKV + g, s = j % C::NVS;
                    uint64_t* const empty_bar = &X->v_empty[s];
                    if (!wait_or_abort(&X->v_full[s], (j / C::NVS) & 1, X, status, 32)) return false;
                    tc_fence_after_sync();
                    const uint32_t va = sbase + C::V_OFF + s * C::VSB;
                    if constexpr (VQ) {
                        // A: the tile as E4M3, 128 tokens x 128 bytes (dims contiguous: MN-major, one 128-byte swizzle atom
                        // wide); B: this kv head's weight rows, MN-major without swizzle (groups of 8 tokens 128 bytes
                        // apart, MN groups of 16 rows 2 KB apart); K = 32 tokens per instruction
                        const uint64_t v8_desc = smem_desc(va, 0, 1024, SWZ_128B);
                        const uint64_t p8_desc = smem_desc(sbase + C::P_OFF + pb * P_BYTES + g * PG8, 128, NPV == 16 ? 128 : PKV_PAGE_TOKENS * 16, SWZ_NONE);
#ifndef PKV_VQ_SKIP_PV
#pragma unroll
                        for (int k = 0; k < PKV_PAGE_TOKENS / 32; ++k)
                            mma_f8(tb + TM_O + NPV * g, v8_desc + (uint64_t)(k * 32 * 128 / 16), p8_desc + (uint64_t)(k * 32 * 16 / 16), idesc_o,
                                   !(i == 0 && k == 0));
#endif
                        tc_commit(empty_bar);
                        continue;
                    }
                    // B operand: 16 rows = the hi weights of the 8-head group holding this kv head's heads, then their lo parts
                    const uint32_t pa = sbase + C::P_OFF + pb * P_BYTES + ((g * REP) >> 3) * 256;
                    const uint64_t v_desc = smem_desc(va, V_STAGE_BYTES / 2, 1024, SWZ_128B);
                    const uint64_t p_desc = smem_desc(pa, PGS, 128, SWZ_NONE);
#ifndef PKV_VQ_SKIP_PV                                                // (development switch: no P.V MMAs)
#pragma unroll
                    for (int k = 0; k < PKV_PAGE_TOKENS / 16; ++k)
                        mma_bf16(tb + TM_O + 16 * g, v_desc + (uint64_t)(k * 2048 / 16), p_desc + (uint64_t)(k * 2 * PGS / 16), idesc_o,
                                 !(i == 0 && k == 0));
#else
                    (void)v_desc; (void)p_desc;
#endif
                    tc_commit(empty_bar);
                }
                tc_commit(&X->pv_done[pb]);
                return true;
            };
            // stage, buffer and their barrier phases advance by counters (this thread's instruction chain is the
            // critical path: no divisions by run-time values in it)
            if (pv_only) {                                   // the second P.V issuer: every page, odd kv heads
                for (int i = 0; i < P && ok; ++i) ok = do_pv(i);
            }
            int s = first % nks, buf = first % NSB;
            uint32_t k_phase = 0, s_round = 0;               // s_round = i / NSB
            for (int i = first; i < P && ok && !pv_only; i += STEP) {
                ok = wait_or_abort(&X->k_full[s], k_phase, X, status, 33);
                if (ok && s_round > 0) ok = wait_or_abort(&X->s_empty[buf], (s_round - 1) & 1, X, status, 34);
                if (!ok) break;
                if (i == 0) PKV_TL(8);
                tc_fence_after_sync();
                const uint32_t ka = sbase + C::K_OFF + s * C::PAGE;
                // descriptors differ from page to page only in the start-address field (units of 16 bytes): the
                // constant parts are formed once, the loops below are fully unrolled
                const uint64_t sf_desc = smem_desc(ka + C::CODES, 0, 128, SWZ_NONE);
                const uint64_t a_desc = smem_desc(ka, 0, C::SBO, C::SWZ);
                const uint32_t s_tm = tb + TM_S + 128 * buf, sfa_tm = tb + TM_SFA + 16 * buf;
#pragma unroll
                for (int k = 0; k < C::KB; ++k) tmem_cp_32x128b_warpx4(sfa_tm + 4 * k, sf_desc + (uint64_t)(k * 512 / 16));
                // the four residual terms of the query are the four 32-row blocks of its tile: one pass with N = 128,
                // the softmax warps add the four column blocks (an MMA costs ~75 cycles whatever its N)
#pragma unroll
                for (int k = 0; k < C::KB; ++k)
                    mma_nvfp4(s_tm, a_desc + (uint64_t)(k * 32 / 16), q_desc + (uint64_t)(k * 32 / 16), idesc_s, sfa_tm + 4 * k,
                              sfb_tm + 4 * k, k != 0);
                tc_commit(&X->k_empty[s]);
                tc_commit(&X->s_full[buf]);
                if (i + STEP >= P) PKV_TL(9);
                if (with_v && !VQ && i >= 1) ok = do_pv(i - 1);
                s += STEP;
                if (s >= nks) { s -= nks; k_phase ^= 1u; }
                buf += STEP;
                if (buf >= NSB) { buf -= NSB; ++s_round; }
            }
            if (ok && with_v && !VQ && !pv_only) do_pv(P - 1);
        }
    } else if (VQ && warp >= 12) {
        // ================================================================== V converter (quantised V pages)
        // A token's 64 bytes of E2M1 codes become 128 E4M3 bytes (exactly the same numbers) in the 128-byte-swizzled
        // MN-major layout the P.V descriptors expect; the token's scale is not applied here but folded into the weights.
        // Two converter warps share every fourth tile (a lane takes two token rows of it), so that four tiles are in
        // work at once and the waits of one hide behind the arithmetic of the others.
        const int cw = (warp - 12) & 3, half = (warp - 12) >> 2;
        // E4M3 bytes of the eight E2M1 magnitudes 0 .5 1 1.5 2 3 4 6 (00 30 38 3C 40 44 48 4C) as byte tables for prmt
        constexpr uint32_t LUT_A = 0x3C383000u, LUT_B = 0x4C484440u;
        auto prmt = [](uint32_t a, uint32_t b, uint32_t c) -> uint32_t {
            uint32_t d;
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
            return d;
        };
        bool ok = true;
        const int n_tiles = P * NKV;
        for (int j = cw; j < n_tiles && ok; j += 4) {
            const int rs = j % NVR, bs = j % C::NVS;
            ok = __all_sync(0xffffffffu, wait_or_abort(&X->vr_full[rs], (j / NVR) & 1, X, status, 50));
            if (ok && j >= C::NVS) ok = __all_sync(0xffffffffu, wait_or_abort(&X->v_empty[bs], ((j / C::NVS) - 1) & 1, X, status, 51));
            if (!ok) break;
            const uint8_t* raw = smem + C::R_OFF + rs * RAW_BYTES;
            uint8_t* stage = smem + C::V_OFF + bs * C::VSB;
#ifdef PKV_WAITPROF
            long long wp_t = clock64();
#endif
#ifndef PKV_VQ_SKIP_CONVERT                                           // (development switch: barrier traffic only)
            // (a compact loop on purpose: unrolled, this code and the softmax loop no longer fit the instruction cache
            // together, and both then run at the speed of instruction fetch)
#pragma unroll 1
            for (int rg = 2 * half; rg < 2 * half + 2; ++rg) {
                const int r = rg * 32 + lane;
                const uint32_t sw = ((uint32_t)r >> 1) & 3u;
                uint8_t* dst = stage + r * 128;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint4 w4 = *reinterpret_cast<const uint4*>(raw + r * 64 + ((c ^ sw) << 4));
                    const uint32_t wv[4] = {w4.x, w4.y, w4.z, w4.w};
                    uint32_t o[8];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {                    // 8 codes -> 8 bytes: magnitude by table, sign on top
                        const uint32_t w = wv[u], m = w & 0x77777777u, up = w << 4;
                        o[2 * u] = prmt(LUT_A, LUT_B, m) | (prmt(up, w, 0xD9C8u) & 0x80808080u);
                        o[2 * u + 1] = prmt(LUT_A, LUT_B, m >> 16) | (prmt(up, w, 0xFBEAu) & 0x80808080u);
                    }
                    // 32 dims = two 16-byte chunks of the token's 128-byte row (128-byte swizzle: chunk ^ (row & 7))
                    *reinterpret_cast<uint4*>(dst + (((2 * c) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(dst + (((2 * c + 1) ^ (r & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                }
            }
#else
            (void)stage; (void)raw; (void)prmt; (void)LUT_A; (void)LUT_B;
#endif
            fence_proxy_async_smem();                                // generic-proxy writes -> visible to the tensor core
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&X->v_full[bs]);
                mbar_arrive(&X->vr_empty[rs]);
            }
            PKV_WPM(58);                                    // one tile converted
        }
    } else {
        // ================================================================== softmax (128 threads, one token row each)
        const int quad = warp & 3;                          // TMEM lane quadrant this warp may access
        const int sg = VQ ? 0 : (warp - W_SM) >> 2;         // softmax group: pages sg, sg + SG, ...
        const int hg = VQ ? (warp - 4) >> 2 : 0;            // quantised V: group hg takes kv heads hg * NKV / 2 .. of every page
        constexpr int GPG = VQ ? NKV / 2 : NKV;             // kv heads per group
        const int g_lo = hg * GPG, g_hi = g_lo + GPG;
        (void)hg; (void)g_lo; (void)g_hi;
        (void)W_SM;
        const int row = quad * 32 + lane;
        const uint32_t tl = tb + ((uint32_t)(quad * 32) << 16);
        const float* rs = reinterpret_cast<const float*>(smem + C::Q_OFF + C::PAGE);     // [head] tensor scale of the query operand
        // waits are made warp-uniform: the warp-collective instructions below need all 32 lanes
        auto wait_all = [&](uint64_t* bar, uint32_t parity, int where) -> bool {
            return __all_sync(0xffffffffu, wait_or_abort(bar, parity, X, status, where));
        };
        int sync_phase = 0;
        auto softmax_sync = [&]() -> bool {                 // all softmax threads meet here
            mbar_arrive(&X->sm_bar);
            return wait_all(&X->sm_bar, (sync_phase++) & 1, 45);
        };
        if constexpr (!WV) {
            // ---------------- scores only: no weights, no P.V. The four softmax groups split the HEADS of every page
            // (group hs takes heads 8 hs .. 8 hs + 7): a thread's state is 8 heads instead of 32 and the loop body a
            // quarter of the code, every warp keeps its own statistics (reference maximum and row sums per head) and no
            // rendezvous is needed inside the loop. A score buffer is free again when all four groups have read it.
            constexpr int HS = 4, HPT = NQ / HS;
            const int hs = (warp - W_SM) >> 2, h0 = hs * HPT;
            if constexpr (INLQ) if (hs == 0) {
                if (early && !(flags & PKV_ATTN_QUERY_READY)) pkv_grid_wait();
                pkv_absorb_impl::body_tile<WP>(qa, b, smem + C::Q_OFF, reinterpret_cast<float*>(smem + C::P_OFF), tid - W_SM * 32);
                fence_proxy_async_smem();                   // generic-proxy writes -> visible to tcgen05.mma / tcgen05.cp
                mbar_arrive(&X->q_full);
            }
            bool ok = wait_all(&X->q_full, 0, 40);
            float cs[HPT], m[HPT], l[HPT];
#pragma unroll
            for (int j = 0; j < HPT; ++j) { cs[j] = ok ? rs[h0 + j] * col_scale : 0.0f; m[j] = -INFINITY; l[j] = 0.0f; }
            for (int i = 0; i < P && ok; ++i) {
                const int sb = i % NSB;
                ok = wait_all(&X->s_full[sb], (i / NSB) & 1, 41);
                if (!ok) break;
                if (i == 0 && warp == W_SM && lane == 0) PKV_TL(10);
                tc_fence_after_sync();
#ifdef PKV_WAITPROF
                long long wp_t = clock64();
#endif
                float sv[HPT];
                {
                    uint32_t r[PKV_QUERY_TERMS][HPT];
#pragma unroll
                    for (int t = 0; t < PKV_QUERY_TERMS; ++t) tmem_ldn<HPT>(tl + TM_S + 128 * sb + 32 * t + h0, r[t]);
                    tmem_ld_wait();
                    tc_fence_before_sync();
                    mbar_arrive(&X->s_empty[sb]);           // one of the 512 arrivals that free this S buffer
#pragma unroll
                    for (int j = 0; j < HPT; ++j) {
                        float a = __uint_as_float(r[0][j]);
#pragma unroll
                        for (int t = 1; t < PKV_QUERY_TERMS; ++t) a += __uint_as_float(r[t][j]);   // the terms share the head's tensor scale
                        sv[j] = a * cs[j];
                    }
                }
                PKV_WPM(52);
                const int token = (p_lo + i) * PKV_PAGE_TOKENS + row;
                const bool valid = token < T;
                if (scores_out && valid) {
#pragma unroll
                    for (int j = 0; j < HPT; ++j) scores_out[((size_t)b * NQ + h0 + j) * scores_stride + token] = sv[j] * inv_logit_scale;
                }
                float e2[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < HPT; ++j) {
                    if (!valid) sv[j] = -INFINITY;
                    e2[j & 1] = fmaxf(e2[j & 1], sv[j] - m[j]);       // +inf while the head has no reference yet
                }
                const bool grow = __any_sync(0xffffffffu, fmaxf(e2[0], e2[1]) > RESCALE_THRESHOLD);
                PKV_WPM(53);
                if (grow) {
#pragma unroll
                    for (int j = 0; j < HPT; ++j) {
                        const float m_new = fmaxf(m[j], ord2f(__reduce_max_sync(0xffffffffu, f2ord(sv[j]))));
                        l[j] *= m[j] > -INFINITY ? exp2f(m[j] - m_new) : 1.0f;      // nothing accumulated yet: leave as is
                        m[j] = m_new;
                    }
                }
                PKV_WPM(54);
#pragma unroll
                for (int j = 0; j < HPT; ++j) l[j] += ex2_fast(sv[j] - (m[j] > -INFINITY ? m[j] : 0.0f));   // exp2(-inf) = 0 for masked rows
                PKV_WPM(56);
            }
            if (warp == W_SM && lane == 0) PKV_TL(11);
            if (early) pkv_grid_wait();                     // (see the note at the same place of the other branch)
            if (ok) {
#pragma unroll
                for (int j = 0; j < HPT; ++j) part[(h0 + j) * (DH + 2) + row] = 0.0f;
                float lw = 0.0f, mw = -INFINITY;
#pragma unroll
                for (int j = 0; j < HPT; ++j) {
                    float v = l[j];
#pragma unroll
                    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (lane == h0 + j) { lw = v; mw = m[j]; }
                }
                if (lane >= h0 && lane < h0 + HPT) {            // a head's sums come from the group that owns it, one set per warp
                    X->lsum[0][quad][lane] = lw;
                    X->mfin[0][quad][lane] = mw;
                }
                if (softmax_sync() && quad == 0 && hs == 0) {
                    float M = -INFINITY, lt = 0.0f;
#pragma unroll
                    for (int w = 0; w < 4; ++w) M = fmaxf(M, X->mfin[0][w][lane]);
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const float mw2 = X->mfin[0][w][lane];
                        if (mw2 > -INFINITY) lt = fmaf(X->lsum[0][w][lane], exp2f(mw2 - M), lt);
                    }
                    part[lane * (DH + 2) + DH] = M;
                    part[lane * (DH + 2) + DH + 1] = lt;
                }
            } else {
                softmax_sync();                             // keep the rendezvous count whole when a group gave up
            }
            if (warp == W_SM && lane == 0) PKV_TL(12);
        } else {
        // Per head (all kept in registers, identical in every thread that shares statistics): the
        // column scale that turns the MMA result into a base-2 logit, the reference maximum, and
        // this thread's share of the sum of 2^(s - m).
        // (With quantised V the loops over the heads are not unrolled, so nothing per head can live in a register
        // array: the column scales stay in shared memory, where the query operand's tail holds them, and are read
        // as broadcasts; the reference maxima, identical in every lane, are kept one per lane -- lane h holds head
        // h's -- and fetched by shuffle, so are the rescale factors; the row sums live in spare tensor-memory columns,
        // which a thread can index at run time.)
        // (Scores only: 16 warps leave 128 registers per thread, so the column scales are read from shared memory there too.)
        constexpr bool CS_REG = WV && !VQ;
        float cs[CS_REG ? HPC : 1], m[VQ ? 1 : HPC], l[VQ ? 1 : HPC];
        float m_lane = -INFINITY;
        const uint32_t l_tm = tl + TM_L;                    // row sums: tensor-memory columns, one per head, this thread's lane
        auto m_of = [&](int h) -> float { return __shfl_sync(0xffffffffu, m_lane, h); };
        (void)l_tm; (void)m_of; (void)m_lane;
        if constexpr (INLQ) if (sg == 0) {
            // the query may come from the launch before this one unless the caller says it was ready earlier
            if (early && !(flags & PKV_ATTN_QUERY_READY)) pkv_grid_wait();
            pkv_absorb_impl::body_tile<WP>(qa, b, smem + C::Q_OFF, reinterpret_cast<float*>(smem + C::P_OFF), tid - W_SM * 32);
            fence_proxy_async_smem();                       // generic-proxy writes -> visible to tcgen05.mma / tcgen05.cp
            mbar_arrive(&X->q_full);
        }
        bool ok = wait_all(&X->q_full, 0, 40);
        if constexpr (VQ) {
            const uint32_t zero[REP] = {};
#pragma unroll 1
            for (int g = g_lo; g < g_hi; ++g) tmem_stn<REP>(l_tm + g * REP, zero);
            tmem_st_wait();
        } else {
#pragma unroll
            for (int h = 0; h < HPC; ++h) {
                if constexpr (CS_REG) cs[h] = ok ? rs[h_base + h] * col_scale : 0.0f;
                m[h] = -INFINITY;
                l[h] = 0.0f;
            }
        }
        (void)cs; (void)m; (void)l;
        for (int i = sg; i < P && ok; i += SG) {
            const int sb = i % NSB;                         // score buffer
            const int buf = i & 1;                          // P buffer and exchange slots
            ok = wait_all(&X->s_full[sb], (i / NSB) & 1, 41);
            if (!ok) break;
            if (i == 0 && warp == W_SM && lane == 0) PKV_TL(10);
            tc_fence_after_sync();
#ifdef PKV_WAITPROF
            long long wp_t = clock64();
#endif
            if constexpr (VQ) {
                // ---------------- quantised V pages. Compact loops over the kv heads: unrolled over all 32 heads, this
                // code and the converter's no longer fit the instruction cache together, and both roles then run at the
                // speed of instruction fetch. The scores are read from tensor memory twice (vote, then weights) instead
                // of kept in 32 registers, the row sums live in shared memory.
                const int token = (p_lo + i) * PKV_PAGE_TOKENS + row;
                const bool valid = token < T;
                const float* hs = rs + h_base;
                const uint32_t s_tm = tl + TM_S + 128 * sb + h_base;
                // the loads of kv head g + 1 are on their way while g is worked on: ask, wait, copy, ask for the next, compute
                auto ask_scores = [&](int g, uint32_t (&r)[PKV_QUERY_TERMS][REP]) {
#pragma unroll
                    for (int t = 0; t < PKV_QUERY_TERMS; ++t) tmem_ldn<REP>(s_tm + 32 * t + g * REP, r[t]);
                };
                auto take_scores = [&](int g, uint32_t (&rn)[PKV_QUERY_TERMS][REP], float (&sv)[REP]) {
                    uint32_t r[PKV_QUERY_TERMS][REP];
#pragma unroll
                    for (int t = 0; t < PKV_QUERY_TERMS; ++t)
#pragma unroll
                        for (int hh = 0; hh < REP; ++hh) r[t][hh] = rn[t][hh];
                    if (g + 1 < g_hi) ask_scores(g + 1, rn);
#pragma unroll
                    for (int hh = 0; hh < REP; ++hh) {
                        float a = __uint_as_float(r[0][hh]);
#pragma unroll
                        for (int t = 1; t < PKV_QUERY_TERMS; ++t) a += __uint_as_float(r[t][hh]);   // the terms share the head's tensor scale
                        a *= hs[g * REP + hh] * col_scale;
                        sv[hh] = valid ? a : -INFINITY;
                    }
                };
                // ---- does any head of any row outgrow its reference maximum by more than the threshold?
                float exc = -INFINITY;
                uint32_t rn[PKV_QUERY_TERMS][REP];
                ask_scores(g_lo, rn);
#pragma unroll 1
                for (int g = g_lo; g < g_hi; ++g) {
                    float sv[REP];
                    tmem_ld_wait();
                    take_scores(g, rn, sv);
#pragma unroll
                    for (int hh = 0; hh < REP; ++hh) exc = fmaxf(exc, sv[hh] - m_of(g * REP + hh));   // +inf while the head has no reference yet
                }
                PKV_WPM(52);
                bool grow = __any_sync(0xffffffffu, exc > RESCALE_THRESHOLD);
                if (lane == 0) X->wflag[buf][hg * 4 + quad] = grow ? 1 : 0;
                ok = softmax_sync();
                if (!ok) break;
                grow = (X->wflag[buf][0] | X->wflag[buf][1] | X->wflag[buf][2] | X->wflag[buf][3] | X->wflag[buf][4] | X->wflag[buf][5] |
                        X->wflag[buf][6] | X->wflag[buf][7]) != 0;
                PKV_WPM(53);
                if (grow) {
                    float wm = -INFINITY;                   // lane h: the tile maximum of head h (this group's heads)
                    ask_scores(g_lo, rn);
#pragma unroll 1
                    for (int g = g_lo; g < g_hi; ++g) {
                        float sv[REP];
                        tmem_ld_wait();
                        take_scores(g, rn, sv);
#pragma unroll
                        for (int hh = 0; hh < REP; ++hh) {
                            const uint32_t red = __reduce_max_sync(0xffffffffu, f2ord(sv[hh]));
                            if (lane == g * REP + hh) wm = ord2f(red);
                        }
                    }
                    if (lane >= g_lo * REP && lane < g_hi * REP) X->wmax[buf][quad][lane] = wm;
                    ok = softmax_sync();
                    if (!ok) break;
                    const float tm = fmaxf(fmaxf(X->wmax[buf][0][lane], X->wmax[buf][1][lane]),
                                           fmaxf(X->wmax[buf][2][lane], X->wmax[buf][3][lane]));
                    if (i > 0) {                            // the accumulators must be at rest before they are rescaled
                        ok = wait_all(&X->pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1, 42);
                        if (!ok) break;
                        tc_fence_after_sync();
                    }
                    const float m_new = fmaxf(m_lane, tm);
                    const float corr_lane = m_lane > -INFINITY ? exp2f(m_lane - m_new) : 1.0f;     // nothing accumulated yet: leave as is
                    m_lane = m_new;
#pragma unroll 1
                    for (int g = g_lo; g < g_hi; ++g) {
                        uint32_t lr[REP];
                        tmem_ldn<REP>(l_tm + g * REP, lr);
                        tmem_ld_wait();
#pragma unroll
                        for (int hh = 0; hh < REP; ++hh) lr[hh] = __float_as_uint(__uint_as_float(lr[hh]) * __shfl_sync(0xffffffffu, corr_lane, g * REP + hh));
                        tmem_stn<REP>(l_tm + g * REP, lr);
                    }
                    tmem_st_wait();
                    if (i > 0) {
#pragma unroll 1
                        for (int g = g_lo; g < g_hi; ++g)
#pragma unroll 1
                            for (int c0 = 0; c0 < NPV; c0 += 16) {   // column n = term * REP + head of the group
                                uint32_t r[16];
                                tmem_ld16(tl + TM_O + NPV * g + c0, r);
                                tmem_ld_wait();
#pragma unroll
                                for (int c = 0; c < 16; ++c)
                                    r[c] = __float_as_uint(__uint_as_float(r[c]) * __shfl_sync(0xffffffffu, corr_lane, g * REP + ((c0 + c) % REP)));
                                tmem_st16(tl + TM_O + NPV * g + c0, r);
                            }
                        tmem_st_wait();
                        tc_fence_before_sync();
                    }
                }
                PKV_WPM(54);
                if (i >= 2) {
                    ok = wait_all(&X->pv_done[buf], ((i >> 1) - 1) & 1, 43);      // P buffer free again
                    if (!ok) break;
                }
                ok = wait_all(&X->sc_full[buf], (i >> 1) & 1, 46);               // this page's scales
                if (!ok) break;
                PKV_WPM(55);
                // ---- weights relative to the reference maximum, times the token's scale of the kv head, as E5M2 terms:
                // in half precision (two heads per register) a term is the number's top byte (E5M2 = a half cut after two
                // mantissa bits) and the remainder is an exact subtraction; four terms leave less than 2^-11 of the value.
                // The kv head's operand row of this token is 16 contiguous bytes per MN group, byte n = term * REP + head.
                const uint16_t* sc = reinterpret_cast<const uint16_t*>(smem + C::SC_OFF + buf * VQ_SCALE_BYTES) + row;
                uint8_t* pdst = smem + C::P_OFF + buf * P_BYTES + row * 16;
                uint32_t ln[REP];
                ask_scores(g_lo, rn);
                tmem_ldn<REP>(l_tm + g_lo * REP, ln);       // (the row sums travel with the scores)
#pragma unroll 1
                for (int g = g_lo; g < g_hi; ++g) {
                    float sv[REP], pw[REP];
                    uint32_t lr[REP];
                    tmem_ld_wait();
#pragma unroll
                    for (int hh = 0; hh < REP; ++hh) lr[hh] = ln[hh];
                    take_scores(g, rn, sv);
                    if (g + 1 < g_hi) tmem_ldn<REP>(l_tm + (g + 1) * REP, ln);
                    const float vsg = pkv_bf16_bits_to_float(sc[g * PKV_PAGE_TOKENS]);
#pragma unroll
                    for (int hh = 0; hh < REP; ++hh) {
                        const int h = g * REP + hh;
                        if (scores_out && valid) scores_out[((size_t)b * NQ + h_base + h) * scores_stride + token] = sv[hh] * inv_logit_scale;
                        const float mh = m_of(h);
                        const float p = ex2_fast(sv[hh] - (mh > -INFINITY ? mh : 0.0f));  // exp2(-inf) = 0 for masked rows
                        pw[hh] = p > 0.0f ? fminf(p * vsg, 57344.0f) : 0.0f;            // a masked row's scale may be anything
                        lr[hh] = __float_as_uint(__uint_as_float(lr[hh]) + p);
                    }
                    tmem_stn<REP>(l_tm + g * REP, lr);
                    constexpr int NP = (REP + 1) / 2, NW = (REP + 3) / 4;
                    uint32_t x[NP], wd[VQ_TERMS][NW];
#pragma unroll
                    for (int k = 0; k < NP; ++k) {
                        const __half2 h2 = __floats2half2_rn(pw[2 * k], 2 * k + 1 < REP ? pw[2 * k + 1 < REP ? 2 * k + 1 : 0] : 0.0f);
                        x[k] = *reinterpret_cast<const uint32_t*>(&h2);
                    }
#pragma unroll
                    for (int t = 0; t < VQ_TERMS; ++t) {
#pragma unroll
                        for (int w = 0; w < NW; ++w)              // top bytes of four heads, in head order
                            asm("prmt.b32 %0, %1, %2, 0x7531;" : "=r"(wd[t][w]) : "r"(x[2 * w]), "r"(2 * w + 1 < NP ? x[2 * w + 1 < NP ? 2 * w + 1 : 0] : 0u));
                        if (t + 1 < VQ_TERMS) {
#pragma unroll
                            for (int k = 0; k < NP; ++k) {
                                const uint32_t top = x[k] & 0xFF00FF00u;
                                const __half2 r2 = __hsub2(*reinterpret_cast<const __half2*>(&x[k]), *reinterpret_cast<const __half2*>(&top));
                                x[k] = *reinterpret_cast<const uint32_t*>(&r2);
                            }
                        }
                    }
                    uint4* dst = reinterpret_cast<uint4*>(pdst + g * PG8);
                    if constexpr (REP == 8) {                     // 32 rows: terms 0, 1 in the first MN group, 2, 3 in the second
                        dst[0] = make_uint4(wd[0][0], wd[0][1], wd[1][0], wd[1][1]);
                        dst[PKV_PAGE_TOKENS] = make_uint4(wd[2][0], wd[2][1], wd[3][0], wd[3][1]);
                    } else if constexpr (REP == 4) {
                        dst[0] = make_uint4(wd[0][0], wd[1][0], wd[2][0], wd[3][0]);
                    } else {                                      // one head: rows 0 .. 3 are its terms, the rest stay zero
                        dst[0] = make_uint4((wd[0][0] & 0xFFu) | ((wd[1][0] & 0xFFu) << 8) | ((wd[2][0] & 0xFFu) << 16) | (wd[3][0] << 24), 0u, 0u, 0u);
                    }
                }
                tmem_st_wait();                             // the row sums are read again with the next page
                mbar_arrive(&X->sc_empty[buf]);
                tc_fence_before_sync();
                mbar_arrive(&X->s_empty[sb]);               // the MMA warp may overwrite this S buffer
                fence_proxy_async_smem();                   // generic-proxy writes -> visible to the tensor core
                mbar_arrive(&X->p_full[buf]);
            } else {
            float s[HPC];
            {
#pragma unroll
                for (int t = 0; t < PKV_QUERY_TERMS; ++t) {     // the terms share the head's tensor scale: plain sum
                    uint32_t r[HPC];
                    if constexpr (HPC == 32) tmem_ld32(tl + TM_S + 128 * sb + 32 * t, r);
                    else tmem_ld8(tl + TM_S + 128 * sb + 32 * t + h_base, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int h = 0; h < HPC; ++h) s[h] = t == 0 ? __uint_as_float(r[h]) : s[h] + __uint_as_float(r[h]);
                }
                tc_fence_before_sync();
                mbar_arrive(&X->s_empty[sb]);               // the MMA warp may overwrite this S buffer
#pragma unroll
                for (int h = 0; h < HPC; ++h) s[h] *= CS_REG ? cs[CS_REG ? h : 0] : rs[h_base + h] * col_scale;
            }
            PKV_WPM(52);                                    // scores out of tensor memory
            const int token = (p_lo + i) * PKV_PAGE_TOKENS + row;
            const bool valid = token < T;
            if (scores_out && valid) {
#pragma unroll
                for (int h = 0; h < HPC; ++h) scores_out[((size_t)b * NQ + h_base + h) * scores_stride + token] = s[h] * inv_logit_scale;
            }
            // ---- does any head of any row outgrow its reference maximum by more than the threshold?
            float ex4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};     // four chains instead of one of 32 dependent maxima
#pragma unroll
            for (int h = 0; h < HPC; ++h) {
                if (!valid) s[h] = -INFINITY;
                ex4[h & 3] = fmaxf(ex4[h & 3], s[h] - m[h]);                 // +inf while the head has no reference yet
            }
            const float exc = fmaxf(fmaxf(ex4[0], ex4[1]), fmaxf(ex4[2], ex4[3]));
            bool grow = __any_sync(0xffffffffu, exc > RESCALE_THRESHOLD);
            if (with_v) {                                   // P.V needs one reference per head for all 128 rows
                if (lane == 0) X->wflag[buf][quad] = grow ? 1 : 0;
                ok = softmax_sync();
                if (!ok) break;
                grow = (X->wflag[buf][0] | X->wflag[buf][1] | X->wflag[buf][2] | X->wflag[buf][3]) != 0;
            }                                               // scores only: every warp keeps its own statistics
            PKV_WPM(53);                                    // vote (with its rendezvous)
            if (grow) {
                // exact tile maximum per head: warp reduction, then (with V) across the four warps
                float wm = -INFINITY;
#pragma unroll
                for (int h = 0; h < HPC; ++h) {
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
                float corr[HPC];
#pragma unroll
                for (int h = 0; h < HPC; ++h) {
                    const float m_new = fmaxf(m[h], __shfl_sync(0xffffffffu, tm, h));
                    corr[h] = m[h] > -INFINITY ? exp2f(m[h] - m_new) : 1.0f;     // nothing accumulated yet: leave as is
                    m[h] = m_new;
                    l[h] *= corr[h];
                }
                if (with_v && i > 0) {
#pragma unroll
                    for (int g = 0; g < NKV; ++g) {
                        // the 16 columns of kv head g are the hi and lo weights of the 8-head group that holds its
                        // REP query heads (the columns of the group's other heads are never read: any factor does)
                        uint32_t r[16];
                        tmem_ld16(tl + TM_O + 16 * g, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 16; ++c)
                            r[c] = __float_as_uint(__uint_as_float(r[c]) * corr[((g * REP) >> 3) * 8 + (c & 7)]);
                        tmem_st16(tl + TM_O + 16 * g, r);
                    }
                    tmem_st_wait();
                    tc_fence_before_sync();
                }
            }
            PKV_WPM(54);                                    // new reference maxima, rescale
            // ---- probabilities relative to the reference maximum; row sums stay per thread
            if (with_v && i >= 2) {
                ok = wait_all(&X->pv_done[buf], ((i >> 1) - 1) & 1, 43);      // P buffer free again
                if (!ok) break;
            }
            PKV_WPM(55);                                    // weight buffer free, scales there
            // weights of token `row`, head h: 8-token group (row / 8) of 1024 bytes = per 8-head group
            // [hi | lo] x (8 heads x 16 bytes), token (row % 8) inside the 16 bytes
            uint8_t* pbuf = smem + C::P_OFF + buf * P_BYTES + (row >> 3) * PGS + (row & 7) * 2;
#pragma unroll
            for (int h = 0; h < HPC; ++h) {
                const float mh = m[h];
                float p = ex2_fast(s[h] - (mh > -INFINITY ? mh : 0.0f));              // exp2(-inf) = 0 for masked rows
                if (with_v) {
                    // the weight goes to the tensor core as hi + lo bf16; the row sum is taken over exactly
                    // that value, so numerator and denominator of softmax . V carry the same rounding
                    const __nv_bfloat16 hi = __float2bfloat16(p);
                    const __nv_bfloat16 lo = __float2bfloat16(p - __bfloat162float(hi));
                    uint8_t* dst = pbuf + (h >> 3) * 256 + (h & 7) * 16;
                    *reinterpret_cast<__nv_bfloat16*>(dst) = hi;
                    *reinterpret_cast<__nv_bfloat16*>(dst + 128) = lo;
                    p = __bfloat162float(hi) + __bfloat162float(lo);
                }
                l[h] += p;
            }
            if (with_v) {
                fence_proxy_async_smem();                   // generic-proxy writes -> visible to the tensor core
                mbar_arrive(&X->p_full[buf]);
            }
            }
            PKV_WPM(56);                                    // weights written
        }
        if (warp == W_SM && lane == 0) PKV_TL(11);
        // ---- epilogue: O^T back from TMEM, row sums reduced over the 128 token rows
        if (ok && with_v) ok = wait_all(&X->pv_done[(P - 1) & 1], ((P - 1) >> 1) & 1, 44);
        // A CTA that streamed early may never have waited for the launch before this one. It does so now, at no
        // cost: every launch of the chain then completes only after its predecessor, so a launch further
        // back that still reads these partials (the merge of the step before) is known to have finished.
        if (early) pkv_grid_wait();
        if (ok) {
            tc_fence_after_sync();
            if constexpr (VQ) {
#pragma unroll 1
                for (int g = g_lo; g < g_hi; ++g) {             // columns term * REP + head: the terms of a head add up
                    float acc[REP];
#pragma unroll
                    for (int c = 0; c < REP; ++c) acc[c] = 0.0f;
#pragma unroll
                    for (int c0 = 0; c0 < VQ_TERMS * REP; c0 += 8) {
                        uint32_t r[8];
                        tmem_ld8(tl + TM_O + NPV * g + c0, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            if (c0 + c < VQ_TERMS * REP) acc[(c0 + c) % REP] += __uint_as_float(r[c]);
                    }
#pragma unroll
                    for (int c = 0; c < REP; ++c) part[(h_base + g * REP + c) * (DH + 2) + row] = acc[c];
                }
            } else if (with_v) {
#pragma unroll
                for (int g = 0; g < NKV; ++g) {
                    uint32_t r[16];
                    tmem_ld16(tl + TM_O + 16 * g, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < REP; ++c) {
                        const int col = ((g * REP) & 7) + c;                  // hi column; its lo part 8 further
                        part[(h_base + g * REP + c) * (DH + 2) + row] = __uint_as_float(r[col]) + __uint_as_float(r[8 + col]);
                    }
                }
            } else {
                if (sg == 0)
                    for (int h = 0; h < NQ; ++h) part[h * (DH + 2) + row] = 0.0f;
            }
            float lw = 0.0f, mw = -INFINITY;
            if constexpr (VQ) {
#pragma unroll 1
                for (int g = g_lo; g < g_hi; ++g) {
                    uint32_t lr[REP];
                    tmem_ldn<REP>(l_tm + g * REP, lr);
                    tmem_ld_wait();
#pragma unroll
                    for (int hh = 0; hh < REP; ++hh) {
                        float v = __uint_as_float(lr[hh]);
#pragma unroll
                        for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                        if (lane == g * REP + hh) { lw = v; mw = m_lane; }
                    }
                }
                if (lane >= g_lo * REP && lane < g_hi * REP) {  // a head's sums come from the group that owns it
                    X->lsum[0][quad][lane] = lw;
                    X->mfin[0][quad][lane] = mw;
                }
            } else {
#pragma unroll
                for (int h = 0; h < HPC; ++h) {
                    float v = l[VQ ? 0 : h];
#pragma unroll
                    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (lane == h) { lw = v; mw = m[VQ ? 0 : h]; }
                }
                X->lsum[sg][quad][lane] = lw;
                X->mfin[sg][quad][lane] = mw;               // per warp in scores-only mode, identical otherwise
            }
            if (softmax_sync() && quad == 0 && sg == 0 && hg == 0 && lane < HPC) {
                float M = -INFINITY, lt = 0.0f;
#pragma unroll
                for (int w = 0; w < 4 * SG; ++w) M = fmaxf(M, X->mfin[w >> 2][w & 3][lane]);
#pragma unroll
                for (int w = 0; w < 4 * SG; ++w) {
                    const float mw2 = X->mfin[w >> 2][w & 3][lane];
                    if (mw2 > -INFINITY) lt = fmaf(X->lsum[w >> 2][w & 3][lane], exp2f(mw2 - M), lt);
                }
                part[(h_base + lane) * (DH + 2) + DH] = M;
                part[(h_base + lane) * (DH + 2) + DH + 1] = lt;
            }
        } else {
            softmax_sync();                                 // keep the rendezvous count whole when a group gave up
        }
        if (warp == W_SM && lane == 0) PKV_TL(12);
        }
    }
    // ---- teardown: everyone meets, tensor memory goes back
    tc_fence_before_sync();
    __syncthreads();
#ifdef PKV_TIMELINE
    if (tid == 0) { PKV_TL(13); tl_buf[14] = pkv_globaltimer(); }
#endif
#ifdef PKV_WAITPROF
    if (tid < 64) wp_buf[tid] = tid == 0 ? (unsigned long long)(clock64() - wp_t0) : X->waited[tid];
#endif
    operand_released();
    if (X->abort_flag) {
        // A role gave up (status says why). The slot of this CTA gets the neutral triple, so that a merge
        // enqueued behind this launch never folds in what an earlier call left in the partials.
        for (int i = tid; i < HPC * (DH + 2); i += blockDim.x)
            part[h_base * (DH + 2) + i] = (i % (DH + 2)) == DH ? -INFINITY : 0.0f;
    }
    if (warp == 2) tmem_dealloc(tb, TM_COLS);
}

// ------------------------------------------------------------------------------------------------ host
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

int init_encoder() {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        PKV_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return PKV_ERR_CUDA;
        g_encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    }
    return PKV_OK;
}

int encode_v_map(CUtensorMap* map, const pkv_cache_t* C) {
    // V pool as a 2-D bf16 tensor [n_pages * n_kv * 128 tokens, head_dim] (pages are head-major: the tile of one kv head
    // is one contiguous block); box = 64 dims x 128 tokens, 128-byte swizzle
    cuuint64_t dims[2] = {(cuuint64_t)C->head_dim, (cuuint64_t)C->n_pages * C->n_kv * PKV_PAGE_TOKENS};
    cuuint64_t strides[1] = {(cuuint64_t)C->head_dim * 2};
    cuuint32_t box[2] = {64, PKV_PAGE_TOKENS};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C->v_dev, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { g_pkv_last_cuda_error = (int)r; return PKV_ERR_CUDA; }
    return PKV_OK;
}

// a buffer of `rows` 128-byte rows as a 2-D uint8 tensor; box = box_rows whole rows, no swizzle (the latent
// pages and the query operand are stored in their shared-memory layout already)
int encode_rows128_map(CUtensorMap* map, const void* base, uint64_t rows, uint32_t box_rows) {
    cuuint64_t dims[2] = {128, rows};
    cuuint64_t strides[1] = {128};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { g_pkv_last_cuda_error = (int)r; return PKV_ERR_CUDA; }
    return PKV_OK;
}

struct VMaps { CUtensorMap v, s; };

template <int WP, int REP, bool WV, bool INLQ, bool VQ = false>
int launch_tc_impl(const VMaps& vm, const pkv_layer_t* L, const pkv_cache_t* C, const uint8_t* qop, const int32_t* pt,
              int max_pages, const int32_t* seqlens, int batch, int n_split, uint32_t flags, float* partials, float* scores,
              long scores_stride, int32_t* status, const pkv_absorb_impl::Args& qa, cudaStream_t st) {
    auto kern = pkv_attn_tc_kernel<WP, REP, WV, INLQ, VQ>;
    constexpr int smem = Cfg<WP, VQ>::SMEM;
    static pkv_attr_flags attr;                                     // per instantiation and device
    PKV_CUDA_TRY(pkv_set_max_smem(kern, smem, attr));
    const float logit_scale = PKV_LOG2E / sqrtf((float)L->head_dim);
    CUtensorMap kmap, qmap;
    int rc = encode_rows128_map(&kmap, C->latent_dev, (uint64_t)C->n_pages * (Cfg<WP>::PAGE / 128), Cfg<WP>::PAGE / 128);
    if (rc) return rc;
    // with in-kernel absorption the operand map is never used: it is encoded over the latent pool to stay well formed
    rc = qa.q ? encode_rows128_map(&qmap, C->latent_dev, (uint64_t)C->n_pages * (Cfg<WP>::PAGE / 128), Cfg<WP>::QBLOB / 128)
              : encode_rows128_map(&qmap, qop, (uint64_t)batch * (Cfg<WP>::QBLOB / 128), Cfg<WP>::QBLOB / 128);
    if (rc) return rc;
    PKV_CUDA_TRY(pkv_launch_chained(kern, dim3(n_split, batch, WV && REP == 1 ? NQ / 8 : 1), dim3(n_threads<WV, VQ>()), smem, st, vm.v, kmap, qmap, vm.s,
                                    pt, max_pages, seqlens, n_split, C->n_pages, L->second * logit_scale,
                                    1.0f / logit_scale, flags, partials, scores, scores_stride, status, qa));
    return PKV_OK;
}

template <int WP, int REP, bool WV, bool VQ = false>
int launch_tc(const VMaps& vm, const pkv_layer_t* L, const pkv_cache_t* C, const uint8_t* qop, const int32_t* pt,
              int max_pages, const int32_t* seqlens, int batch, int n_split, uint32_t flags, float* partials, float* scores,
              long scores_stride, int32_t* status, const pkv_absorb_impl::Args& qa, cudaStream_t st) {
    if constexpr (VQ) {                              // quantised V pages: the operand comes from pkv_absorb
        if (qa.q) return PKV_ERR_UNSUPPORTED;
        return launch_tc_impl<WP, REP, WV, false, true>(vm, L, C, qop, pt, max_pages, seqlens, batch, n_split, flags, partials,
                                                        scores, scores_stride, status, qa, st);
    } else {
        return qa.q ? launch_tc_impl<WP, REP, WV, true>(vm, L, C, qop, pt, max_pages, seqlens, batch, n_split, flags, partials, scores,
                                                        scores_stride, status, qa, st)
                    : launch_tc_impl<WP, REP, WV, false>(vm, L, C, qop, pt, max_pages, seqlens, batch, n_split, flags, partials,
                                                         scores, scores_stride, status, qa, st);
    }
}

}  // namespace

int pkv_attn_tc_launch(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* q_dev,
                       const int32_t* page_table_dev, int32_t max_pages, const int32_t* seqlens_dev, int32_t batch,
                       int32_t n_split, uint32_t flags, float* partials_dev, float* scores_out_dev,
                       int64_t scores_stride, int32_t* status_dev, float* out_dev, cudaStream_t stream,
                       const float* q_raw_dev, const int32_t* q_positions_dev, int32_t* qsync_dev) {
    const int rep = layer->n_q / layer->n_kv;
    pkv_absorb_impl::Args qa;
    memset(&qa, 0, sizeof(qa));
    if (q_raw_dev) {                                // raw queries: absorbed inside the kernel
        if (!q_positions_dev || (((uintptr_t)q_raw_dev) & 15u)) return PKV_ERR_INVALID;
        if (layer->head_dim / 2 > pkv_absorb_impl::MAX_H) return PKV_ERR_UNSUPPORTED;
        qa = pkv_absorb_impl::make_args(layer, q_raw_dev, q_positions_dev, nullptr, nullptr, nullptr);
    } else if (!q_dev) {
        return PKV_ERR_INVALID;
    }
    if (qsync_dev) {                                // operand-ready counters: only with the operand of a launch directly before
        if (q_raw_dev || !(flags & PKV_ATTN_EARLY_STREAM)) return PKV_ERR_INVALID;
        qa.qsync = qsync_dev;
    }
    if (rep != 1 && rep != 4 && rep != 8) return PKV_ERR_UNSUPPORTED;
    if (q_dev && (((uintptr_t)q_dev) & 15u)) return PKV_ERR_INVALID;
    const bool with_v = !(flags & PKV_ATTN_SCORES_ONLY);
    VMaps vm;                                       // V tiles (bf16 pages, or the code tiles of quantised pages) and their scale blocks
    memset(&vm, 0, sizeof(vm));
    CUtensorMap& vmap = vm.v;
    CUtensorMap& smap = vm.s;
    {
        int st = init_encoder();
        if (st) return st;
    }
    const bool vq = with_v && cache->v_bits != 0;    // V pages hold per-token low-bit codes (pkv_vq_write)
    if (vq) {
        if (!cache->vq_dev || (((uintptr_t)cache->vq_dev) & 127u) || cache->head_dim != DH) return PKV_ERR_INVALID;
        const uint64_t rows = (uint64_t)cache->n_pages * cache->n_kv * (PKV_VQ_TILE_BYTES / 128);
        int st = encode_rows128_map(&vmap, cache->vq_dev, rows, RAW_BYTES / 128);           // the codes of a (page, kv head) tile
        if (st) return st;
        st = encode_rows128_map(&smap, cache->vq_dev, rows, VQ_SCALE_BYTES / 128);          // the scales of 8 kv heads of a page
        if (st) return st;
    } else if (with_v) {
        if (!cache->v_dev || (((uintptr_t)cache->v_dev) & 15u)) return PKV_ERR_INVALID;
        int st = encode_v_map(&vmap, cache);
        if (st) return st;
    }
    const bool wide = pkv_padded_width(cache->W) == 256;
    const uint8_t* qop = (const uint8_t*)q_dev;
    int rc;
#define PKV_TC_CASE(WP_, R_)                                                                                         \
    rc = with_v ? launch_tc<WP_, R_, true>(vm, layer, cache, qop, page_table_dev, max_pages, seqlens_dev, batch, n_split, \
                                           flags, partials_dev, scores_out_dev, scores_stride, status_dev, qa, stream)       \
                : launch_tc<WP_, R_, false>(vm, layer, cache, qop, page_table_dev, max_pages, seqlens_dev, batch, n_split, \
                                            flags, partials_dev, scores_out_dev, scores_stride, status_dev, qa, stream)
#define PKV_TC_VQ(WP_, R_)                                                                                                \
    rc = launch_tc<WP_, R_, true, true>(vm, layer, cache, qop, page_table_dev, max_pages, seqlens_dev, batch, n_split, flags, \
                                        partials_dev, scores_out_dev, scores_stride, status_dev, qa, stream)
    if (vq) {
        if (rep == 1) { if (wide) PKV_TC_VQ(256, 1); else PKV_TC_VQ(128, 1); }
        else if (rep == 8) { if (wide) PKV_TC_VQ(256, 8); else PKV_TC_VQ(128, 8); }
        else { if (wide) PKV_TC_VQ(256, 4); else PKV_TC_VQ(128, 4); }
    } else if (rep == 1 && with_v) {                // one query head per kv head: 4 CTAs of 8 heads per (sequence, split)
        rc = wide ? launch_tc<256, 1, true>(vm, layer, cache, qop, page_table_dev, max_pages, seqlens_dev, batch, n_split, flags,
                                            partials_dev, scores_out_dev, scores_stride, status_dev, qa, stream)
                  : launch_tc<128, 1, true>(vm, layer, cache, qop, page_table_dev, max_pages, seqlens_dev, batch, n_split, flags,
                                            partials_dev, scores_out_dev, scores_stride, status_dev, qa, stream);
    } else if (rep == 8) { if (wide) PKV_TC_CASE(256, 8); else PKV_TC_CASE(128, 8); }
    else { if (wide) PKV_TC_CASE(256, 4); else PKV_TC_CASE(128, 4); }      // scores only never touches V: any grouping
#undef PKV_TC_CASE
#undef PKV_TC_VQ
    if (rc == PKV_OK && out_dev) {                  // the merge of the splits: a second, latency-tuned launch
        const int64_t pw = DH + 2;
        const bool packed = (flags & PKV_ATTN_PACKED_OUT) != 0;
        rc = pkv_merge(partials_dev, (int64_t)n_split * NQ * pw, NQ * pw, n_split, batch, NQ, DH, packed ? nullptr : out_dev,
                       packed ? out_dev : nullptr, stream);
    }
    return rc;
}
