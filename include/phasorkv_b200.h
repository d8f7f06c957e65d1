/* phasorkv_b200 -- C ABI of the B200 (sm_100a) PhasorKey decode path.
 *
 * One shared library, libphasorkv_b200.so, loaded with dlopen/ctypes. Every entry point
 *   - is extern "C", takes plain pointers and sizes (no C++ or torch types),
 *   - enqueues work on the CUDA stream it is given and returns without synchronising,
 *   - allocates nothing: inputs, outputs and scratch are all owned by the caller,
 *   - returns 0 on success or a negative pkv_status code (never throws, never exits).
 * (Three calls say otherwise in their own comments: pkv_layer_create / pkv_layer_destroy allocate and free
 * the device copy of a layer for hosts without a tensor library, pkv_status_read waits for the stream.)
 * Process-wide state, all of it stated here: (1) the shared-memory opt-in of each kernel is remembered per
 * device, so one process may drive several GPUs (make the device current before the call, as for any
 * CUDA stream); (2) the rounding mode of pkv_set_scale_round_up is one switch for the whole process;
 * (3) pkv_decode_attn_noalloc keeps the address of its built-in scratch per device.  None of it is
 * guarded by a lock: two host threads that race on (1) or (3) store the same value.
 * This is the convention of the reference's own FFI, which launches extern "C" kernels on torch's
 * current stream with caller-owned buffers (phasorkv/kernels/cubin.py:34-55,
 * phasorkv/kernels/latent_attn.py:610-629).  "file:line" citations below are paths inside the
 * reference project and name the Python routine each entry point stands in for.
 *
 * Pointers named *_dev point to device memory of the current device; *_host to host memory.
 */
#ifndef PHASORKV_B200_H
#define PHASORKV_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PKV_PAGE_TOKENS 128          /* tokens per cache page */
#define PKV_MAX_WIDTH   256          /* largest supported latent width W = 2R + R_s */
#ifndef PKV_QUERY_TERMS
#define PKV_QUERY_TERMS 4            /* NVFP4 residual terms of the absorbed query operand */
#endif
#define PKV_NOALLOC_MAX_PARTS 320     /* pkv_decode_attn_noalloc: upper bound on batch * n_split */
#define PKV_SMALL_WRITE_TOKENS 64    /* pkv_cache_write spreads the projection over the GPU up to this n */
#define PKV_VQ_TILE_BYTES 8448       /* quantised V: bytes per (page, kv head): 128 tokens x 64 bytes of codes + 128 bf16 scales */

enum pkv_status {
    PKV_OK = 0,
    PKV_ERR_INVALID = -1,            /* null pointer, negative size, misaligned buffer */
    PKV_ERR_UNSUPPORTED = -2,        /* shape outside what the kernels are built for */
    PKV_ERR_CUDA = -3,               /* a CUDA runtime call failed; see pkv_last_cuda_error */
    PKV_ERR_ARCH = -4                /* the current device is not sm_100 */
};

enum pkv_dtype { PKV_F32 = 0, PKV_BF16 = 1, PKV_F64 = 2 };    /* PKV_F64: pkv_scores_exact only */

/* flags of pkv_decode_attn */
#define PKV_ATTN_SCORES_ONLY 1u      /* K path only: logits and log-sum-exp, V is not read */
#define PKV_ATTN_SIMT        2u      /* CUDA-core scaffold kernel on the fp32 absorbed query */
#define PKV_ATTN_EARLY_STREAM 8u     /* the launch directly before this one on the stream is pkv_absorb (it writes
                                        neither cache nor page table nor lengths): cache pages are streamed
                                        while it still runs, only the query operand is waited for */
#define PKV_ATTN_TAIL_WRITTEN 16u    /* with PKV_ATTN_EARLY_STREAM: the launch before is pkv_decode_prologue, which also
                                        writes the newest token (position seqlen-1) of each sequence: the last page
                                        of a sequence is fetched only after that launch has completed */
#define PKV_ATTN_QUERY_READY 32u     /* pkv_decode_attn_q with PKV_ATTN_EARLY_STREAM: the queries and their positions were
                                        complete before the launch directly before this one was enqueued (they do
                                        not come from it): the kernel absorbs them without waiting for that launch */
#define PKV_ATTN_PACKED_OUT  4u      /* out_dev receives the merged triple [B, n_q, head_dim+2] (o, m, l), not normalised */

/* One layer's factors, in the attribute convention of phasorkv.latent.PhasorKey
 * (phasorkv/latent.py:47-54).  All arrays live in device memory and belong to the caller. */
typedef struct pkv_layer {
    int32_t d_model;                 /* D */
    int32_t n_q, n_kv, head_dim;     /* query heads, kv heads, d */
    int32_t R, R_s, n_slow;          /* complex latent dims, real slow dims, slow frequencies */
    float   attn_scale;              /* rotary attention_scaling (phasorkv/rope.py:31) */
    float   second;                  /* fp32 tensor scale of this layer's NVFP4 latent */
    const float*   Bw_dev;           /* [2R + R_s, D]: rows Re B | Im B | B_s */
    const float*   A_re_dev;         /* [n_kv, R] */
    const float*   A_im_dev;         /* [n_kv, R] */
    const float*   A_s_dev;          /* [n_kv, 2*n_slow, R_s] or NULL */
    const int32_t* freq_dev;         /* [R] frequency index of each complex latent dim */
    const int32_t* slow_dev;         /* [n_slow] or NULL */
    const double*  inv_freq_dev;     /* [head_dim/2] rotary inverse frequencies */
    const void*    Bw_bf16x3_dev;    /* optional bf16 [3][Wp][D], Wp = 128 if 2R+R_s <= 128 else 256: Bw as the sum of
                                        three bf16 matrices (hi, mid, lo; rows past 2R+R_s zero).  Enables the
                                        tensor-core cache write for bf16 x; NULL selects the CUDA-core kernels */
    const float*   second_blocks_dev;/* optional fp32 [(2R+R_s)/16]: the tensor scale of every 16-column block of the
                                        latent, for tiers -- one static scale per 16-aligned span of the
                                        energy-sorted latent, as the reference fixes them offline
                                        (phasorkv/quant.py:119-124, phasorkv/kernels/latent_attn.py:149-152).  The
                                        quantising calls use it in place of `second`; pkv_absorb / the prologue
                                        multiply the query's columns by second_blocks[j] / second, so that the decode
                                        kernels, which know one scale per layer, stay as they are (the fp32 absorbed
                                        rows they write are then in the cache's units, not the reference's).  NULL:
                                        `second` for every block */
} pkv_layer_t;

/* The paged cache of one layer.  A page holds PKV_PAGE_TOKENS tokens.
 *   latent page (pkv_latent_page_bytes(W) bytes, pool base 1024-byte aligned):
 *     codes : 128 rows x RB bytes (RB = 64 if W <= 128 else 128), two E2M1 codes per byte, even
 *             column in the low nibble (phasorkv/kernels/nvfp4.py:34-36); byte `o = row*RB + col/2`
 *             is stored at `o ^ ((o >> 3) & (RB == 128 ? 0x70 : 0x30))`, the shared-memory swizzle
 *             of a K-major tcgen05 operand, so a page is copied to shared memory verbatim.
 *     scales: after the codes, one 512-byte block per 64 columns; the E4M3 scale of row r,
 *             16-column block j sits at `(j/4)*512 + (r%32)*16 + (r/32)*4 + j%4`.
 *   V page: [n_kv][128][head_dim] bf16 (head-major: the 128 x head_dim tile of one kv head is one
 *           contiguous block); the value of (slot, kv head g, dim) sits at element
 *           ((page * n_kv + g) * 128 + row) * head_dim + dim.  pkv_v_write / pkv_cache_write place rows there.
 *   Quantised V page (v_bits = 3 or 2; head_dim 128): n_kv * 66 rows of 128 bytes -- the per-token low-bit tier of
 *           the reference (phasorkv/kernels/nvfp4.py:58-67) applied to each (token, kv head) value row.  Rows
 *           g*64 .. g*64+63 hold the codes of kv head g: 128 E2M1 codes per token, two per byte with the even dim in
 *           the low nibble, 64 bytes per token whose 16-byte chunk c is stored at chunk position c ^ ((row >> 1) & 3);
 *           the rows from n_kv*64 on hold the bf16 scales, 128 per kv head.  pkv_vq_write fills it.
 * A token's place is its *slot*: page_index * 128 + row. */
typedef struct pkv_cache {
    uint8_t* latent_dev;
    void*    v_dev;                  /* bf16, may be NULL when only the K path is used or the V pages are quantised */
    int32_t  n_pages;
    int32_t  W;                      /* 2R + R_s, a multiple of 16, <= PKV_MAX_WIDTH */
    int32_t  n_kv, head_dim;
    void*    vq_dev;                 /* quantised V pool (128-byte aligned) or NULL */
    int32_t  v_bits;                 /* 0: V pages are bf16 in v_dev; 3 or 2: per-token low-bit codes in vq_dev */
} pkv_cache_t;

int pkv_abi_version(void);
const char* pkv_status_string(int status);
/* cudaError_t of the last failing CUDA call made by this library on the calling thread. */
int pkv_last_cuda_error(void);
/* 0 when the current device can run the library (compute capability 10.x), else PKV_ERR_ARCH. */
int pkv_device_check(void);

int64_t pkv_latent_page_bytes(int32_t W);
int64_t pkv_v_page_bytes(int32_t n_kv, int32_t head_dim);

/* Host-side description of a layer for pkv_layer_create: the arrays of phasorkv.latent.PhasorKey
 * (phasorkv/latent.py:47-54) in HOST memory, complex arrays as separate real and imaginary parts. */
typedef struct pkv_layer_host {
    int32_t d_model, n_q, n_kv, head_dim, R, R_s, n_slow;
    float   attn_scale, second;
    const float*   B_re;             /* [R, D] */
    const float*   B_im;             /* [R, D] */
    const float*   B_s;              /* [R_s, D] or NULL */
    const float*   A_re;             /* [n_kv, R] */
    const float*   A_im;             /* [n_kv, R] */
    const float*   A_s;              /* [n_kv, 2*n_slow, R_s] or NULL */
    const int32_t* freq;             /* [R] */
    const int32_t* slow;             /* [n_slow] or NULL */
    const double*  inv_freq;         /* [head_dim/2] */
} pkv_layer_host_t;
/* Layer handle for hosts without a tensor library: uploads the factors (and builds the three bf16
 * terms of the tensor-core cache write) into device memory owned by the handle.  These two calls are
 * the only ones that allocate, free or synchronise; `second` may be changed in the returned struct at
 * any time (it is read at every call).  Python callers fill pkv_layer_t from torch tensors instead. */
int pkv_layer_create(const pkv_layer_host_t* host, pkv_layer_t** out);
int pkv_layer_destroy(pkv_layer_t* layer);

/* Rounding of the E4M3 block scales in every quantising entry point.  0 (default): round to nearest,
 * the reference's default.  1: round up, so that a block's largest element is never clipped by a scale
 * that was rounded down -- the reference's PHASORKV_SCALE_UP=1 (phasorkv/quant.py:57,85-88).  Like
 * there the switch is process-wide; it is taken from the same environment variable at first use unless
 * this call has set it. */
int pkv_set_scale_round_up(int32_t on);

/* NVFP4 quantise-and-pack of given fp32 latent rows into the paged cache: the bit-exact
 * counterpart of quantize_nv_block + pack_nibbles (phasorkv/kernels/nvfp4.py:34-55;
 * rounding rules of phasorkv/quant.py:70-89).  rows_dev [n, W]; slots_dev [n]. */
int pkv_quantize_rows(const pkv_cache_t* cache, const float* rows_dev, const int32_t* slots_dev,
                      int32_t n_tokens, float second, void* stream);
/* The same with one tensor scale per 16-column block (second_blocks_dev fp32 [W/16]): quantize_nv_block applied
 * tier by tier (phasorkv/kernels/latent_attn.py:255-262).  pkv_cache_read_tiered is the matching read-back. */
int pkv_quantize_rows_tiered(const pkv_cache_t* cache, const float* rows_dev, const int32_t* slots_dev,
                             int32_t n_tokens, const float* second_blocks_dev, void* stream);

/* Fused cache write: c = x B^T (complex), rotation by e^{i theta t} * attn_scale, slow block
 * unrotated, NVFP4 quantisation, paged store.  Replaces PhasorKey.write (phasorkv/latent.py:61-70)
 * followed by the quantiser above.  x_dev [n, D] of x_dtype; slots_dev [n].  The phasor of token i is
 * either computed from positions_dev[i] (angle position * inv_freq formed in double, as
 * phasorkv/rope.py:29-32 does) or, when phasors_dev is given, read from it: [n, head_dim/2] complex64
 * (re, im interleaved), the `ph` argument of the reference with attention_scaling already inside.
 * latent_out_dev: optional fp32 [n, W] copy of the unquantised rows (what PhasorKey.write returns);
 * cache may be NULL when only that copy is wanted.
 * scratch_dev: optional fp32 scratch of pkv_write_scratch_floats(n, d_model) floats (16-byte
 * aligned).  When it is given and n <= PKV_SMALL_WRITE_TOKENS (the decode-time write of one token per
 * sequence) the projection is split by latent column and by d_model slice over many SMs and staged
 * through it; otherwise one CTA per 64 tokens does everything on chip and the scratch is not touched.
 * v_rows_dev: optional bf16 value rows [n, n_kv*head_dim] stored into the V pages at the same slots
 * (the same effect as a following pkv_v_write, without a further launch on the small path).
 * Larger n with bf16 x and layer->Bw_bf16x3_dev set run on the tensor cores (128 tokens per CTA,
 * three bf16 passes that reproduce the fp32 factors to 2^-24); status_dev (optional int32[4]) receives
 * a give-up of one of that kernel's bounded waits. */
int pkv_cache_write(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* x_dev, int32_t x_dtype,
                    const int32_t* positions_dev, const float* phasors_dev, const int32_t* slots_dev,
                    int32_t n_tokens, float* latent_out_dev, float* scratch_dev, const void* v_rows_dev,
                    int32_t* status_dev, void* stream);
int64_t pkv_write_scratch_floats(int32_t n_tokens, int32_t d_model);

/* bf16 value rows v_dev [n, n_kv*head_dim] into the V pages at slots_dev [n]. */
int pkv_v_write(const pkv_cache_t* cache, const void* v_dev, const int32_t* slots_dev, int32_t n_tokens,
                void* stream);

/* Quantised V pages (cache->vq_dev, cache->v_bits = 3 or 2): every value row v_dev [n, n_kv*head_dim] bf16 is
 * quantised per (token, kv head) exactly as quantize_per_token does (phasorkv/kernels/nvfp4.py:58-67: one bf16
 * scale = bf16(max(amax, 1e-5) / 3) and integers -4 .. 3 rounded half to even for 3 bits; bf16(max(amax, 1e-5)
 * / 1.5) and levels +-0.5, +-1.5 for 2 bits; E2M1 codes, four bits of storage each) and stored at slots_dev [n].
 * pkv_decode_attn reads such pages when cache->v_bits != 0 (tensor-core kernel only): the codes become E4M3
 * operands (the same numbers), the scales go into the softmax weights, P.V runs on the 8-bit tensor-core path; V
 * costs 528 instead of 2048 bytes per token at 8 kv heads.
 * pkv_vq_read returns, per (token, kv head): rows_out [n, n_kv, 128] fp32 = value(code) * scale,
 * codes_out [n, n_kv, 128] one code per byte, scales_out [n, n_kv] bf16 bit patterns; any may be NULL. */
int64_t pkv_vq_page_bytes(int32_t n_kv, int32_t head_dim);
int pkv_vq_write(const pkv_cache_t* cache, const void* v_dev, const int32_t* slots_dev, int32_t n_tokens, void* stream);
int pkv_vq_read(const pkv_cache_t* cache, const int32_t* slots_dev, int32_t n_tokens, float* rows_out_dev,
                uint8_t* codes_out_dev, uint16_t* scales_out_dev, void* stream);

/* Read tokens back in the reference's layout (tests, debugging): any of the outputs may be NULL.
 * rows_out [n, W] fp32 = value(code) * (scale * second) (phasorkv/kernels/nvfp4.py:55);
 * codes_out [n, W/2] packed nibbles; scales_out [n, W/16] E4M3 bytes. */
int pkv_cache_read(const pkv_cache_t* cache, const int32_t* slots_dev, int32_t n_tokens, float second,
                   float* rows_out_dev, uint8_t* codes_out_dev, uint8_t* scales_out_dev, void* stream);
int pkv_cache_read_tiered(const pkv_cache_t* cache, const int32_t* slots_dev, int32_t n_tokens,
                          const float* second_blocks_dev, float* rows_out_dev, uint8_t* codes_out_dev,
                          uint8_t* scales_out_dev, void* stream);

/* The same entry points under the names of the reference's vocabulary: pkv_quantize_nvfp4 is
 * pkv_quantize_rows (quantize_nv_block, phasorkv/kernels/nvfp4.py:43-55); pkv_dequant is pkv_cache_read
 * with the fp32 rows only (nvfp4.py:55).  pkv_status_read copies the 4 status words a kernel may have
 * written (0 = fine; 1 = a pipeline wait gave up, 2 = page index outside the pool, 3 = a peer never
 * delivered; word 1 says where) to host memory and waits for the stream: the one call that synchronises. */
int pkv_quantize_nvfp4(const pkv_cache_t* cache, const float* rows_dev, const int32_t* slots_dev, int32_t n_tokens,
                       float second, void* stream);
int pkv_dequant(const pkv_cache_t* cache, const int32_t* slots_dev, int32_t n_tokens, float second,
                float* rows_out_dev, void* stream);
int pkv_status_read(const int32_t* status_dev, int32_t* status_host, void* stream);

/* Query absorption, PhasorKey.absorb for one query position per sequence
 * (phasorkv/latent.py:72-83).  q_dev [B, n_q, head_dim] fp32 pre-RoPE; positions_dev [B] or, as for
 * pkv_cache_write, phasors_dev [B, head_dim/2] complex64 (one of the two must be given).
 * qabs_out_dev: optional fp32 [B, n_q, W] in the reference layout [Re q' | Im q' | slow].
 * qop_out_dev: optional tensor-core operand, pkv_query_operand_bytes(W) per sequence: the absorbed
 * query as PKV_QUERY_TERMS NVFP4 residual terms that share one fp32 tensor scale per head: a
 * 128-row tile (row = term*32 + head) in exactly the layout of a cache page, then the 32 per-head
 * tensor scales (padded to 512 bytes). */
int pkv_absorb(const pkv_layer_t* layer, const float* q_dev, const int32_t* positions_dev,
               const float* phasors_dev, int32_t batch, float* qabs_out_dev, uint8_t* qop_out_dev, void* stream);
int64_t pkv_query_operand_bytes(int32_t W);

/* The reference's calls in the precision of their arguments, without quantisation -- what host code written
 * against phasorkv.latent.PhasorKey and its exactness statement (README.md:75-77) expect.  Plain CUDA-core
 * kernels, not the decode path.
 *   pkv_scores_exact    PhasorKey.scores (phasorkv/latent.py:85-88): out [n_query_rows, n_tokens] =
 *                       q_abs [n_query_rows, W] . rows [n_tokens, W]^T, all of `dtype` PKV_F32 or PKV_F64.
 *   pkv_write_rows_f64  PhasorKey.write for fp64 x (phasorkv/latent.py:63-64 keeps fp64): Bw_dev [2R+R_s, D]
 *                       (rows Re B | Im B | B_s), x_dev [n, D], phasors_dev [n, half_dim] complex128
 *                       (re, im interleaved) -> rows_out_dev [n, 2R+R_s].  fp32 / bf16 x go to pkv_cache_write.
 *   pkv_absorb_rows_f64 PhasorKey.absorb for fp64 q (phasorkv/latent.py:72-83): q_dev [n_positions, n_q,
 *                       head_dim], phasors_dev [n_positions, head_dim/2] complex128 -> out_dev
 *                       [n_positions, n_q, 2R+R_s]; A_re/A_im [n_kv, R], A_s [n_kv, 2*n_slow, R_s]. */
int pkv_scores_exact(const void* q_abs_dev, const void* rows_dev, int32_t n_query_rows, int32_t n_tokens, int32_t W,
                     int32_t dtype, void* out_dev, void* stream);
int pkv_write_rows_f64(const double* Bw_dev, const int32_t* freq_dev, int32_t d_model, int32_t R, int32_t R_s,
                       int32_t half_dim, const double* x_dev, const double* phasors_dev, int32_t n_tokens,
                       double* rows_out_dev, void* stream);
int pkv_absorb_rows_f64(const double* A_re_dev, const double* A_im_dev, const double* A_s_dev, const int32_t* freq_dev,
                        const int32_t* slow_dev, int32_t n_q, int32_t n_kv, int32_t head_dim, int32_t R, int32_t R_s,
                        int32_t n_slow, const double* q_dev, const double* phasors_dev, int32_t n_positions,
                        double* out_dev, void* stream);

/* The two calls a decode step makes before it attends -- pkv_cache_write of the newest token of each
 * of the `batch` sequences (x_dev [batch, d_model], write_positions_dev / slots_dev / v_rows_dev
 * [batch]) and pkv_absorb of the step's queries (q_dev at query_positions_dev [batch]) -- as ONE
 * launch: the reference's per-layer patch makes them back to back (PhasorKey.write, then
 * PhasorKey.absorb: phasorkv/latent.py:57-83) and neither depends on the other. The absorbed queries are
 * those of pkv_absorb bit for bit; the latent rows are those of pkv_cache_write up to the order in which a
 * row's partial sums are added (the last bit of a value may differ; the stored codes and scales are the
 * quantiser's bits of the rows this call forms). The single launch needs batch <= PKV_SMALL_WRITE_TOKENS, R a
 * multiple of 16 and d_model a multiple of 32 and at most 16384; otherwise the two separate launches
 * are made (scratch_dev, optional, is only used then). latent_out_dev, qabs_out_dev, qop_out_dev,
 * v_rows_dev are optional as in the separate calls (with quantised V pages, cache->v_bits != 0, the value rows
 * are quantised and stored by the same launch, bit for bit as pkv_vq_write does). q_dev NULL: the write alone
 * (the queries are then absorbed by pkv_decode_attn_q). */
int pkv_decode_prologue(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* x_dev, int32_t x_dtype,
                        const int32_t* write_positions_dev, const int32_t* slots_dev, const void* v_rows_dev,
                        const float* q_dev, const int32_t* query_positions_dev, int32_t batch,
                        float* latent_out_dev, float* scratch_dev, float* qabs_out_dev, uint8_t* qop_out_dev,
                        int32_t* status_dev, void* stream);

/* Decode attention on the latent cache: scores (PhasorKey.scores, phasorkv/latent.py:85-88),
 * softmax(S * head_dim^-0.5) and P.V with kv heads shared by n_q/n_kv query heads
 * (phasorkv/metrics.py:23,29-35), as split-T flash decoding.
 *   q_dev       : fp32 [B, n_q, W] (PKV_ATTN_SIMT) or the operand blob written by pkv_absorb
 *   page_table  : [B, max_pages] page indices; seqlens [B] tokens per sequence
 *   partials    : scratch AND result, fp32 [B, n_split, n_q, head_dim + 2]: per split the
 *                 unnormalised output o[head_dim], the maximum m of the base-2 logits and
 *                 l = sum 2^(s - m)
 *   scores_out  : optional fp32 [B, n_q, scores_stride] unscaled scores (tests)
 *   status_dev  : optional int32[4]; kernels record a give-up of a bounded wait or an index out
 *                 of range here instead of trapping
 *   out_dev     : optional fp32 [B, n_q, head_dim] (with PKV_ATTN_PACKED_OUT: [B, n_q, head_dim+2], the
 *                 not normalised triple a rank of a token-sharded sequence hands to the exchange);
 *                 when given, the splits are merged as well (pkv_merge on `partials`, enqueued
 *                 right behind the attention kernel) */
int pkv_decode_attn(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* q_dev,
                    const int32_t* page_table_dev, int32_t max_pages, const int32_t* seqlens_dev,
                    int32_t batch, int32_t n_split, uint32_t flags, float* partials_dev,
                    float* scores_out_dev, int64_t scores_stride, int32_t* status_dev, float* out_dev,
                    void* stream);

/* Operand-ready counters: the three calls of a decode step with one more argument, qsync_dev -- int32
 * [2 * batch] in device memory, zero before its first use, owned by the caller, one array per operand buffer.
 * pkv_absorb_sync / pkv_decode_prologue_sync raise qsync_dev[b] once for each group of 8 query heads of
 * sequence b whose operand rows are in place; pkv_decode_attn_sync (tensor-core kernel, PKV_ATTN_EARLY_STREAM
 * required, launched directly behind one of the two on the same stream) then polls that counter (bounded; a
 * give-up is status 1 / where 11) instead of waiting for the whole launch before it: the attention starts as
 * soon as the queries are absorbed, while e.g. the prologue's cache write of the newest token still runs
 * (the last page of a sequence is still only fetched after that launch has completed, PKV_ATTN_TAIL_WRITTEN).
 * The attention launch clears the counters when its last CTA of a sequence is done with the operand.
 * qsync_dev NULL: exactly the plain calls.  No counterpart in the reference (its host waits for whole
 * launches). */
int pkv_absorb_sync(const pkv_layer_t* layer, const float* q_dev, const int32_t* positions_dev, const float* phasors_dev,
                    int32_t batch, float* qabs_out_dev, uint8_t* qop_out_dev, int32_t* qsync_dev, void* stream);
int pkv_decode_prologue_sync(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* x_dev, int32_t x_dtype,
                             const int32_t* write_positions_dev, const int32_t* slots_dev, const void* v_rows_dev,
                             const float* q_dev, const int32_t* query_positions_dev, int32_t batch,
                             float* latent_out_dev, float* scratch_dev, float* qabs_out_dev, uint8_t* qop_out_dev,
                             int32_t* qsync_dev, int32_t* status_dev, void* stream);
int pkv_decode_attn_sync(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* q_dev, int32_t* qsync_dev,
                         const int32_t* page_table_dev, int32_t max_pages, const int32_t* seqlens_dev,
                         int32_t batch, int32_t n_split, uint32_t flags, float* partials_dev,
                         float* scores_out_dev, int64_t scores_stride, int32_t* status_dev, float* out_dev,
                         void* stream);

/* pkv_decode_attn on RAW queries: q_dev [B, n_q, head_dim] fp32 pre-RoPE at query_positions_dev [B].
 * The tensor-core kernel absorbs them itself (every CTA forms the NVFP4 operand of its sequence in
 * shared memory with the arithmetic of pkv_absorb: same bits, same results) - no pkv_absorb launch, no
 * operand in global memory.  Flags as for pkv_decode_attn except PKV_ATTN_SIMT (unsupported);
 * PKV_ATTN_EARLY_STREAM here means that the launch directly before writes neither page table nor
 * lengths nor cache rows (except, with PKV_ATTN_TAIL_WRITTEN, rows of each sequence's last page), and
 * the queries are waited for unless PKV_ATTN_QUERY_READY is given as well. */
int pkv_decode_attn_q(const pkv_layer_t* layer, const pkv_cache_t* cache, const float* q_dev,
                      const int32_t* query_positions_dev, const int32_t* page_table_dev, int32_t max_pages,
                      const int32_t* seqlens_dev, int32_t batch, int32_t n_split, uint32_t flags, float* partials_dev,
                      float* scores_out_dev, int64_t scores_stride, int32_t* status_dev, float* out_dev, void* stream);

/* Log-sum-exp merge of n_parts partial triples per (sequence, head): M = max m, w = 2^(m - M),
 * O = sum w o / sum w l (phasorkv/kernels/dense_attn.py:72-74).  parts_dev is addressed as
 * parts[b*stride_b + p*stride_p + head*(head_dim+2) + i].  out_dev: optional normalised
 * [B, n_q, head_dim]; packed_out_dev: optional merged triple [B, n_q, head_dim+2] (what a rank
 * contributes to the all-gather of a token-sharded sequence). */
int pkv_merge(const float* parts_dev, int64_t stride_b, int64_t stride_p, int32_t n_parts, int32_t batch,
              int32_t n_q, int32_t head_dim, float* out_dev, float* packed_out_dev, void* stream);

/* Exact-token side path: the tokens a serving stack keeps as rotated bf16 keys instead of latent rows
 * (attention sinks, the recent window) take part in the same softmax
 * (phasorkv/kernels/latent_attn.py:448-495,548-596: exact = (k, v) bf16 [B, n_kv, E, d], k after RoPE).
 * pkv_exact_partial forms their partial triple (o unnormalised, base-2 max m, sum l) per (sequence,
 * head) into exact_out_dev [B, n_q, head_dim+2]; pkv_merge_exact is pkv_merge with that triple as one
 * more part (exact_dev NULL: plain pkv_merge).
 *   q_dev [B, n_q, head_dim] fp32 pre-RoPE, rotated by the kernel to positions_dev [B] (double angle,
 *   the layer's attn_scale; band layouts leave their slow frequencies unrotated, as the keys are);
 *   k_exact_dev, v_exact_dev bf16 [B, n_kv, e_max, head_dim], n_exact_dev [B] valid tokens (NULL: e_max).
 * Limits: e_max <= 512, head_dim <= 128, at most 8 query heads per kv head. */
int pkv_exact_partial(const pkv_layer_t* layer, const float* q_dev, const int32_t* positions_dev,
                      const void* k_exact_dev, const void* v_exact_dev, const int32_t* n_exact_dev, int32_t e_max,
                      int32_t batch, float* exact_out_dev, void* stream);
int pkv_merge_exact(const float* parts_dev, int64_t stride_b, int64_t stride_p, int32_t n_parts, int32_t batch,
                    int32_t n_q, int32_t head_dim, const float* exact_dev, float* out_dev, float* packed_out_dev,
                    void* stream);

/* Token-sharded sequences (the token axis of every sequence split over the GPUs of one box; no
 * counterpart in the reference, which is single-GPU): exchange of the per-rank merged triples
 * [B, n_q, head_dim+2] over NVLink peer memory and their merge, in one launch per rank.
 * The caller provides, on every rank, memory that all ranks can address (CUDA IPC, or
 * torch.distributed._symmetric_memory): a gather buffer of 8-byte words
 *   data : uint64 [2][world][B*n_q*(head_dim+2)], zero at start, 8-byte aligned
 * (low half: a float of a triple; high half: the number of the exchange it belongs to, so that a
 * value and its "arrived" mark travel in one store) and passes a device array with the addresses of
 * all ranks' copies.  epoch_dev is local, uint32 [n_cta], zero at start.  All ranks must call with the
 * same shapes, the same n_cta and the same number of calls.  A rank waits for its peers' words with a
 * bounded poll; when it gives up, status[0] = 3 and out is left incomplete.  phases = PUSH | MERGE in
 * production; the two phases can be launched separately (all pushes, then all merges) to drive
 * several ranks' buffers from one GPU in tests. */
#define PKV_EXCHANGE_PUSH  1u
#define PKV_EXCHANGE_MERGE 2u
typedef struct pkv_exchange {
    int32_t world, rank;
    int32_t batch, n_q, head_dim;
    int32_t n_cta;                       /* CTAs of the launch; the rows = batch*n_q are split evenly over them */
    void* const*     peer_data_dev;      /* device array [world]: address of rank r's gather buffer */
    uint32_t*        epoch_dev;          /* local, [n_cta] */
} pkv_exchange_t;
int pkv_exchange_merge(const pkv_exchange_t* x, const float* packed_dev, float* out_dev, uint32_t phases,
                       int32_t* status_dev, void* stream);
/* pkv_merge of the local split-T partials (same parts_dev / strides / n_parts as pkv_merge, batch, n_q and
 * head_dim <= 128 taken from x) and pkv_exchange_merge in ONE launch: the merged local triple of a row
 * goes from registers straight to the peers. One CTA per row: x->n_cta must equal batch * n_q (and
 * epoch_dev hold that many counters). A handle is used with either this entry point or
 * pkv_exchange_merge, not both in turn. */
int pkv_merge_exchange(const pkv_exchange_t* x, const float* parts_dev, int64_t stride_b, int64_t stride_p,
                       int32_t n_parts, float* out_dev, int32_t* status_dev, void* stream);

/* Decode attention and merge for callers that cannot allocate device memory (no counterpart in the
 * reference, whose callers always allocate their own scratch with torch).  It is meant for hosts that
 * only ever receive input and output buffers -- a plugin inside another runtime's fixed memory plan, a
 * serving loop after its allocator has been frozen -- and therefore cannot provide the `partials`
 * scratch that pkv_decode_attn asks for.  The scratch lives inside the library instead: a fixed array
 * of PKV_NOALLOC_MAX_PARTS * 32 * 130 floats (about 5.3 MB) in the device memory of every GPU that
 * loads the library, held until the process exits.
 *   - same inputs as pkv_decode_attn with the tensor-core kernel (qop_dev is the operand blob of
 *     pkv_absorb; 32 query heads, head_dim 128, 1, 4 or 8 query heads per kv head) and the V cache
 *     present; the result is the normalised output out_dev [B, n_q, head_dim], as pkv_merge gives
 *   - batch * n_split must not exceed PKV_NOALLOC_MAX_PARTS; larger requests return
 *     PKV_ERR_UNSUPPORTED and do nothing
 *   - the first call on each device looks up the array's address (cudaGetSymbolAddress); make that
 *     first call outside any stream capture.  No call allocates or frees anything.
 *   - all calls on one GPU share the one array: two calls whose kernels may overlap on the GPU
 *     (different streams, different threads) race on it.  Issue them on one stream or serialise
 *     them.  Nothing in the array needs clearing between calls: each call overwrites every slot it
 *     later reads -- also when a CTA of the attention launch gives up (bad page index, a bounded wait
 *     that ran out): it then stores the neutral triple (o = 0, m = -inf, l = 0) in its slot, status_dev
 *     says what happened, and out_dev is then NOT the attention output (rows whose splits all gave up
 *     are zero).  Pass status_dev and check it when the inputs are not trusted. */
int pkv_decode_attn_noalloc(const pkv_layer_t* layer, const pkv_cache_t* cache, const void* qop_dev,
                            const int32_t* page_table_dev, int32_t max_pages, const int32_t* seqlens_dev,
                            int32_t batch, int32_t n_split, float* out_dev, int32_t* status_dev, void* stream);

/* Measurement aid (no counterpart in the reference): reads `bytes` (16-byte aligned buffer) once with plain
 * 16-byte loads from every SM and discards them; sink_dev is one uint32 the kernel may add to.  Timed by
 * the benchmark beside the attention kernel: the bandwidth a pure reader gets on this GPU. */
int pkv_read_probe(const void* src_dev, int64_t bytes, uint32_t* sink_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PHASORKV_B200_H */
