// Shared definitions of the phasorkv_b200 CUDA library: page layout, NVFP4 arithmetic, error plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/phasorkv_b200.h"

#define PKV_LOG2E 1.4426950408889634f

extern thread_local int g_pkv_last_cuda_error;
int pkv_scale_round_up_mode();     // 1: block scales are rounded up (pkv_set_scale_round_up / PHASORKV_SCALE_UP=1)

#define PKV_CUDA_TRY(expr)                                   \
    do {                                                     \
        cudaError_t e__ = (expr);                            \
        if (e__ != cudaSuccess) {                            \
            g_pkv_last_cuda_error = (int)e__;                \
            return PKV_ERR_CUDA;                             \
        }                                                    \
    } while (0)

#define PKV_LAUNCH_CHECK() PKV_CUDA_TRY(cudaGetLastError())

// Opt-in to more than 48 KB of dynamic shared memory. The attribute belongs to a (kernel, device) pair, so
// it is set once per kernel on every device this process launches on (a process may drive several GPUs);
// `done` is the kernel's own flag table. The race of two host threads on a flag is benign: both set the
// same attribute value.
constexpr int PKV_MAX_DEVICES = 64;
struct pkv_attr_flags { bool done[PKV_MAX_DEVICES]; };
template <typename K>
inline cudaError_t pkv_set_max_smem(K kern, int bytes, pkv_attr_flags& f) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < PKV_MAX_DEVICES && f.done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && dev >= 0 && dev < PKV_MAX_DEVICES) f.done[dev] = true;
    return e;
}

// ------------------------------------------------------------------------------------------------
// Programmatic dependent launch. The kernels of a decode step form a chain on one stream; each is
// launched with the "programmatic stream serialization" attribute, lets its successor come onto the
// SMs early (pkv_grid_launch_dependents) and waits for the complete result of its predecessor
// (pkv_grid_wait) before it touches global data. One kernel, pkv_absorb, triggers only AFTER its own
// wait: the attention kernel behind it may then stream cache pages before waiting, knowing that every
// kernel up to absorb's predecessor (the cache writers) has completed.
// A kernel launched without the attribute sees both calls as no-ops.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void pkv_grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pkv_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t pkv_launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                      Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ------------------------------------------------------------------------------------------------
// page layout (documented in include/phasorkv_b200.h)
// ------------------------------------------------------------------------------------------------

__host__ __device__ __forceinline__ int pkv_padded_width(int W) { return W <= 128 ? 128 : 256; }
__host__ __device__ __forceinline__ int pkv_row_bytes(int W) { return pkv_padded_width(W) / 2; }
__host__ __device__ __forceinline__ int pkv_codes_bytes(int W) { return PKV_PAGE_TOKENS * pkv_row_bytes(W); }
__host__ __device__ __forceinline__ int pkv_scales_bytes(int W) { return (pkv_padded_width(W) / 64) * 512; }
__host__ __device__ __forceinline__ int pkv_page_bytes(int W) { return pkv_codes_bytes(W) + pkv_scales_bytes(W); }

// byte offset inside the code region of (row, byte column) for a row pitch of RB bytes: the
// 128-byte (RB = 128) or 64-byte (RB = 64) shared-memory swizzle applied to the linear offset
__host__ __device__ __forceinline__ uint32_t pkv_code_offset(uint32_t row, uint32_t byte_col, uint32_t RB) {
    uint32_t o = row * RB + byte_col;
    return o ^ ((o >> 3) & (RB == 128 ? 0x70u : 0x30u));
}

// V pool: per page [n_kv][128 tokens][head_dim] bf16, so that the tile of one (page, kv head) is one contiguous
// block (a token-major page makes every tile 128 rows of 2 * head_dim bytes at a stride of the whole token
// row: measured 2 % slower to stream). Index, in 16-byte vectors, of vector c of the value row of `slot`
// (a row has n_kv * vec_per_head vectors, vec_per_head = head_dim / 8).
__host__ __device__ __forceinline__ size_t pkv_v_vec_index(int slot, int c, int n_kv, int vec_per_head) {
    const int page = slot / PKV_PAGE_TOKENS, r = slot % PKV_PAGE_TOKENS, g = c / vec_per_head, w = c % vec_per_head;
    return (((size_t)page * n_kv + g) * PKV_PAGE_TOKENS + r) * vec_per_head + w;
}

// byte offset inside the scale region of (row, 16-column block j)
__host__ __device__ __forceinline__ uint32_t pkv_scale_offset(uint32_t row, uint32_t j) {
    return (j >> 2) * 512u + (row & 31u) * 16u + (row >> 5) * 4u + (j & 3u);
}

// ------------------------------------------------------------------------------------------------
// NVFP4 arithmetic. Every step is a single correctly rounded fp32 operation in the order the
// reference performs it (phasorkv/kernels/nvfp4.py:49-55): no reciprocal, no fused multiply-add.
// ------------------------------------------------------------------------------------------------

__device__ __forceinline__ float pkv_e4m3_to_float(uint8_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
}

// round to nearest even with saturation; the input is already clamped to [0, 448]
__device__ __forceinline__ uint8_t pkv_float_to_e4m3(float x) {
    return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ float pkv_e2m1_value(uint32_t code) {
    // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 : code bits 0-2 (2 exponent bits, bias 1, and 1 mantissa bit), sign bit 3.
    // The float is assembled from its fields (integer ALU only: int -> float conversions share a slow pipe):
    // exponent field e >= 1 -> 2^(e-1) * (1 + mant/2); e == 0 -> mant * 0.5
    const uint32_t e = (code >> 1) & 3u, mant = code & 1u;
    const uint32_t bits = e ? (((126u + e) << 23) | (mant << 22)) : (mant ? 0x3F000000u : 0u);
    return __uint_as_float(bits | ((code & 8u) << 28));
}

// E4M3 scale byte of a block with the given max magnitude
// round_up (PHASORKV_SCALE_UP=1 of the reference, phasorkv/quant.py:57,85-88): a scale that round-to-nearest put
// below the unclamped ratio moves one E4M3 step up, so the block maximum is never clipped. Consecutive
// non-negative E4M3 values are consecutive bytes; 0x7e (448) is the largest.
__device__ __forceinline__ uint8_t pkv_block_scale_byte(float amax, float second, bool round_up = false) {
    const float ratio = __fdiv_rn(__fdiv_rn(amax, 6.0f), second);
    uint8_t b = pkv_float_to_e4m3(fminf(fmaxf(ratio, 0.0f), 448.0f));
    if (round_up && pkv_e4m3_to_float(b) < ratio && b < 0x7e) ++b;
    return b;
}

// E2M1 code of x under `scale` (= e4m3 * second): midpoints are compared with ">" so that an
// exact tie takes the lower magnitude, and a value that rounds to zero carries no sign
__device__ __forceinline__ uint32_t pkv_e2m1_code(float x, float scale) {
    if (!(scale > 0.0f)) return 0u;
    float y = __fdiv_rn(x, fmaxf(scale, 1e-30f));
    float a = fabsf(y);
    uint32_t idx = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
    return idx | ((idx != 0u && y < 0.0f) ? 8u : 0u);
}

// The fp32 tensor scale of block j of a latent row: one per layer, or one per 16-column block (tiers)
struct pkv_second {
    float s;
    const float* blocks;
    __device__ __forceinline__ float of(int j) const { return blocks ? blocks[j] : s; }
};
inline pkv_second pkv_second_of(const pkv_layer_t* L) { return pkv_second{L->second, L->second_blocks_dev}; }

// quantise 16 consecutive values; returns the 8 packed code bytes (low nibble = even column)
__device__ __forceinline__ uint2 pkv_quantize_block16(const float (&v)[16], float second, uint8_t& scale_byte,
                                                      bool round_up = false) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    scale_byte = pkv_block_scale_byte(amax, second, round_up);
    float scale = __fmul_rn(pkv_e4m3_to_float(scale_byte), second);
    uint32_t lo = 0u, hi = 0u;
#pragma unroll
    for (int i = 0; i < 8; ++i) lo |= pkv_e2m1_code(v[i], scale) << (4 * i);
#pragma unroll
    for (int i = 0; i < 8; ++i) hi |= pkv_e2m1_code(v[8 + i], scale) << (4 * i);
    return make_uint2(lo, hi);
}

__device__ __forceinline__ float pkv_bf16_bits_to_float(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
