// Per-token low-bit quantisation of one (token, kv head) value row by one warp (the reference's quantize_per_token,
// phasorkv/kernels/nvfp4.py:58-67), shared by the stand-alone writer and the decode-step prologue.
#pragma once
#include "pkv_common.cuh"

// one warp per (token, kv head) row of 128 bf16 values; lane l holds dims 4l .. 4l+3 (`u`: its four values)
__device__ __forceinline__ void pkv_vq_store_row(uint2 u, int lane, int slot, int g, int n_kv, int bits, uint8_t* __restrict__ pool) {
    float x[4] = {pkv_bf16_bits_to_float(u.x & 0xffffu), pkv_bf16_bits_to_float(u.x >> 16), pkv_bf16_bits_to_float(u.y & 0xffffu),
                  pkv_bf16_bits_to_float(u.y >> 16)};
    float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float qmax = bits == 2 ? 1.5f : 3.0f;
    const __nv_bfloat16 sb = __float2bfloat16_rn(__fdiv_rn(fmaxf(amax, 1e-5f), qmax));
    const float s = __bfloat162float(sb);
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float y = __fdiv_rn(x[i], s);
        uint32_t code;
        if (bits == 2) {
            code = (fabsf(y) > 1.0f ? 3u : 1u) | (y < 0.0f ? 8u : 0u);            // +-0.5 / +-1.5, no zero level
        } else {
            const float v = fminf(fmaxf(rintf(y), -4.0f), 3.0f);                   // round half to even, clamp to -4 .. 3
            const int m = (int)fabsf(v);                                           // 0 1 2 3 4 -> E2M1 index 0 2 4 5 6
            code = (m == 0 ? 0u : m == 1 ? 2u : m == 2 ? 4u : m == 3 ? 5u : 6u) | (v < 0.0f ? 8u : 0u);
        }
        packed |= code << (4 * i);
    }
    uint8_t* page = pool + (size_t)(slot / PKV_PAGE_TOKENS) * n_kv * PKV_VQ_TILE_BYTES;
    uint8_t* tile = page + (size_t)g * 8192;
    const uint32_t r = slot % PKV_PAGE_TOKENS;
    const uint32_t chunk = (lane >> 3) ^ ((r >> 1) & 3u);
    *reinterpret_cast<uint16_t*>(tile + r * 64 + chunk * 16 + (lane & 7) * 2) = (uint16_t)packed;
    if (lane == 0) *reinterpret_cast<__nv_bfloat16*>(page + (size_t)n_kv * 8192 + g * 256 + r * 2) = sb;
}
