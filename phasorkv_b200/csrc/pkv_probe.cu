// A plain read-only stream over a buffer: what the memory system gives a kernel that only reads, as a
// yardstick beside the copy bandwidth (read + write) that roofline fractions are usually quoted against.
// The decode attention kernel is such a reader; the benchmark times this probe in the same run.
#include "pkv_common.cuh"

namespace {

__global__ void __launch_bounds__(512) pkv_read_probe_kernel(const uint4* __restrict__ src, size_t n_vec, uint32_t* __restrict__ sink) {
    uint32_t acc = 0;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n_vec; i += 4 * stride) {            // four independent 16-byte loads in flight per thread
        const uint4 a = __ldcs(src + i), b = __ldcs(src + i + stride), c = __ldcs(src + i + 2 * stride),
                    d = __ldcs(src + i + 3 * stride);
        acc ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c.x ^ c.y ^ c.z ^ c.w ^ d.x ^ d.y ^ d.z ^ d.w;
    }
    for (; i < n_vec; i += stride) {
        const uint4 a = __ldcs(src + i);
        acc ^= a.x ^ a.y ^ a.z ^ a.w;
    }
    if (acc == 0x9e3779b9u) atomicAdd(sink, 1u);                 // keeps the loads alive; practically never taken
}

}  // namespace

extern "C" int pkv_read_probe(const void* src_dev, int64_t bytes, uint32_t* sink_dev, void* stream) {
    if (!src_dev || !sink_dev || bytes < 0 || (((uintptr_t)src_dev) & 15u)) return PKV_ERR_INVALID;
    if (bytes < 16) return PKV_OK;
    int dev = 0, sms = 0;
    PKV_CUDA_TRY(cudaGetDevice(&dev));
    PKV_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    pkv_read_probe_kernel<<<sms * 4, 512, 0, (cudaStream_t)stream>>>((const uint4*)src_dev, (size_t)(bytes / 16), sink_dev);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}
