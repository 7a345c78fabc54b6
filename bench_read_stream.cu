// bench_read_stream.cu — measurement helper of bench.py, not part of the library: read-only streaming bandwidth
// of the device the caller is on, the second denominator the decode roofline is quoted against (the reference
// measures its ceiling the same way: a kernel that only reads and sums, tools/probe_bw.cu:18-28, timed with
// events over repeated launches, :99-113).  A copy (read + write) understates what a read-mostly kernel can
// reach.  bench.py builds this file into libbench_read_stream.so next to itself.
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace {

// 4 independent 16-byte loads in flight per thread and trip, grid-stride over the buffer.
__global__ void __launch_bounds__(512) read_stream_kernel(const uint4* __restrict__ src, size_t n, uint32_t* sink) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t acc = 0;
    for (; i + 3 * stride < n; i += 4 * stride) {
        const uint4 a = __ldg(src + i), b = __ldg(src + i + stride), c = __ldg(src + i + 2 * stride), d = __ldg(src + i + 3 * stride);
        acc ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c.x ^ c.y ^ c.z ^ c.w ^ d.x ^ d.y ^ d.z ^ d.w;
    }
    for (; i < n; i += stride) {
        const uint4 a = __ldg(src + i);
        acc ^= a.x ^ a.y ^ a.z ^ a.w;
    }
    if (acc == 0x9e3779b9u) *sink = acc;             // keeps the loads alive; practically never taken
}

}  // namespace

// GB/s over `bytes` of device memory at `buf` (use more than the L2 holds): CUDA events around `iters` launches after
// two warm-ups.  Returns 0, or a negative number / a cudaError_t value on failure.
extern "C" __attribute__((visibility("default"))) int bench_read_stream_gbs(const void* buf, size_t bytes, int iters,
                                                                            void* stream_, double* gb_per_s) {
    if (!buf || bytes < (1u << 20) || iters < 1 || !gb_per_s) return -1;
    cudaStream_t stream = (cudaStream_t)stream_;
    int dev = 0, sms = 0;
    uint32_t* sink = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce == cudaSuccess) ce = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (ce == cudaSuccess) ce = cudaMalloc(&sink, sizeof(uint32_t));
    if (ce == cudaSuccess) ce = cudaEventCreate(&e0);
    if (ce == cudaSuccess) ce = cudaEventCreate(&e1);
    float ms = 0.f;
    if (ce == cudaSuccess) {
        const size_t n = bytes / sizeof(uint4);
        const int grid = sms * 4;                    // 4 CTAs of 512 threads per SM
        for (int i = 0; i < 2; i++) read_stream_kernel<<<grid, 512, 0, stream>>>(static_cast<const uint4*>(buf), n, sink);
        cudaEventRecord(e0, stream);
        for (int i = 0; i < iters; i++) read_stream_kernel<<<grid, 512, 0, stream>>>(static_cast<const uint4*>(buf), n, sink);
        cudaEventRecord(e1, stream);
        ce = cudaEventSynchronize(e1);
        if (ce == cudaSuccess) ce = cudaEventElapsedTime(&ms, e0, e1);
        if (ce == cudaSuccess) ce = cudaGetLastError();
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (sink) cudaFree(sink);
    if (ce != cudaSuccess) return (int)ce;
    *gb_per_s = (double)(bytes / sizeof(uint4) * sizeof(uint4)) * iters / (ms * 1e-3) / 1e9;
    return 0;
}
