// Host-memory stand-ins for the few CUDA runtime calls that the reference's
// Memoria host sources make (block_pool.cpp, cache_manager.cpp, kv_swapper.cpp).
// Test infrastructure only: lets those sources run unmodified on a machine
// without a GPU so that their block tables, free counts and eviction order can
// be recorded.  "Device" memory is plain malloc memory, streams are dummies.
#include <cuda_runtime.h>
#include <cstdlib>
#include <cstring>

extern "C" {

cudaError_t cudaMalloc(void** p, size_t n) {
    // The reference zero-fills the slab right after; calloc keeps large pools cheap
    // (untouched pages are never committed).
    *p = calloc(n ? n : 1, 1);
    return *p ? cudaSuccess : cudaErrorMemoryAllocation;
}
cudaError_t cudaFree(void* p) { free(p); return cudaSuccess; }
cudaError_t cudaMemset(void* p, int v, size_t n) {
    if (v != 0) memset(p, v, n);   // calloc'd memory is already zero
    return cudaSuccess;
}
cudaError_t cudaMemcpyAsync(void* d, const void* s, size_t n, cudaMemcpyKind, cudaStream_t) {
    memcpy(d, s, n);
    return cudaSuccess;
}
const char* cudaGetErrorString(cudaError_t) { return "stub"; }
cudaError_t cudaHostAlloc(void** p, size_t n, unsigned) {
    *p = malloc(n ? n : 1);
    return *p ? cudaSuccess : cudaErrorMemoryAllocation;
}
cudaError_t cudaFreeHost(void* p) { free(p); return cudaSuccess; }
cudaError_t cudaStreamCreate(cudaStream_t* s) { *s = (cudaStream_t)0x1; return cudaSuccess; }
cudaError_t cudaStreamDestroy(cudaStream_t) { return cudaSuccess; }
cudaError_t cudaStreamSynchronize(cudaStream_t) { return cudaSuccess; }

}  // extern "C"
