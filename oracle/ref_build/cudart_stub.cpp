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
cudaError_t cudaMemcpy(void* d, const void* s, size_t n, cudaMemcpyKind) {
    memcpy(d, s, n);
    return cudaSuccess;
}

// The reference's importance_scorer.cu is compiled by nvcc, so its object registers a device binary
// and launches one kernel.  Registration is a no-op here.  The only kernel these libraries can launch
// is importance_update_kernel(scores, new_scores, num_blocks, decay)
// (src/memoria/importance_scorer.cu:27-37); so that scores can be fed to the reference's host-side
// policy code without a GPU, the launch applies that kernel's one statement on the host, fused the
// way the device compiler contracts it.  (The kernel's arithmetic itself is checked on a GPU.)
void** __cudaRegisterFatBinary(void*) { static void* handle = nullptr; return &handle; }
void __cudaRegisterFatBinaryEnd(void**) {}
void __cudaUnregisterFatBinary(void**) {}
void __cudaRegisterFunction(void**, const char*, char*, const char*, int, void*, void*, void*, void*, int*) {}
char __cudaInitModule(void**) { return 0; }
static dim3 g_grid, g_block;
unsigned __cudaPushCallConfiguration(dim3 grid, dim3 block, size_t, struct CUstream_st*) {
    g_grid = grid;
    g_block = block;
    return 0;
}
cudaError_t __cudaPopCallConfiguration(dim3* grid, dim3* block, size_t* smem, void* stream) {
    *grid = g_grid;
    *block = g_block;
    *smem = 0;
    *(cudaStream_t*)stream = nullptr;
    return cudaSuccess;
}
cudaError_t cudaLaunchKernel(const void*, dim3, dim3, void** args, size_t, cudaStream_t) {
    float* scores = *(float**)args[0];
    const float* fresh = *(const float**)args[1];
    const int n = *(int*)args[2];
    const float decay = *(float*)args[3];
    for (int b = 0; b < n; b++) scores[b] = __builtin_fmaf(scores[b], decay, fresh[b]);
    return cudaSuccess;
}

}  // extern "C"
