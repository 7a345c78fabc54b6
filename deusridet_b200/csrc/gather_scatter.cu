// gather_scatter.cu — flat <-> paged K/V copies (SSD staging, prefix store / restore).
//
// B200 versions of extract_kv_from_pages_kernel / inject_kv_to_pages_kernel
// (src/memoria/cache_kernels.cu:30-141): the reference moves one fp16 element per thread with
// 32-bit index arithmetic (overflows beyond 2^31 elements); here one thread moves a 16-byte vector
// and every index is 64-bit.  Flat layout [layer][K|V][token][kv_head][dim]
// (src/memoria/cache_kernels.h:29).  A token whose table entry is < 0 reads as zeros on extract
// (cache_kernels.cu:66-69) and is skipped on inject (cache_kernels.cu:127).
// Pure data movement: HBM-bound, 2 bytes moved per byte of payload (one read, one write).
#include "kernels.hpp"
#include "kv_common.cuh"

namespace drkv {

namespace {

template <bool TO_FLAT>
__global__ void __launch_bounds__(256) flat_paged_copy_kernel(const FlatCopyParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const int D8 = p.layout.head_dim / 8;                       // 16-byte vectors per head row
    const int64_t per_token = (int64_t)p.layout.num_kv_heads * D8;
    const int64_t per_kv = (int64_t)p.num_tokens * per_token;
    const int64_t per_layer = 2 * per_kv;
    const int64_t total = (int64_t)p.num_layers * per_layer;
    char* flat = reinterpret_cast<char*>(p.flat);
    char* pool = reinterpret_cast<char*>(p.pool);
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        int64_t rem = idx;
        const int layer = (int)(rem / per_layer);
        rem -= (int64_t)layer * per_layer;
        const int kv = (int)(rem / per_kv);
        rem -= (int64_t)kv * per_kv;
        const int tok = (int)(rem / per_token);
        rem -= (int64_t)tok * per_token;
        const int head = (int)(rem / D8), d8 = (int)(rem - (int64_t)head * D8);
        const int pos = p.start_token + tok;
        const int logical = pos / p.layout.page_size, slot = pos - logical * p.layout.page_size;
        int page = -1;
        if (logical < p.table_stride) page = p.table[logical];
        if (page >= p.layout.max_pages) page = -1;
        if (TO_FLAT) {
            Vec16 v = {{0u, 0u, 0u, 0u}};
            if (page >= 0) v = ldg16(pool + (p.layout.row(layer, page, kv, head, slot) + 8 * d8) * 2);
            stg16(flat + idx * 16, v);
        } else if (page >= 0) {
            stg16(pool + (p.layout.row(layer, page, kv, head, slot) + 8 * d8) * 2, ldg16(flat + idx * 16));
        }
    }
}

}  // namespace

cudaError_t launch_flat_paged_copy(const FlatCopyParams& p, bool to_flat, int num_sms, cudaStream_t stream) {
    const int64_t total = (int64_t)p.num_layers * 2 * p.num_tokens * p.layout.num_kv_heads * (p.layout.head_dim / 8);
    if (total <= 0) return cudaSuccess;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)num_sms * 16;                  // grid-stride beyond 16 CTAs per SM
    if (blocks > cap) blocks = cap;
    if (to_flat) return launch_pdl(flat_paged_copy_kernel<true>, dim3((unsigned)blocks), dim3(256), 0, stream, p);
    return launch_pdl(flat_paged_copy_kernel<false>, dim3((unsigned)blocks), dim3(256), 0, stream, p);
}

}  // namespace drkv
