// gather_scatter.cu — flat <-> paged K/V copies (SSD staging, prefix store / restore).
//
// B200 versions of extract_kv_from_pages_kernel / inject_kv_to_pages_kernel
// (src/memoria/cache_kernels.cu:30-141): the reference moves one fp16 element per thread with
// 32-bit index arithmetic (overflows beyond 2^31 elements); here a warp moves a token's K or V rows in
// 16-byte vectors and every index is 64-bit.  Flat layout [layer][K|V][token][kv_head][dim]
// (src/memoria/cache_kernels.h:29).  A token whose table entry is < 0 reads as zeros on extract
// (cache_kernels.cu:66-69) and is skipped on inject (cache_kernels.cu:127).
// Pure data movement: HBM-bound, 2 bytes moved per byte of payload (one read, one write).
#include "kernels.hpp"
#include "kv_common.cuh"

namespace drkv {

namespace {

// One warp per (layer, plane, token): its num_kv_heads * head_dim elements are one contiguous run on the flat
// side and num_kv_heads rows of head_dim elements in the page.  The index arithmetic (one 64-bit division, the
// table look-up) is done once per warp and token; every lane then has up to four independent 16-byte loads in
// flight before the first store.
template <bool TO_FLAT>
__global__ void __launch_bounds__(256) flat_paged_copy_kernel(const FlatCopyParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const int D8 = p.layout.head_dim / 8;                       // 16-byte vectors per head row
    const int vec_per_tok = p.layout.num_kv_heads * D8;         // vectors of one token in one plane
    const int64_t n_rows = (int64_t)p.num_layers * 2 * p.num_tokens;
    const int lane = threadIdx.x & 31;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    char* flat = reinterpret_cast<char*>(p.flat);
    char* pool = reinterpret_cast<char*>(p.pool);
    for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < n_rows; r += n_warps) {
        const int64_t lk = r / p.num_tokens;                    // layer * 2 + plane
        const int tok = (int)(r - lk * p.num_tokens);
        const int kv = (int)(lk & 1), layer = (int)(lk >> 1);
        const int pos = p.start_token + tok;
        const int logical = pos / p.layout.page_size, slot = pos - logical * p.layout.page_size;
        int page = -1;
        if (logical < p.table_stride) page = __ldg(p.table + logical);
        if (page >= p.layout.max_pages) page = -1;
        char* frow = flat + r * vec_per_tok * 16;
        if (!TO_FLAT && page < 0) continue;                     // nowhere to write
        for (int v0 = 0; v0 < vec_per_tok; v0 += 128) {
            Vec16 v[4];
            char* prow[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int vi = v0 + lane + 32 * i;
                v[i] = Vec16{{0u, 0u, 0u, 0u}};
                prow[i] = nullptr;
                if (vi < vec_per_tok) {
                    const int head = vi / D8, d8 = vi - head * D8;
                    if (page >= 0) prow[i] = pool + (p.layout.row(layer, page, kv, head, slot) + 8 * d8) * 2;
                    if (TO_FLAT) {
                        if (page >= 0) v[i] = ldg16(prow[i]);
                    } else {
                        v[i] = ldg16(frow + (int64_t)vi * 16);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int vi = v0 + lane + 32 * i;
                if (vi < vec_per_tok) {
                    if (TO_FLAT) stg16(frow + (int64_t)vi * 16, v[i]);
                    else stg16(prow[i], v[i]);
                }
            }
        }
    }
}

}  // namespace

cudaError_t launch_flat_paged_copy(const FlatCopyParams& p, bool to_flat, int num_sms, cudaStream_t stream) {
    const int64_t n_rows = (int64_t)p.num_layers * 2 * p.num_tokens;
    if (n_rows <= 0 || p.layout.num_kv_heads <= 0) return cudaSuccess;
    int64_t blocks = (n_rows + 7) / 8;                          // eight warps per CTA, one (layer, plane, token) each
    const int64_t cap = (int64_t)num_sms * 8;                   // the warps stride over the rest
    if (blocks > cap) blocks = cap;
    if (to_flat) return launch_pdl(flat_paged_copy_kernel<true>, dim3((unsigned)blocks), dim3(256), 0, stream, p);
    return launch_pdl(flat_paged_copy_kernel<false>, dim3((unsigned)blocks), dim3(256), 0, stream, p);
}

}  // namespace drkv
