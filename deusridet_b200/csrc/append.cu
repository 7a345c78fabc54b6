// append.cu — fused K/V append: RoPE on K, then scatter of K and V into their pages.
//
// Replaces three reference launches (rope_kernel / paged_rope_batch_kernel on K,
// paged_kv_cache_write[_batch]_kernel; src/machina/layer_attention.cu:32-79,
// src/machina/paged_attention.cu:73-167, 412-451) with one kernel that reads each source
// element once and writes it once, in 16-byte vectors.  Pure data movement plus 3 flops per
// rotated element: HBM/latency bound; the rows written are 256-byte contiguous runs.
#include "kernels.hpp"
#include "kv_common.cuh"

namespace drkv {

namespace {

constexpr int kAppendThreads = 128;
constexpr int kMaxPairs = 128;  // rotary_dim / 2 <= head_dim / 2 <= 128

// One CTA per token.  `tok` tokens come either from a batch of sequences (one token each:
// rows[i], pos[i]) or from one sequence (row fixed, pos_start + i).
template <typename T>
__global__ void __launch_bounds__(kAppendThreads)
append_rope_kernel(AppendParams p) {
    const int tok = blockIdx.x;
    // Positions, rows, the block table and the frequencies are written by copies or by kernels further back
    // than the one directly in front (which, when it belongs to this library, released this launch only after
    // its own wait): the angles and the page id are worked out under that kernel's tail.  The sources and
    // the pool are touched after the wait.
    if (p.wait_first) pdl_wait();    // a foreign caller's kernel in front may have written the position or the table
    int row, pos;
    if (p.rows != nullptr) {
        row = p.rows[tok];
        pos = p.pos[tok];
    } else {
        row = p.row;
        pos = (p.pos != nullptr ? p.pos[0] : p.pos_start) + tok;
    }
    const int D = p.layout.head_dim, P = p.layout.page_size, H = p.layout.num_kv_heads;
    const int half = p.rotary_dim >> 1;

    __shared__ float s_cos[kMaxPairs], s_sin[kMaxPairs];
    for (int i = threadIdx.x; i < half; i += kAppendThreads) {
        // angle = pos * freq in fp32, as the reference (layer_attention.cu:45-46)
        float angle = __fmul_rn((float)pos, p.inv_freq[i]);
        float s, c;
        sincos_det(angle, s, c);
        s_cos[i] = c;
        s_sin[i] = s;
    }
    const int logical = pos >= 0 ? pos / P : 0, slot = pos - logical * P;
    const int page = (pos >= 0 && logical < p.table_stride) ? p.tables[(int64_t)row * p.table_stride + logical] : -1;
    __syncthreads();
    pdl_wait();
    pdl_launch_dependents();
    if (page < 0 || page >= p.layout.max_pages) return;  // hole or no position: nothing to write into

    const T* ksrc = reinterpret_cast<const T*>(p.k_src) + (int64_t)tok * H * D;
    const T* vsrc = reinterpret_cast<const T*>(p.v_src) + (int64_t)tok * H * D;
    T* pool = reinterpret_cast<T*>(p.pool);

    const int vec_per_head = D / 8;            // 16-byte vectors per head row
    const int rope_vecs = half / 8;            // vectors in each rotated half
    const int items_k_rope = H * rope_vecs;    // pairs of vectors (i, i + half)
    const int items_k_copy = H * (vec_per_head - 2 * rope_vecs);
    const int items_v = H * vec_per_head;
    const int total = items_k_rope + items_k_copy + items_v;

    for (int it = threadIdx.x; it < total; it += kAppendThreads) {
        if (it < items_k_rope) {
            const int h = it / rope_vecs, j = it - h * rope_vecs;  // dims [8j, 8j+8) and + half
            const T* src = ksrc + h * D;
            Vec16 a = ldg16(src + 8 * j), b = ldg16(src + half + 8 * j);
            Vec16 ya, yb;
#pragma unroll
            for (int w = 0; w < 4; w++) {
                float2 x0 = Elem<T>::unpack2(a.w[w]), x1 = Elem<T>::unpack2(b.w[w]);
                const int i0 = 8 * j + 2 * w;
                float r00, r01, r10, r11;
                rope_pair(x0.x, x1.x, s_cos[i0], s_sin[i0], r00, r10);
                rope_pair(x0.y, x1.y, s_cos[i0 + 1], s_sin[i0 + 1], r01, r11);
                ya.w[w] = Elem<T>::pack2(r00, r01);
                yb.w[w] = Elem<T>::pack2(r10, r11);
            }
            T* dst = pool + p.layout.row(p.layer, page, 0, h, slot);
            stg16(dst + 8 * j, ya);
            stg16(dst + half + 8 * j, yb);
        } else if (it < items_k_rope + items_k_copy) {
            const int r = it - items_k_rope;
            const int per = vec_per_head - 2 * rope_vecs;
            const int h = r / per, j = r - h * per;
            const int off = p.rotary_dim + 8 * j;
            stg16(pool + p.layout.row(p.layer, page, 0, h, slot) + off, ldg16(ksrc + h * D + off));
        } else {
            const int r = it - items_k_rope - items_k_copy;
            const int h = r / vec_per_head, j = r - h * vec_per_head;
            stg16(pool + p.layout.row(p.layer, page, 1, h, slot) + 8 * j, ldg16(vsrc + h * D + 8 * j));
        }
    }
}

// Copy-on-write of a partially filled page: slots [0, n_slots) of K and V, every layer
// and KV head.  One CTA per (layer, plane, head) run of n_slots * D contiguous elements.
__global__ void __launch_bounds__(128) cow_copy_kernel(CowParams p) {
    const int head = blockIdx.x, kv = blockIdx.y, layer = blockIdx.z;
    const int D = p.layout.head_dim;
    pdl_wait();
    pdl_launch_dependents();
    const size_t esize = 2;
    const char* src = reinterpret_cast<const char*>(p.pool) + p.layout.row(layer, p.src_page, kv, head, 0) * esize;
    char* dst = reinterpret_cast<char*>(p.pool) + p.layout.row(layer, p.dst_page, kv, head, 0) * esize;
    const int vecs = p.n_slots * D / 8;
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) stg16(dst + 16 * i, ldg16(src + 16 * i));
}

}  // namespace

cudaError_t launch_append_rope(const AppendParams& p, int n_tokens, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return cudaSuccess;
    if (dtype == DRKV_DTYPE_F16)
        return launch_pdl(append_rope_kernel<__half>, dim3(n_tokens), dim3(kAppendThreads), 0, stream, p);
    return launch_pdl(append_rope_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(kAppendThreads), 0, stream, p);
}

cudaError_t launch_cow_copy(const CowParams& p, int num_layers, cudaStream_t stream) {
    if (p.n_slots <= 0) return cudaSuccess;
    dim3 grid(p.layout.num_kv_heads, 2, num_layers);
    return launch_pdl(cow_copy_kernel, grid, dim3(128), 0, stream, p);
}

}  // namespace drkv
