// stateless.cu — the reference's free functions as C entry points: one sequence, one block
// table, raw device pointers, geometry passed in (the reference reads it from ModelConfig
// statics; src/machina/paged_attention.cu:104-115, 155-167, 271-282).  Nothing here owns
// memory: the decode attention takes its split-KV scratch from the caller.
#include <climits>
#include <cstdio>
#include <string>

#include "../../include/drkv.h"
#include "kernels.hpp"
#include "stateless.hpp"

using namespace drkv;

namespace drkv {

static int fail(int code, const char* msg) {
    set_last_error(msg);
    return code;
}

bool stateless_geometry_ok(const drkv_geometry* g) {
    if (!g) return false;
    if (g->num_layers <= 0 || g->num_q_heads <= 0 || g->num_kv_heads <= 0) return false;
    if (g->num_q_heads % g->num_kv_heads != 0 || g->num_q_heads / g->num_kv_heads > 16) return false;
    if (g->head_dim != 64 && g->head_dim != 128 && g->head_dim != 256) return false;
    if (g->page_size <= 0 || g->page_size % 16 != 0) return false;
    if (g->dtype != DRKV_DTYPE_F16 && g->dtype != DRKV_DTYPE_BF16) return false;
    return true;
}

int stateless_pick_chunk(const drkv_geometry* g, int seq_len, int num_sms) {
    const int group = g->num_q_heads / g->num_kv_heads;
    int chunk = group > 4 ? 512 : 256;
    const long warps = (long)num_sms * decode_warps_per_cta(g->head_dim);
    const long hkv = g->num_kv_heads;
    {
        // one equal item per warp, the fewest partials, whenever such an item keeps at least 64 keys
        const long per_head = warps / hkv > 0 ? warps / hkv : 1;
        const long c = ((seq_len + per_head - 1) / per_head + 15) / 16 * 16;
        if (c >= 64) return (int)c;
    }
    while (chunk > 64 && hkv * ((seq_len + chunk - 1) / chunk) < warps) chunk >>= 1;
    return chunk;
}

size_t stateless_scratch_bytes(const drkv_geometry* g, int seq_len, int chunk) {
    const size_t chunks = (size_t)(seq_len + chunk - 1) / chunk;
    return kStatelessHeaderBytes + (size_t)g->num_q_heads * chunks * (g->head_dim + 2) * sizeof(float);
}

// Shared by the caller-scratch and the built-in-scratch entry points.
int stateless_decode(const drkv_geometry* g, const void* q, const void* kv_pool, const int32_t* d_block_table,
                     void* out, int layer, int seq_len, int max_pages, float scale, void* scratch, int chunk,
                     cudaStream_t stream) {
    int dev = 0, num_sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return fail(DRKV_ERR_NO_DEVICE, "no CUDA device is current");
    CUtensorMap tmap;
    const char* terr = nullptr;
    if (!make_pool_slot_tensor_map(&tmap, kv_pool, g->num_layers, max_pages, g->num_kv_heads, g->page_size, g->head_dim, &terr))
        return fail(DRKV_ERR_CUDA, terr ? terr : "tensor map");
    // header: [0] queue head, [1] error word, [2] exit count; all start at zero for every call
    if (cudaMemsetAsync(scratch, 0, kStatelessHeaderBytes, stream) != cudaSuccess)
        return fail(DRKV_ERR_CUDA, "cudaMemsetAsync(scratch header) failed");
    int* header = reinterpret_cast<int*>(scratch);
    float* parts = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + kStatelessHeaderBytes);
    const int max_chunks = (seq_len + chunk - 1) / chunk;
    const size_t n_slots = (size_t)g->num_q_heads * max_chunks;

    DecodeParams p{};
    p.tables = d_block_table;
    // The caller's table covers ceil(seq_len / page_size) entries by contract and not one more: the kernel
    // fetches page ids a window of 32 ahead, and this bound turns every entry past the end into a hole
    // instead of a read outside the caller's allocation.
    p.table_stride = (seq_len + g->page_size - 1) / g->page_size;
    p.rows = nullptr;
    p.kv_len = nullptr;
    p.row = 0;
    p.kv_begin = 0;
    p.kv_end = seq_len;
    p.q = q;
    p.part_o = parts;
    p.part_m = parts + n_slots * g->head_dim;
    p.part_l = p.part_m + n_slots;
    p.layer = layer;
    p.max_pages = max_pages;
    p.num_q_heads = g->num_q_heads;
    p.num_kv_heads = g->num_kv_heads;
    p.group = g->num_q_heads / g->num_kv_heads;
    p.page_size = g->page_size;
    p.chunk_tokens = chunk;
    p.max_chunks = max_chunks;
    p.n_seq = 1;
    p.few_keys_possible = seq_len > 1024 ? 0 : 1;       // the length comes from the host: see DecodeParams
    p.total_items = g->num_kv_heads * max_chunks;
    p.work_counter = header;
    p.exit_count = header + 2;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.error_word = header + 1;
    p.wait_first = 1;                  // the caller's own kernel may have written the table directly in front
    if (launch_attend_decode(tmap, p, num_sms, g->head_dim, g->dtype, stream) != cudaSuccess)
        return fail(DRKV_ERR_CUDA, "decode attention launch failed");

    CombineParams c{};
    c.part_o = p.part_o;
    c.part_m = p.part_m;
    c.part_l = p.part_l;
    c.kv_len = nullptr;
    c.kv_begin = 0;
    c.kv_end = seq_len;
    c.num_q_heads = g->num_q_heads;
    c.head_dim = g->head_dim;
    c.chunk_tokens = chunk;
    c.max_chunks = max_chunks;
    c.out = out;
    c.out_partial = nullptr;
    if (launch_combine(c, 1, g->dtype, stream) != cudaSuccess) return fail(DRKV_ERR_CUDA, "combine launch failed");
    return DRKV_OK;
}

}  // namespace drkv

extern "C" {

int drkv_k_cache_write(const drkv_geometry* g, const void* src_k, const void* src_v, void* kv_pool,
                       const int32_t* d_block_table, int layer, const int32_t* d_pos, int max_pages, void* stream) {
    if (!stateless_geometry_ok(g) || !src_k || !src_v || !kv_pool || !d_block_table || !d_pos || layer < 0 ||
        layer >= g->num_layers || max_pages <= 0)
        return fail(DRKV_ERR_INVALID, "cache_write: bad argument");
    AppendParams p{};
    p.layout = PoolLayout::make(g->num_kv_heads, g->page_size, g->head_dim, max_pages);
    p.pool = kv_pool;
    p.tables = d_block_table;
    p.table_stride = INT_MAX;
    p.rows = nullptr;
    p.pos = d_pos;                 // position read on the device (paged_attention.cu:87)
    p.row = 0;
    p.layer = layer;
    p.rotary_dim = 0;              // the reference rotates K before this call
    p.wait_first = 1;              // d_pos and the table may come from the caller's kernel directly in front
    p.inv_freq = nullptr;
    p.k_src = src_k;
    p.v_src = src_v;
    if (launch_append_rope(p, 1, g->dtype, (cudaStream_t)stream) != cudaSuccess)
        return fail(DRKV_ERR_CUDA, "cache_write launch failed");
    return DRKV_OK;
}

int drkv_k_cache_write_batch(const drkv_geometry* g, const void* src_k, const void* src_v, void* kv_pool,
                             const int32_t* d_block_table, int layer, int pos_start, int m, int max_pages,
                             void* stream) {
    if (!stateless_geometry_ok(g) || !src_k || !src_v || !kv_pool || !d_block_table || layer < 0 ||
        layer >= g->num_layers || max_pages <= 0 || pos_start < 0 || m < 0)
        return fail(DRKV_ERR_INVALID, "cache_write_batch: bad argument");
    AppendParams p{};
    p.layout = PoolLayout::make(g->num_kv_heads, g->page_size, g->head_dim, max_pages);
    p.pool = kv_pool;
    p.tables = d_block_table;
    p.table_stride = INT_MAX;
    p.rows = nullptr;
    p.pos = nullptr;
    p.row = 0;
    p.pos_start = pos_start;
    p.layer = layer;
    p.rotary_dim = 0;
    p.wait_first = 1;
    p.inv_freq = nullptr;
    p.k_src = src_k;
    p.v_src = src_v;
    if (launch_append_rope(p, m, g->dtype, (cudaStream_t)stream) != cudaSuccess)
        return fail(DRKV_ERR_CUDA, "cache_write_batch launch failed");
    return DRKV_OK;
}

static int flat_copy(const drkv_geometry* g, void* pool, void* flat, const int32_t* table, int start_token,
                     int num_tokens, int max_pages, bool to_flat, void* stream) {
    if (!stateless_geometry_ok(g) || !pool || !flat || !table || start_token < 0 || num_tokens < 0 || max_pages <= 0)
        return fail(DRKV_ERR_INVALID, "extract/inject: bad argument");
    int dev = 0, num_sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    FlatCopyParams p{};
    p.layout = PoolLayout::make(g->num_kv_heads, g->page_size, g->head_dim, max_pages);
    p.pool = pool;
    p.flat = flat;
    p.table = table;
    p.table_stride = INT_MAX;
    p.start_token = start_token;
    p.num_tokens = num_tokens;
    p.num_layers = g->num_layers;
    if (launch_flat_paged_copy(p, to_flat, num_sms, (cudaStream_t)stream) != cudaSuccess)
        return fail(DRKV_ERR_CUDA, "extract/inject launch failed");
    return DRKV_OK;
}

int drkv_k_extract_kv(const drkv_geometry* g, void* dst, const void* kv_pool, const int32_t* d_block_table,
                      int start_token, int num_tokens, int max_pages, void* stream) {
    return flat_copy(g, const_cast<void*>(kv_pool), dst, d_block_table, start_token, num_tokens, max_pages, true, stream);
}

int drkv_k_inject_kv(const drkv_geometry* g, void* kv_pool, const void* src, const int32_t* d_block_table,
                     int start_token, int num_tokens, int max_pages, void* stream) {
    return flat_copy(g, kv_pool, const_cast<void*>(src), d_block_table, start_token, num_tokens, max_pages, false, stream);
}

int drkv_k_decode_kernel_error(const void* scratch, void* stream) {
    const void* area = scratch;
    if (area == nullptr) {
        void* builtin = nullptr;
        int rc = noalloc_scratch_for_current_device(&builtin);
        if (rc != DRKV_OK) return rc;
        area = builtin;
    }
    int code = 0;
    // header word 1 is the error word of the last call that used this scratch (stateless_decode)
    if (cudaMemcpyAsync(&code, reinterpret_cast<const int*>(area) + 1, sizeof(int), cudaMemcpyDeviceToHost,
                        (cudaStream_t)stream) != cudaSuccess ||
        cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess)
        return fail(DRKV_ERR_CUDA, "decode_kernel_error: reading the scratch header failed");
    if (code != 0) {
        char msg[160];
        snprintf(msg, sizeof(msg),
                 "a kernel reported error code %d (1 = load wait, 2 = ring wait, 3 = page id, 4 = peer wait)", code);
        return fail(DRKV_ERR_CUDA, msg);
    }
    return DRKV_OK;
}

size_t drkv_k_decode_scratch_bytes(const drkv_geometry* g, int seq_len) {
    if (!stateless_geometry_ok(g) || seq_len <= 0) return 0;
    // sized for the smallest chunk the launcher may pick, so it is valid on any device
    return stateless_scratch_bytes(g, seq_len, 64);
}

int drkv_k_decode_attention(const drkv_geometry* g, const void* q, const void* kv_pool, const int32_t* d_block_table,
                            void* out, int layer, int seq_len, int max_pages, float scale, void* scratch,
                            size_t scratch_bytes, void* stream) {
    if (!stateless_geometry_ok(g) || !q || !kv_pool || !d_block_table || !out || !scratch || layer < 0 ||
        layer >= g->num_layers || max_pages <= 0 || seq_len < 0)
        return fail(DRKV_ERR_INVALID, "decode_attention: bad argument");
    if (seq_len == 0) return DRKV_OK;   // no key: the output stays untouched (paged_attention.cu:266-268)
    if ((reinterpret_cast<uintptr_t>(scratch) & 255) != 0)
        return fail(DRKV_ERR_INVALID, "decode_attention: scratch must be 256-byte aligned");
    int dev = 0, num_sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    int chunk = stateless_pick_chunk(g, seq_len, num_sms);
    while (stateless_scratch_bytes(g, seq_len, chunk) > scratch_bytes && chunk < (1 << 24)) chunk <<= 1;
    if (stateless_scratch_bytes(g, seq_len, chunk) > scratch_bytes)
        return fail(DRKV_ERR_CAPACITY, "decode_attention: scratch too small (see drkv_k_decode_scratch_bytes)");
    return stateless_decode(g, q, kv_pool, d_block_table, out, layer, seq_len, max_pages, scale, scratch, chunk,
                            (cudaStream_t)stream);
}

}  // extern "C"
