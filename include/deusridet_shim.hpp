// deusridet_shim.hpp — the reference's C++ call surface on top of the C ABI (drkv.h).
//
// Header-only.  A DeusRidet build that includes this instead of memoria/block_pool.h,
// memoria/cache_manager.h and machina/paged_attention.h, and links libdrkv.so instead of
// compiling block_pool.cpp / cache_manager.cpp / paged_attention.cu, keeps its callers
// (src/conscientia/stream.cpp:145-255, 261-401; src/actus/awaken_consciousness.cpp:82-100)
// unchanged: same class names, method names, argument meaning, bool / -1 failure convention.
//
//   BlockPool      src/memoria/block_pool.h:58-123
//   CacheManager   src/memoria/cache_manager.h:52-169
//   KVSwapper      src/memoria/kv_swapper.h:36-120 (SwapRequest, submit, drain, prefetch, is_prefetched, drop_prefetch):
//                  a non-null swapper together with a cache_dir switches the engine's storage tier on
//                  (cache_manager.cpp:132, 56-66); its calls forward to that tier
//   ImportanceScorer src/memoria/importance_scorer.h:25-67: init / update / sync_to_host / score /
//                  least_important forward to the engine's scorer once a CacheManager has adopted it
//   paged_kv_cache_write / _batch, paged_gqa_decode_attention
//                  src/machina/paged_attention.h:27-71
//   invoke_extract_kv_from_pages / invoke_inject_kv_to_pages
//                  src/memoria/cache_kernels.h:44-74
//
// The reference reads head counts and dims from process-wide ModelConfig statics
// (src/machina/paged_attention.cu:110-114); here the integrator fills shim_geometry() once,
// before the first init(), from the same statics.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <functional>
#include <mutex>
#include <string>
#include <unordered_set>
#include <vector>

#include "drkv.h"

namespace deusridet {

// Defaults are the reference's compile-time PagedKVConfig (src/memoria/block_pool.h:34-40) and
// Qwen3.5-27B's attention shape; set every field from ModelConfig in a real build.
inline drkv_geometry& shim_geometry() {
    static drkv_geometry g = {16, 24, 4, 256, 256, DRKV_DTYPE_F16, 64, 10000000.0f};
    return g;
}
// CUDA device the pool lives on; -1 keeps bookkeeping only (host-side tests).
inline int& shim_device() {
    static int d = [] {
        const char* s = std::getenv("DRKV_SHIM_DEVICE");
        return s ? std::atoi(s) : 0;
    }();
    return d;
}

struct PagedKVConfig {
    static constexpr int BLOCK_SIZE = 256;
};

class BlockPool;

// src/memoria/kv_swapper.h:36-44
enum class SwapDirection { GPU_TO_SSD, SSD_TO_GPU };
struct SwapRequest {
    SwapDirection direction;
    int logical_block_idx;
    int physical_block_id;                 // pool page (source for out, target for in)
    std::string ssd_path;                  // file path
    std::function<void(bool)> callback;    // completion callback (success)
};

// src/memoria/kv_swapper.h:52-120.  The engine moves evicted pages itself once a CacheManager has adopted the
// swapper (cache_manager.cpp:132, 215-292); the swapper's own calls forward to the engine's storage tier.  A
// request is carried out before submit() returns (the reference queues it for its I/O thread and its only caller
// drains at once, cache_manager.cpp:226-229); drkv_tier_set_write_behind is how file writes leave the caller's thread.
class KVSwapper {
public:
    bool init(BlockPool& pool, const std::string& ssd_dir, int /*staging_blocks*/ = 2);
    void submit(SwapRequest req) {
        bool ok = false;
        if (e_ != nullptr)
            ok = (req.direction == SwapDirection::GPU_TO_SSD
                      ? drkv_tier_page_to_file(e_, req.physical_block_id, req.ssd_path.c_str())
                      : drkv_tier_file_to_page(e_, req.ssd_path.c_str(), req.physical_block_id)) == DRKV_OK;
        if (!ok) std::fprintf(stderr, "[Memoria] KVSwapper: %s\n", e_ ? drkv_last_error() : "not initialised");
        if (req.callback) req.callback(ok);
    }
    void drain() {
        if (e_) drkv_tier_drain(e_);
    }
    void shutdown() { drain(); }
    int pending() const { return 0; }
    // the file of a logical block is the engine's own (cache_manager.cpp:211-213): the path argument is not needed
    void prefetch(int logical_block_idx, const std::string& /*ssd_path*/) {
        if (e_) drkv_tier_prefetch(e_, seq_, logical_block_idx);
    }
    bool is_prefetched(int logical_block_idx) const { return e_ && drkv_tier_is_prefetched(e_, seq_, logical_block_idx) == 1; }
    void drop_prefetch(int logical_block_idx) {
        if (e_) drkv_tier_drop_prefetch(e_, seq_, logical_block_idx);
    }
    const std::string& dir() const { return dir_; }

private:
    friend class CacheManager;
    std::string dir_;
    drkv_engine* e_ = nullptr;
    int seq_ = 0;
};

class ImportanceScorer {
public:
    bool init(int max_blocks, float decay = 0.95f) {
        max_blocks_ = max_blocks;
        decay_ = decay;
        return max_blocks > 0;
    }
    // d_block_scores: device memory (host memory when the engine has no device), as in the reference.
    void update(const float* d_block_scores, int num_blocks) {
        if (e_ && drkv_scorer_update(e_, seq_, d_block_scores, num_blocks, nullptr) != DRKV_OK)
            std::fprintf(stderr, "[Memoria] ImportanceScorer: %s\n", drkv_last_error());
    }
    void sync_to_host() {
        if (e_) drkv_scorer_sync(e_, nullptr);
    }
    float score(int logical_block) const {
        if (!e_ || logical_block < 0 || logical_block >= max_blocks_) return 0.0f;   // importance_scorer.cu:86-89
        std::string buf((size_t)max_blocks_ * sizeof(float), '\0');
        float* f = reinterpret_cast<float*>(&buf[0]);
        const int n = drkv_scorer_scores(e_, seq_, f, max_blocks_);
        return logical_block < n ? f[logical_block] : 0.0f;
    }
    int least_important(const int* gpu_resident, int n) const {                   // importance_scorer.cu:75-87
        if (n <= 0) return -1;
        int min_idx = gpu_resident[0];
        float min_score = score(min_idx);
        for (int i = 1; i < n; i++) {
            const float sc = score(gpu_resident[i]);
            if (sc < min_score) {
                min_score = sc;
                min_idx = gpu_resident[i];
            }
        }
        return min_idx;
    }
    void destroy() { e_ = nullptr; }
    float decay() const { return decay_; }

private:
    friend class CacheManager;
    drkv_engine* e_ = nullptr;
    int seq_ = 0, max_blocks_ = 0;
    float decay_ = 0.95f;
};

class BlockPool {
public:
    BlockPool() = default;
    ~BlockPool() { destroy(); }
    BlockPool(const BlockPool&) = delete;
    BlockPool& operator=(const BlockPool&) = delete;

    bool init(size_t budget_bytes, int block_size = PagedKVConfig::BLOCK_SIZE) {
        return init_rows(budget_bytes, block_size, 1, 0, 0);
    }
    int alloc_block() { return e_ ? drkv_pool_alloc(e_) : -1; }
    void free_block(int id) {
        if (e_ && drkv_pool_free(e_, id) != DRKV_OK)
            std::fprintf(stderr, "[Memoria] free_block(%d): %s\n", id, drkv_last_error());
    }
    int free_count() const { return e_ ? drkv_pool_free_count(e_) : 0; }
    int max_blocks() const { return e_ ? drkv_pool_max_pages(e_) : 0; }
    int block_size() const { return e_ ? drkv_pool_page_size(e_) : block_size_; }
    __half* pool_ptr() const { return e_ ? static_cast<__half*>(drkv_pool_ptr(e_)) : nullptr; }
    __half* k_ptr(int layer, int id) const {
        return reinterpret_cast<__half*>(reinterpret_cast<char*>(pool_ptr()) + k_offset(layer, id));
    }
    __half* v_ptr(int layer, int id) const {
        return reinterpret_cast<__half*>(reinterpret_cast<char*>(pool_ptr()) + v_offset(layer, id));
    }
    size_t k_offset(int layer, int id) const { return e_ ? drkv_pool_k_offset(e_, layer, id) : 0; }
    size_t v_offset(int layer, int id) const { return e_ ? drkv_pool_v_offset(e_, layer, id) : 0; }
    size_t total_bytes() const { return e_ ? drkv_pool_total_bytes(e_) : 0; }
    void destroy() {
        if (e_) drkv_destroy(e_);
        e_ = nullptr;
    }

    drkv_engine* engine() const { return e_; }

private:
    friend class CacheManager;
    bool init_rows(size_t budget_bytes, int block_size, int max_seqs, int row_width, int stream_evict) {
        destroy();
        block_size_ = block_size;
        drkv_geometry g = shim_geometry();
        g.page_size = block_size;
        drkv_config c = {};
        c.budget_bytes = budget_bytes;
        c.max_seqs = max_seqs;
        c.max_pages_per_seq = row_width;   // 0 = 2 x physical pages, CacheManager's logical space
        c.device = shim_device();
        c.stream_evict = stream_evict;
        if (drkv_create(&g, &c, &e_) != DRKV_OK) {
            std::fprintf(stderr, "[Memoria] BlockPool: %s\n", drkv_last_error());
            e_ = nullptr;
            return false;
        }
        return true;
    }
    drkv_engine* e_ = nullptr;
    int block_size_ = PagedKVConfig::BLOCK_SIZE;
};

inline bool KVSwapper::init(BlockPool& pool, const std::string& ssd_dir, int) {
    dir_ = ssd_dir;
    e_ = pool.engine();                    // null until the pool is initialised; a CacheManager sets it when it adopts the swapper
    if (e_ != nullptr && !ssd_dir.empty() && drkv_tier_enable(e_, ssd_dir.c_str()) != DRKV_OK) {
        std::fprintf(stderr, "[Memoria] KVSwapper: %s\n", drkv_last_error());
        return false;
    }
    return true;
}

class CacheManager {
public:
    CacheManager() = default;
    ~CacheManager() { destroy(); }
    CacheManager(const CacheManager&) = delete;
    CacheManager& operator=(const CacheManager&) = delete;

    bool init(size_t kv_budget_bytes, const std::string& cache_dir = "",
              int block_size = PagedKVConfig::BLOCK_SIZE, KVSwapper* swapper = nullptr,
              ImportanceScorer* scorer = nullptr) {
        if (!pool_.init_rows(kv_budget_bytes, block_size, 1, 0, 1)) return false;
        if (scorer != nullptr) {                       // before the row exists, so that it starts scored
            if (!ok(drkv_scorer_enable(pool_.e_, scorer->decay()))) return false;
            scorer->e_ = pool_.e_;
        }
        seq_ = drkv_seq_create(pool_.e_);
        if (scorer != nullptr) scorer->seq_ = seq_;
        // cache_manager.cpp:56-66, 132: stored only with a directory AND a swapper; a directory that
        // cannot be created switches the tier off with a warning
        if (seq_ >= 0 && swapper != nullptr && !cache_dir.empty() && drkv_tier_enable(pool_.e_, cache_dir.c_str()) != DRKV_OK)
            std::fprintf(stderr, "[Memoria] Cannot create SSD cache dir: %s\n", cache_dir.c_str());
        if (swapper != nullptr) {
            swapper->e_ = pool_.e_;
            swapper->seq_ = seq_;
        }
        return seq_ >= 0;
    }
    bool ensure_blocks_for(int pos) { return ok(drkv_seq_ensure_pos(pool_.e_, seq_, pos, nullptr)); }
    bool ensure_blocks_for_range(int pos_start, int m) {
        return ok(drkv_seq_ensure_range(pool_.e_, seq_, pos_start, m, nullptr));
    }
    const int* d_block_table() const { return pool_.e_ ? drkv_device_tables(pool_.e_) : nullptr; }
    void sync_block_table(cudaStream_t stream = 0) {
        if (pool_.e_) drkv_sync_tables(pool_.e_, stream);
    }
    int seq_len() const { return pool_.e_ ? drkv_seq_len(pool_.e_, seq_) : 0; }
    void set_seq_len(int n) {
        if (pool_.e_) drkv_seq_set_len(pool_.e_, seq_, n);
    }
    int num_logical_blocks() const { return pool_.e_ ? drkv_seq_num_pages(pool_.e_, seq_) : 0; }
    int evict_blocks(int n) { return pool_.e_ ? drkv_seq_evict(pool_.e_, seq_, n) : 0; }
    bool ensure_free_blocks(int n_free) { return pool_.e_ && drkv_ensure_free(pool_.e_, seq_, n_free) == 1; }
    void prefetch_block(int logical_idx) {
        if (pool_.e_) drkv_tier_prefetch(pool_.e_, seq_, logical_idx);
    }
    BlockPool& block_pool() { return pool_; }
    const BlockPool& block_pool() const { return pool_; }
    int gpu_blocks_used() const { return pool_.max_blocks() - pool_.free_count(); }
    int ssd_blocks_used() const {
        drkv_tier_stats st = {};
        return (pool_.e_ && drkv_tier_get_stats(pool_.e_, &st) == DRKV_OK) ? (int)st.pages_stored : 0;
    }
    int free_blocks() const { return pool_.free_count(); }
    void destroy() {
        pool_.destroy();
        seq_ = -1;
    }
    // Host copy of the table, for tests.
    int host_table(int* out, int cap) const { return pool_.e_ ? drkv_seq_table(pool_.e_, seq_, out, cap) : 0; }

private:
    bool ok(int rc) {
        if (rc == DRKV_OK) return true;
        std::fprintf(stderr, "[Memoria] %s\n", drkv_last_error());
        return false;
    }
    BlockPool pool_;
    int seq_ = -1;
};

// ---- src/machina/paged_attention.h:27-71 -------------------------------------------------------
inline void paged_kv_cache_write(const __half* src_k, const __half* src_v, __half* kv_pool,
                                 const int* d_block_table, int fa_layer_idx, const int* d_pos,
                                 int max_phys_blocks, int block_size, cudaStream_t stream = 0) {
    drkv_geometry g = shim_geometry();
    g.page_size = block_size;
    if (drkv_k_cache_write(&g, src_k, src_v, kv_pool, d_block_table, fa_layer_idx, d_pos, max_phys_blocks, stream) !=
        DRKV_OK)
        std::fprintf(stderr, "[Machina] paged_kv_cache_write: %s\n", drkv_last_error());
}

inline void paged_kv_cache_write_batch(const __half* src_k, const __half* src_v, __half* kv_pool,
                                       const int* d_block_table, int fa_layer_idx, int pos_start, int M,
                                       int max_phys_blocks, int block_size, cudaStream_t stream = 0) {
    drkv_geometry g = shim_geometry();
    g.page_size = block_size;
    if (drkv_k_cache_write_batch(&g, src_k, src_v, kv_pool, d_block_table, fa_layer_idx, pos_start, M,
                                 max_phys_blocks, stream) != DRKV_OK)
        std::fprintf(stderr, "[Machina] paged_kv_cache_write_batch: %s\n", drkv_last_error());
}

// The reference signature has no workspace argument; the shim keeps one split-KV scratch buffer per CUDA
// device, shared by every call on that device: calls must be ordered on one stream (or otherwise not overlap
// on the GPU).  A buffer grows on demand and is never shrunk; the old buffer of a grown one is kept until the
// process exits, because kernels already enqueued (or captured in a graph) may still use it.  Growth calls
// cudaMalloc, which synchronises the device and is illegal during stream capture: call
// shim_reserve_decode_scratch() for the longest sequence once, before capturing a decode step.
namespace detail {
struct DecodeScratch {
    void* ptr = nullptr;
    size_t bytes = 0;
};
inline std::mutex& decode_scratch_mutex() {
    static std::mutex m;
    return m;
}
inline DecodeScratch* decode_scratch_slots() {
    static DecodeScratch slots[64];
    return slots;
}
// Returns the current device's buffer, at least `need` bytes (nullptr on failure).
inline void* decode_scratch(size_t need, size_t* bytes_out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(decode_scratch_mutex());
    DecodeScratch& sc = decode_scratch_slots()[dev];
    if (need > sc.bytes) {
        void* fresh = nullptr;
        const size_t bytes = need * 2;
        if (cudaMalloc(&fresh, bytes) != cudaSuccess) return nullptr;
        sc.ptr = fresh;       // the previous buffer stays allocated, see above
        sc.bytes = bytes;
    }
    *bytes_out = sc.bytes;
    return sc.ptr;
}
}  // namespace detail

inline bool shim_reserve_decode_scratch(int max_seq_len, int block_size = PagedKVConfig::BLOCK_SIZE) {
    drkv_geometry g = shim_geometry();
    g.page_size = block_size;
    size_t bytes = 0;
    return detail::decode_scratch(drkv_k_decode_scratch_bytes(&g, max_seq_len > 0 ? max_seq_len : 1), &bytes) != nullptr;
}

inline void paged_gqa_decode_attention(const __half* Q, __half* kv_pool, const int* d_block_table, __half* out,
                                       int fa_layer_idx, int seq_len, int max_phys_blocks, int block_size,
                                       float scale, cudaStream_t stream = 0) {
    drkv_geometry g = shim_geometry();
    g.page_size = block_size;
    size_t scratch_bytes = 0;
    void* scratch = detail::decode_scratch(drkv_k_decode_scratch_bytes(&g, seq_len > 0 ? seq_len : 1), &scratch_bytes);
    if (scratch == nullptr) {
        std::fprintf(stderr, "[Machina] paged_gqa_decode_attention: scratch allocation failed\n");
        return;
    }
    if (drkv_k_decode_attention(&g, Q, kv_pool, d_block_table, out, fa_layer_idx, seq_len, max_phys_blocks, scale,
                                scratch, scratch_bytes, stream) != DRKV_OK)
        std::fprintf(stderr, "[Machina] paged_gqa_decode_attention: %s\n", drkv_last_error());
}

// What the kernels of the last paged_gqa_decode_attention call on this device reported (a bounded wait that gave
// up, a table entry beyond the pool): true = nothing.  Synchronises the stream.  The reference's kernels have no
// error path (src/machina/paged_attention.cu:219-230 index the pool unchecked).
inline bool shim_decode_kernels_ok(cudaStream_t stream = 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    void* ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(detail::decode_scratch_mutex());
        ptr = detail::decode_scratch_slots()[dev].ptr;
    }
    if (ptr == nullptr) return true;
    if (drkv_k_decode_kernel_error(ptr, stream) == DRKV_OK) return true;
    std::fprintf(stderr, "[Machina] paged_gqa_decode_attention: %s\n", drkv_last_error());
    return false;
}

// ---- src/memoria/cache_kernels.h:44-74 -----------------------------------------------------------
inline void invoke_extract_kv_from_pages(__half* dst, const __half* kv_pool, const int* block_table, int start_token,
                                         int num_tokens, int num_layers, int num_kv_heads, int head_dim,
                                         int block_size, int max_phys_blocks, cudaStream_t stream) {
    drkv_geometry g = shim_geometry();
    g.num_layers = num_layers;
    g.num_kv_heads = num_kv_heads;
    g.num_q_heads = num_kv_heads * (shim_geometry().num_q_heads / shim_geometry().num_kv_heads);
    g.head_dim = head_dim;
    g.page_size = block_size;
    if (drkv_k_extract_kv(&g, dst, kv_pool, block_table, start_token, num_tokens, max_phys_blocks, stream) != DRKV_OK)
        std::fprintf(stderr, "[Memoria] invoke_extract_kv_from_pages: %s\n", drkv_last_error());
}

inline void invoke_inject_kv_to_pages(__half* kv_pool, const __half* src, const int* block_table, int start_token,
                                      int num_tokens, int num_layers, int num_kv_heads, int head_dim, int block_size,
                                      int max_phys_blocks, cudaStream_t stream) {
    drkv_geometry g = shim_geometry();
    g.num_layers = num_layers;
    g.num_kv_heads = num_kv_heads;
    g.num_q_heads = num_kv_heads * (shim_geometry().num_q_heads / shim_geometry().num_kv_heads);
    g.head_dim = head_dim;
    g.page_size = block_size;
    if (drkv_k_inject_kv(&g, kv_pool, src, block_table, start_token, num_tokens, max_phys_blocks, stream) != DRKV_OK)
        std::fprintf(stderr, "[Memoria] invoke_inject_kv_to_pages: %s\n", drkv_last_error());
}

}  // namespace deusridet
