// C entry points over the reference's own BlockPool / CacheManager objects
// (src/memoria/block_pool.h:58-123, src/memoria/cache_manager.h:52-169), so that
// a test can drive them through ctypes and record what they do.
// Test infrastructure only; compiled together with the reference sources where
// they lie, never shipped.
#include "memoria/block_pool.h"
#include "memoria/cache_manager.h"
#include "memoria/kv_swapper.h"
#include "memoria/importance_scorer.h"
#include "communis/log.h"
#include <cstdio>
#include <cstdlib>
#include <cstring>

using namespace deusridet;

static size_t budget_for(int num_fa_layers, int n_pages, int block_size) {
    ModelConfig::NUM_FA_LAYERS = num_fa_layers;
    size_t per_page = (size_t)num_fa_layers * 2 * PagedKVConfig::NUM_KV_HEADS * block_size *
                      PagedKVConfig::HEAD_DIM * sizeof(__half);
    return per_page * (size_t)n_pages;
}

extern "C" {

void ref_quiet(int quiet) {
    deusridet::log::set_level(quiet ? deusridet::log::Level::ERROR : deusridet::log::Level::INFO);
}

// ---- BlockPool ------------------------------------------------------------
void* ref_bp_create(int num_fa_layers, int n_pages, int block_size, size_t extra_bytes) {
    BlockPool* p = new BlockPool();
    if (!p->init(budget_for(num_fa_layers, n_pages, block_size) + extra_bytes, block_size)) {
        delete p;
        return nullptr;
    }
    return p;
}
void ref_bp_destroy(void* h) { delete (BlockPool*)h; }
int ref_bp_alloc(void* h) { return ((BlockPool*)h)->alloc_block(); }
void ref_bp_free(void* h, int id) { ((BlockPool*)h)->free_block(id); }
int ref_bp_free_count(void* h) { return ((BlockPool*)h)->free_count(); }
int ref_bp_max_blocks(void* h) { return ((BlockPool*)h)->max_blocks(); }
int ref_bp_block_size(void* h) { return ((BlockPool*)h)->block_size(); }
size_t ref_bp_total_bytes(void* h) { return ((BlockPool*)h)->total_bytes(); }
size_t ref_bp_k_offset(void* h, int layer, int id) { return ((BlockPool*)h)->k_offset(layer, id); }
size_t ref_bp_v_offset(void* h, int layer, int id) { return ((BlockPool*)h)->v_offset(layer, id); }
size_t ref_bp_k_ptr_offset(void* h, int layer, int id) {
    BlockPool* p = (BlockPool*)h;
    return (size_t)((char*)p->k_ptr(layer, id) - (char*)p->pool_ptr());
}
size_t ref_bp_v_ptr_offset(void* h, int layer, int id) {
    BlockPool* p = (BlockPool*)h;
    return (size_t)((char*)p->v_ptr(layer, id) - (char*)p->pool_ptr());
}

// ---- CacheManager ---------------------------------------------------------
void* ref_cm_create(int num_fa_layers, int n_pages, int block_size) {
    CacheManager* c = new CacheManager();
    if (!c->init(budget_for(num_fa_layers, n_pages, block_size), "", block_size)) {
        delete c;
        return nullptr;
    }
    return c;
}
void ref_cm_destroy(void* h) { delete (CacheManager*)h; }

// CacheManager with the reference's ImportanceScorer attached (cache_manager.h:67-71; the manager
// borrows the scorer).  One handle owns both.
struct ScoredManager {
    ImportanceScorer scorer;
    CacheManager cm;
};
void* ref_scored_create(int num_fa_layers, int n_pages, int block_size, float decay, void** cm_out) {
    ScoredManager* s = new ScoredManager();
    if (!s->scorer.init(2 * n_pages, decay) ||
        !s->cm.init(budget_for(num_fa_layers, n_pages, block_size), "", block_size, nullptr, &s->scorer)) {
        delete s;
        return nullptr;
    }
    *cm_out = &s->cm;
    return s;
}
void ref_scored_destroy(void* h) { delete (ScoredManager*)h; }
// ImportanceScorer::update followed by sync_to_host, the sequence a caller needs before the policy
// sees new values.  new_scores is "device" memory of the stub runtime, i.e. host memory.
void ref_scored_update(void* h, const float* new_scores, int n) {
    ScoredManager* s = (ScoredManager*)h;
    s->scorer.update(new_scores, n);
    s->scorer.sync_to_host();
}
float ref_scored_score(void* h, int idx) { return ((ScoredManager*)h)->scorer.score(idx); }
int ref_cm_ensure(void* h, int pos) { return ((CacheManager*)h)->ensure_blocks_for(pos) ? 1 : 0; }
int ref_cm_ensure_range(void* h, int pos, int m) {
    return ((CacheManager*)h)->ensure_blocks_for_range(pos, m) ? 1 : 0;
}
int ref_cm_evict(void* h, int n) { return ((CacheManager*)h)->evict_blocks(n); }
int ref_cm_ensure_free(void* h, int n) { return ((CacheManager*)h)->ensure_free_blocks(n) ? 1 : 0; }
void ref_cm_set_seq_len(void* h, int n) { ((CacheManager*)h)->set_seq_len(n); }
int ref_cm_seq_len(void* h) { return ((CacheManager*)h)->seq_len(); }
int ref_cm_num_logical_blocks(void* h) { return ((CacheManager*)h)->num_logical_blocks(); }
int ref_cm_gpu_blocks_used(void* h) { return ((CacheManager*)h)->gpu_blocks_used(); }
int ref_cm_ssd_blocks_used(void* h) { return ((CacheManager*)h)->ssd_blocks_used(); }
int ref_cm_free_blocks(void* h) { return ((CacheManager*)h)->free_blocks(); }
int ref_cm_max_blocks(void* h) { return ((CacheManager*)h)->block_pool().max_blocks(); }
// Direct pool access, as Conscientia has through block_pool().
int ref_cm_pool_alloc(void* h) { return ((CacheManager*)h)->block_pool().alloc_block(); }
void ref_cm_pool_free(void* h, int id) { ((CacheManager*)h)->block_pool().free_block(id); }
// Mirrors the table exactly as the kernels would see it: sync, then read the
// "device" copy (host memory under the stub).
int ref_cm_table(void* h, int* out, int cap) {
    CacheManager* c = (CacheManager*)h;
    c->sync_block_table(0);
    int n = c->block_pool().max_blocks() * 2;
    if (n > cap) n = cap;
    memcpy(out, c->d_block_table(), (size_t)n * sizeof(int));
    return n;
}

}  // extern "C"
