/*
 * drkv.h — C ABI of the B200 paged KV-cache engine.
 *
 * One shared library (libdrkv.so) exports everything below with C linkage, plain
 * pointers and sizes.  It replaces, for the KV-cache hot path only, what the
 * DeusRidet reference links statically from its `memoria` and `machina` libraries:
 *
 *   page pool            src/memoria/block_pool.h:58-123     (BlockPool)
 *   block tables/evict   src/memoria/cache_manager.h:52-169  (CacheManager)
 *   K/V append           src/machina/paged_attention.h:27-52 (paged_kv_cache_write[_batch])
 *   RoPE on K            src/machina/layer.h:127-130, src/machina/layer_attention.cu:32-79
 *   decode attention     src/machina/paged_attention.h:61-71 (paged_gqa_decode_attention)
 *   prefill attention    src/machina/paged_attention.cu:465-554 (paged_prefill_attention_kernel)
 *   split-KV merge       src/sensus/auditus/asr/asr_ops_attn.cu:88-108 (semantic analogue)
 *
 * Conventions: every call returns DRKV_OK (0) or a negative drkv_status; nothing throws
 * across this boundary; kernels are enqueued on the caller's stream (a cudaStream_t
 * passed as void*) and never synchronise; device memory is owned by the engine and
 * released by drkv_destroy().  There is no CPU fallback: a compute entry point called
 * on an engine without a device returns DRKV_ERR_NO_DEVICE.
 *
 * Pool layout, identical to the reference (src/machina/paged_attention.cu:13-18,
 * src/memoria/block_pool.cpp:23-24,81-95), in elements of the storage type:
 *   elem(layer, page, kv, head, slot, d) =
 *       layer * layer_stride + page * block_stride + kv * kv_plane
 *       + head * page_size * head_dim + slot * head_dim + d
 *   kv_plane = num_kv_heads * page_size * head_dim, block_stride = 2 * kv_plane,
 *   layer_stride = max_pages * block_stride.
 */
#ifndef DRKV_H_
#define DRKV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DRKV_API __attribute__((visibility("default")))

typedef enum drkv_status {
    DRKV_OK = 0,
    DRKV_ERR_INVALID = -1,     /* bad argument (range, alignment, unsupported geometry) */
    DRKV_ERR_EXHAUSTED = -2,   /* no free page and nothing evictable */
    DRKV_ERR_NO_DEVICE = -3,   /* compute call on a bookkeeping-only engine, or no GPU */
    DRKV_ERR_CUDA = -4,        /* a CUDA runtime/driver call failed; see drkv_last_error */
    DRKV_ERR_STATE = -5,       /* double free, unknown sequence, released sequence ... */
    DRKV_ERR_CAPACITY = -6     /* position beyond the table, too many sequences, scratch too small */
} drkv_status;

enum { DRKV_DTYPE_F16 = 0, DRKV_DTYPE_BF16 = 1 };

/* Runtime geometry.  The reference fixes these at compile time (PagedKVConfig,
 * src/memoria/block_pool.h:34-52) or in process-wide statics (ModelConfig,
 * src/machina/model.h:30-83). */
typedef struct drkv_geometry {
    int32_t num_layers;    /* full-attention layers sharing the pool (NUM_FA_LAYERS) */
    int32_t num_q_heads;
    int32_t num_kv_heads;
    int32_t head_dim;      /* 64, 128 or 256 */
    int32_t page_size;     /* tokens per page, a multiple of 16 */
    int32_t dtype;         /* DRKV_DTYPE_* : storage type of Q, K, V, out and the pool */
    int32_t rotary_dim;    /* leading dims of each K head that RoPE rotates (0 = none) */
    float rope_theta;
} drkv_geometry;

typedef struct drkv_config {
    size_t budget_bytes;        /* pool budget; used when max_pages == 0 (BlockPool::init) */
    int32_t max_pages;          /* explicit page count (0 = derive from budget_bytes) */
    int32_t max_seqs;           /* rows of the device table */
    int32_t max_pages_per_seq;  /* row width; 0 = 2 * max_pages as in CacheManager::init */
    int32_t device;             /* CUDA device ordinal; -1 = bookkeeping only, no device memory */
    int32_t stream_evict;       /* 1 = a sequence that cannot get a page discards its own oldest
                                   page (CacheManager behaviour); 0 = fail with DRKV_ERR_EXHAUSTED */
} drkv_config;

typedef struct drkv_stats {
    int64_t pages_total, pages_free, pages_cached, pages_active;
    int64_t evictions_cached, evictions_stream, cow_copies, cow_bytes;
    int64_t table_sync_bytes, table_syncs;
    int64_t live_seqs;
} drkv_stats;

/* One eviction, in the order it happened.  kind 0: an unreferenced cached page was
 * reclaimed (seq = logical = -1).  kind 1: a sequence discarded one of its own pages.
 * kind 2: a sequence's page was written to the storage tier and its pool page freed. */
typedef struct drkv_evict_record {
    int32_t kind, seq, logical, page;
} drkv_evict_record;

typedef struct drkv_engine drkv_engine;

/* ---- lifetime ------------------------------------------------------------------- */
/* CacheManager::init + BlockPool::init (src/memoria/cache_manager.cpp:24-71,
 * src/memoria/block_pool.cpp:18-61): page count = budget / bytes per page over all layers,
 * fails below 4 pages, slab zero-filled, page ids pop 0,1,2,... */
DRKV_API int drkv_create(const drkv_geometry* geom, const drkv_config* cfg, drkv_engine** out);
/* CacheManager::destroy / BlockPool::destroy (cache_manager.cpp:328-338, block_pool.cpp:97-105) */
DRKV_API void drkv_destroy(drkv_engine* e);
/* Text of the last failure on this thread (the reference logs with LOG_ERROR instead). */
DRKV_API const char* drkv_last_error(void);
DRKV_API int drkv_get_geometry(const drkv_engine* e, drkv_geometry* out);
DRKV_API int drkv_get_stats(const drkv_engine* e, drkv_stats* out);

/* ---- page pool: BlockPool (src/memoria/block_pool.h:69-107) --------------------- */
DRKV_API int drkv_pool_alloc(drkv_engine* e);                 /* alloc_block: id or -1 */
DRKV_API int drkv_pool_free(drkv_engine* e, int page);        /* free_block, with double-free/range check */
DRKV_API int drkv_pool_free_count(const drkv_engine* e);      /* free_count */
DRKV_API int drkv_pool_max_pages(const drkv_engine* e);       /* max_blocks */
DRKV_API int drkv_pool_page_size(const drkv_engine* e);       /* block_size */
DRKV_API void* drkv_pool_ptr(const drkv_engine* e);           /* pool_ptr (device) */
DRKV_API size_t drkv_pool_total_bytes(const drkv_engine* e);  /* total_bytes */
DRKV_API size_t drkv_pool_k_offset(const drkv_engine* e, int layer, int page);  /* k_offset (bytes) */
DRKV_API size_t drkv_pool_v_offset(const drkv_engine* e, int layer, int page);  /* v_offset (bytes) */

/* ---- sequences and block tables: CacheManager (src/memoria/cache_manager.h:67-125) */
/* The reference has one implicit sequence; here each sequence owns one table row. */
DRKV_API int drkv_seq_create(drkv_engine* e);                 /* new empty sequence: id (lowest free) */
/* Drops the sequence.  Pages whose reference count reaches 0 keep their contents and
 * join the tail of the evictable LRU list (discard = 0), or go straight back to the
 * free stack (discard = 1), in ascending logical order. */
DRKV_API int drkv_seq_release(drkv_engine* e, int seq, int discard);
/* Decode branch: the child shares every page of the parent (reference count + 1).
 * No counterpart in the reference code; intent in docs/en/architecture/02-memoria.md:25-26. */
DRKV_API int drkv_seq_fork(drkv_engine* e, int parent);
/* ensure_blocks_for(pos) (cache_manager.cpp:73-95): make the page holding `pos` resident
 * and private to this sequence (copy-on-write when it is shared). */
DRKV_API int drkv_seq_ensure_pos(drkv_engine* e, int seq, int pos, void* stream);
/* ensure_blocks_for_range(pos_start, m) (cache_manager.cpp:97-106): stops at the first
 * failure and keeps earlier allocations. */
DRKV_API int drkv_seq_ensure_range(drkv_engine* e, int seq, int pos_start, int m, void* stream);
/* ensure_blocks_for_range(seq_len, n): room for n more tokens after the current length. */
DRKV_API int drkv_seq_reserve(drkv_engine* e, int seq, int n_tokens, void* stream);
/* The per-token pair of a decode loop for a whole batch in one call each (the reference makes the
 * two calls once per token for its single sequence, src/conscientia/stream.cpp:297, 369-370):
 * reserve n_tokens more for every listed sequence (stops at the first failure, earlier allocations
 * stay), and set_seq_len(seq_len + n_tokens) for every listed sequence. */
DRKV_API int drkv_seq_reserve_batch(drkv_engine* e, int n, const int32_t* seqs, int n_tokens, void* stream);
DRKV_API int drkv_seq_advance_batch(drkv_engine* e, int n, const int32_t* seqs, int n_tokens);
DRKV_API int drkv_seq_set_len(drkv_engine* e, int seq, int len);   /* set_seq_len */
DRKV_API int drkv_seq_len(const drkv_engine* e, int seq);          /* seq_len */
DRKV_API int drkv_seq_num_pages(const drkv_engine* e, int seq);    /* num_logical_blocks = ceil(len / page) */
/* Host copy of the row (h_block_table_); returns entries written. */
DRKV_API int drkv_seq_table(const drkv_engine* e, int seq, int32_t* out, int cap);
/* Attach existing pages (active or cached) to an empty sequence as its first
 * ceil(n_tokens / page) logical pages: prefix reuse after the owner was released. */
DRKV_API int drkv_seq_adopt(drkv_engine* e, int seq, const int32_t* pages, int n_pages, int n_tokens);

/* ---- eviction (src/memoria/cache_manager.cpp:118-205) ----------------------------- */
/* evict_blocks(n) for one sequence: discard its n oldest-allocated resident pages that
 * nobody else references; returns the number evicted. */
DRKV_API int drkv_seq_evict(drkv_engine* e, int seq, int n);
/* Reclaim up to n unreferenced cached pages, least recently released first. */
DRKV_API int drkv_evict_cached(drkv_engine* e, int n);
/* ensure_free_blocks(n_free): cached pages first, then (stream_evict) pages of `seq`
 * (seq = -1: cached pages only).  Returns 1 if the target is met, 0 if not. */
DRKV_API int drkv_ensure_free(drkv_engine* e, int seq, int n_free);

/* ---- inspection (bit-exact bookkeeping artefacts) ---------------------------------- */
DRKV_API int drkv_refcounts(const drkv_engine* e, int32_t* out, int cap);
DRKV_API int drkv_free_stack(const drkv_engine* e, int32_t* out, int cap);   /* bottom..top */
DRKV_API int drkv_cached_lru(const drkv_engine* e, int32_t* out, int cap);   /* head(oldest)..tail */
DRKV_API int drkv_evict_log(drkv_engine* e, drkv_evict_record* out, int cap, int clear);

/* ---- device block tables (src/memoria/cache_manager.cpp:108-112) ------------------- */
/* sync_block_table: uploads only the entries changed since the last call. */
DRKV_API int drkv_sync_tables(drkv_engine* e, void* stream);
DRKV_API const int32_t* drkv_device_tables(const drkv_engine* e);  /* d_block_table: [max_seqs][stride] */
DRKV_API int drkv_table_stride(const drkv_engine* e);
/* Reads (and clears) the device error word that kernels set instead of trapping when a
 * bounded wait gives up or a table holds an impossible page id.  Synchronises the device.
 * The reference has no counterpart: its kernels index the pool unchecked. */
DRKV_API int drkv_kernel_error(drkv_engine* e);
/* Keys per split-KV chunk of the decode kernel: 0 = chosen per call from the batch shape,
 * else a positive multiple of 16.  Tuning knob, no counterpart in the reference. */
DRKV_API int drkv_set_chunk_tokens(drkv_engine* e, int chunk_tokens);
/* Tail split of the batched decode pass: the last `mode` chunks of every sequence are queued last and in
 * 64-key pieces so that the persistent warps finish close together.  -1: automatic (the default: on, with
 * 512-key chunks and one tail chunk, when the pass is at least three chunks deep per warp), 0: off,
 * 1..4: forced. */
DRKV_API int drkv_set_tail_split(drkv_engine* e, int mode);
/* Measurement aid (the reference brackets its kernels with cudaEvents the same way,
 * src/machina/forward.cu:265-275): while enabled, every launch of the decode attention kernel
 * is bracketed by CUDA events on its own stream (up to 512 launches).  A call first returns,
 * if the pointers are non-null, the summed duration and the count since the last call
 * (synchronises the device), then sets the new mode. */
DRKV_API int drkv_kernel_timing(drkv_engine* e, int enable, double* total_ms, int* launches);

/* ---- K/V append with RoPE on K ------------------------------------------------------ */
/* paged_kv_cache_write + rope_kernel's K half (paged_attention.cu:73-115,
 * layer_attention.cu:32-69), batched over sequences: sequence i of the batch uses table
 * row d_rows[i] and writes its token at d_pos[i] (both device int32 arrays).
 * k_src/v_src: [n_seq][num_kv_heads][head_dim] device, storage type.
 * As with drkv_attend_decode, d_rows, d_pos and the block table are read while the launch directly in
 * front may still be running: a caller's kernel that writes them and signals programmatic completion
 * early must not be that launch. */
DRKV_API int drkv_append_rope(drkv_engine* e, int layer, int n_seq, const int32_t* d_rows,
                              const int32_t* d_pos, const void* k_src, const void* v_src,
                              void* stream);
/* paged_kv_cache_write_batch + paged_rope_batch_kernel's K half (paged_attention.cu:123-167,
 * 412-451): m consecutive tokens of one sequence from pos_start.
 * k_src/v_src: [m][num_kv_heads][head_dim]. */
DRKV_API int drkv_append_rope_chunk(drkv_engine* e, int layer, int seq, int pos_start, int m,
                                    const void* k_src, const void* v_src, void* stream);

/* ---- flat <-> paged copies ------------------------------------------------------------ */
/* invoke_extract_kv_from_pages / invoke_inject_kv_to_pages (src/memoria/cache_kernels.h:44-74,
 * cache_kernels.cu:30-187) for tokens [start_token, start_token + num_tokens) of one sequence, all
 * layers.  Flat layout [layer][K|V][token][kv_head][dim].  Pages missing from the table read as
 * zeros (extract) or are skipped (inject). */
DRKV_API int drkv_seq_extract(drkv_engine* e, int seq, int start_token, int num_tokens, void* dst, void* stream);
DRKV_API int drkv_seq_inject(drkv_engine* e, int seq, int start_token, int num_tokens, const void* src, void* stream);

/* ---- attention ---------------------------------------------------------------------- */
/* paged_gqa_decode_attention (paged_attention.cu:179-282), batched: q/out
 * [n_seq][num_q_heads][head_dim]; sequence i attends to keys 0..d_kv_len[i]-1 of table row
 * d_rows[i].  max_kv_len is a host-side upper bound of the d_kv_len values (it sizes the
 * grid).  Table entries < 0 are skipped.  A sequence with no visible key leaves its output
 * rows untouched (paged_attention.cu:266-268).
 * The kernels are launched with programmatic dependent launch, and the attention kernel reads
 * d_rows, d_kv_len and the block table while the kernel in front of it may still be running
 * (everything before THAT kernel has completed).  Arrays written by copies, by ordinary kernels
 * or by this library's kernels are therefore safe; a caller's own kernel that writes them AND
 * signals programmatic completion early must not be the launch directly in front. */
DRKV_API int drkv_attend_decode(drkv_engine* e, int layer, int n_seq, const int32_t* d_rows,
                                const int32_t* d_kv_len, int max_kv_len, const void* q, void* out,
                                float scale, void* stream);
/* The decode step of one layer in one call: paged_kv_cache_write + rope_kernel's K half + paged_gqa_decode_attention
 * (paged_attention.cu:353-367 runs them as three launches).  d_kv_len[i] counts the new token: it is appended at
 * position d_kv_len[i] - 1 of table row d_rows[i] from k_src / v_src [n_seq][num_kv_heads][head_dim] and attended
 * to with the rest.  There is no append launch: the work item of the attention kernel that
 * reaches the new position rotates K, uses both rows from the caller's buffers and writes them into the page (the
 * same bytes drkv_append_rope writes).  A hole at the new position
 * writes nothing, as in drkv_append_rope. */
DRKV_API int drkv_append_attend_decode(drkv_engine* e, int layer, int n_seq, const int32_t* d_rows,
                                       const int32_t* d_kv_len, int max_kv_len, const void* k_src, const void* v_src,
                                       const void* q, void* out, float scale, void* stream);
/* Shared-prefix decode.  The reference's decode kernel (paged_attention.cu:179-282) walks every
 * sequence's whole block table, so branches forked from one prompt (CacheManager block tables that
 * start with the same page ids) each read the shared pages again.  A plan finds, among CONSECUTIVE
 * batch entries, families whose host tables start with the same pages; the planned pass reads those
 * pages once per 16 query rows of the family, and every sequence's remaining keys as before.  The
 * result is the same attention (same partial/merge arithmetic, different grouping of rows).
 * seqs / kv_len are HOST arrays of n_seq (<= 2048) entries; the plan is uploaded on `stream` and
 * holds until the next call that changes a block table.  No counterpart in the reference. */
typedef struct drkv_plan_info {
    int32_t n_seq, n_families, n_blocks, chunk_tokens;
    int64_t keys_per_sequence_pass; /* sum of kv_len: key positions an unplanned pass reads per kv head */
    int64_t keys_planned_pass;      /* key positions the planned pass reads per kv head */
} drkv_plan_info;
DRKV_API int drkv_plan_decode(drkv_engine* e, int n_seq, const int32_t* seqs, const int32_t* kv_len,
                              void* stream);
DRKV_API int drkv_plan_get_info(const drkv_engine* e, drkv_plan_info* out);
/* The plan as the kernel reads it, for inspection (works on an engine without a device; returns the
 * number of ints): rows[n_seq], kv_len[n_seq], first_chunk[n_seq] (chunks of each sequence that its
 * family's blocks cover), then per block: table row of the family's first member [n_blocks], shared
 * chunks [n_blocks], batch indices of up to 16 members, -1 padded [n_blocks][16]. */
DRKV_API int drkv_plan_dump(const drkv_engine* e, int32_t* out, int cap);
/* q/out [n_seq][num_q_heads][head_dim] in the plan's batch order. */
DRKV_API int drkv_attend_decode_planned(drkv_engine* e, int layer, const void* q, void* out,
                                        float scale, void* stream);
/* The planned pass with the append of each entry's new token in the same call, as drkv_append_attend_decode does
 * for the per-sequence pass: the plan's lengths count the token, whose position is kv_len - 1; k_src / v_src
 * [n_seq][num_kv_heads][head_dim] in the plan's batch order.  The token always falls into an item of its own
 * sequence (the chunks a family shares are whole chunks of cached keys), which rotates K, writes both rows into the
 * page and attends over them. */
DRKV_API int drkv_append_attend_decode_planned(drkv_engine* e, int layer, const void* k_src, const void* v_src,
                                               const void* q, void* out, float scale, void* stream);
/* ---- storage tier behind the pool --------------------------------------------------------------
 * KVSwapper (kv_swapper.h:52-120, kv_swapper.cpp:179-300) and CacheManager's swap paths
 * (cache_manager.cpp:132-141, 215-292): with a tier enabled, a page that a sequence evicts from
 * itself is written to `dir` (row 0: block_<logical>.kv as cache_manager.cpp:211-213, other rows
 * seq<row>_block_<logical>.kv) instead of discarded, and drkv_seq_ensure_pos / _range / _reserve on a
 * stored page allocates a pool page (discarding, never storing, a victim if the pool is empty) and
 * reads it back.  File = for every layer the K plane then the V plane of the page, sized from the
 * engine's geometry (the reference sizes it from compile-time constants).  Both moves are synchronous
 * unless drkv_tier_set_write_behind turns deferred file writes on.  On an engine without a device the files
 * are empty markers. */
typedef struct drkv_tier_stats {
    int64_t pages_stored, swap_outs, swap_ins, bytes_out, bytes_in, prefetch_hits, page_file_bytes;
    int64_t writes_deferred, write_failures;   /* write-behind: file writes handed to the worker thread / that failed there */
} drkv_tier_stats;
DRKV_API int drkv_tier_enable(drkv_engine* e, const char* dir);
DRKV_API int drkv_tier_disable(drkv_engine* e);       /* refused while pages are stored */
/* CacheManager::prefetch_block (cache_manager.cpp:166-180): background read of a stored page into host
 * memory, so that the swap-in skips the file.  Returns 1 if queued, 0 if the page is not stored. */
DRKV_API int drkv_tier_prefetch(drkv_engine* e, int seq, int logical);
DRKV_API int drkv_tier_drain(drkv_engine* e);          /* waits for queued prefetches and deferred file writes */
/* Write-behind (off by default).  The reference moves pages on an I/O thread with its own stream
 * (kv_swapper.cpp:154-177) but CacheManager waits for it (submit + drain, cache_manager.cpp:215-241), so its moves
 * are synchronous in effect.  With write-behind on, a swap-out returns once the page's bytes are in pinned host
 * memory (the pool page is free from then on) and a worker thread writes the file; whatever touches that page
 * next (swap-in, prefetch, release) waits for its write.  Up to four pages may wait for their files. */
DRKV_API int drkv_tier_set_write_behind(drkv_engine* e, int on);
/* KVSwapper::is_prefetched / drop_prefetch (kv_swapper.h:85-88): 1 if a background read of the page has landed. */
DRKV_API int drkv_tier_is_prefetched(drkv_engine* e, int seq, int logical);
DRKV_API int drkv_tier_drop_prefetch(drkv_engine* e, int seq, int logical);
/* What one KVSwapper::submit request does (SwapRequest, kv_swapper.h:36-44): pool page `page` to the file `path`
 * (GPU_TO_SSD) or back (SSD_TO_GPU), file layout as above.  Synchronous; the bookkeeping is the caller's. */
DRKV_API int drkv_tier_page_to_file(drkv_engine* e, int page, const char* path);
DRKV_API int drkv_tier_file_to_page(drkv_engine* e, const char* path, int page);
DRKV_API int drkv_tier_get_stats(const drkv_engine* e, drkv_tier_stats* out);
/* BlockLocation per logical page of a sequence (cache_manager.h:42-46): 0 invalid, 1 in the pool, 2 stored. */
DRKV_API int drkv_seq_locations(const drkv_engine* e, int seq, int8_t* out, int cap);

/* ---- importance-guided eviction ------------------------------------------------------------
 * ImportanceScorer (importance_scorer.h:25-67, importance_scorer.cu:27-99) attached to the eviction
 * policy (cache_manager.cpp:185-205): one fp32 score per (sequence, logical page), updated as
 * score = score * decay + new, copied to a host mirror on request; a sequence's victim becomes the
 * resident, unshared page with the lowest mirrored score (the first such in allocation order)
 * instead of its oldest.  The reference never produces `new` (no caller of update()); here
 * drkv_attend_decode and drkv_attend_decode_planned accumulate, while the scorer is enabled, the
 * softmax probability mass each page received, summed over query heads and layers ("per-block
 * attention weights across all Full Attention layers", importance_scorer.h:8-10), and
 * drkv_scorer_step folds that into the scores once per token. */
/* ImportanceScorer::init: decay >= 0 enables (scores start at 0), decay < 0 detaches. */
DRKV_API int drkv_scorer_enable(drkv_engine* e, float decay);
/* ImportanceScorer::update for the first num_blocks logical pages of one sequence with values the
 * caller provides: a device pointer on an engine with a device, a host pointer on one without. */
DRKV_API int drkv_scorer_update(drkv_engine* e, int seq, const float* new_scores, int num_blocks, void* stream);
/* score = score * decay + accumulated attention mass, for every sequence; the accumulator restarts. */
DRKV_API int drkv_scorer_step(drkv_engine* e, void* stream);
/* ImportanceScorer::sync_to_host: device scores to the host mirror eviction reads; synchronises the stream. */
DRKV_API int drkv_scorer_sync(drkv_engine* e, void* stream);
/* ImportanceScorer::score for a whole sequence: the mirrored scores of its logical pages; returns the count. */
DRKV_API int drkv_scorer_scores(const drkv_engine* e, int seq, float* out, int cap);

/* paged_prefill_attention_kernel (paged_attention.cu:465-554): q/out
 * [m][num_q_heads][head_dim]; token t attends keys 0..pos_start+t.  Runs on the tensor-core (tcgen05) kernel at
 * head_dim 64, 128 and 256 (the reference model's own, block_pool.h:34-40).  A pool with more than 2^31 head rows,
 * which one TMA descriptor cannot address, or an engine told so by drkv_set_prefill_on_decode_kernel(e, 1), runs
 * the chunk as a batch of one-token decodes on the split-KV decode kernel: same results within the tolerance, every
 * token re-reads its keys (about ten times slower). */
DRKV_API int drkv_set_prefill_on_decode_kernel(drkv_engine* e, int on);
DRKV_API int drkv_attend_prefill_chunk(drkv_engine* e, int layer, int seq, int pos_start, int m,
                                       const void* q, void* out, float scale, void* stream);
/* The same for several sequences in one launch (host arrays of n_seq entries; q[i] / out[i] are
 * device pointers): independent sequences prefilling in step fill the GPU better than one chunk.
 * No counterpart in the reference, whose prefill handles one sequence. */
DRKV_API int drkv_attend_prefill_batch(drkv_engine* e, int layer, int n_seq, const int32_t* seqs,
                                       const int32_t* pos_start, const int32_t* m, const void* const* q,
                                       void* const* out, float scale, void* stream);
/* One sequence whose pages are split across GPUs by contiguous key range: this rank
 * attends keys [kv_begin, kv_end) of table row `seq` and returns the un-normalised partial
 * (m, l, o) per query head in fp32: part[0 .. Hq*D) = o, then Hq values m, then Hq values l.
 * Empty range: m = -1e20, l = 0, o = 0 (asr_ops_attn.cu:38-42). */
DRKV_API int drkv_attend_partial(drkv_engine* e, int layer, int seq, int kv_begin, int kv_end,
                                 const void* q, float* part, float scale, void* stream);
/* The same split across GPUs with the merge fused with the exchange: drkv_attend_exchange computes this
 * rank's partial over [kv_begin, kv_end) and then ONE kernel pushes it into every rank's exchange area
 * with peer stores over NVLink, every value as one 64-bit {fp32 value, call number} word, polls the words the
 * peers push (bounded: a rank that never arrives ends the wait after 2 s with kernel error 4, the outputs are
 * left as they were, nothing traps) and writes the merged output; no library collective is called.  Every rank makes the same sequence of drkv_attend_exchange
 * calls.  Set-up: each rank (one process per GPU, same node) creates its area and gets a 64-byte CUDA IPC
 * handle, the ranks exchange handles by any host-side means, each connects to all.  No counterpart in the
 * reference, which is single-GPU. */
#define DRKV_IPC_HANDLE_BYTES 64
DRKV_API int drkv_exchange_create(drkv_engine* e, int world, int rank, uint8_t* handle_out /* [64] */);
DRKV_API int drkv_exchange_connect(drkv_engine* e, const uint8_t* handles /* [world][64] */);
/* Ranks that live in ONE process (one engine per GPU, peer access enabled by the host) connect with plain device
 * pointers instead of IPC handles: areas[r] = drkv_exchange_area() of rank r's engine. */
DRKV_API int drkv_exchange_connect_local(drkv_engine* e, void* const* areas /* [world] */);
DRKV_API void* drkv_exchange_area(const drkv_engine* e);
/* How long the merge kernel waits for a peer's words before it gives up with kernel error 4 (default 2000 ms). */
DRKV_API int drkv_exchange_set_wait_ms(drkv_engine* e, int ms);
DRKV_API int drkv_exchange_destroy(drkv_engine* e);   /* after a host-side barrier: peers must be done */
DRKV_API int drkv_attend_exchange(drkv_engine* e, int layer, int seq, int kv_begin, int kv_end,
                                  const void* q, void* out, float scale, void* stream);
/* drkv_attend_exchange with the new token's append fused as in drkv_append_attend_decode: the rank whose range ends
 * at the sequence's end (kv_end = length including the new token) passes the token's k_src / v_src
 * [num_kv_heads][head_dim]; every other rank passes NULL for both. */
DRKV_API int drkv_append_attend_exchange(drkv_engine* e, int layer, int seq, int kv_begin, int kv_end,
                                         const void* k_src, const void* v_src, const void* q, void* out, float scale,
                                         void* stream);
/* contiguous_split_k_merge_kernel (asr_ops_attn.cu:88-108): merges n_parts partials laid
 * out as drkv_attend_partial writes them (parts[p] at p * (Hq*(D+2)) floats). */
DRKV_API int drkv_combine_partials(drkv_engine* e, int n_parts, const float* parts, void* out,
                                   void* stream);
DRKV_API size_t drkv_partial_floats(const drkv_engine* e);   /* Hq * (D + 2) */

/* ---- partitioning across the GPUs of one box (one process per GPU) ---------------------------
 * No counterpart in the reference, which is single-GPU.  One long sequence is split by contiguous page range:
 * rank r owns pages [lo, hi) (sizes differ by at most one, earlier ranks take the larger shares), attends keys
 * [begin, end) = that range clipped to the sequence, and the rank whose range holds a position appends it.
 * Independent sequences are placed by greedy balance of their cost (context length), largest unit first;
 * families[i] (NULL: none) groups forks that share pages: a family goes to one rank as a unit.
 * rank_of[i] receives the rank of sequence i. */
DRKV_API int drkv_shard_page_range(int n_pages, int rank, int world, int* lo, int* hi);
DRKV_API int drkv_shard_key_range(int seq_len, int page_size, int rank, int world, int* begin, int* end);
DRKV_API int drkv_shard_owner_of_position(int pos, int seq_len_after, int page_size, int world);   /* rank, or < 0 */
DRKV_API int drkv_shard_sequences(int n, const int64_t* costs, const int32_t* families, int world, int32_t* rank_of);

/* ---- stateless kernel entry points: the reference's free functions -------------------
 * Same argument meaning as src/machina/paged_attention.h:27-71 plus the geometry the
 * reference reads from ModelConfig statics.  One sequence, one table.  These kernels read nothing
 * (positions, block table, sources) before every earlier launch on the stream has completed: a caller's
 * own kernel may write d_pos or the table directly in front of them, as with the reference's launches.
 * (The engine's batched calls above read lengths and tables early; see drkv_attend_decode.) */
DRKV_API int drkv_k_cache_write(const drkv_geometry* g, const void* src_k, const void* src_v,
                                void* kv_pool, const int32_t* d_block_table, int layer,
                                const int32_t* d_pos, int max_pages, void* stream);
DRKV_API int drkv_k_cache_write_batch(const drkv_geometry* g, const void* src_k, const void* src_v,
                                      void* kv_pool, const int32_t* d_block_table, int layer,
                                      int pos_start, int m, int max_pages, void* stream);
/* `scratch`: device memory of at least drkv_k_decode_scratch_bytes(g, seq_len) bytes, 256-byte aligned.
 * d_block_table needs ceil(seq_len / page_size) entries and is not read beyond them. */
DRKV_API int drkv_k_decode_attention(const drkv_geometry* g, const void* q, const void* kv_pool,
                                     const int32_t* d_block_table, void* out, int layer,
                                     int seq_len, int max_pages, float scale, void* scratch,
                                     size_t scratch_bytes, void* stream);
DRKV_API size_t drkv_k_decode_scratch_bytes(const drkv_geometry* g, int seq_len);
/* The error word of the last drkv_k_decode_attention call that used `scratch` (NULL: of the last
 * drkv_k_decode_attention_noalloc call on the current device): DRKV_OK, or DRKV_ERR_CUDA with the
 * code in drkv_last_error() when a kernel gave up a bounded wait or met a page id >= max_pages (such
 * an entry is treated as a hole; nothing outside the pool is touched).  Synchronises `stream`.  Each
 * decode call clears the word when it starts, so ask before the next call on the same scratch.  The
 * reference's kernels have no counterpart: they index the pool unchecked (paged_attention.cu:219-230). */
DRKV_API int drkv_k_decode_kernel_error(const void* scratch, void* stream);
/* invoke_extract_kv_from_pages / invoke_inject_kv_to_pages with raw pointers
 * (src/memoria/cache_kernels.h:44-74); num_layers, heads, dims and block size come from g. */
DRKV_API int drkv_k_extract_kv(const drkv_geometry* g, void* dst, const void* kv_pool,
                               const int32_t* d_block_table, int start_token, int num_tokens,
                               int max_pages, void* stream);
DRKV_API int drkv_k_inject_kv(const drkv_geometry* g, void* kv_pool, const void* src,
                              const int32_t* d_block_table, int start_token, int num_tokens,
                              int max_pages, void* stream);

/* No counterpart in the reference.  drkv_k_decode_attention for callers that cannot get
 * device memory at all: hosts that own the whole GPU through their own allocator, threads that
 * must not take cudaMalloc's device-wide synchronisation, processes that have filled HBM with
 * KV pages.  The split-KV partials go to a scratch area built into the library
 * (DRKV_NOALLOC_SCRATCH_BYTES, resident on every GPU that loads the library until the process
 * exits); the call itself allocates and frees nothing, on the host side of CUDA or the device.
 *   - Limit: num_q_heads * ceil(seq_len / 4096) * (head_dim + 2) * 4 + 256 bytes must fit in the
 *     scratch (e.g. 32 heads, head_dim 128: about one million keys); beyond that the call
 *     returns DRKV_ERR_CAPACITY and launches nothing.
 *   - The first call on each device looks the scratch address up and configures the kernel;
 *     make that call before any stream capture begins.
 *   - All calls in the process share the one scratch area per GPU: two calls whose kernels can
 *     overlap on the GPU (different streams, no ordering between them) race on it.  Calls
 *     ordered on one stream are safe; each call re-initialises what it needs. */
#define DRKV_NOALLOC_SCRATCH_BYTES (4u << 20)
DRKV_API int drkv_k_decode_attention_noalloc(const drkv_geometry* g, const void* q, const void* kv_pool,
                                             const int32_t* d_block_table, void* out, int layer,
                                             int seq_len, int max_pages, float scale, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DRKV_H_ */
