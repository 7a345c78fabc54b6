// engine.cu — the C ABI (include/drkv.h): owns the pool slab, the device block tables and
// the split-KV scratch, keeps the host bookkeeping (page_book.hpp) and launches the kernels.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/drkv.h"
#include "kernels.hpp"
#include "page_book.hpp"
#include "page_store.hpp"
#include "stateless.hpp"

using namespace drkv;

namespace {

thread_local std::string g_err;

int set_err(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

bool geometry_ok(const drkv_geometry& g, std::string* why) {
    auto bad = [&](const char* m) {
        *why = m;
        return false;
    };
    if (g.num_layers <= 0 || g.num_q_heads <= 0 || g.num_kv_heads <= 0) return bad("layer/head counts must be positive");
    if (g.num_q_heads % g.num_kv_heads != 0) return bad("num_q_heads must be a multiple of num_kv_heads");
    if (g.num_q_heads / g.num_kv_heads > 16) return bad("GQA group larger than 16 is not supported");
    if (g.head_dim != 64 && g.head_dim != 128 && g.head_dim != 256) return bad("head_dim must be 64, 128 or 256");
    if (g.page_size <= 0 || g.page_size % 16 != 0) return bad("page_size must be a positive multiple of 16");
    if (g.dtype != DRKV_DTYPE_F16 && g.dtype != DRKV_DTYPE_BF16) return bad("dtype must be f16 or bf16");
    if (g.rotary_dim < 0 || g.rotary_dim > g.head_dim || g.rotary_dim % 16 != 0)
        return bad("rotary_dim must be a multiple of 16 within head_dim");
    if (g.rotary_dim > 0 && !(g.rope_theta > 0.f)) return bad("rope_theta must be positive");
    return true;
}

// freq_i = 1 / theta^(2i / rot) in fp32, the reference's expression
// (src/machina/layer_attention.cu:45) evaluated once on the host.
void fill_inv_freq(float theta, int rot, std::vector<float>* out) {
    out->resize(rot / 2);
    for (int i = 0; i < rot / 2; i++) (*out)[i] = 1.0f / powf(theta, (2.0f * (float)i) / (float)rot);
}

size_t page_bytes_all_layers(const drkv_geometry& g) {
    return (size_t)g.num_layers * 2 * g.num_kv_heads * g.page_size * g.head_dim * 2;
}

// Keys per work item, given a function that counts the items a chunk size produces.  Each item writes one
// fp32 partial per query row (rows * (D + 2) * 4 bytes against chunk * 2 * D * 2 bytes of K/V read), so
// the chunk starts large enough to keep that a few percent.  It shrinks when that shortens the longest
// warp's queue: warps take whole items, so the pass lasts about ceil(items / warps) items of (chunk +
// a fixed cost per item worth ~64 keys: start-up, the partial's write and its share of the merge) each.
template <typename ItemsFn>
int pick_chunk_by_cost(int group, long warps, bool exact, ItemsFn items) {
    int best = 0;
    long best_cost = 0;
    // Every multiple of 16 is a legal chunk.  With exact item counts (a decode plan knows every length) the
    // search goes down in steps of 16 and can land on a size whose items just fit a whole number of rounds;
    // with only an upper bound of the lengths it stays on powers of two.  Ties go to the larger chunk.
    for (int c = group > 4 ? 512 : 256; c >= 64; c = exact ? c - 16 : c >> 1) {
        const long n = items(c);
        const long cost = ((n + warps - 1) / warps) * (c + 64);
        if (best == 0 || cost < best_cost) {
            best = c;
            best_cost = cost;
        }
    }
    return best;
}

int pick_chunk(int n_seq, int hkv, int group, int max_kv_span, long warps) {
    auto items = [&](int c) { return (long)n_seq * hkv * ((max_kv_span + c - 1) / c); };
    if (n_seq == 1) {
        // One sequence: equal items, one per warp, is a perfect partition with the fewest partials, as long as an item
        // is not shorter than the smallest chunk the cost model would pick.
        const long per_head = warps / hkv > 0 ? warps / hkv : 1;
        const long c = ((max_kv_span + per_head - 1) / per_head + 15) / 16 * 16;
        if (c >= 64) return (int)c;
    }
    return pick_chunk_by_cost(group, warps, false, items);
}

}  // namespace

namespace drkv {
void set_last_error(const char* msg) { g_err = msg ? msg : ""; }
}  // namespace drkv

struct drkv_engine {
    drkv_geometry geom{};
    drkv_config cfg{};
    PageBook book;
    std::mutex mu;  // the reference guards the pool and ensure_blocks_for the same way

    bool has_device = false;
    int device = -1;
    void* pool = nullptr;
    size_t pool_bytes = 0;
    int32_t* d_tables = nullptr;
    float* d_inv_freq = nullptr;
    int* d_error = nullptr;
    float* d_scratch = nullptr;
    size_t scratch_bytes = 0;
    CUtensorMap tmap_pf{};     // 5-D view, one box per 16 keys x 128 dims x (K, V): the prefill kernel's (head_dim 128)
    bool has_tmap_pf = false;
    std::string tmap_pf_err;
    CUtensorMap tmap_slot{};   // 4-D view, one box per 16 keys x head_dim x (K, V): the decode kernel's
    PoolLayout layout{};
    int forced_chunk = 0;
    bool prefill_on_decode = false;   // chunk attention as one-token decodes even where the tensor-memory kernel could run
    int tail_mode = -1;        // tail split of the decode pass: -1 automatic (default), 0 off, n > 0: the last n chunks
    int num_sms = 148;
    int* d_work = nullptr;   // decode kernel's work-queue head
    int* d_exit = nullptr;   // decode kernel's count of warps that have left

    // optional per-launch timing of the decode attention kernel (events on the launch stream)
    bool timing = false;
    std::vector<cudaEvent_t> tev;   // pairs: start, stop
    size_t tev_used = 0;

    // staging for table updates: two pinned buffers used alternately
    int32_t* h_stage[2] = {nullptr, nullptr};
    cudaEvent_t stage_done[2] = {nullptr, nullptr};
    bool stage_busy[2] = {false, false};
    int stage_next = 0;
    size_t stage_ints = 0;
    int64_t sync_bytes = 0, syncs = 0, cow_bytes = 0;

    // shared-prefix decode plan: device arrays in one allocation, uploaded from two pinned buffers
    struct Plan {
        bool valid = false;
        int n_seq = 0, n_fb = 0, n_fam = 0, chunk = 0, max_chunks = 0, rows_per_item = 0, min_kv = 0;
        int64_t keys_seq = 0, keys_plan = 0;
        const int32_t *rows = nullptr, *kv_len = nullptr, *first_chunk = nullptr;
        const int32_t *fb_row = nullptr, *fb_chunks = nullptr, *fb_members = nullptr;
    } plan;
    std::vector<int32_t> plan_image;   // what the device holds: rows, kv_len, first_chunk, fb_row, fb_chunks, fb_members
    int32_t* d_plan = nullptr;
    int32_t* h_plan[2] = {nullptr, nullptr};
    cudaEvent_t plan_done[2] = {nullptr, nullptr};
    bool plan_busy[2] = {false, false};
    int plan_next = 0;

    // importance scorer (off until drkv_scorer_enable): scores per (sequence row, logical page)
    struct Scorer {
        bool on = false;
        float decay = 0.95f;
        std::vector<float> h_scores;                 // host mirror [max_seqs][row_width], what eviction reads
        float* d_scores = nullptr;                   // running scores
        float* d_fresh = nullptr;                    // attention mass accumulated since the last step
        float* d_tile_lse = nullptr;                 // decode kernel's per-tile values of one launch
        float* d_lse2 = nullptr;                     // merge kernel's log-sum-exp per (sequence, head)
        int max_tiles = 0;
        std::vector<std::pair<int, int>> pending;    // rows to reset (src = -1) or copy from src, at the next stream call
    } scorer;

    // cross-GPU exchange of one sequence's split-KV partials (off until drkv_exchange_create)
    struct Exchange {
        int world = 0, rank = 0;
        uint32_t seq_no = 0;
        void* area = nullptr;                        // this rank's slots + flags, one allocation
        void* peer_area[kMaxExchangeRanks] = {};     // every rank's area as mapped here (own = area)
        bool connected = false;
        bool local = false;                          // peers' areas were given as pointers, not opened through IPC
        unsigned long long wait_ns = 2000000000ull;  // bounded wait for a peer's flag
    } xchg;

    // storage tier behind the pool (off until drkv_tier_enable)
    std::unique_ptr<PageStore> store;
    cudaStream_t last_stream = nullptr;              // stream of the most recent kernel launches
};

// Remembers the stream kernels were last launched on: page copies to the storage tier wait for it.
static inline void note_stream(drkv_engine* e, cudaStream_t s) {
    e->last_stream = s;
    if (e->store) e->store->set_order_stream(s);
}

// ints of a plan: rows, kv_len, first_chunk per sequence; row, chunks and 16 members per family block
static constexpr size_t kPlanInts = (size_t)kMaxDecodeSeqs * 3 + (size_t)kMaxDecodeSeqs * 18;

#define LOCK(e) std::lock_guard<std::mutex> lock_((e)->mu)
#define NEED(e)                                                        \
    if ((e) == nullptr) return set_err(DRKV_ERR_INVALID, "null engine")
#define NEED_DEVICE(e)                                                                           \
    if (!(e)->has_device) return set_err(DRKV_ERR_NO_DEVICE, "engine was created without a device")
#define CUDA_TRY(expr)                                                                             \
    do {                                                                                           \
        cudaError_t ce_ = (expr);                                                                  \
        if (ce_ != cudaSuccess) return set_err(DRKV_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(ce_)); \
    } while (0)

static int book_err(drkv_engine* e, int rc) {
    if (rc < 0) g_err = e->book.error();
    return rc;
}

static int run_cow(drkv_engine* e, const std::vector<CowJob>& jobs, cudaStream_t stream) {
    for (const CowJob& j : jobs) {
        e->cow_bytes += (int64_t)j.n_slots * e->geom.head_dim * 2 * 2 * e->geom.num_kv_heads * e->geom.num_layers;
        if (!e->has_device) continue;
        CowParams cp;
        cp.layout = e->layout;
        cp.pool = e->pool;
        cp.src_page = j.src_page;
        cp.dst_page = j.dst_page;
        cp.n_slots = j.n_slots;
        CUDA_TRY(launch_cow_copy(cp, e->geom.num_layers, stream));
    }
    return DRKV_OK;
}

extern "C" {

static void exchange_release(drkv_engine* e);

const char* drkv_last_error(void) { return g_err.c_str(); }

int drkv_create(const drkv_geometry* geom, const drkv_config* cfg, drkv_engine** out) {
    if (!geom || !cfg || !out) return set_err(DRKV_ERR_INVALID, "null argument");
    *out = nullptr;
    std::string why;
    if (!geometry_ok(*geom, &why)) return set_err(DRKV_ERR_INVALID, "geometry: %s", why.c_str());
    if (cfg->max_seqs <= 0) return set_err(DRKV_ERR_INVALID, "max_seqs must be positive");

    const size_t per_page = page_bytes_all_layers(*geom);
    long max_pages = cfg->max_pages > 0 ? cfg->max_pages : (long)(cfg->budget_bytes / per_page);  // block_pool.cpp:30
    if (max_pages > 0x7fffffffL) return set_err(DRKV_ERR_INVALID, "too many pages");

    drkv_engine* e = new drkv_engine();
    e->geom = *geom;
    e->cfg = *cfg;
    std::string err;
    if (!e->book.init((int)max_pages, geom->page_size, cfg->max_seqs, cfg->max_pages_per_seq,
                      cfg->stream_evict != 0, &err)) {
        delete e;
        return set_err(DRKV_ERR_INVALID, "%s (budget %.1f MB, %.1f MB per page)", err.c_str(),
                       cfg->budget_bytes / 1048576.0, per_page / 1048576.0);
    }
    e->layout = PoolLayout::make(geom->num_kv_heads, geom->page_size, geom->head_dim, (int)max_pages);
    e->pool_bytes = per_page * (size_t)max_pages;

    if (cfg->device >= 0) {
        auto fail = [&](int code, const char* what, cudaError_t ce) {
            set_err(code, "%s: %s", what, cudaGetErrorString(ce));
            drkv_destroy(e);
            return code;
        };
        cudaError_t ce = cudaSetDevice(cfg->device);
        if (ce != cudaSuccess) return fail(DRKV_ERR_NO_DEVICE, "cudaSetDevice", ce);
        e->device = cfg->device;
        e->has_device = true;
        if ((ce = cudaMalloc(&e->pool, e->pool_bytes)) != cudaSuccess) return fail(DRKV_ERR_CUDA, "cudaMalloc(pool)", ce);
        if ((ce = cudaMemset(e->pool, 0, e->pool_bytes)) != cudaSuccess) return fail(DRKV_ERR_CUDA, "cudaMemset(pool)", ce);
        const size_t table_ints = (size_t)cfg->max_seqs * e->book.row_width();
        if ((ce = cudaMalloc(&e->d_tables, table_ints * 4)) != cudaSuccess) return fail(DRKV_ERR_CUDA, "cudaMalloc(tables)", ce);
        if ((ce = cudaMemset(e->d_tables, 0xFF, table_ints * 4)) != cudaSuccess)  // -1 = not resident (cache_manager.cpp:53)
            return fail(DRKV_ERR_CUDA, "cudaMemset(tables)", ce);
        e->stage_ints = table_ints;
        for (int i = 0; i < 2; i++) {
            if ((ce = cudaHostAlloc(&e->h_stage[i], table_ints * 4, cudaHostAllocDefault)) != cudaSuccess)
                return fail(DRKV_ERR_CUDA, "cudaHostAlloc(stage)", ce);
            if ((ce = cudaEventCreateWithFlags(&e->stage_done[i], cudaEventDisableTiming)) != cudaSuccess)
                return fail(DRKV_ERR_CUDA, "cudaEventCreate", ce);
        }
        if ((ce = cudaMalloc(&e->d_plan, kPlanInts * 4)) != cudaSuccess) return fail(DRKV_ERR_CUDA, "cudaMalloc(plan)", ce);
        for (int i = 0; i < 2; i++) {
            if ((ce = cudaHostAlloc(&e->h_plan[i], kPlanInts * 4, cudaHostAllocDefault)) != cudaSuccess)
                return fail(DRKV_ERR_CUDA, "cudaHostAlloc(plan)", ce);
            if ((ce = cudaEventCreateWithFlags(&e->plan_done[i], cudaEventDisableTiming)) != cudaSuccess)
                return fail(DRKV_ERR_CUDA, "cudaEventCreate", ce);
        }
        const size_t ctl_ints = 4;   // error word, queue head, exit count, padding
        if ((ce = cudaMalloc(&e->d_error, ctl_ints * sizeof(int))) != cudaSuccess) return fail(DRKV_ERR_CUDA, "cudaMalloc(error)", ce);
        if ((ce = cudaMemset(e->d_error, 0, ctl_ints * sizeof(int))) != cudaSuccess) return fail(DRKV_ERR_CUDA, "cudaMemset(error)", ce);
        e->d_work = e->d_error + 1;
        e->d_exit = e->d_error + 2;
        if ((ce = cudaDeviceGetAttribute(&e->num_sms, cudaDevAttrMultiProcessorCount, cfg->device)) != cudaSuccess)
            return fail(DRKV_ERR_CUDA, "cudaDeviceGetAttribute", ce);
        std::vector<float> inv;
        fill_inv_freq(geom->rope_theta, geom->rotary_dim, &inv);
        if ((ce = cudaMalloc(&e->d_inv_freq, sizeof(float) * (inv.size() + 1))) != cudaSuccess)
            return fail(DRKV_ERR_CUDA, "cudaMalloc(inv_freq)", ce);
        if (!inv.empty() &&
            (ce = cudaMemcpy(e->d_inv_freq, inv.data(), sizeof(float) * inv.size(), cudaMemcpyHostToDevice)) != cudaSuccess)
            return fail(DRKV_ERR_CUDA, "cudaMemcpy(inv_freq)", ce);
        // split-KV scratch: every sequence at full length in 256-key chunks, at least 64 MB.  A sequence is
        // never longer than its table row nor than the pool (the default row is twice the pool, CacheManager's
        // logical space); a pass that needs more partials than this gets larger chunks (decode_common).
        size_t row_tokens = (size_t)e->book.row_width() * geom->page_size;
        const size_t pool_tokens = (size_t)max_pages * geom->page_size;
        if (row_tokens > pool_tokens) row_tokens = pool_tokens;
        size_t need = (size_t)cfg->max_seqs * geom->num_q_heads * ((row_tokens + 255) / 256) * (geom->head_dim + 2) * 4;
        e->scratch_bytes = need < (64u << 20) ? (64u << 20) : need;
        if ((ce = cudaMalloc(&e->d_scratch, e->scratch_bytes)) != cudaSuccess) return fail(DRKV_ERR_CUDA, "cudaMalloc(scratch)", ce);
        const char* terr = nullptr;
        {
            const char* perr = nullptr;
            e->has_tmap_pf = make_pool_kv16_tensor_map(&e->tmap_pf, e->pool, geom->num_layers, (int)max_pages,
                                                       geom->num_kv_heads, geom->page_size, geom->head_dim, &perr);
            if (!e->has_tmap_pf) e->tmap_pf_err = perr ? perr : "tensor map";   // prefill then runs on the decode kernel
        }
        if (!make_pool_slot_tensor_map(&e->tmap_slot, e->pool, geom->num_layers, (int)max_pages, geom->num_kv_heads,
                                       geom->page_size, geom->head_dim, &terr)) {
            set_err(DRKV_ERR_CUDA, "%s", terr ? terr : "tensor map");
            drkv_destroy(e);
            return DRKV_ERR_CUDA;
        }
    }
    *out = e;
    return DRKV_OK;
}

void drkv_destroy(drkv_engine* e) {
    if (!e) return;
    e->book.attach_tier(nullptr);
    e->store.reset();                                // joins the prefetch thread; stored files stay on disk
    if (e->has_device) {
        cudaSetDevice(e->device);
        cudaDeviceSynchronize();
        exchange_release(e);
    }
    if (e->has_device) {
        cudaSetDevice(e->device);
        cudaDeviceSynchronize();
        cudaFree(e->pool);
        cudaFree(e->d_tables);
        cudaFree(e->d_inv_freq);
        cudaFree(e->d_error);
        cudaFree(e->d_scratch);
        cudaFree(e->d_plan);
        cudaFree(e->scorer.d_scores);
        cudaFree(e->scorer.d_fresh);
        cudaFree(e->scorer.d_tile_lse);
        cudaFree(e->scorer.d_lse2);
        for (int i = 0; i < 2; i++) {
            if (e->h_plan[i]) cudaFreeHost(e->h_plan[i]);
            if (e->plan_done[i]) cudaEventDestroy(e->plan_done[i]);
        }
        for (auto& ev : e->tev) cudaEventDestroy(ev);
        for (int i = 0; i < 2; i++) {
            if (e->h_stage[i]) cudaFreeHost(e->h_stage[i]);
            if (e->stage_done[i]) cudaEventDestroy(e->stage_done[i]);
        }
    }
    delete e;
}

int drkv_get_geometry(const drkv_engine* e, drkv_geometry* out) {
    NEED(e);
    if (!out) return set_err(DRKV_ERR_INVALID, "null argument");
    *out = e->geom;
    return DRKV_OK;
}

int drkv_get_stats(const drkv_engine* ce, drkv_stats* out) {
    drkv_engine* e = const_cast<drkv_engine*>(ce);
    NEED(e);
    if (!out) return set_err(DRKV_ERR_INVALID, "null argument");
    LOCK(e);
    out->pages_total = e->book.max_pages();
    out->pages_free = e->book.free_count();
    out->pages_cached = (int64_t)e->book.cached_lru().size();
    out->pages_active = out->pages_total - out->pages_free - out->pages_cached;
    out->evictions_cached = e->book.n_evict_cached;
    out->evictions_stream = e->book.n_evict_stream;
    out->cow_copies = e->book.n_cow;
    out->cow_bytes = e->cow_bytes;
    out->table_sync_bytes = e->sync_bytes;
    out->table_syncs = e->syncs;
    out->live_seqs = e->book.live_seqs();
    return DRKV_OK;
}

// ---- pool -------------------------------------------------------------------------------
int drkv_pool_alloc(drkv_engine* e) {
    if (!e) return -1;
    LOCK(e);
    return e->book.pool_alloc();
}
int drkv_pool_free(drkv_engine* e, int page) {
    NEED(e);
    LOCK(e);
    return book_err(e, e->book.pool_free(page));
}
int drkv_pool_free_count(const drkv_engine* ce) {
    drkv_engine* e = const_cast<drkv_engine*>(ce);
    if (!e) return 0;
    LOCK(e);
    return e->book.free_count();
}
int drkv_pool_max_pages(const drkv_engine* e) { return e ? e->book.max_pages() : 0; }
int drkv_pool_page_size(const drkv_engine* e) { return e ? e->book.page_size() : 0; }
void* drkv_pool_ptr(const drkv_engine* e) { return e ? e->pool : nullptr; }
size_t drkv_pool_total_bytes(const drkv_engine* e) { return e ? e->pool_bytes : 0; }
size_t drkv_pool_k_offset(const drkv_engine* e, int layer, int page) {
    return e ? (size_t)e->layout.row(layer, page, 0, 0, 0) * 2 : 0;  // block_pool.cpp:89-91
}
size_t drkv_pool_v_offset(const drkv_engine* e, int layer, int page) {
    return e ? (size_t)e->layout.row(layer, page, 1, 0, 0) * 2 : 0;  // block_pool.cpp:93-95
}

// ---- sequences --------------------------------------------------------------------------
// A new row starts with zero scores, a fork with its parent's: the host mirror now, the device at
// the next scorer call that carries a stream.
static void scorer_new_row(drkv_engine* e, int row, int src) {
    if (!e->scorer.on || row < 0) return;
    const size_t w = (size_t)e->book.row_width();
    float* dst = e->scorer.h_scores.data() + (size_t)row * w;
    if (src >= 0)
        memcpy(dst, e->scorer.h_scores.data() + (size_t)src * w, w * sizeof(float));
    else
        memset(dst, 0, w * sizeof(float));
    e->scorer.pending.push_back({row, src});
}

static int scorer_flush_pending(drkv_engine* e, cudaStream_t stream) {
    if (!e->has_device) {
        e->scorer.pending.clear();
        return DRKV_OK;
    }
    const size_t w = (size_t)e->book.row_width();
    for (const auto& pr : e->scorer.pending) {
        float* dst = e->scorer.d_scores + (size_t)pr.first * w;
        if (pr.second >= 0)
            CUDA_TRY(cudaMemcpyAsync(dst, e->scorer.d_scores + (size_t)pr.second * w, w * 4, cudaMemcpyDeviceToDevice, stream));
        else
            CUDA_TRY(cudaMemsetAsync(dst, 0, w * 4, stream));
        CUDA_TRY(cudaMemsetAsync(e->scorer.d_fresh + (size_t)pr.first * w, 0, w * 4, stream));
    }
    e->scorer.pending.clear();
    return DRKV_OK;
}

int drkv_seq_create(drkv_engine* e) {
    NEED(e);
    LOCK(e);
    const int row = book_err(e, e->book.seq_create());
    scorer_new_row(e, row, -1);
    return row;
}
int drkv_seq_release(drkv_engine* e, int seq, int discard) {
    NEED(e);
    LOCK(e);
    return book_err(e, e->book.seq_release(seq, discard != 0));
}
int drkv_seq_fork(drkv_engine* e, int parent) {
    NEED(e);
    LOCK(e);
    const int row = book_err(e, e->book.seq_fork(parent));
    scorer_new_row(e, row, parent);
    return row;
}
int drkv_seq_ensure_pos(drkv_engine* e, int seq, int pos, void* stream) {
    NEED(e);
    LOCK(e);
    std::vector<CowJob> jobs;
    int rc = e->book.seq_ensure_pos(seq, pos, &jobs);
    int rc2 = run_cow(e, jobs, (cudaStream_t)stream);
    return rc < 0 ? book_err(e, rc) : rc2;
}
int drkv_seq_ensure_range(drkv_engine* e, int seq, int pos_start, int m, void* stream) {
    NEED(e);
    LOCK(e);
    std::vector<CowJob> jobs;
    int rc = e->book.seq_ensure_range(seq, pos_start, m, &jobs);
    int rc2 = run_cow(e, jobs, (cudaStream_t)stream);
    return rc < 0 ? book_err(e, rc) : rc2;
}
int drkv_seq_reserve(drkv_engine* e, int seq, int n_tokens, void* stream) {
    NEED(e);
    LOCK(e);
    int len = e->book.seq_len(seq);
    if (len < 0) return set_err(DRKV_ERR_STATE, "reserve: unknown sequence");
    std::vector<CowJob> jobs;
    int rc = e->book.seq_ensure_range(seq, len, n_tokens, &jobs);
    int rc2 = run_cow(e, jobs, (cudaStream_t)stream);
    return rc < 0 ? book_err(e, rc) : rc2;
}
int drkv_seq_reserve_batch(drkv_engine* e, int n, const int32_t* seqs, int n_tokens, void* stream) {
    NEED(e);
    if (n < 0 || (n > 0 && !seqs)) return set_err(DRKV_ERR_INVALID, "reserve_batch: bad argument");
    LOCK(e);
    std::vector<CowJob> jobs;
    int rc = DRKV_OK;
    for (int i = 0; i < n && rc == DRKV_OK; i++) {
        const int len = e->book.seq_len(seqs[i]);
        rc = len < 0 ? DRKV_ERR_STATE : e->book.seq_ensure_range(seqs[i], len, n_tokens, &jobs);
        if (len < 0) return set_err(DRKV_ERR_STATE, "reserve_batch: unknown sequence %d", seqs[i]);
    }
    int rc2 = run_cow(e, jobs, (cudaStream_t)stream);
    return rc < 0 ? book_err(e, rc) : rc2;
}
int drkv_seq_advance_batch(drkv_engine* e, int n, const int32_t* seqs, int n_tokens) {
    NEED(e);
    if (n < 0 || (n > 0 && !seqs)) return set_err(DRKV_ERR_INVALID, "advance_batch: bad argument");
    LOCK(e);
    for (int i = 0; i < n; i++) {
        const int len = e->book.seq_len(seqs[i]);
        if (len < 0) return set_err(DRKV_ERR_STATE, "advance_batch: unknown sequence %d", seqs[i]);
        int rc = e->book.seq_set_len(seqs[i], len + n_tokens);
        if (rc < 0) return book_err(e, rc);
    }
    return DRKV_OK;
}
int drkv_seq_set_len(drkv_engine* e, int seq, int len) {
    NEED(e);
    LOCK(e);
    return book_err(e, e->book.seq_set_len(seq, len));
}
int drkv_seq_len(const drkv_engine* ce, int seq) {
    drkv_engine* e = const_cast<drkv_engine*>(ce);
    NEED(e);
    LOCK(e);
    return e->book.seq_len(seq);
}
int drkv_seq_num_pages(const drkv_engine* ce, int seq) {
    drkv_engine* e = const_cast<drkv_engine*>(ce);
    NEED(e);
    LOCK(e);
    return e->book.seq_num_pages(seq);
}
int drkv_seq_table(const drkv_engine* ce, int seq, int32_t* out, int cap) {
    drkv_engine* e = const_cast<drkv_engine*>(ce);
    NEED(e);
    LOCK(e);
    const PageBook::Seq* s = e->book.seq(seq);
    if (!s) return set_err(DRKV_ERR_STATE, "table: unknown sequence");
    int n = (int)s->table.size() < cap ? (int)s->table.size() : cap;
    if (n > 0) memcpy(out, s->table.data(), (size_t)n * 4);
    return n;
}
int drkv_seq_adopt(drkv_engine* e, int seq, const int32_t* pages, int n_pages, int n_tokens) {
    NEED(e);
    LOCK(e);
    return book_err(e, e->book.seq_adopt(seq, pages, n_pages, n_tokens));
}

// ---- eviction ---------------------------------------------------------------------------
int drkv_seq_evict(drkv_engine* e, int seq, int n) {
    NEED(e);
    LOCK(e);
    return book_err(e, e->book.seq_evict(seq, n));
}
int drkv_evict_cached(drkv_engine* e, int n) {
    NEED(e);
    LOCK(e);
    return e->book.evict_cached(n);
}
int drkv_ensure_free(drkv_engine* e, int seq, int n_free) {
    NEED(e);
    LOCK(e);
    return e->book.ensure_free(seq, n_free);
}

// ---- inspection -------------------------------------------------------------------------
int drkv_refcounts(const drkv_engine* ce, int32_t* out, int cap) {
    drkv_engine* e = const_cast<drkv_engine*>(ce);
    NEED(e);
    LOCK(e);
    const auto& v = e->book.refcounts();
    int n = (int)v.size() < cap ? (int)v.size() : cap;
    if (n > 0) memcpy(out, v.data(), (size_t)n * 4);
    return n;
}
int drkv_free_stack(const drkv_engine* ce, int32_t* out, int cap) {
    drkv_engine* e = const_cast<drkv_engine*>(ce);
    NEED(e);
    LOCK(e);
    const auto& v = e->book.free_stack();
    int n = (int)v.size() < cap ? (int)v.size() : cap;
    if (n > 0) memcpy(out, v.data(), (size_t)n * 4);
    return n;
}
int drkv_cached_lru(const drkv_engine* ce, int32_t* out, int cap) {
    drkv_engine* e = const_cast<drkv_engine*>(ce);
    NEED(e);
    LOCK(e);
    int n = 0;
    for (int p : e->book.cached_lru()) {
        if (n >= cap) break;
        out[n++] = p;
    }
    return n;
}
int drkv_evict_log(drkv_engine* e, drkv_evict_record* out, int cap, int clear) {
    NEED(e);
    LOCK(e);
    auto& log = e->book.evict_log();
    int n = (int)log.size() < cap ? (int)log.size() : cap;
    for (int i = 0; i < n; i++) out[i] = {log[i].kind, log[i].seq, log[i].logical, log[i].page};
    int total = (int)log.size();
    if (clear) log.clear();
    return out ? n : total;
}

// ---- device tables ----------------------------------------------------------------------
int drkv_sync_tables(drkv_engine* e, void* stream_) {
    NEED(e);
    NEED_DEVICE(e);
    LOCK(e);
    cudaStream_t stream = (cudaStream_t)stream_;
    std::vector<DirtyRange> dirty;
    e->book.take_dirty(&dirty);
    if (dirty.empty()) return DRKV_OK;
    const int b = e->stage_next;
    if (e->stage_busy[b]) CUDA_TRY(cudaEventSynchronize(e->stage_done[b]));
    int32_t* stage = e->h_stage[b];
    size_t off = 0;
    const int width = e->book.row_width();
    // Many changed rows (a wave of sequences released and another admitted): one copy of the whole rows from the
    // first to the last changed one costs less than a copy per row, each of which is a few microseconds of stream
    // time whatever its size.  Unchanged entries in between are re-sent with their current values.
    long dirty_ints = 0;
    for (const DirtyRange& r : dirty) dirty_ints += r.hi - r.lo;
    const int row_lo = dirty.front().row, row_hi = dirty.back().row;      // take_dirty lists rows in ascending order
    const long span_ints = (long)(row_hi - row_lo + 1) * width;
    if (dirty.size() > 4 && span_ints <= 8 * dirty_ints && (size_t)span_ints <= e->stage_ints) {
        for (int row = row_lo; row <= row_hi; row++) {
            const PageBook::Seq* s = e->book.seq(row);       // a released slot has no Seq any more: all -1
            if (s)
                memcpy(stage + off, s->table.data(), (size_t)width * 4);
            else
                memset(stage + off, 0xFF, (size_t)width * 4);
            off += width;
        }
        CUDA_TRY(cudaMemcpyAsync(e->d_tables + (size_t)row_lo * width, stage, (size_t)span_ints * 4, cudaMemcpyHostToDevice,
                                 stream));
        e->sync_bytes += span_ints * 4;
    } else {
        for (const DirtyRange& r : dirty) {
            // A released slot has no Seq to read from any more: its row is all -1.
            const PageBook::Seq* s = e->book.seq(r.row);
            const int n = r.hi - r.lo;
            if (s)
                memcpy(stage + off, s->table.data() + r.lo, (size_t)n * 4);
            else
                memset(stage + off, 0xFF, (size_t)n * 4);
            CUDA_TRY(cudaMemcpyAsync(e->d_tables + (size_t)r.row * width + r.lo, stage + off, (size_t)n * 4,
                                     cudaMemcpyHostToDevice, stream));
            off += n;
            e->sync_bytes += (int64_t)n * 4;
        }
    }
    CUDA_TRY(cudaEventRecord(e->stage_done[b], stream));
    e->stage_busy[b] = true;
    e->stage_next ^= 1;
    e->syncs++;
    return DRKV_OK;
}
const int32_t* drkv_device_tables(const drkv_engine* e) { return e ? e->d_tables : nullptr; }
int drkv_table_stride(const drkv_engine* e) { return e ? e->book.row_width() : 0; }

int drkv_kernel_error(drkv_engine* e) {
    NEED(e);
    NEED_DEVICE(e);
    int code = 0;
    CUDA_TRY(cudaMemcpy(&code, e->d_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (code != 0) {
        cudaMemset(e->d_error, 0, sizeof(int));
        return set_err(DRKV_ERR_CUDA, "a kernel reported error code %d (1 = load wait, 2 = ring wait, 3 = page id, 4 = peer wait)", code);
    }
    return DRKV_OK;
}

int drkv_set_tail_split(drkv_engine* e, int mode) {
    NEED(e);
    if (mode < -1 || mode > 4) return set_err(DRKV_ERR_INVALID, "tail split: -1 (automatic), 0 (off) or 1..4 chunks");
    e->tail_mode = mode;
    return DRKV_OK;
}

int drkv_set_prefill_on_decode_kernel(drkv_engine* e, int on) {
    NEED(e);
    e->prefill_on_decode = on != 0;
    return DRKV_OK;
}

int drkv_set_chunk_tokens(drkv_engine* e, int chunk_tokens) {
    NEED(e);
    if (chunk_tokens != 0 && (chunk_tokens % 16 != 0 || chunk_tokens < 16))
        return set_err(DRKV_ERR_INVALID, "chunk_tokens must be 0 (automatic) or a positive multiple of 16");
    e->forced_chunk = chunk_tokens;
    return DRKV_OK;
}


int drkv_kernel_timing(drkv_engine* e, int enable, double* total_ms, int* launches) {
    NEED(e);
    NEED_DEVICE(e);
    if (total_ms || launches) {
        double sum = 0;
        CUDA_TRY(cudaDeviceSynchronize());
        for (size_t i = 0; i + 1 < e->tev_used; i += 2) {
            float ms = 0;
            CUDA_TRY(cudaEventElapsedTime(&ms, e->tev[i], e->tev[i + 1]));
            sum += ms;
        }
        if (total_ms) *total_ms = sum;
        if (launches) *launches = (int)(e->tev_used / 2);
    }
    e->tev_used = 0;
    e->timing = enable != 0;
    if (e->timing && e->tev.empty()) {
        e->tev.resize(2 * 512);
        for (auto& ev : e->tev) CUDA_TRY(cudaEventCreate(&ev));
    }
    return DRKV_OK;
}

// ---- append -----------------------------------------------------------------------------
static AppendParams append_params(drkv_engine* e, int layer) {
    AppendParams p{};
    p.layout = e->layout;
    p.pool = e->pool;
    p.tables = e->d_tables;
    p.table_stride = e->book.row_width();
    p.layer = layer;
    p.rotary_dim = e->geom.rotary_dim;
    p.inv_freq = e->d_inv_freq;
    return p;
}

int drkv_append_rope(drkv_engine* e, int layer, int n_seq, const int32_t* d_rows, const int32_t* d_pos,
                     const void* k_src, const void* v_src, void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    if (layer < 0 || layer >= e->geom.num_layers || n_seq < 0 || !d_rows || !d_pos || !k_src || !v_src)
        return set_err(DRKV_ERR_INVALID, "append_rope: bad argument");
    note_stream(e, (cudaStream_t)stream);
    AppendParams p = append_params(e, layer);
    p.rows = d_rows;
    p.pos = d_pos;
    p.k_src = k_src;
    p.v_src = v_src;
    CUDA_TRY(launch_append_rope(p, n_seq, e->geom.dtype, (cudaStream_t)stream));
    return DRKV_OK;
}

int drkv_append_rope_chunk(drkv_engine* e, int layer, int seq, int pos_start, int m, const void* k_src,
                           const void* v_src, void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    if (layer < 0 || layer >= e->geom.num_layers || m < 0 || pos_start < 0 || !k_src || !v_src || seq < 0 ||
        seq >= e->book.max_seqs())
        return set_err(DRKV_ERR_INVALID, "append_rope_chunk: bad argument");
    note_stream(e, (cudaStream_t)stream);
    AppendParams p = append_params(e, layer);
    p.rows = nullptr;
    p.pos = nullptr;
    p.row = seq;
    p.pos_start = pos_start;
    p.k_src = k_src;
    p.v_src = v_src;
    CUDA_TRY(launch_append_rope(p, m, e->geom.dtype, (cudaStream_t)stream));
    return DRKV_OK;
}

static int seq_flat_copy(drkv_engine* e, int seq, int start_token, int num_tokens, void* flat, bool to_flat,
                         void* stream) {
    if (seq < 0 || seq >= e->book.max_seqs() || start_token < 0 || num_tokens < 0 || !flat)
        return set_err(DRKV_ERR_INVALID, "extract/inject: bad argument");
    FlatCopyParams p{};
    p.layout = e->layout;
    p.pool = e->pool;
    p.flat = flat;
    p.table = e->d_tables + (size_t)seq * e->book.row_width();
    p.table_stride = e->book.row_width();
    p.start_token = start_token;
    p.num_tokens = num_tokens;
    p.num_layers = e->geom.num_layers;
    CUDA_TRY(launch_flat_paged_copy(p, to_flat, e->num_sms, (cudaStream_t)stream));
    return DRKV_OK;
}

int drkv_seq_extract(drkv_engine* e, int seq, int start_token, int num_tokens, void* dst, void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    return seq_flat_copy(e, seq, start_token, num_tokens, dst, true, stream);
}

int drkv_seq_inject(drkv_engine* e, int seq, int start_token, int num_tokens, const void* src, void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    return seq_flat_copy(e, seq, start_token, num_tokens, const_cast<void*>(src), false, stream);
}

// ---- attention --------------------------------------------------------------------------
static int decode_common(drkv_engine* e, int layer, int n_seq, const int32_t* d_rows, const int32_t* d_kv_len,
                         int row, int kv_begin, int kv_end, int max_span, const void* q, void* out,
                         float* out_partial, float scale, cudaStream_t stream,
                         const drkv_engine::Plan* plan = nullptr, const ExchangeParams* xchg = nullptr,
                         int kv_step = 0, const void* k_new = nullptr, const void* v_new = nullptr) {
    const drkv_geometry& g = e->geom;
    note_stream(e, stream);
    int chunk = 0;
    if (plan) {
        chunk = plan->chunk;   // the plan's chunk was checked against the scratch when it was made
    } else {
        const long warps = (long)e->num_sms * decode_warps_per_cta(g.head_dim);
        chunk = e->forced_chunk ? e->forced_chunk
                                : pick_chunk(n_seq, g.num_kv_heads, g.num_q_heads / g.num_kv_heads, max_span, warps);
        // A batch several 512-key items deep per warp: long items (fewer starts, fewer partials), and the last
        // chunk of every sequence in 64-key pieces at the end of the queue, which evens out the finish
        // (measured on 64 sequences of 1-8 k keys: 2.5-4 % off the launch against 256-key items).
        if (!e->forced_chunk && e->tail_mode < 0 && d_rows != nullptr &&
            (long)n_seq * g.num_kv_heads * ((max_span + 511) / 512) >= 3 * warps)
            chunk = 512;
        auto need_bytes = [&](int c) {
            return (size_t)n_seq * g.num_q_heads * ((max_span + c - 1) / c) * (g.head_dim + 2) * 4;
        };
        while (need_bytes(chunk) > e->scratch_bytes && chunk < (1 << 24)) chunk <<= 1;
        if (need_bytes(chunk) > e->scratch_bytes)
            return set_err(DRKV_ERR_CAPACITY, "attend: split-KV scratch too small for %d sequences x %d keys", n_seq, max_span);
    }
    const int max_chunks = (max_span + chunk - 1) / chunk;
    // Tail split: when the pass is several chunks deep per warp, the last chunk of every sequence is
    // queued last and in 64-key pieces, so that the warps finish within a piece of one another.
    int tail_chunks = 0, tail_split = 1;
    {
        const long warps = (long)e->num_sms * decode_warps_per_cta(g.head_dim, plan && plan->n_fb > 0), streams = (long)n_seq * g.num_kv_heads;
        const long items = streams * max_chunks;
        const bool forced = e->tail_mode > 0 && chunk >= 32 && chunk % 32 == 0;
        const bool automatic = e->tail_mode < 0 && chunk >= 128 && chunk % 64 == 0 && items >= 3 * warps;
        if (d_rows != nullptr && (forced || automatic)) {
            tail_split = chunk >= 128 && chunk % 64 == 0 ? chunk / 64 : 2;
            tail_chunks = forced ? e->tail_mode : 1;      // two chunks in pieces measured slower than one
            if (tail_chunks < 1) tail_chunks = 1;
            if (tail_chunks > 4) tail_chunks = 4;
            const size_t need = (size_t)n_seq * g.num_q_heads * (max_chunks + tail_chunks * tail_split) * (g.head_dim + 2) * 4;
            if (need > e->scratch_bytes) tail_chunks = 0;
        }
    }
    const int slot_stride = max_chunks + tail_chunks * tail_split;
    const size_t n_slots = (size_t)n_seq * g.num_q_heads * slot_stride;

    DecodeParams p{};
    p.tables = e->d_tables;
    p.table_stride = e->book.row_width();
    p.rows = d_rows;
    p.kv_len = d_kv_len;
    p.row = row;
    p.kv_begin = kv_begin;
    p.kv_end = kv_end;
    p.kv_step = kv_step;
    p.q = q;
    p.part_o = e->d_scratch;
    p.part_m = e->d_scratch + n_slots * g.head_dim;
    p.part_l = p.part_m + n_slots;
    p.layer = layer;
    p.max_pages = e->book.max_pages();
    p.num_q_heads = g.num_q_heads;
    p.num_kv_heads = g.num_kv_heads;
    p.group = g.num_q_heads / g.num_kv_heads;
    p.page_size = g.page_size;
    p.chunk_tokens = chunk;
    p.max_chunks = max_chunks;
    p.tail_chunks = tail_chunks;
    p.tail_split = tail_split;
    p.n_seq = n_seq;
    // Lengths given on the host (one sequence, a range of it, the tokens of a chunk: every entry sees at least kv_end
    // keys once its partials are merged) or known from the plan: the pass may leave out the residue term of P.
    p.few_keys_possible = 1;
    if (d_kv_len == nullptr && kv_end > 1024) p.few_keys_possible = 0;
    if (plan && plan->min_kv > 1024) p.few_keys_possible = 0;
    p.total_items = n_seq * g.num_kv_heads * max_chunks;
    if (plan && plan->n_fb > 0) {
        p.n_fb = plan->n_fb;
        p.rows_per_item = plan->rows_per_item;
        p.fb_row = plan->fb_row;
        p.fb_chunks = plan->fb_chunks;
        p.fb_members = plan->fb_members;
        p.seq_first_chunk = plan->first_chunk;
    }
    const bool scored = e->scorer.on && d_rows != nullptr && out_partial == nullptr;
    if (scored) {
        int rc = scorer_flush_pending(e, stream);
        if (rc != DRKV_OK) return rc;
        p.tile_lse = e->scorer.d_tile_lse;
        p.max_tiles = e->scorer.max_tiles;
    }
    p.work_counter = e->d_work;
    p.exit_count = e->d_exit;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.error_word = e->d_error;
    if (k_new != nullptr) {                 // fused append of each entry's new token (see DecodeParams)
        p.k_new = k_new;
        p.v_new = v_new;
        p.pool = e->pool;
        p.inv_freq = e->d_inv_freq;
        p.rotary_dim = g.rotary_dim;
    }
    const bool timed = e->timing && e->tev_used + 2 <= e->tev.size();
    if (timed) CUDA_TRY(cudaEventRecord(e->tev[e->tev_used], stream));
    CUDA_TRY(launch_attend_decode(e->tmap_slot, p, e->num_sms, g.head_dim, g.dtype, stream));
    if (timed) {
        CUDA_TRY(cudaEventRecord(e->tev[e->tev_used + 1], stream));
        e->tev_used += 2;
    }

    CombineParams c{};
    c.part_o = p.part_o;
    c.part_m = p.part_m;
    c.part_l = p.part_l;
    c.kv_len = d_kv_len;
    c.kv_begin = kv_begin;
    c.kv_end = kv_end;
    c.kv_step = kv_step;
    c.num_q_heads = g.num_q_heads;
    c.head_dim = g.head_dim;
    c.chunk_tokens = chunk;
    c.max_chunks = max_chunks;
    c.tail_chunks = tail_chunks;
    c.tail_split = tail_split;
    c.seq_first_chunk = (plan && plan->n_fb > 0) ? plan->first_chunk : nullptr;
    c.out = out;
    c.out_partial = out_partial;
    c.lse2_out = scored ? e->scorer.d_lse2 : nullptr;
    if (xchg) c.xchg = *xchg;
    CUDA_TRY(launch_combine(c, n_seq, g.dtype, stream));
    if (scored) {
        PageMassParams pm{};
        pm.tile_lse = e->scorer.d_tile_lse;
        pm.lse2 = e->scorer.d_lse2;
        pm.rows = d_rows;
        pm.kv_len = d_kv_len;
        pm.fresh = e->scorer.d_fresh;
        pm.num_q_heads = g.num_q_heads;
        pm.num_kv_heads = g.num_kv_heads;
        pm.max_tiles = e->scorer.max_tiles;
        pm.page_size = g.page_size;
        pm.table_stride = e->book.row_width();
        CUDA_TRY(launch_page_mass(pm, n_seq, max_span, stream));
    }
    return DRKV_OK;
}

int drkv_attend_decode(drkv_engine* e, int layer, int n_seq, const int32_t* d_rows, const int32_t* d_kv_len,
                       int max_kv_len, const void* q, void* out, float scale, void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    if (layer < 0 || layer >= e->geom.num_layers || n_seq < 0 || !d_rows || !d_kv_len || !q || !out || max_kv_len < 0)
        return set_err(DRKV_ERR_INVALID, "attend_decode: bad argument");
    if (n_seq == 0 || max_kv_len == 0) return DRKV_OK;
    // one launch takes up to kMaxDecodeSeqs sequences; larger batches go in slices
    const size_t row_bytes = (size_t)e->geom.num_q_heads * e->geom.head_dim * 2;
    for (int s0 = 0; s0 < n_seq; s0 += kMaxDecodeSeqs) {
        const int n = n_seq - s0 < kMaxDecodeSeqs ? n_seq - s0 : kMaxDecodeSeqs;
        int rc = decode_common(e, layer, n, d_rows + s0, d_kv_len + s0, 0, 0, 0, max_kv_len,
                               (const char*)q + s0 * row_bytes, (char*)out + s0 * row_bytes, nullptr, scale,
                               (cudaStream_t)stream);
        if (rc != DRKV_OK) return rc;
    }
    return DRKV_OK;
}

int drkv_append_attend_decode(drkv_engine* e, int layer, int n_seq, const int32_t* d_rows, const int32_t* d_kv_len,
                              int max_kv_len, const void* k_src, const void* v_src, const void* q, void* out, float scale,
                              void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    if (layer < 0 || layer >= e->geom.num_layers || n_seq < 0 || !d_rows || !d_kv_len || !k_src || !v_src || !q || !out ||
        max_kv_len < 0)
        return set_err(DRKV_ERR_INVALID, "append_attend_decode: bad argument");
    if (n_seq == 0 || max_kv_len == 0) return DRKV_OK;
    // every head dim appends inside the decode kernel (at head dim 256, whose ring holds K and V of a group in separate
    // entries, the K row is staged and the V row taken from its source)
    const size_t q_bytes = (size_t)e->geom.num_q_heads * e->geom.head_dim * 2;
    const size_t kv_bytes = (size_t)e->geom.num_kv_heads * e->geom.head_dim * 2;
    for (int s0 = 0; s0 < n_seq; s0 += kMaxDecodeSeqs) {
        const int n = n_seq - s0 < kMaxDecodeSeqs ? n_seq - s0 : kMaxDecodeSeqs;
        int rc = decode_common(e, layer, n, d_rows + s0, d_kv_len + s0, 0, 0, 0, max_kv_len,
                               (const char*)q + s0 * q_bytes, (char*)out + s0 * q_bytes, nullptr, scale,
                               (cudaStream_t)stream, nullptr, nullptr, 0,
                               (const char*)k_src + s0 * kv_bytes, (const char*)v_src + s0 * kv_bytes);
        if (rc != DRKV_OK) return rc;
    }
    return DRKV_OK;
}

int drkv_plan_decode(drkv_engine* e, int n_seq, const int32_t* seqs, const int32_t* kv_len, void* stream_) {
    NEED(e);
    if (n_seq < 0 || n_seq > kMaxDecodeSeqs || (n_seq > 0 && (!seqs || !kv_len)))
        return set_err(DRKV_ERR_INVALID, "plan_decode: bad argument (at most %d sequences)", kMaxDecodeSeqs);
    LOCK(e);
    cudaStream_t stream = (cudaStream_t)stream_;
    const drkv_geometry& g = e->geom;
    const int P = g.page_size, group = g.num_q_heads / g.num_kv_heads;
    const int per_block = 16 / group;   // sequences whose query rows fill one 16-row tile
    drkv_engine::Plan& pl = e->plan;
    pl.valid = false;

    // families: runs of consecutive entries whose tables start with the same pages as the run's first
    struct Fam { int first, count, shared_tokens; };
    std::vector<Fam> fams;
    std::vector<int> fam_of(n_seq, -1);
    int max_kv = 0;
    int64_t keys_seq = 0;
    for (int i = 0; i < n_seq; i++) {
        if (seqs[i] < 0 || seqs[i] >= e->book.max_seqs() || e->book.seq(seqs[i]) == nullptr || kv_len[i] < 0)
            return set_err(DRKV_ERR_INVALID, "plan_decode: entry %d is not a live sequence", i);
        if (kv_len[i] > e->book.row_width() * P)
            return set_err(DRKV_ERR_INVALID, "plan_decode: entry %d is longer than a block table", i);
        max_kv = kv_len[i] > max_kv ? kv_len[i] : max_kv;
        keys_seq += kv_len[i];
    }
    for (int i = 0; i < n_seq && per_block >= 2;) {
        const std::vector<int32_t>& lead = e->book.seq(seqs[i])->table;
        int shared = kv_len[i], j = i + 1;
        for (; j < n_seq; j++) {
            const std::vector<int32_t>& t = e->book.seq(seqs[j])->table;
            const size_t lim = lead.size() < t.size() ? lead.size() : t.size();
            size_t c = 0;
            while (c < lim && lead[c] >= 0 && lead[c] == t[c]) c++;
            int common = (int)c * P;
            if (kv_len[j] < common) common = kv_len[j];
            if (common < 64 || common * 2 < shared) break;   // too little in common with the run so far
            if (common < shared) shared = common;
        }
        if (j - i >= 2) {
            for (int k = i; k < j; k++) fam_of[k] = (int)fams.size();
            fams.push_back(Fam{i, j - i, shared});
        }
        i = j;
    }

    // chunk: as for an unplanned pass, but counted over the planned items
    auto planned_items = [&](int c, int64_t* keys) {
        int64_t items = 0, k = 0;
        for (const Fam& f : fams) {
            const int sc = f.shared_tokens / c;
            items += (int64_t)((f.count + per_block - 1) / per_block) * sc;
            k += (int64_t)((f.count + per_block - 1) / per_block) * sc * c;
        }
        for (int i = 0; i < n_seq; i++) {
            const int first = fam_of[i] >= 0 ? fams[fam_of[i]].shared_tokens / c : 0;
            const int nch = (kv_len[i] + c - 1) / c;
            items += nch > first ? nch - first : 0;
            k += kv_len[i] > first * c ? kv_len[i] - first * c : 0;
        }
        if (keys) *keys = k;
        return items * g.num_kv_heads;
    };
    int chunk = e->forced_chunk;
    if (!chunk) {
        auto items = [&](int c) { return (long)planned_items(c, nullptr); };
        auto blocks_at = [&](int c) {
            for (const Fam& f : fams)
                if (f.shared_tokens / c > 0) return true;
            return false;
        };
        // a pass with family blocks runs on more warps per CTA (head_dim 128): pick the chunk for the CTA it will get
        chunk = pick_chunk_by_cost(group, (long)e->num_sms * decode_warps_per_cta(e->geom.head_dim, !fams.empty()), true, items);
        if (!fams.empty() && !blocks_at(chunk))
            chunk = pick_chunk_by_cost(group, (long)e->num_sms * decode_warps_per_cta(e->geom.head_dim, false), true, items);
    }
    if (e->has_device) {
        auto need_bytes = [&](int c) {
            return (size_t)n_seq * g.num_q_heads * ((max_kv + c - 1) / c) * (g.head_dim + 2) * 4;
        };
        while (need_bytes(chunk) > e->scratch_bytes && chunk < (1 << 24)) chunk <<= 1;
        if (need_bytes(chunk) > e->scratch_bytes)
            return set_err(DRKV_ERR_CAPACITY, "plan_decode: split-KV scratch too small for %d sequences x %d keys", n_seq, max_kv);
    }

    // the plan's image (an engine without a device keeps it for inspection only)
    e->plan_image.assign(3 * (size_t)n_seq + 18 * (size_t)(n_seq / 2 + 1), 0);
    int32_t* h = e->plan_image.data();
    int32_t* h_rows = h;
    int32_t* h_len = h + n_seq;
    int32_t* h_first = h + 2 * (size_t)n_seq;
    int n_fb = 0, n_fam = 0, max_members = 0;
    for (const Fam& f : fams)
        if (f.shared_tokens / chunk > 0) n_fb += (f.count + per_block - 1) / per_block;
    int32_t* h_fb_row = h + 3 * (size_t)n_seq;
    int32_t* h_fb_chunks = h_fb_row + n_fb;
    int32_t* h_fb_members = h_fb_chunks + n_fb;
    for (int i = 0; i < n_seq; i++) {
        h_rows[i] = seqs[i];
        h_len[i] = kv_len[i];
        h_first[i] = fam_of[i] >= 0 ? fams[fam_of[i]].shared_tokens / chunk : 0;
    }
    int k = 0;
    for (const Fam& f : fams) {
        const int sc = f.shared_tokens / chunk;
        if (sc == 0) continue;
        n_fam++;
        for (int m0 = 0; m0 < f.count; m0 += per_block, k++) {
            h_fb_row[k] = seqs[f.first];
            h_fb_chunks[k] = sc;
            const int nm = f.count - m0 < per_block ? f.count - m0 : per_block;
            max_members = nm > max_members ? nm : max_members;
            for (int i = 0; i < 16; i++) h_fb_members[16 * k + i] = i < nm ? f.first + m0 + i : -1;
        }
    }
    const size_t ints = 3 * (size_t)n_seq + 18 * (size_t)n_fb;
    e->plan_image.resize(ints);
    if (e->has_device) {
        const int b = e->plan_next;
        if (e->plan_busy[b]) CUDA_TRY(cudaEventSynchronize(e->plan_done[b]));
        if (ints > 0) {
            memcpy(e->h_plan[b], e->plan_image.data(), ints * 4);
            CUDA_TRY(cudaMemcpyAsync(e->d_plan, e->h_plan[b], ints * 4, cudaMemcpyHostToDevice, stream));
        }
        CUDA_TRY(cudaEventRecord(e->plan_done[b], stream));
        e->plan_busy[b] = true;
        e->plan_next ^= 1;
    }

    pl.n_seq = n_seq;
    pl.n_fb = n_fb;
    pl.n_fam = n_fam;
    pl.chunk = chunk;
    pl.max_chunks = (max_kv + chunk - 1) / chunk;
    pl.min_kv = n_seq > 0 ? kv_len[0] : 0;
    for (int i = 1; i < n_seq; i++) pl.min_kv = kv_len[i] < pl.min_kv ? kv_len[i] : pl.min_kv;
    pl.rows_per_item = max_members * group;
    pl.keys_seq = keys_seq;
    planned_items(chunk, &pl.keys_plan);
    pl.rows = e->d_plan;
    pl.kv_len = e->d_plan + n_seq;
    pl.first_chunk = e->d_plan + 2 * (size_t)n_seq;
    pl.fb_row = e->d_plan + 3 * (size_t)n_seq;
    pl.fb_chunks = pl.fb_row + n_fb;
    pl.fb_members = pl.fb_chunks + n_fb;
    pl.valid = true;
    return DRKV_OK;
}

int drkv_plan_get_info(const drkv_engine* e, drkv_plan_info* out) {
    NEED(e);
    if (!out) return set_err(DRKV_ERR_INVALID, "null argument");
    if (!e->plan.valid) return set_err(DRKV_ERR_INVALID, "no decode plan");
    out->n_seq = e->plan.n_seq;
    out->n_families = e->plan.n_fam;
    out->n_blocks = e->plan.n_fb;
    out->chunk_tokens = e->plan.chunk;
    out->keys_per_sequence_pass = e->plan.keys_seq;
    out->keys_planned_pass = e->plan.keys_plan;
    return DRKV_OK;
}

int drkv_plan_dump(const drkv_engine* e, int32_t* out, int cap) {
    NEED(e);
    if (!e->plan.valid) return set_err(DRKV_ERR_INVALID, "no decode plan");
    const int n = (int)e->plan_image.size();
    if (out) memcpy(out, e->plan_image.data(), (size_t)(n < cap ? n : cap) * 4);
    return n;
}

int drkv_attend_decode_planned(drkv_engine* e, int layer, const void* q, void* out, float scale, void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    if (layer < 0 || layer >= e->geom.num_layers || !q || !out)
        return set_err(DRKV_ERR_INVALID, "attend_decode_planned: bad argument");
    const drkv_engine::Plan& pl = e->plan;
    if (!pl.valid) return set_err(DRKV_ERR_INVALID, "attend_decode_planned: no decode plan");
    if (pl.n_seq == 0 || pl.max_chunks == 0) return DRKV_OK;
    return decode_common(e, layer, pl.n_seq, pl.rows, pl.kv_len, 0, 0, 0, pl.max_chunks * pl.chunk, q, out, nullptr,
                         scale, (cudaStream_t)stream, &pl);
}

int drkv_append_attend_decode_planned(drkv_engine* e, int layer, const void* k_src, const void* v_src, const void* q,
                                      void* out, float scale, void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    if (layer < 0 || layer >= e->geom.num_layers || !k_src || !v_src || !q || !out)
        return set_err(DRKV_ERR_INVALID, "append_attend_decode_planned: bad argument");
    const drkv_engine::Plan& pl = e->plan;
    if (!pl.valid) return set_err(DRKV_ERR_INVALID, "append_attend_decode_planned: no decode plan");
    if (pl.n_seq == 0 || pl.max_chunks == 0) return DRKV_OK;
    return decode_common(e, layer, pl.n_seq, pl.rows, pl.kv_len, 0, 0, 0, pl.max_chunks * pl.chunk, q, out, nullptr,
                         scale, (cudaStream_t)stream, &pl, nullptr, 0, k_src, v_src);
}

// ---- storage tier --------------------------------------------------------------------------
int drkv_tier_enable(drkv_engine* e, const char* dir) {
    NEED(e);
    if (!dir || !*dir) return set_err(DRKV_ERR_INVALID, "tier_enable: empty directory");
    LOCK(e);
    std::unique_ptr<PageStore> st(new PageStore());
    std::string err;
    const size_t page_bytes = (size_t)2 * e->geom.num_kv_heads * e->geom.page_size * e->geom.head_dim * 2;
    if (!st->init(dir, e->pool, e->geom.num_layers, page_bytes * (size_t)e->book.max_pages(), page_bytes, &err))
        return set_err(DRKV_ERR_STATE, "%s", err.c_str());
    st->set_order_stream(e->last_stream);
    e->store = std::move(st);
    e->book.attach_tier(e->store.get());
    return DRKV_OK;
}

int drkv_tier_disable(drkv_engine* e) {
    NEED(e);
    LOCK(e);
    if (e->book.stored_pages() > 0)
        return set_err(DRKV_ERR_STATE, "tier_disable: %d pages are still stored", e->book.stored_pages());
    e->book.attach_tier(nullptr);
    e->store.reset();
    return DRKV_OK;
}

int drkv_tier_prefetch(drkv_engine* e, int seq, int logical) {
    NEED(e);
    LOCK(e);
    if (!e->store) return set_err(DRKV_ERR_STATE, "tier_prefetch: no storage tier");
    if (e->book.seq_location(seq, logical) != LOC_SSD) return 0;    // cache_manager.cpp:168-169: nothing to do
    return e->store->prefetch(seq, logical) ? 1 : 0;
}

int drkv_tier_set_write_behind(drkv_engine* e, int on) {
    NEED(e);
    LOCK(e);
    if (!e->store) return set_err(DRKV_ERR_STATE, "tier_set_write_behind: no storage tier");
    if (!on) e->store->drain();
    e->store->set_write_behind(on != 0);
    return DRKV_OK;
}

int drkv_tier_is_prefetched(drkv_engine* e, int seq, int logical) {
    NEED(e);
    if (!e->store) return set_err(DRKV_ERR_STATE, "tier_is_prefetched: no storage tier");
    return e->store->is_prefetched(seq, logical) ? 1 : 0;
}

int drkv_tier_drop_prefetch(drkv_engine* e, int seq, int logical) {
    NEED(e);
    if (!e->store) return set_err(DRKV_ERR_STATE, "tier_drop_prefetch: no storage tier");
    e->store->drop_prefetch(seq, logical);
    return DRKV_OK;
}

int drkv_tier_page_to_file(drkv_engine* e, int page, const char* path) {
    NEED(e);
    LOCK(e);
    if (!e->store) return set_err(DRKV_ERR_STATE, "tier_page_to_file: no storage tier");
    if (!path || page < 0 || page >= e->book.max_pages()) return set_err(DRKV_ERR_INVALID, "tier_page_to_file: bad argument");
    if (!e->store->page_to_file(page, path)) return set_err(DRKV_ERR_STATE, "tier_page_to_file: copy or write failed (%s)", path);
    return DRKV_OK;
}

int drkv_tier_file_to_page(drkv_engine* e, const char* path, int page) {
    NEED(e);
    LOCK(e);
    if (!e->store) return set_err(DRKV_ERR_STATE, "tier_file_to_page: no storage tier");
    if (!path || page < 0 || page >= e->book.max_pages()) return set_err(DRKV_ERR_INVALID, "tier_file_to_page: bad argument");
    if (!e->store->file_to_page(path, page)) return set_err(DRKV_ERR_STATE, "tier_file_to_page: read or copy failed (%s)", path);
    return DRKV_OK;
}

int drkv_tier_drain(drkv_engine* e) {
    NEED(e);
    if (!e->store) return set_err(DRKV_ERR_STATE, "tier_drain: no storage tier");
    e->store->drain();
    return DRKV_OK;
}

int drkv_tier_get_stats(const drkv_engine* ce, drkv_tier_stats* out) {
    drkv_engine* e = const_cast<drkv_engine*>(ce);
    NEED(e);
    if (!out) return set_err(DRKV_ERR_INVALID, "null argument");
    LOCK(e);
    memset(out, 0, sizeof(*out));
    out->pages_stored = e->book.stored_pages();
    out->swap_outs = e->book.n_swap_out;
    out->swap_ins = e->book.n_swap_in;
    if (e->store) {
        out->bytes_out = e->store->bytes_out;
        out->bytes_in = e->store->bytes_in;
        out->prefetch_hits = e->store->prefetch_hits;
        out->page_file_bytes = (int64_t)e->store->file_bytes();
        out->writes_deferred = e->store->writes_deferred;
        out->write_failures = e->store->write_failures;
    }
    return DRKV_OK;
}

int drkv_seq_locations(const drkv_engine* ce, int seq, int8_t* out, int cap) {
    drkv_engine* e = const_cast<drkv_engine*>(ce);
    NEED(e);
    LOCK(e);
    if (!e->book.seq_live(seq) || !out || cap < 0) return set_err(DRKV_ERR_INVALID, "seq_locations: bad argument");
    const int n = cap < e->book.row_width() ? cap : e->book.row_width();
    for (int i = 0; i < n; i++) out[i] = (int8_t)e->book.seq_location(seq, i);
    return n;
}

// ---- importance scorer ---------------------------------------------------------------------
int drkv_scorer_enable(drkv_engine* e, float decay) {
    NEED(e);
    LOCK(e);
    drkv_engine::Scorer& sc = e->scorer;
    if (!(decay >= 0.f)) {                               // negative: detach; eviction is oldest-first again
        sc.on = false;
        e->book.attach_scores(nullptr);
        return DRKV_OK;
    }
    const size_t n = (size_t)e->book.max_seqs() * e->book.row_width();
    sc.decay = decay;
    if (sc.h_scores.size() != n) sc.h_scores.assign(n, 0.f);
    if (e->has_device && sc.d_scores == nullptr) {
        const drkv_geometry& g = e->geom;
        sc.max_tiles = e->book.row_width() * (g.page_size / 16);
        const size_t launch_seqs = e->book.max_seqs() < kMaxDecodeSeqs ? e->book.max_seqs() : kMaxDecodeSeqs;
        CUDA_TRY(cudaMalloc(&sc.d_scores, n * 4));
        CUDA_TRY(cudaMalloc(&sc.d_fresh, n * 4));
        CUDA_TRY(cudaMalloc(&sc.d_tile_lse, launch_seqs * g.num_q_heads * sc.max_tiles * 4 * sizeof(float)));   // 4 values per row-tile
        CUDA_TRY(cudaMalloc(&sc.d_lse2, launch_seqs * g.num_q_heads * 4));
        CUDA_TRY(cudaMemset(sc.d_scores, 0, n * 4));     // importance_scorer.cu:57
        CUDA_TRY(cudaMemset(sc.d_fresh, 0, n * 4));
    }
    sc.on = true;
    e->book.attach_scores(sc.h_scores.data());
    return DRKV_OK;
}

int drkv_scorer_update(drkv_engine* e, int seq, const float* new_scores, int num_blocks, void* stream) {
    NEED(e);
    LOCK(e);
    if (!e->scorer.on) return set_err(DRKV_ERR_STATE, "scorer_update: the scorer is not enabled");
    if (seq < 0 || seq >= e->book.max_seqs() || num_blocks < 0 || num_blocks > e->book.row_width() ||
        (num_blocks > 0 && !new_scores))
        return set_err(DRKV_ERR_INVALID, "scorer_update: bad argument");
    const size_t off = (size_t)seq * e->book.row_width();
    if (!e->has_device) {
        float* row = e->scorer.h_scores.data() + off;
        for (int i = 0; i < num_blocks; i++) row[i] = fmaf(row[i], e->scorer.decay, new_scores[i]);
        return DRKV_OK;
    }
    int rc = scorer_flush_pending(e, (cudaStream_t)stream);
    if (rc != DRKV_OK) return rc;
    CUDA_TRY(launch_importance_add(e->scorer.d_scores + off, new_scores, num_blocks, e->scorer.decay, (cudaStream_t)stream));
    return DRKV_OK;
}

int drkv_scorer_step(drkv_engine* e, void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    LOCK(e);
    if (!e->scorer.on) return set_err(DRKV_ERR_STATE, "scorer_step: the scorer is not enabled");
    int rc = scorer_flush_pending(e, (cudaStream_t)stream);
    if (rc != DRKV_OK) return rc;
    const int64_t n = (int64_t)e->book.max_seqs() * e->book.row_width();
    CUDA_TRY(launch_importance_update(e->scorer.d_scores, e->scorer.d_fresh, n, e->scorer.decay, (cudaStream_t)stream));
    return DRKV_OK;
}

int drkv_scorer_sync(drkv_engine* e, void* stream) {
    NEED(e);
    LOCK(e);
    if (!e->scorer.on) return set_err(DRKV_ERR_STATE, "scorer_sync: the scorer is not enabled");
    if (!e->has_device) return DRKV_OK;
    int rc = scorer_flush_pending(e, (cudaStream_t)stream);
    if (rc != DRKV_OK) return rc;
    CUDA_TRY(cudaMemcpyAsync(e->scorer.h_scores.data(), e->scorer.d_scores, e->scorer.h_scores.size() * 4,
                             cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));   // importance_scorer.cu:91-96 is synchronous too
    return DRKV_OK;
}

int drkv_scorer_scores(const drkv_engine* e, int seq, float* out, int cap) {
    NEED(e);
    if (!e->scorer.on) return set_err(DRKV_ERR_STATE, "scorer_scores: the scorer is not enabled");
    if (seq < 0 || seq >= e->book.max_seqs() || !out || cap < 0) return set_err(DRKV_ERR_INVALID, "scorer_scores: bad argument");
    const int w = e->book.row_width();
    const int n = cap < w ? cap : w;
    memcpy(out, e->scorer.h_scores.data() + (size_t)seq * w, (size_t)n * 4);
    return n;
}

int drkv_attend_partial(drkv_engine* e, int layer, int seq, int kv_begin, int kv_end, const void* q, float* part,
                        float scale, void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    if (layer < 0 || layer >= e->geom.num_layers || seq < 0 || seq >= e->book.max_seqs() || kv_begin < 0 || !q || !part)
        return set_err(DRKV_ERR_INVALID, "attend_partial: bad argument");
    int span = kv_end - (kv_begin / 16) * 16;
    if (span < 1) span = 1;   // an empty range still has to produce the (-1e20, 0, 0) partial
    return decode_common(e, layer, 1, nullptr, nullptr, seq, kv_begin, kv_end, span, q, nullptr, part, scale,
                         (cudaStream_t)stream);
}

// ---- cross-GPU exchange ---------------------------------------------------------------------
static void exchange_release(drkv_engine* e) {
    drkv_engine::Exchange& x = e->xchg;
    for (int r = 0; r < x.world; r++)
        if (x.connected && !x.local && r != x.rank && x.peer_area[r]) cudaIpcCloseMemHandle(x.peer_area[r]);
    if (x.area) cudaFree(x.area);
    const unsigned long long keep = x.wait_ns;
    x = drkv_engine::Exchange();
    x.wait_ns = keep;
}

int drkv_exchange_create(drkv_engine* e, int world, int rank, uint8_t* handle_out) {
    NEED(e);
    NEED_DEVICE(e);
    if (world < 1 || world > kMaxExchangeRanks || rank < 0 || rank >= world || !handle_out)
        return set_err(DRKV_ERR_INVALID, "exchange_create: bad argument (at most %d ranks)", kMaxExchangeRanks);
    static_assert(sizeof(cudaIpcMemHandle_t) == DRKV_IPC_HANDLE_BYTES, "IPC handle size");
    LOCK(e);
    CUDA_TRY(cudaSetDevice(e->device));
    exchange_release(e);
    drkv_engine::Exchange& x = e->xchg;
    // {value, sequence number} words: 2 parities x world ranks x Hq * (D + 2)
    const size_t per_rank = (size_t)e->geom.num_q_heads * (e->geom.head_dim + 2) * sizeof(float2);
    const size_t bytes = (2 * (size_t)world * per_rank + 255) / 256 * 256;
    CUDA_TRY(cudaMalloc(&x.area, bytes));
    CUDA_TRY(cudaMemset(x.area, 0, bytes));
    CUDA_TRY(cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    CUDA_TRY(cudaIpcGetMemHandle(&h, x.area));
    memcpy(handle_out, &h, sizeof(h));
    x.world = world;
    x.rank = rank;
    x.peer_area[rank] = x.area;
    return DRKV_OK;
}

int drkv_exchange_connect(drkv_engine* e, const uint8_t* handles) {
    NEED(e);
    NEED_DEVICE(e);
    LOCK(e);
    drkv_engine::Exchange& x = e->xchg;
    if (x.world == 0 || !handles) return set_err(DRKV_ERR_STATE, "exchange_connect: no exchange area / null handles");
    CUDA_TRY(cudaSetDevice(e->device));
    for (int r = 0; r < x.world; r++) {
        if (r == x.rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * DRKV_IPC_HANDLE_BYTES, sizeof(h));
        CUDA_TRY(cudaIpcOpenMemHandle(&x.peer_area[r], h, cudaIpcMemLazyEnablePeerAccess));
    }
    x.connected = true;
    return DRKV_OK;
}

int drkv_exchange_connect_local(drkv_engine* e, void* const* areas) {
    NEED(e);
    NEED_DEVICE(e);
    LOCK(e);
    drkv_engine::Exchange& x = e->xchg;
    if (x.world == 0 || !areas) return set_err(DRKV_ERR_STATE, "exchange_connect_local: no exchange area / null areas");
    for (int r = 0; r < x.world; r++) {
        if (r == x.rank) continue;
        if (areas[r] == nullptr) return set_err(DRKV_ERR_INVALID, "exchange_connect_local: rank %d has no area", r);
        x.peer_area[r] = areas[r];
    }
    x.connected = true;
    x.local = true;
    return DRKV_OK;
}

void* drkv_exchange_area(const drkv_engine* e) { return e ? e->xchg.area : nullptr; }

int drkv_exchange_set_wait_ms(drkv_engine* e, int ms) {
    NEED(e);
    if (ms < 1 || ms > 60000) return set_err(DRKV_ERR_INVALID, "exchange wait limit: 1 .. 60000 ms");
    e->xchg.wait_ns = (unsigned long long)ms * 1000000ull;
    return DRKV_OK;
}

int drkv_exchange_destroy(drkv_engine* e) {
    NEED(e);
    NEED_DEVICE(e);
    LOCK(e);
    CUDA_TRY(cudaSetDevice(e->device));
    CUDA_TRY(cudaDeviceSynchronize());
    exchange_release(e);
    return DRKV_OK;
}

static int attend_exchange(drkv_engine* e, int layer, int seq, int kv_begin, int kv_end, const void* k_src,
                           const void* v_src, const void* q, void* out, float scale, void* stream);

int drkv_attend_exchange(drkv_engine* e, int layer, int seq, int kv_begin, int kv_end, const void* q, void* out,
                         float scale, void* stream) {
    return attend_exchange(e, layer, seq, kv_begin, kv_end, nullptr, nullptr, q, out, scale, stream);
}

int drkv_append_attend_exchange(drkv_engine* e, int layer, int seq, int kv_begin, int kv_end, const void* k_src,
                                const void* v_src, const void* q, void* out, float scale, void* stream) {
    if ((k_src == nullptr) != (v_src == nullptr))
        return set_err(DRKV_ERR_INVALID, "append_attend_exchange: k_src and v_src come together");
    return attend_exchange(e, layer, seq, kv_begin, kv_end, k_src, v_src, q, out, scale, stream);
}

static int attend_exchange(drkv_engine* e, int layer, int seq, int kv_begin, int kv_end, const void* k_src,
                           const void* v_src, const void* q, void* out, float scale, void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    drkv_engine::Exchange& x = e->xchg;
    if (x.world == 0 || (x.world > 1 && !x.connected))
        return set_err(DRKV_ERR_STATE, "attend_exchange: create and connect the exchange first");
    if (layer < 0 || layer >= e->geom.num_layers || seq < 0 || seq >= e->book.max_seqs() || kv_begin < 0 || !q || !out)
        return set_err(DRKV_ERR_INVALID, "attend_exchange: bad argument");
    int span = kv_end - (kv_begin / 16) * 16;
    if (span < 1) span = 1;
    ExchangeParams p{};
    for (int r = 0; r < x.world; r++) {
        p.peer_slots[r] = static_cast<float2*>(x.peer_area[r]);
    }
    p.world = x.world;
    p.rank = x.rank;
    p.seq_no = ++x.seq_no;
    p.parity = (int)(p.seq_no & 1u);
    p.wait_ns = x.wait_ns;
    p.error_word = e->d_error;
    if (k_src != nullptr && kv_end <= kv_begin) {
        // nothing of this rank's range to attend: the token goes through the append kernel
        if (kv_end < 1) return set_err(DRKV_ERR_INVALID, "append_attend_exchange: no position to append at");
        note_stream(e, (cudaStream_t)stream);
        AppendParams ap = append_params(e, layer);
        ap.rows = nullptr;
        ap.pos = nullptr;
        ap.row = seq;
        ap.pos_start = kv_end - 1;
        ap.k_src = k_src;
        ap.v_src = v_src;
        CUDA_TRY(launch_append_rope(ap, 1, e->geom.dtype, (cudaStream_t)stream));
        k_src = v_src = nullptr;
    }
    // the merge kernel's CTA of head h exchanges that head with the peers and writes the final output
    return decode_common(e, layer, 1, nullptr, nullptr, seq, kv_begin, kv_end, span, q, out, nullptr, scale,
                         (cudaStream_t)stream, nullptr, &p, 0, k_src, v_src);
}

int drkv_combine_partials(drkv_engine* e, int n_parts, const float* parts, void* out, void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    if (n_parts < 0 || !parts || !out) return set_err(DRKV_ERR_INVALID, "combine_partials: bad argument");
    CUDA_TRY(launch_combine_external(n_parts, parts, e->geom.num_q_heads, e->geom.head_dim, out, e->geom.dtype,
                                     (cudaStream_t)stream));
    return DRKV_OK;
}

size_t drkv_partial_floats(const drkv_engine* e) {
    return e ? (size_t)e->geom.num_q_heads * (e->geom.head_dim + 2) : 0;
}

// Prefill attention without the tensor-memory kernel (a pool that one TMA descriptor cannot address, or on request:
// drkv_set_prefill_on_decode_kernel): the causal rule "token t sees
// keys [0, pos_start + t]" (paged_attention.cu:465-554) is a batch of m one-token decodes over one block table, which
// the split-KV decode kernel runs as it stands: batch entry t reads the same table row and sees pos_start + t + 1
// keys (kv_step = 1), the query rows of a GQA group share each K/V tile, every token re-reads the keys (mostly from
// L2).  Same arithmetic as decode attention; q/out are [m][Hq][D] in both.
static int prefill_by_decode(drkv_engine* e, int layer, int seq, int pos_start, int m, const void* q, void* out,
                             float scale, cudaStream_t stream) {
    const size_t row_bytes = (size_t)e->geom.num_q_heads * e->geom.head_dim * 2;
    for (int t0 = 0; t0 < m; t0 += kMaxDecodeSeqs) {
        const int n = m - t0 < kMaxDecodeSeqs ? m - t0 : kMaxDecodeSeqs;
        int rc = decode_common(e, layer, n, nullptr, nullptr, seq, 0, pos_start + t0 + 1, pos_start + t0 + n,
                               (const char*)q + t0 * row_bytes, (char*)out + t0 * row_bytes, nullptr, scale, stream,
                               nullptr, nullptr, /*kv_step=*/1);
        if (rc != DRKV_OK) return rc;
    }
    return DRKV_OK;
}

int drkv_attend_prefill_batch(drkv_engine* e, int layer, int n_seq, const int32_t* seqs, const int32_t* pos_start,
                              const int32_t* m, const void* const* q, void* const* out, float scale, void* stream) {
    NEED(e);
    NEED_DEVICE(e);
    const drkv_geometry& g = e->geom;
    if (layer < 0 || layer >= g.num_layers || n_seq < 0 || !seqs || !pos_start || !m || !q || !out)
        return set_err(DRKV_ERR_INVALID, "attend_prefill: bad argument");
    for (int i = 0; i < n_seq; i++)
        if (seqs[i] < 0 || seqs[i] >= e->book.max_seqs() || pos_start[i] < 0 || m[i] < 0 || (m[i] > 0 && (!q[i] || !out[i])))
            return set_err(DRKV_ERR_INVALID, "attend_prefill: bad sequence entry %d", i);
    if (!e->has_tmap_pf || e->prefill_on_decode) {
        // no 16-key view of this pool for the tensor-memory kernel (a pool beyond what one TMA descriptor addresses),
        // or the caller asked for it: the chunk runs on the split-KV decode kernel, a batch of one-token decodes over
        // one block table
        note_stream(e, (cudaStream_t)stream);
        for (int i = 0; i < n_seq; i++) {
            if (m[i] == 0) continue;
            int rc = prefill_by_decode(e, layer, seqs[i], pos_start[i], m[i], q[i], out[i], scale, (cudaStream_t)stream);
            if (rc != DRKV_OK) return rc;
        }
        return DRKV_OK;
    }
    for (int s0 = 0; s0 < n_seq; s0 += kMaxPrefillSeqs) {
        PrefillParams p{};
        p.tables = e->d_tables;
        p.table_stride = e->book.row_width();
        p.n_seq = n_seq - s0 < kMaxPrefillSeqs ? n_seq - s0 : kMaxPrefillSeqs;
        for (int i = 0; i < p.n_seq; i++) {
            p.row[i] = seqs[s0 + i];
            p.pos_start[i] = pos_start[s0 + i];
            p.m[i] = m[s0 + i];
            p.q[i] = q[s0 + i];
            p.out[i] = out[s0 + i];
        }
        p.layer = layer;
        p.max_pages = e->book.max_pages();
        p.num_q_heads = g.num_q_heads;
        p.num_kv_heads = g.num_kv_heads;
        p.group = g.num_q_heads / g.num_kv_heads;
        p.page_size = g.page_size;
        p.scale_log2 = scale * 1.4426950408889634f;
        p.error_word = e->d_error;
        CUDA_TRY(launch_attend_prefill(e->tmap_pf, p, g.head_dim, g.dtype, e->num_sms, e->d_scratch, e->scratch_bytes,
                                       (cudaStream_t)stream));
    }
    return DRKV_OK;
}

int drkv_attend_prefill_chunk(drkv_engine* e, int layer, int seq, int pos_start, int m, const void* q, void* out,
                              float scale, void* stream) {
    const int32_t s = seq, ps = pos_start, mm = m;
    return drkv_attend_prefill_batch(e, layer, 1, &s, &ps, &mm, &q, &out, scale, stream);
}

}  // extern "C"
