// attend_decode.cu — split-KV paged GQA decode attention for sm_100a, plus the LSE combine.
//
// Replaces paged_gqa_decode_attention_kernel (src/machina/paged_attention.cu:179-269): one
// CTA per query head walking every key with two block barriers per key.  Here:
//   * the keys of one sequence are split into chunks; (sequence, KV head, chunk) work items
//     are pulled from an atomic queue by a persistent grid of one CTA per SM; every item
//     yields an un-normalised partial (m, l, o) per query head of the GQA group, a second
//     small kernel merges the partials (same arithmetic as contiguous_split_k_merge_kernel,
//     src/sensus/auditus/asr/asr_ops_attn.cu:88-108);
//   * every K/V byte is read from HBM once per KV head: the query heads of a group share
//     the tile (the reference re-reads it once per query head);
//   * pages are gathered by TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast): ONE 4-D box per
//     ring slot brings the K and V rows of 16 keys of one head (8 KB at head_dim 128) into the shared-memory
//     ring that every warp owns (two slots: one gather lands while the previous group is computed;
//     mbarrier-guarded), laid out [plane][128-byte segment][row] so that the fragment loads are free of bank
//     conflicts; lane 0 of the warp walks the block table, 32 page ids at a time, and issues the copies
//     ahead of the tile being computed, across item boundaries;
//   * QK^T and PV run as m16n8k16 tensor-core tiles with fp32 accumulation: the 4..16 query rows of a GQA
//     group are far from a dense contraction (the tensor pipe is about a quarter busy), they only keep the
//     SM's issue slots free so that the kernel stays HBM-bound; softmax statistics are reduced with warp
//     shuffles in fp32.  P is fed to the PV product as a two-term (hi + lo) split so that it carries ~16
//     significant bits;
//   * a shared-prefix plan adds work items whose 16 query rows come from several forked sequences over the
//     chunks their block tables have in common, and the importance scorer's per-tile probability masses
//     are a by-product (both compiled only into the EXT instantiation).
// Holes (table entry < 0) contribute nothing.  All waits are bounded; a wait that gives
// up records a code in the engine's error word and the CTA retires without trapping.
#include <atomic>
#include <mutex>

#include "kernels.hpp"
#include "kv_common.cuh"
#include "sm100_primitives.cuh"
#include "exchange.cuh"

namespace drkv {

namespace {

constexpr int kGroupTokens = 16;                               // keys per ring slot
constexpr float kNegBig = -1.0e30f;                            // "no key seen yet" in the log2 domain

// Ring geometry per head_dim: consumer warps per CTA and slots per warp ring.  At head_dim 128 a warp
// has one 8 KB gather landing while it computes the previous one: 148 SMs x 8 warps x 8 KB = 9.7 MB in
// flight, about bandwidth x loaded latency.  A third slot per warp (19 MB in flight) made the pass over
// long items 8 % slower, and so do more warps with two slots each (12 warps: c2 +4 %, one long sequence +12 %;
// only a short launch over few items gains, c3 -13 %): the memory system serves fewer, not more, concurrent
// streams better.  At 64 and 256 the pass is bound by the instruction stream of the warps, not by the loads in
// flight (2 to 6 slots within 1 %): at 64, where a slot is 4 KB and the registers allow it, sixteen warps with two
// slots each run 45 % faster than eight with six (4.0 -> 5.8 TB/s on a 64-sequence batch, 4.3 -> 6.3 on one long
// sequence).  At 256 a ring entry holds ONE plane (kSplit): the K and the V rows of a group
// are separate 8 KB gathers, three entries per warp, so that eight warps fit (192 KB) where whole groups
// of 16 KB allowed six; the warp releases a group's K entry after the softmax, sends the next gather and
// only then waits for the group's V entry.
template <int D> struct RingShape;
template <> struct RingShape<64>  { static constexpr int kWarps = 16, kDepth = 2; static constexpr bool kSplit = false; };
template <> struct RingShape<128> { static constexpr int kWarps = 8, kDepth = 2; static constexpr bool kSplit = false; };
template <> struct RingShape<256> { static constexpr int kWarps = 8, kDepth = 3; static constexpr bool kSplit = true; };

enum SlotFlags : int { SLOT_FIRST = 1, SLOT_LAST = 2, SLOT_SKIP = 4, SLOT_DONE = 8 };

// What lane 0 leaves for its warp about one ring slot: one 8-byte store per group; everything that is the
// same for all groups of an item is written once per item.
struct alignas(16) SlotMeta {
    int flags;                      // SlotFlags | (item entry << kItemShift)
    int tok0;                       // first key of the group (a multiple of 16)
    int page;                       // pool page of the group (< 0: hole)
    int pad;
};
struct alignas(16) ItemMeta {
    int b, kvh, part_slot, fam;     // part_slot: index of the partial of query row 0; fam: family block + 1 or 0
    int tok_hi, append, trow, pad2; // keys of the item end here; append: the item ends at the sequence's new token, which it appends; table row
};
constexpr int kItemShift = 4, kItemEntries = 8;   // a ring holds at most 6 groups, so at most 7 items are live


template <typename T>
struct Mma;
template <>
struct Mma<__half> {
    static __device__ __forceinline__ void run(float& d0, float& d1, float& d2, float& d3, uint32_t a0,
                                               uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d0), "+f"(d1), "+f"(d2), "+f"(d3)
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};
template <>
struct Mma<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float& d0, float& d1, float& d2, float& d3, uint32_t a0,
                                               uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d0), "+f"(d1), "+f"(d2), "+f"(d3)
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};

// Two-term split of a pair of probabilities into the storage type: hi = rn(p), lo = rn(p - hi).
template <typename T>
__device__ __forceinline__ void split_pack(float p0, float p1, uint32_t& hi, uint32_t& lo) {
    hi = Elem<T>::pack2(p0, p1);
    float2 h = Elem<T>::unpack2(hi);
    lo = Elem<T>::pack2(p0 - h.x, p1 - h.y);
}

// Fused append, the rare path of one work item per (sequence, KV head): the token at `pos` is not in the pool yet.
// When the item that will reach it STARTS, its warp rotates the K row exactly as append_rope_kernel does (same
// operations, same rounding: the pool bytes are identical), leaves the K and the V row in a small staging area of
// its own in shared memory, and writes both to the pool page with 16-byte stores; the item's first gathers are
// in flight meanwhile.  When the item's last group has landed, the staged rows replace the row of the K and V
// tiles that the gather brought from the pool (stale there, or racing with the store above).  Kept out of line so
// that the main loop's register allocation does not see the fp64 sine/cosine evaluation.
// STAGE_V = false (head_dim 256, where shared memory has room for the K row only): the V row is not staged; it goes
// from its source to the pool here and from its source into the V tile later (it is not rotated, so both are copies).
template <typename T, int D, bool STAGE_V>
__device__ __noinline__ void fused_append_prepare(const T* ksrc, const T* vsrc, T* pool_krow, int64_t plane_elems,
                                                  const float* inv_freq, int rotary_dim, uint8_t* stage, int pos, int lane) {
    const int half = rotary_dim >> 1;
    T* krow = reinterpret_cast<T*>(stage);
    for (int i = lane; i < half; i += 32) {
        const float x0 = Elem<T>::to_f(ksrc[i]), x1 = Elem<T>::to_f(ksrc[i + half]);
        float sn, cs, y0, y1;
        sincos_det(__fmul_rn((float)pos, __ldg(inv_freq + i)), sn, cs);
        rope_pair(x0, x1, cs, sn, y0, y1);
        krow[i] = Elem<T>::from_f(y0);
        krow[i + half] = Elem<T>::from_f(y1);
    }
    for (int d = rotary_dim + lane; d < D; d += 32) krow[d] = ksrc[d];
    if (STAGE_V)
        for (int c = lane; c < D / 8; c += 32) *reinterpret_cast<Vec16*>(stage + D * 2 + 16 * c) = ldg16(vsrc + 8 * c);
    __syncwarp();
    if (pool_krow != nullptr) {
        // the token's pool rows: the V plane of a page starts plane_elems after its K plane
        for (int c = lane; c < 2 * (D / 8); c += 32) {
            const int pl = c / (D / 8), cc = c - pl * (D / 8);
            const Vec16 v = (pl && !STAGE_V) ? ldg16(vsrc + 8 * cc) : *reinterpret_cast<const Vec16*>(stage + pl * (D * 2) + 16 * cc);
            stg16(pool_krow + pl * plane_elems + 8 * cc, v);
        }
    }
}

// Prefix sums of per-sequence chunk counts live in shared memory: kMaxDecodeSeqs + 1 ints.

// Persistent kernel, one CTA per SM, every warp on its own.  Work item = (sequence, KV head,
// chunk of keys); a block-wide prefix sum of the per-sequence chunk counts turns the atomic
// queue index into (sequence, head, chunk) without empty items.  A warp owns a private ring
// of DEPTH slots (16 keys of K and V each; at head_dim 256 of one plane each), its 16-row query
// fragments and its (m, l, o) state.  Its lane 0 issues the TMA gathers DEPTH - 1 groups ahead of the group being
// computed, across item boundaries, and the next item (queue index, length, table row, first
// 32 page ids) is fetched while the current one is processed, so that neither the atomic nor the
// table look-ups sit on the critical path.  An item's partial goes straight from the
// accumulators to global memory; there is no block-level barrier after start-up.
// HI: the GQA group has more than 8 query heads, so rows 8..15 of the 16-row tile are live.
// EXT compiles in the two extensions that cost the plain pass time when merely present: shared-prefix
// family blocks and the per-tile masses of the importance scorer.
// WARPS: consumer warps per CTA; RingShape<D>::kWarps except for passes over family blocks at head_dim 128.
// LO: P enters PV as two terms, its value rounded to the storage type and the residue of that rounding (about 16
// significant bits together).  Without it P has the storage type's precision, as in the prefill kernel: enough
// once a row sees more than kLoTermMaxKeys keys, whose residues average out far below the tolerance.  Only the
// head_dim 256 pass, which is bound by its warps' instruction stream, has the variant without (9 % faster); the
// host asks for it when it knows that every row of the launch sees more keys than that.
template <typename T, int D, bool HI, bool EXT, int WARPS, bool LO = true>
__global__ void __launch_bounds__(WARPS * 32, 1)
attend_decode_kernel(const __grid_constant__ CUtensorMap tmap, const DecodeParams p) {
    constexpr int DEPTH = RingShape<D>::kDepth;
    constexpr int THREADS = WARPS * 32;
    constexpr int NH = D / 64;                       // 128-byte sub-rows per head row
    constexpr int KSTEPS = D / 16;
    constexpr int NT = D / 8;
    constexpr int TILE_BYTES = NH * 2048;            // 16 keys of K (or V)
    constexpr bool SPLIT = RingShape<D>::kSplit;     // ring entries hold one plane: K and V of a group travel separately
    constexpr int SLOT_BYTES = SPLIT ? TILE_BYTES : 2 * TILE_BYTES;
    constexpr int NR = HI ? 2 : 1;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    SlotMeta* metas = reinterpret_cast<SlotMeta*>(smem + WARPS * DEPTH * SLOT_BYTES);   // [WARPS][DEPTH]
    uint64_t* bars = reinterpret_cast<uint64_t*>(metas + WARPS * DEPTH);               // full[WARPS][DEPTH]
    int* cum = reinterpret_cast<int*>(bars + WARPS * DEPTH);                           // [n_seq + 1]
    __shared__ int s_warp_tot[WARPS];
    __shared__ ItemMeta s_items[WARPS][kItemEntries];
    __shared__ __align__(16) uint8_t s_new_kv[WARPS][SPLIT ? D * 2 : 2 * D * 2];   // fused append: a warp's new K row (and V row)

    const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
    const uint32_t bar_full = smem_u32(bars);
    const int base_tok = (p.kv_begin / kGroupTokens) * kGroupTokens;
    const int CT = p.chunk_tokens;

    if (tid == 0) {
        for (int i = 0; i < WARPS * DEPTH; i++) mbar_init(bar_full + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap) : "memory");
    }
    if (p.wait_first) pdl_wait();   // raw-pointer entry points: the table may come from the caller's kernel in front
    // What runs before pdl_wait() overlaps the tail of the preceding kernel.  That kernel may still be writing
    // the pool (an append), the query or the scratch; everything launched before it has completed, because a
    // kernel of this library releases its dependents only after its own wait, and any other kernel releases
    // them by completing.  Lengths, rows, block tables and plan arrays are written by copies or by kernels
    // further back, never by the kernel directly in front of an attention launch, so the prefix sum, the
    // warp's first item and its page ids are worked out up here; the first gather comes after the wait.
    // ---- items per entry, exclusive prefix sum into cum[] ----
    // Entries: first the family blocks of a shared-prefix plan (up to 16 query rows of several forked
    // sequences over the chunks they have in common), then the sequences (their remaining chunks).
    // With a tail split (p.tail_chunks > 0) the last tail_chunks chunks of every sequence are cut into
    // p.tail_split pieces that form a third group of entries at the END of the queue: the warps run out
    // of work within a quarter-chunk of one another instead of a whole chunk.
    const int n_fb = EXT ? p.n_fb : 0;
    const int TAILC = p.tail_chunks, TAILS = p.tail_split;
    const int SUBK = TAILC > 0 ? CT / TAILS : CT;     // keys per tail piece
    const int slot_stride = p.max_chunks + TAILC * TAILS;   // partial slots per query row: chunks, then tail pieces
    const int n_ent = n_fb + p.n_seq + (TAILC > 0 ? p.n_seq : 0);
    struct SeqShape { int kv_end, first, nbig, nsmall; };
    auto seq_shape = [&](int b) -> SeqShape {
        SeqShape q;
        q.kv_end = p.kv_len != nullptr ? __ldg(p.kv_len + b) : p.kv_end + b * p.kv_step;
        int nch = q.kv_end > base_tok ? (q.kv_end - base_tok + CT - 1) / CT : 0;
        nch = min(nch, p.max_chunks);
        q.first = n_fb > 0 ? min(__ldg(p.seq_first_chunk + b), nch) : 0;
        q.nbig = max(q.first, nch - TAILC);           // chunks [first, nbig) whole, [nbig, nch) in pieces
        const int ntail = nch - q.nbig;
        q.nsmall = 0;
        if (ntail > 0) {
            const int rem_last = min(q.kv_end - base_tok, nch * CT) - (nch - 1) * CT;
            q.nsmall = (ntail - 1) * TAILS + (rem_last + SUBK - 1) / SUBK;
        }
        return q;
    };
    auto entry_items = [&](int e) -> int {
        if (e < n_fb) return __ldg(p.fb_chunks + e) * p.num_kv_heads;
        if (e < n_fb + p.n_seq) {
            const SeqShape q = seq_shape(e - n_fb);
            return (q.nbig - q.first) * p.num_kv_heads;
        }
        return seq_shape(e - n_fb - p.n_seq).nsmall * p.num_kv_heads;
    };
    {
        const int per = (n_ent + THREADS - 1) / THREADS;
        const int lo = min(tid * per, n_ent), hi = min(lo + per, n_ent);
        int local = 0;
        for (int e = lo; e < hi; e++) local += entry_items(e);
        int incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) s_warp_tot[w] = incl;
        __syncthreads();
        int offset = 0;
        for (int i = 0; i < w; i++) offset += s_warp_tot[i];
        int run = offset + incl - local;
        for (int e = lo; e < hi; e++) {
            cum[e] = run;
            run += entry_items(e);
        }
        if (tid == THREADS - 1) cum[n_ent] = offset + incl;
    }
    __syncthreads();
    const int total_items = cum[n_ent];

    // ---- next-item prefetch state (warp-uniform except raw_next, which lane 0 owns) ----
    // n_state: 0 nothing requested, 1 queue index requested (atomic in flight), 2 decoded (length and
    // table row requested), 3 first page id requested.  The next item is requested only when the
    // current one is within kPrefetchGroups of its end, so that a warp never sits on work that an
    // idle warp could have taken, yet the atomic and the look-ups are off the critical path.
#ifndef DRKV_PREFETCH_GROUPS
#define DRKV_PREFETCH_GROUPS 3
#endif
    constexpr int kPrefetchGroups = DRKV_PREFETCH_GROUPS;
    int raw_next = 0, n_state = 0;
    bool exhausted = false;
    int n_b = 0, n_kvh = 0, n_slot = 0, n_tok_lo = 0, n_tok_hi = 0, n_trow = 0, n_fam = 0;   // n_fam: family block + 1, 0 = plain
    int n_end = 0;              // the next item ends where its sequence ends (it meets the token a fused append brings)
    int n_pv = -1;              // per lane: page id of logical page (n_tok_lo / page_size) + lane of the next item
    // ---- issue cursor ----
    bool c_valid = false;
    int c_b = 0, c_kvh = 0, c_slot = 0, c_trow = 0, c_tok_hi = 0, c_tok_lo = 0, c_ngroups = 0, c_gi = 0, c_fam = 0, c_end = 0;
    // Page ids come 32 at a time: lane i holds the id of logical page c_pv_base + i (c_pv) and of the 32 after
    // those (c_pvn), loaded a window ahead; a group's id is a shuffle away.  A table load per group would sit
    // on the issue path with the latency of a saturated memory system.
    int c_pv = -1, c_pvn = -1, c_pv_base = 0, c_logical = 0, c_off = 0;
    int c_item = 0;             // entry of s_items[w] that describes the item being issued
    int c_half = 0;             // SPLIT: 0 = the group's K entry is next, 1 = its V entry
    bool zero_filled = false;   // some lane has written zeros into a ring slot since the last proxy fence
    int i_slot = 0, outstanding = 0;
    // ---- compute cursor ----
    int slot = 0, phase = 0;
    int mass_row[2] = {-1, -1};     // with tile masses on: this lane's query rows as (sequence, head) indices, -1 = padding
    const int64_t rows_per_plane = (int64_t)p.num_kv_heads * p.page_size;

    // The first item of every warp is its own index in the grid (no atomic on the way to the first
    // gather); later items come from the queue, which therefore starts behind those.
    const int grid_warps = (int)gridDim.x * WARPS;
    bool first_fetch = true;
    auto fetch_raw = [&]() {
        if (first_fetch) {
            raw_next = (int)blockIdx.x * WARPS + w;
            first_fetch = false;
        } else if (lane == 0) {
            raw_next = atomicAdd(p.work_counter, 1) + grid_warps;
        }
        n_state = 1;
    };
    // queue index -> (sequence, head, chunk); requests the sequence's length and table row
    auto decode_next = [&]() {
        const int raw = __shfl_sync(0xffffffffu, raw_next, 0);
        if (raw >= total_items) {
            exhausted = true;
            n_state = 0;
            return;
        }
        int lo = 0, hi = n_ent;                        // largest entry with cum[e] <= raw
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (cum[mid] <= raw) lo = mid; else hi = mid;
        }
        const int per_head = (cum[lo + 1] - cum[lo]) / p.num_kv_heads;
        const int j = raw - cum[lo];
        n_kvh = j / per_head;
        const int i = j - n_kvh * per_head;
        if (lo < n_fb) {                               // shared chunks of a family block
            n_fam = lo + 1;
            n_end = 0;
            n_b = 0;
            n_slot = i;
            n_tok_lo = base_tok + i * CT;
            n_tok_hi = n_tok_lo + CT;
            n_trow = __ldg(p.fb_row + lo);
        } else {
            n_fam = 0;
            const bool piece = lo >= n_fb + p.n_seq;
            n_b = lo - n_fb - (piece ? p.n_seq : 0);
            const SeqShape q = seq_shape(n_b);
            if (!piece) {                              // a whole chunk
                n_slot = q.first + i;
                n_tok_lo = base_tok + n_slot * CT;
                n_tok_hi = min(n_tok_lo + CT, q.kv_end);
            } else {                                   // a piece of one of the last chunks
                n_slot = p.max_chunks + i;
                n_tok_lo = base_tok + (q.nbig + i / TAILS) * CT + (i % TAILS) * SUBK;
                n_tok_hi = min(n_tok_lo + SUBK, q.kv_end);
            }
            n_end = n_tok_hi == q.kv_end;
            n_trow = p.rows != nullptr ? __ldg(p.rows + n_b) : p.row;
        }
        n_state = 2;
    };
    auto load_window = [&](int trow, int first_logical) -> int {
        const int logical = first_logical + lane;
        return logical < p.table_stride ? __ldg(p.tables + (int64_t)trow * p.table_stride + logical) : -1;
    };
    const int plane2 = 2 * (int)rows_per_plane;                  // head rows of one (layer, page): K plane + V plane
    const int layer_page0 = p.layer * p.max_pages;

    float m2[2] = {kNegBig, kNegBig};
    float lsum[2] = {0.f, 0.f};
    float o[NT][2 * NR];
    uint32_t qf[KSTEPS][4];
    const int col = (lane & 3) * 2;
    const int qrow = lane >> 2;

    // One ring entry: the gather of the cursor's group (SPLIT: of its K or its V plane), then the cursor moves on.
    auto issue_entry = [&]() {
        const int ring = w * DEPTH + i_slot;
        const int tok0 = c_tok_lo + c_gi * kGroupTokens;
        if (c_logical - c_pv_base >= 32) {             // next window of page ids (requested 32 pages ago)
            c_pv = c_pvn;
            c_pv_base += 32;
            c_pvn = load_window(c_trow, c_pv_base + 32);
        }
        int page = __shfl_sync(0xffffffffu, c_pv, c_logical - c_pv_base);
        if (page >= p.max_pages) {
            page = -1;
            if (lane == 0) atomicExch(p.error_word, (int)KERR_BAD_PAGE);
        }
        const bool last = (c_gi == c_ngroups - 1);
        if (lane == 0) {
            if (!SPLIT || c_half == 0) {
                SlotMeta m;
                m.flags = (c_gi == 0 ? SLOT_FIRST : 0) | (last ? SLOT_LAST : 0) | (page < 0 ? SLOT_SKIP : 0) | (c_item << kItemShift);
                m.tok0 = tok0;
                m.page = page;
                m.pad = 0;
                metas[ring] = m;
            }
            // Generic-proxy WRITES to the ring (the zero fill of an end group's hidden V rows, made visible
            // to this lane by the __syncwarp that closed that group) are ordered before the async-proxy
            // writes of the new gather.  Reads need no fence: the ldmatrix results have been consumed.
            if (zero_filled) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive_expect_tx(bar_full + 8 * ring, page >= 0 ? SLOT_BYTES : 0);
            if (page >= 0) {
                const uint32_t dst = smem_u32(smem + ring * SLOT_BYTES);
                // head row of the group's first key in the K plane (the descriptor has fewer than 2^31 rows)
                const int rk = (layer_page0 + page) * plane2 + c_kvh * p.page_size + c_off;
                // one box: 16 key rows x the whole head dim x the K and the V plane (8 KB at D = 128);
                // SPLIT: x one plane (8 KB at D = 256)
                tma_load_4d(dst, &tmap, 0, rk, 0, SPLIT ? c_half : 0, bar_full + 8 * ring);
            }
        }
        zero_filled = false;
        if (++i_slot == DEPTH) i_slot = 0;
        outstanding++;
        if (SPLIT && c_half == 0) {                    // the V entry of the same group comes next
            c_half = 1;
            return;
        }
        c_half = 0;
        if (last) {
            c_valid = false;
        } else {
            c_gi++;
            c_off += kGroupTokens;
            if (c_off == p.page_size) {
                c_off = 0;
                c_logical++;
            }
        }
        // one step of the next-item pipeline per issued group, started near the end of this item
        if (!exhausted) {
            if (n_state == 0) {
                if (!c_valid || c_ngroups - c_gi <= kPrefetchGroups) fetch_raw();
            } else if (n_state == 1) {
                decode_next();
            } else if (n_state == 2) {
                n_pv = load_window(n_trow, n_tok_lo / p.page_size);
                n_state = 3;
            }
        }
    };

    // SPLIT: the warp is done with the group's K entry; one more gather goes out (the V plane of the group
    // whose K plane went out last) and the warp waits for the V entry of the group it is computing.
    auto next_entry = [&]() -> bool {
        __syncwarp();
        outstanding--;
        if (++slot == DEPTH) { slot = 0; phase ^= 1; }
        if (c_valid && c_half == 1 && outstanding < DEPTH) issue_entry();
        if (!mbar_wait(bar_full + 8 * (w * DEPTH + slot), phase)) {
            if (lane == 0) atomicExch(p.error_word, (int)KERR_WAIT_FULL);
            return false;
        }
        __syncwarp();
        return true;
    };

    // the warp's first item (its own index in the grid: no queue access) and the first window of its page ids
    fetch_raw();
    decode_next();
    if (n_state == 2) {
        n_pv = load_window(n_trow, n_tok_lo / p.page_size);
        n_state = 3;
    }
    pdl_wait();
    pdl_launch_dependents();

    while (true) {
        // ------------- issue: keep DEPTH groups in flight, across item boundaries -------------
        while (outstanding < DEPTH) {
            if (!c_valid) {
                if (n_state == 0 && !exhausted) fetch_raw();
                if (n_state == 1) decode_next();       // waits for the atomic only if it was just issued
                if (n_state < 2) break;                // queue drained
                c_b = n_b; c_kvh = n_kvh; c_slot = n_slot; c_trow = n_trow; c_tok_lo = n_tok_lo; c_tok_hi = n_tok_hi; c_fam = n_fam;
                c_end = n_end;
                c_ngroups = (c_tok_hi - c_tok_lo + kGroupTokens - 1) / kGroupTokens;
                c_gi = 0;
                c_logical = c_tok_lo / p.page_size;
                c_off = c_tok_lo - c_logical * p.page_size;
                c_pv_base = c_logical;
                c_pv = n_state == 3 ? n_pv : load_window(c_trow, c_logical);
                c_pvn = load_window(c_trow, c_logical + 32);
                c_valid = true;
                n_state = 0;
                c_item = (c_item + 1) & (kItemEntries - 1);
                if (lane == 0) {
                    ItemMeta im;
                    im.b = c_b;
                    im.kvh = c_kvh;
                    im.part_slot = (EXT && c_fam) ? c_slot : (c_b * p.num_q_heads + c_kvh * p.group) * slot_stride + c_slot;
                    im.fam = c_fam;
                    im.tok_hi = c_tok_hi;
                    im.append = (c_end && p.k_new != nullptr) ? 1 : 0;
                    im.trow = c_trow;
                    im.pad2 = 0;
                    s_items[w][c_item] = im;
                }
                if (!EXT || c_fam == 0) {
                    // the item's query rows into L1, a group's time before the warp loads them into fragments
                    const char* qb = reinterpret_cast<const char*>(p.q) +
                                     ((int64_t)c_b * p.num_q_heads + (int64_t)c_kvh * p.group) * (D * (int)sizeof(T));
                    if (lane * 128 < p.group * D * (int)sizeof(T))
                        asm volatile("prefetch.global.L1 [%0];" ::"l"(qb + lane * 128));
                    if (c_end && p.k_new != nullptr && lane < 2 * (D * (int)sizeof(T) / 128)) {
                        // the new token's K and V rows, which this item will append when it starts
                        const int64_t src = ((int64_t)c_b * p.num_kv_heads + c_kvh) * (D * (int)sizeof(T));
                        const int hl = D * (int)sizeof(T) / 128;                 // 128-byte lines per row
                        const char* base = reinterpret_cast<const char*>(lane < hl ? p.k_new : p.v_new) + src;
                        asm volatile("prefetch.global.L1 [%0];" ::"l"(base + (lane % hl) * 128));
                    }
                }
            }
            issue_entry();
        }
        if (outstanding == 0) break;                   // queue drained and every group consumed

        // ------------- compute the oldest group in flight -------------
        const int ring = w * DEPTH + slot;
        if (!mbar_wait(bar_full + 8 * ring, phase)) {
            if (lane == 0) atomicExch(p.error_word, (int)KERR_WAIT_FULL);
            break;
        }
        __syncwarp();
        const SlotMeta meta = metas[ring];
        const ItemMeta* item = &s_items[w][(meta.flags >> kItemShift) & (kItemEntries - 1)];
        if (meta.flags & SLOT_FIRST) {
            // query rows straight into m16k16 A fragments.  Plain item: row r is query head r of the group;
            // family block: row r is head r % g of member r / g (several forked sequences share the keys).
            // Rows beyond that are zero.
            const T* qall = reinterpret_cast<const T*>(p.q);
            const T* qr0 = nullptr;
            const T* qr1 = nullptr;
            if (!EXT || item->fam == 0) {
                const T* qb = qall + ((int64_t)item->b * p.num_q_heads + (int64_t)item->kvh * p.group) * D;
                if (qrow < p.group) qr0 = qb + (int64_t)qrow * D;
                if (HI && qrow + 8 < p.group) qr1 = qb + (int64_t)(qrow + 8) * D;
            } else {
                const int32_t* mem = p.fb_members + (item->fam - 1) * 16;
                const int r0i = qrow / p.group, r1i = (qrow + 8) / p.group;
                const int b0 = r0i < 16 ? __ldg(mem + r0i) : -1, b1 = (HI && r1i < 16) ? __ldg(mem + r1i) : -1;
                if (b0 >= 0) qr0 = qall + ((int64_t)b0 * p.num_q_heads + (int64_t)item->kvh * p.group + qrow % p.group) * D;
                if (b1 >= 0) qr1 = qall + ((int64_t)b1 * p.num_q_heads + (int64_t)item->kvh * p.group + (qrow + 8) % p.group) * D;
            }
            if (EXT && p.tile_lse != nullptr) {
                // value of (sequence b, kv head, tile, head-in-group j) at ((b * Hkv + kvh) * max_tiles + tile) * g + j:
                // the rows of one group land in one 32-byte sector per tile
                auto base_of = [&](const T* qr) -> int {
                    if (qr == nullptr) return -1;
                    const int rowi = (int)((qr - qall) / (int64_t)D);          // b * Hq + kvh * g + j
                    const int bq = rowi / p.num_q_heads, j = rowi % p.group;
                    return ((bq * p.num_kv_heads + item->kvh) * p.max_tiles * p.group + j) * 4 + (lane & 3);
                };
                mass_row[0] = base_of(qr0);
                mass_row[1] = base_of(qr1);
            }
            const uint32_t* q0 = reinterpret_cast<const uint32_t*>(qr0 + col);
            const uint32_t* q1 = reinterpret_cast<const uint32_t*>(qr1 + col);
#pragma unroll
            for (int kk = 0; kk < KSTEPS; kk++) {
                qf[kk][0] = qr0 ? __ldg(q0 + 8 * kk) : 0u;
                qf[kk][2] = qr0 ? __ldg(q0 + 8 * kk + 4) : 0u;
                qf[kk][1] = qr1 ? __ldg(q1 + 8 * kk) : 0u;
                qf[kk][3] = qr1 ? __ldg(q1 + 8 * kk + 4) : 0u;
            }
            m2[0] = m2[1] = kNegBig;
            lsum[0] = lsum[1] = 0.f;
#pragma unroll
            for (int i = 0; i < NT; i++)
#pragma unroll
                for (int j = 0; j < 2 * NR; j++) o[i][j] = 0.f;
        }
        if ((meta.flags & SLOT_FIRST) && item->append) {
            // this item ends at its sequence's new token: rotate and stage the token's rows now, while the item's
            // first gathers are in flight, and write them into the pool page (nothing if the table has a hole there)
            const int pos = item->tok_hi - 1;
            const int logical = pos / p.page_size;
            int page = logical < p.table_stride ? __ldg(p.tables + (int64_t)item->trow * p.table_stride + logical) : -1;
            if (page >= p.max_pages) page = -1;
            const int64_t src = ((int64_t)item->b * p.num_kv_heads + item->kvh) * D;
            const int64_t plane = rows_per_plane * D;           // elements of one plane of a page
            // element offset of (layer, page, K plane, kv head, slot of the token, 0)
            const int64_t krow = ((int64_t)(layer_page0 + page) * 2) * plane + ((int64_t)item->kvh * p.page_size + pos % p.page_size) * D;
            fused_append_prepare<T, D, !SPLIT>(reinterpret_cast<const T*>(p.k_new) + src, reinterpret_cast<const T*>(p.v_new) + src,
                                               page >= 0 ? reinterpret_cast<T*>(p.pool) + krow : nullptr, plane, p.inv_freq,
                                               p.rotary_dim, &s_new_kv[w][0], pos, lane);
        }
        if (!(meta.flags & SLOT_SKIP)) {
            // keys [v_lo, v_hi) of the 16 in the slot are visible: all of them except in an item's end groups
            int v_lo = 0, v_hi = kGroupTokens;
            if (meta.flags & (SLOT_FIRST | SLOT_LAST)) {
                v_lo = max(0, p.kv_begin - meta.tok0);
                v_hi = min(kGroupTokens, item->tok_hi - meta.tok0);
            }
            uint8_t* kt = smem + ring * SLOT_BYTES;
            uint8_t* vt = kt + TILE_BYTES;              // SPLIT: set once the V entry has landed
            const bool patch_new = (meta.flags & SLOT_LAST) && item->append;
            if (patch_new) {
                // the last key of the item is the sequence's new token: its rows come from the warp's staging area
                // (see fused_append_prepare), whatever the gather found at that slot of the page.  With K and V in
                // separate ring entries only the K row is staged and patched here; the V row follows once its entry
                // has landed.
                const int row = item->tok_hi - 1 - meta.tok0;
                const uint8_t* stage = &s_new_kv[w][0];
                for (int c = lane; c < (SPLIT ? 1 : 2) * (D / 8); c += 32) {
                    const int pl = c / (D / 8), cc = c - pl * (D / 8);
                    *reinterpret_cast<Vec16*>((pl ? vt : kt) + swz_seg16(row, cc)) =
                        *reinterpret_cast<const Vec16*>(stage + pl * (D * 2) + 16 * cc);
                }
                __syncwarp();
                zero_filled = true;                     // generic-proxy writes to the slot: fence before its next gather
            }
            auto zero_hidden_rows = [&]() {
                if (v_hi < kGroupTokens || v_lo > 0) {
                    // Slots outside the visible range may hold anything (stale pages): give the
                    // PV product zeros there so that 0 * garbage cannot produce a NaN.
                    for (int i = lane; i < kGroupTokens * NH * 8; i += 32) {
                        const int r = i / (NH * 8), c = i - r * (NH * 8);
                        if (r >= v_hi || r < v_lo)
                            *reinterpret_cast<Vec16*>(vt + swz_seg16(r, c)) = Vec16{{0u, 0u, 0u, 0u}};
                    }
                    __syncwarp();
                    zero_filled = true;
                }
            };
            if (!SPLIT) zero_hidden_rows();
            // ---- S = Q K^T : 16 rows x 16 keys ----
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
            {
                const int mi = lane >> 3;
                const int key = (mi >> 1) * 8 + (lane & 7);
                const uint32_t kbase = smem_u32(kt);
#pragma unroll
                for (int kk = 0; kk < KSTEPS; kk++) {
                    const int c = 2 * kk + (mi & 1);
                    uint32_t kb[4];
                    ldmatrix_x4(kb, kbase + swz_seg16(key, c));
                    Mma<T>::run(s0[0], s0[1], s0[2], s0[3], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], kb[0], kb[1]);
                    Mma<T>::run(s1[0], s1[1], s1[2], s1[3], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], kb[2], kb[3]);
                }
            }
            // ---- online softmax in the log2 domain ----
            const bool k0 = (col >= v_lo) && (col < v_hi), k1 = (col + 1 >= v_lo) && (col + 1 < v_hi);
            const bool k8 = (col + 8 >= v_lo) && (col + 8 < v_hi), k9 = (col + 9 >= v_lo) && (col + 9 < v_hi);
            uint32_t phi[4], plo[4];
            float alpha[2] = {1.f, 1.f};
#pragma unroll
            for (int r = 0; r < NR; r++) {
                float x0 = k0 ? s0[2 * r] * p.scale_log2 : -INFINITY;
                float x1 = k1 ? s0[2 * r + 1] * p.scale_log2 : -INFINITY;
                float x8 = k8 ? s1[2 * r] * p.scale_log2 : -INFINITY;
                float x9 = k9 ? s1[2 * r + 1] * p.scale_log2 : -INFINITY;
                float mx = fmaxf(fmaxf(x0, x1), fmaxf(x8, x9));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float mnew = fmaxf(m2[r], mx);
                alpha[r] = fast_exp2(m2[r] - mnew);
                m2[r] = mnew;
                const float p0 = fast_exp2(x0 - mnew), p1 = fast_exp2(x1 - mnew);
                const float p8 = fast_exp2(x8 - mnew), p9 = fast_exp2(x9 - mnew);
                lsum[r] = lsum[r] * alpha[r] + ((p0 + p1) + (p8 + p9));
                if (EXT && p.tile_lse != nullptr) {
                    // log2 of the un-normalised probability mass of this lane's four keys of the tile, on the
                    // scale of the final log-sum-exp: mass share = 2^(tile_lse - lse2) once the merge knows lse2.
                    // The four lanes of a row store their own value: no shuffle on the softmax's critical path.
                    const float ts = (p0 + p1) + (p8 + p9);
                    if (mass_row[r] >= 0)
                        p.tile_lse[mass_row[r] + (meta.tok0 / kGroupTokens) * p.group * 4] = ts > 0.f ? mnew + __log2f(ts) : -INFINITY;
                }
                if (LO) {
                    split_pack<T>(p0, p1, phi[r], plo[r]);          // a0 (r=0) / a1 (r=1)
                    split_pack<T>(p8, p9, phi[2 + r], plo[2 + r]);  // a2 / a3
                } else {
                    phi[r] = Elem<T>::pack2(p0, p1);
                    phi[2 + r] = Elem<T>::pack2(p8, p9);
                    plo[r] = plo[2 + r] = 0u;
                }
            }
            if (!HI) { phi[1] = phi[3] = plo[1] = plo[3] = 0u; }
            if (SPLIT) {
                if (!next_entry()) break;
                vt = smem + (w * DEPTH + slot) * SLOT_BYTES;
                if (patch_new) {
                    // the new token's V row, straight from its source (it is not rotated)
                    const int row = item->tok_hi - 1 - meta.tok0;
                    const T* vsrc = reinterpret_cast<const T*>(p.v_new) + ((int64_t)item->b * p.num_kv_heads + item->kvh) * D;
                    for (int c = lane; c < D / 8; c += 32) *reinterpret_cast<Vec16*>(vt + swz_seg16(row, c)) = ldg16(vsrc + 8 * c);
                    __syncwarp();
                    zero_filled = true;
                }
                zero_hidden_rows();
            }
            if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                for (int i = 0; i < NT; i++) {
                    o[i][0] *= alpha[0];
                    o[i][1] *= alpha[0];
                    if (HI) { o[i][2 * NR - 2] *= alpha[1]; o[i][2 * NR - 1] *= alpha[1]; }
                }
            }
            // ---- O += P V : 16 rows x D ----
            {
                const int mi = lane >> 3;
                const int key = (mi & 1) * 8 + (lane & 7);
                const uint32_t vbase = smem_u32(vt);
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    const int c = j + (mi >> 1);
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, vbase + swz_seg16(key, c));
                    if (HI) {
                        Mma<T>::run(o[j][0], o[j][1], o[j][2 * NR - 2], o[j][2 * NR - 1], phi[0], phi[1], phi[2], phi[3], vb[0], vb[1]);
                        if (LO) Mma<T>::run(o[j][0], o[j][1], o[j][2 * NR - 2], o[j][2 * NR - 1], plo[0], plo[1], plo[2], plo[3], vb[0], vb[1]);
                        Mma<T>::run(o[j + 1][0], o[j + 1][1], o[j + 1][2 * NR - 2], o[j + 1][2 * NR - 1], phi[0], phi[1], phi[2], phi[3], vb[2], vb[3]);
                        if (LO) Mma<T>::run(o[j + 1][0], o[j + 1][1], o[j + 1][2 * NR - 2], o[j + 1][2 * NR - 1], plo[0], plo[1], plo[2], plo[3], vb[2], vb[3]);
                    } else {
                        float z0 = 0.f, z1 = 0.f;   // rows 8..15 are padding: their sums are discarded
                        Mma<T>::run(o[j][0], o[j][1], z0, z1, phi[0], 0u, phi[2], 0u, vb[0], vb[1]);
                        if (LO) Mma<T>::run(o[j][0], o[j][1], z0, z1, plo[0], 0u, plo[2], 0u, vb[0], vb[1]);
                        Mma<T>::run(o[j + 1][0], o[j + 1][1], z0, z1, phi[0], 0u, phi[2], 0u, vb[2], vb[3]);
                        if (LO) Mma<T>::run(o[j + 1][0], o[j + 1][1], z0, z1, plo[0], 0u, plo[2], 0u, vb[2], vb[3]);
                    }
                }
            }
        }
        else {
            if (SPLIT && !next_entry()) break;         // a skipped group still has two (empty) ring entries
            if (EXT && p.tile_lse != nullptr) {
#pragma unroll
                for (int r = 0; r < NR; r++)
                    if (mass_row[r] >= 0) p.tile_lse[mass_row[r] + (meta.tok0 / kGroupTokens) * p.group * 4] = -INFINITY;
            }
        }
        __syncwarp();                                  // every lane is done with the slot's shared memory
        outstanding--;
        if (++slot == DEPTH) { slot = 0; phase ^= 1; }

        if (meta.flags & SLOT_LAST) {
            // the item's partial (m, l, o), un-normalised, straight from the accumulators
            const float kLn2 = 0.6931471805599453f;
#pragma unroll
            for (int r = 0; r < NR; r++) {
                float l = lsum[r];
                l += __shfl_xor_sync(0xffffffffu, l, 1);
                l += __shfl_xor_sync(0xffffffffu, l, 2);
                const int row = qrow + 8 * r;
                int64_t ps = -1;                                   // partial slot of this row, -1: padding row
                if (!EXT || item->fam == 0) {
                    if (row < p.group) ps = (int64_t)item->part_slot + (int64_t)row * slot_stride;
                } else {
                    const int mi = row / p.group;
                    const int bm = mi < 16 ? __ldg(p.fb_members + (item->fam - 1) * 16 + mi) : -1;
                    if (bm >= 0)
                        ps = ((int64_t)bm * p.num_q_heads + (int64_t)item->kvh * p.group + row % p.group) * slot_stride +
                             item->part_slot;               // part_slot holds the chunk index for family blocks
                }
                if (ps >= 0) {
                    const bool empty = !(l > 0.f);
                    float* dst = p.part_o + ps * D + col;
#pragma unroll
                    for (int i = 0; i < NT; i++)
                        *reinterpret_cast<float2*>(dst + 8 * i) =
                            empty ? make_float2(0.f, 0.f) : make_float2(o[i][2 * r], o[i][2 * r + 1]);
                    if ((lane & 3) == 0) {
                        p.part_m[ps] = empty ? -1.0e20f : m2[r] * kLn2;
                        p.part_l[ps] = empty ? 0.f : l;
                    }
                }
            }
        }
    }
    // The last warp of the grid to leave rewinds the work queue for the next launch on this stream.
    if (lane == 0) {
        __threadfence();
        const int total_warps = (int)gridDim.x * WARPS;
        if (atomicAdd(p.exit_count, 1) == total_warps - 1) {
            *p.work_counter = 0;
            *p.exit_count = 0;
        }
    }
}

// Merge of chunk partials: m = max m_c, weights exp(m_c - m); out = sum w_c o_c / sum w_c l_c.
// Left unwritten when no key was visible (paged_attention.cu:266-268).  One CTA per (query
// head, sequence); its 8 warps take the chunks round-robin, each lane owning 4 (or 8)
// consecutive dims as float4, and a shared-memory pass adds the warps' partial sums.  Eight warps per CTA
// for batches (a handful of partials per row); 32 for a row with more than 64 partials (one long sequence
// cut into an item per warp of the grid: 148 partials per head), where eight warps would each walk 19
// partials in five dependent round trips to L2.
template <typename T, int kCombineWarps>
__global__ void __launch_bounds__(kCombineWarps * 32) combine_kernel(const CombineParams p) {
    const int h = blockIdx.x, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = p.head_dim;
    const float kLog2e = 1.4426950408889634f;
    __shared__ float s_m[kCombineWarps], s_l[kCombineWarps];
    __shared__ float4 s_acc[kCombineWarps][64];         // D <= 256 -> at most 64 float4 per row

    // lengths and plan arrays are older than the kernel in front (see attend_decode_kernel): the slot arithmetic
    // runs under its tail, the partials are read after the wait
    const int kv_end = p.kv_len != nullptr ? p.kv_len[b] : p.kv_end + b * p.kv_step;
    const int base = (p.kv_begin / kGroupTokens) * kGroupTokens;
    int nch = kv_end > base ? (kv_end - base + p.chunk_tokens - 1) / p.chunk_tokens : 0;
    nch = min(nch, p.max_chunks);
    // partial slots of this row: whole chunks [0, nbig) at their index, then the pieces of the last chunks
    // (see the tail split in attend_decode_kernel) from index max_chunks on
    const int tailc = p.tail_chunks, tails = p.tail_split;
    const int first = (tailc > 0 && p.seq_first_chunk != nullptr) ? min(p.seq_first_chunk[b], nch) : 0;
    const int nbig = tailc > 0 ? max(first, nch - tailc) : nch;
    int nsmall = 0;
    if (nch > nbig) {
        const int subk = p.chunk_tokens / tails;
        const int rem_last = min(kv_end - base, nch * p.chunk_tokens) - (nch - 1) * p.chunk_tokens;
        nsmall = (nch - nbig - 1) * tails + (rem_last + subk - 1) / subk;
    }
    const int nchunks = nbig + nsmall;
    const int skip = p.max_chunks - nbig;                // list index i >= nbig lives at slot i + skip
    const int64_t slot0 = ((int64_t)b * p.num_q_heads + h) * (p.max_chunks + tailc * tails);
    pdl_wait();                                          // partials come from the preceding kernel
    pdl_launch_dependents();

    float mloc = -1.0e20f;
    for (int c = threadIdx.x; c < nchunks; c += kCombineWarps * 32)
        mloc = fmaxf(mloc, p.part_m[slot0 + c + (c >= nbig ? skip : 0)]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
    if (lane == 0) s_m[warp] = mloc;
    __syncthreads();
    float mmax = s_m[0];
#pragma unroll
    for (int i = 1; i < kCombineWarps; i++) mmax = fmaxf(mmax, s_m[i]);

    const int nq = D / 4;                                // float4 per row
    float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
    float l = 0.f;
    // four chunks per trip: their loads are independent, so one round trip to L2 covers all of them
    for (int c0 = warp; c0 < nchunks; c0 += 4 * kCombineWarps) {
        float wgt[4], lv[4];
        float4 v0[4], v1[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int c = c0 + u * kCombineWarps;
            const bool in = c < nchunks;
            const int cc = in ? c : c0;
            const int64_t sl = slot0 + cc + (cc >= nbig ? skip : 0);
            wgt[u] = in ? p.part_m[sl] : -1.0e20f;
            lv[u] = in ? p.part_l[sl] : 0.f;
            const float4* row = reinterpret_cast<const float4*>(p.part_o + sl * D);
            v0[u] = (in && lane < nq) ? row[lane] : make_float4(0.f, 0.f, 0.f, 0.f);
            v1[u] = (in && lane + 32 < nq) ? row[lane + 32] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const float wg = (c0 + u * kCombineWarps < nchunks) ? fast_exp2((wgt[u] - mmax) * kLog2e) : 0.f;
            l += wg * lv[u];
            acc0.x += wg * v0[u].x; acc0.y += wg * v0[u].y; acc0.z += wg * v0[u].z; acc0.w += wg * v0[u].w;
            acc1.x += wg * v1[u].x; acc1.y += wg * v1[u].y; acc1.z += wg * v1[u].z; acc1.w += wg * v1[u].w;
        }
    }
    s_acc[warp][lane] = acc0;
    s_acc[warp][lane + 32] = acc1;
    if (lane == 0) s_l[warp] = l;
    __syncthreads();
    float lt = 0.f;
#pragma unroll
    for (int i = 0; i < kCombineWarps; i++) lt += s_l[i];
    if (p.xchg.world > 0) {
        // one sequence split over several GPUs: this head's partial goes to every rank, theirs come here
        __shared__ int s_ok;
        float acc = 0.f;
        if ((int)threadIdx.x < D) {
#pragma unroll
            for (int i = 0; i < kCombineWarps; i++) acc += reinterpret_cast<const float*>(&s_acc[i][0])[threadIdx.x];
        }
        const bool any = lt > 0.f;
        exchange_and_merge<T>(p.xchg, h, p.num_q_heads, D, any ? acc : 0.f, any ? mmax : -1.0e20f, any ? lt : 0.f, p.out, &s_ok);
        return;
    }
    for (int d = threadIdx.x; d < D; d += kCombineWarps * 32) {
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < kCombineWarps; i++) acc += reinterpret_cast<const float*>(&s_acc[i][0])[d];
        if (p.out_partial != nullptr) {
            p.out_partial[(int64_t)h * D + d] = lt > 0.f ? acc : 0.f;
        } else if (lt > 0.f) {
            reinterpret_cast<T*>(p.out)[((int64_t)b * p.num_q_heads + h) * D + d] = Elem<T>::from_f(acc / lt);
        }
    }
    if (p.lse2_out != nullptr && threadIdx.x == 0)
        p.lse2_out[(int64_t)b * p.num_q_heads + h] = lt > 0.f ? mmax * kLog2e + __log2f(lt) : INFINITY;
    if (p.out_partial != nullptr && threadIdx.x == 0) {
        p.out_partial[(int64_t)p.num_q_heads * D + h] = lt > 0.f ? mmax : -1.0e20f;
        p.out_partial[(int64_t)p.num_q_heads * (D + 1) + h] = lt > 0.f ? lt : 0.f;
    }
}

// Attention mass per page, the importance scorer's input (importance_scorer.h:8-15: "accumulates
// per-block attention weights across all Full Attention layers"): new[row][page] += sum over query
// heads and the page's keys of the softmax probability.  One thread per (sequence, page); a warp's
// lanes take consecutive pages, so the tile values of one head are read contiguously.
__global__ void __launch_bounds__(128) page_mass_kernel(const PageMassParams p) {
    pdl_wait();                                          // tile values and lse2 come from the two preceding kernels
    pdl_launch_dependents();
    // 32 pages x 4 slices of the kv heads per CTA; the slices are added in a fixed order (no atomics: the sums
    // are reproducible)
    __shared__ float s_part[4][32];
    const int b = blockIdx.y, lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
    const int page = blockIdx.x * 32 + lane;
    const int kv_end = p.kv_len[b];
    const int tiles_per_page = p.page_size / kGroupTokens;
    const int n_tiles = (kv_end + kGroupTokens - 1) / kGroupTokens;
    const bool live = page * tiles_per_page < n_tiles;
    const int t1 = min((page + 1) * tiles_per_page, n_tiles);
    const int g = p.num_q_heads / p.num_kv_heads;
    float mass = 0.f;
    if (live) {
        for (int kvh = slice; kvh < p.num_kv_heads; kvh += 4) {
            const float* lse2 = p.lse2 + (int64_t)b * p.num_q_heads + kvh * g;
            const float4* tl = reinterpret_cast<const float4*>(p.tile_lse) + ((int64_t)b * p.num_kv_heads + kvh) * p.max_tiles * g;
            for (int t = page * tiles_per_page; t < t1; t++)
                for (int j = 0; j < g; j++) {
                    const float4 v = tl[t * g + j];      // the four lanes' shares of row j of this tile
                    const float l2 = lse2[j];
                    mass += (fast_exp2(v.x - l2) + fast_exp2(v.y - l2)) + (fast_exp2(v.z - l2) + fast_exp2(v.w - l2));
                }
        }
    }
    s_part[slice][lane] = mass;
    __syncthreads();
    if (slice == 0 && live) {
        float* dst = p.fresh + (int64_t)p.rows[b] * p.table_stride + page;
        *dst += (s_part[0][lane] + s_part[1][lane]) + (s_part[2][lane] + s_part[3][lane]);
    }
}

// score = score * decay + new, then new = 0 (importance_scorer.cu:27-37, one fused multiply-add).
__global__ void importance_update_kernel(float* scores, float* fresh, int64_t n, float decay) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    scores[i] = __fmaf_rn(scores[i], decay, fresh[i]);
    fresh[i] = 0.f;
}

// ImportanceScorer::update with caller-provided values (importance_scorer.cu:27-37,68-73).
__global__ void importance_add_kernel(float* scores, const float* new_scores, int n, float decay) {
    pdl_wait();
    pdl_launch_dependents();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) scores[i] = __fmaf_rn(scores[i], decay, new_scores[i]);
}

// Merge of whole-range partials in the external layout [Hq*D o | Hq m | Hq l] per part, in the
// order and with the running-max update of asr_ops_attn.cu:94-107.
template <typename T>
__global__ void __launch_bounds__(128)
combine_external_kernel(int n_parts, const float* parts, int hq, int D, void* out) {
    const int h = blockIdx.x;
    const int64_t stride = (int64_t)hq * (D + 2);
    const float kLog2e = 1.4426950408889634f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float m = -1.0e20f, l = 0.f, acc = 0.f;
        for (int q = 0; q < n_parts; q++) {
            const float* base = parts + q * stride;
            const float pm = base[(int64_t)hq * D + h], pl = base[(int64_t)hq * (D + 1) + h];
            const float pv = base[(int64_t)h * D + d];
            if (pm > m) {
                const float f = fast_exp2((m - pm) * kLog2e);
                acc = acc * f + pv;
                l = l * f + pl;
                m = pm;
            } else {
                const float f = fast_exp2((pm - m) * kLog2e);
                acc += pv * f;
                l += pl * f;
            }
        }
        if (l > 0.f) reinterpret_cast<T*>(out)[(int64_t)h * D + d] = Elem<T>::from_f(acc / l);
    }
}

template <typename T, int D, bool HI, bool EXT, int WARPS = RingShape<D>::kWarps, bool LO = true>
cudaError_t launch_decode_hi(const CUtensorMap& tmap, const DecodeParams& p, int num_sms, cudaStream_t stream) {
    constexpr int DEPTH = RingShape<D>::kDepth, NH = D / 64;
    constexpr size_t smem = 1024 + (size_t)WARPS * DEPTH * ((RingShape<D>::kSplit ? 1 : 2) * NH * 2048 + sizeof(SlotMeta) + sizeof(uint64_t)) +
                            (3 * kMaxDecodeSeqs + 1) * sizeof(int);   // cum[]: family blocks, sequences, their tail pieces
    // per instantiation and device (the attribute belongs to the context); any thread may be the first caller
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        e = cudaFuncSetAttribute(attend_decode_kernel<T, D, HI, EXT, WARPS, LO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    int grid = (p.total_items + WARPS - 1) / WARPS;
    if (grid > num_sms) grid = num_sms;
    return launch_pdl(attend_decode_kernel<T, D, HI, EXT, WARPS, LO>, dim3(grid), dim3(WARPS * 32), smem, stream, tmap, p);
}

// A pass over family blocks (branches of one prompt: a short launch over few items, its shared pages partly read
// from L2) is not bound by the memory system's taste for few concurrent streams: at head_dim 128 twelve warps per
// CTA run it 13 % faster than eight (168 registers per thread), where a pass that streams from HBM loses 4-12 %.
constexpr int kFamilyWarps128 = 12;

template <typename T, int D>
cudaError_t launch_decode_t(const CUtensorMap& tmap, const DecodeParams& p, int num_sms, cudaStream_t stream) {
    const bool ext = p.n_fb > 0 || p.tile_lse != nullptr;
    if constexpr (D == 256) {
        if (p.few_keys_possible == 0 && !ext)
            return (p.group > 8 || p.rows_per_item > 8)
                       ? launch_decode_hi<T, D, true, false, RingShape<D>::kWarps, false>(tmap, p, num_sms, stream)
                       : launch_decode_hi<T, D, false, false, RingShape<D>::kWarps, false>(tmap, p, num_sms, stream);
    }
    if constexpr (D == 128) {
        if (p.n_fb > 0)
            return (p.group > 8 || p.rows_per_item > 8)
                       ? launch_decode_hi<T, D, true, true, kFamilyWarps128>(tmap, p, num_sms, stream)
                       : launch_decode_hi<T, D, false, true, kFamilyWarps128>(tmap, p, num_sms, stream);
    }
    if (p.group > 8 || p.rows_per_item > 8)
        return ext ? launch_decode_hi<T, D, true, true>(tmap, p, num_sms, stream)
                   : launch_decode_hi<T, D, true, false>(tmap, p, num_sms, stream);
    return ext ? launch_decode_hi<T, D, false, true>(tmap, p, num_sms, stream)
               : launch_decode_hi<T, D, false, false>(tmap, p, num_sms, stream);
}

}  // namespace


// Decode's descriptor: the pool as [plane offset 0/1][head row][64-dim half][64 elements], so that one box
// of {64, D/64, 16, 2} brings 16 key rows of one head, all dims, K and V (the V plane of a page starts
// num_kv_heads * page_size rows after its K plane).  The row dimension stops one plane short of the end so
// that plane offset 1 stays inside the pool.  Shared-memory image: K rows then V rows, full rows of D * 2
// bytes, 128-byte swizzle.
bool make_pool_slot_tensor_map(CUtensorMap* out, const void* pool, int num_layers, int max_pages, int num_kv_heads,
                               int page_size, int head_dim, const char** err) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    // One descriptor per (pool, shape) is kept: the raw-pointer entry points are called once per layer and token
    // with the same pool, and neither the driver look-up nor the encoding belongs on that path.
    struct Key {
        const void* pool;
        int layers, pages, heads, page, dim;
        bool operator==(const Key& o) const {
            return pool == o.pool && layers == o.layers && pages == o.pages && heads == o.heads && page == o.page && dim == o.dim;
        }
    };
    struct Entry { Key key; CUtensorMap map; };
    static std::mutex cache_mu;
    static Entry cache[8];
    static int cache_used = 0, cache_next = 0;
    const Key key{pool, num_layers, max_pages, num_kv_heads, page_size, head_dim};
    std::lock_guard<std::mutex> lock(cache_mu);
    for (int i = 0; i < cache_used; i++)
        if (cache[i].key == key) {
            *out = cache[i].map;
            return true;
        }
    static EncodeFn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || fn == nullptr) {
            if (err) *err = "cuTensorMapEncodeTiled is not available from this driver";
            return false;
        }
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const uint64_t plane_rows = (uint64_t)num_kv_heads * page_size;
    const uint64_t rows = (uint64_t)num_layers * max_pages * 2 * plane_rows;
    if (rows >= (1ull << 31)) {
        if (err) *err = "pool has more than 2^31 head rows: not addressable by one TMA descriptor";
        return false;
    }
    const int nh = head_dim / 64;
    // dimensions: 64 elements of a 128-byte segment, head row, segment of the row, plane.  The row comes BEFORE
    // the segment although its stride is the larger one, so that a box lands as [plane][segment][row][128 B]:
    // rows 128 bytes apart, which is what keeps the ldmatrix reads of the kernel free of bank conflicts.
    cuuint64_t gdim[4] = {64, (cuuint64_t)(rows - plane_rows), (cuuint64_t)nh, 2};
    cuuint64_t gstride[3] = {(cuuint64_t)head_dim * 2, 128, (cuuint64_t)plane_rows * head_dim * 2};
    // head_dim 256: the decode ring holds K and V of a group as separate entries, one plane per box
    cuuint32_t box[4] = {64, 16, (cuuint32_t)nh, (head_dim == 256 && RingShape<256>::kSplit) ? 1u : 2u};
    cuuint32_t estride[4] = {1, 1, 1, 1};
    CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(pool), gdim, gstride, box, estride,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (err) *err = "cuTensorMapEncodeTiled (decode slot descriptor) failed";
        return false;
    }
    cache[cache_next] = Entry{key, *out};
    cache_next = (cache_next + 1) % 8;
    if (cache_used < 8) cache_used++;
    return true;
}

// The prefill kernel's descriptor for head_dim 128: the pool as
//   [octet of 8 head rows (stride 2 KB)][plane K/V (stride Hkv * page rows)][64-dim half (stride 128 B)][row in octet (stride 256 B)][64 elements],
// box {64, 8, 2, 2, 2}: one copy brings the K and the V rows of 16 keys of one head, all dims (8 KB), as sixteen 8-row
// groups of 128 bytes ordered [octet][plane][half], 128-byte swizzle.  The 8-row groups of one (plane, half) are then
// 4 KB apart over a whole block of keys, so a single MMA operand descriptor (one stride between 8-row groups) walks
// them: K-major for K, MN-major for V.  The octet dimension stops one plane short of the end so that plane 1 stays
// inside the pool.
bool make_pool_kv16_tensor_map(CUtensorMap* out, const void* pool, int num_layers, int max_pages, int num_kv_heads,
                               int page_size, int head_dim, const char** err) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) {
        if (err) *err = "the tensor-core prefill kernel is built for head_dim 64, 128 and 256";
        return false;
    }
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || fn == nullptr) {
        if (err) *err = "cuTensorMapEncodeTiled is not available from this driver";
        return false;
    }
    EncodeFn encode = reinterpret_cast<EncodeFn>(fn);
    const uint64_t plane_rows = (uint64_t)num_kv_heads * page_size;
    const uint64_t rows = (uint64_t)num_layers * max_pages * 2 * plane_rows;
    if (rows >= (1ull << 31)) {
        if (err) *err = "pool has more than 2^31 head rows: not addressable by one TMA descriptor";
        return false;
    }
    const cuuint32_t halves = (cuuint32_t)(head_dim / 64);          // 64-element (128-byte) runs of a head row
    cuuint64_t gdim[5] = {64, 8, halves, 2, (cuuint64_t)((rows - plane_rows) / 8)};
    cuuint64_t gstride[4] = {(cuuint64_t)head_dim * 2, 128, (cuuint64_t)plane_rows * head_dim * 2, (cuuint64_t)8 * head_dim * 2};
    cuuint32_t box[5] = {64, 8, halves, 2, 2};
    cuuint32_t estride[5] = {1, 1, 1, 1, 1};
    CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 5, const_cast<void*>(pool), gdim, gstride, box, estride,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (err) *err = "cuTensorMapEncodeTiled refused the 16-key K/V view of the pool";
        return false;
    }
    return true;
}

int decode_warps_per_cta(int head_dim, bool family_blocks) {
    if (head_dim == 128 && family_blocks) return kFamilyWarps128;
    return head_dim == 64 ? RingShape<64>::kWarps : head_dim == 128 ? RingShape<128>::kWarps : RingShape<256>::kWarps;
}

cudaError_t launch_attend_decode(const CUtensorMap& tmap, const DecodeParams& p, int num_sms, int head_dim,
                                 int dtype, cudaStream_t stream) {
    if (p.total_items <= 0) return cudaSuccess;
    if (p.n_seq > kMaxDecodeSeqs || p.n_fb > kMaxDecodeSeqs) return cudaErrorInvalidValue;
    if (p.chunk_tokens % kGroupTokens != 0 || p.chunk_tokens <= 0 || p.group > 16 || p.page_size % kGroupTokens != 0)
        return cudaErrorInvalidValue;
    if (p.tail_chunks < 0 || (p.tail_chunks > 0 && (p.tail_split < 1 || p.chunk_tokens % p.tail_split != 0 ||
                                                    (p.chunk_tokens / p.tail_split) % kGroupTokens != 0)))
        return cudaErrorInvalidValue;
    const bool f16 = dtype == DRKV_DTYPE_F16;
    switch (head_dim) {
        case 64:
            return f16 ? launch_decode_t<__half, 64>(tmap, p, num_sms, stream)
                       : launch_decode_t<__nv_bfloat16, 64>(tmap, p, num_sms, stream);
        case 128:
            return f16 ? launch_decode_t<__half, 128>(tmap, p, num_sms, stream)
                       : launch_decode_t<__nv_bfloat16, 128>(tmap, p, num_sms, stream);
        case 256:
            return f16 ? launch_decode_t<__half, 256>(tmap, p, num_sms, stream)
                       : launch_decode_t<__nv_bfloat16, 256>(tmap, p, num_sms, stream);
        default:
            return cudaErrorInvalidValue;
    }
}

cudaError_t launch_page_mass(const PageMassParams& p, int n_seq, int max_kv_len, cudaStream_t stream) {
    const int pages = (max_kv_len + p.page_size - 1) / p.page_size;
    if (pages <= 0 || n_seq <= 0) return cudaSuccess;
    return launch_pdl(page_mass_kernel, dim3((pages + 31) / 32, n_seq), dim3(128), 0, stream, p);
}

cudaError_t launch_importance_update(float* scores, float* fresh, int64_t n, float decay, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    return launch_pdl(importance_update_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, scores, fresh,
                      n, decay);
}

cudaError_t launch_importance_add(float* scores, const float* new_scores, int n, float decay, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    return launch_pdl(importance_add_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, scores, new_scores, n, decay);
}

cudaError_t launch_combine(const CombineParams& p, int n_seq, int dtype, cudaStream_t stream) {
    if (n_seq <= 0) return cudaSuccess;
    dim3 grid(p.num_q_heads, n_seq);
    const int slots = p.max_chunks + p.tail_chunks * p.tail_split;
    const bool wide = slots > 64;
    constexpr int kNarrow = 4;
    // A handful of partials per row (batched decode): small CTAs, so that the whole grid is resident at once
    // (c2: 2048 CTAs; -1.5 % on the step against eight warps per CTA, two are slower again).  The cross-GPU tail wants a thread per dim.
    const bool narrow = slots <= 32 && (p.xchg.world == 0 || p.head_dim <= kNarrow * 32);
    if (narrow) {
        if (dtype == DRKV_DTYPE_F16)
            return launch_pdl(combine_kernel<__half, kNarrow>, grid, dim3(kNarrow * 32), 0, stream, p);
        return launch_pdl(combine_kernel<__nv_bfloat16, kNarrow>, grid, dim3(kNarrow * 32), 0, stream, p);
    }
    if (dtype == DRKV_DTYPE_F16)
        return wide ? launch_pdl(combine_kernel<__half, 32>, grid, dim3(32 * 32), 0, stream, p)
                    : launch_pdl(combine_kernel<__half, 8>, grid, dim3(8 * 32), 0, stream, p);
    return wide ? launch_pdl(combine_kernel<__nv_bfloat16, 32>, grid, dim3(32 * 32), 0, stream, p)
                : launch_pdl(combine_kernel<__nv_bfloat16, 8>, grid, dim3(8 * 32), 0, stream, p);
}

cudaError_t launch_combine_external(int n_parts, const float* parts, int num_q_heads, int head_dim, void* out,
                                    int dtype, cudaStream_t stream) {
    if (n_parts <= 0) return cudaSuccess;
    if (dtype == DRKV_DTYPE_F16)
        combine_external_kernel<__half><<<num_q_heads, 128, 0, stream>>>(n_parts, parts, num_q_heads, head_dim, out);
    else
        combine_external_kernel<__nv_bfloat16><<<num_q_heads, 128, 0, stream>>>(n_parts, parts, num_q_heads, head_dim, out);
    return cudaGetLastError();
}

}  // namespace drkv
