// attend_prefill.cu — chunked-prefill paged attention on the 5th-generation tensor cores.
//
// Replaces paged_prefill_attention_kernel (src/machina/paged_attention.cu:465-554): one CTA per
// (query head, query token), each re-streaming every earlier key with scalar loads.  Here the
// m tokens of a chunk times the g query heads of a GQA group form the rows of 128-row tiles; a
// CTA owns two such tiles of one KV head (one at head_dim 256) and walks the keys 0 .. pos_start + t in
// blocks of 64, for head dims D = 64, 128 and 256 (the reference's own model is 24/4 heads x 256):
//     S = Q K^T   tcgen05.mma  M128 x N64 x K=D   (A = Q tile, B = K block, both K-major in smem)
//     P = softmax piece (fp32 in registers, one row per thread, read from TMEM with tcgen05.ld)
//     O += P V    tcgen05.mma  M128 x N=D x K64   (A = P in tensor memory, B = V block, MN-major)
// with the S and O accumulators and P in tensor memory (D = 128: 2 x (64 + 128 + 64) = all 512 columns;
// D = 256: 64 + 256 + 64 of one tile, and the tile's Q as the A operand of Q K^T in the remaining 128).
// P is stored as a two-term split (hi + lo, 32 packed columns each); the lo term is multiplied in
// only by CTAs whose rows see at most 1024 keys, where single-term 16-bit weights would cost more
// than the 2e-3 bound on rows dominated by a handful of keys.  One thread per tile
// issues that tile's MMAs (a lone issuing thread is a serial stream of waits, instructions and
// commits: two of them overlap), one warp issues the box loads of a key block (ONE 5-D box per 16 keys
// brings their K and V rows, all dims: the issue rate of copy instructions, not HBM, bounds a producer that
// sends twelve 2-4 KB boxes per block), eight softmax warps (four per tile, one row per thread) do the
// arithmetic, the two warps that share a scheduler taking turns at the exponential unit; the
// K/V block fetched by TMA is used by 256 query rows (128 at head_dim 256).  O stays in
// TMEM across key blocks and is rescaled there only when a row's running maximum has grown by
// more than 2^8 since the scale in use was chosen; the final division by l undoes the stale
// scale.  Same recurrence and mask as the reference: token t sees keys [0, pos_start + t],
// fp32 accumulation, out = o / l, rows without a visible key are left unwritten.
// Block-table holes contribute nothing.  Waits are bounded; a give-up sets the engine's error
// word, and the CTA still frees its tensor memory before it returns.
#include <atomic>

#include "kernels.hpp"
#include "kv_common.cuh"
#include "sm100_primitives.cuh"

namespace drkv {

namespace {

constexpr int kPfBlockN = 64;                  // keys per block
constexpr int kPfSoftmaxWarps = 8;             // 4 per tile
constexpr int kPfProducerWarp = 8;
constexpr int kPfMmaWarp = 9;
constexpr int kPfThreads = 11 * 32;           // 8 softmax warps, TMA producer, one MMA issuer per tile
constexpr int kPfTmemCols = 512;
constexpr int kPfLoTermMaxKeys = 1024;         // CTAs that see at most this many keys add the lo term of P
constexpr int kPfMaxTableSlice = 4096;         // block-table entries staged in shared memory
constexpr float kPfRescaleThreshold = 8.0f;    // log2 units
constexpr float kNegBigPf = -1.0e30f;          // "no key seen yet"

// What depends on the head dim D (64, 128, 256).  Two 128-row tiles per CTA up to D = 128; at 256 the O accumulator
// of one tile takes 256 of the 512 tensor-memory columns and a CTA has one tile.
template <int D>
struct PfShape {
    static constexpr int kTiles = D <= 128 ? 2 : 1;
    static constexpr int kHalves = D / 64;                              // 64-dim (128-byte) runs of a head row
    // At D = 256 the Q tile (64 KB) lives in tensor memory, in the 128 columns that S, O and P of the single tile leave
    // free, as the A operand of Q K^T; shared memory then holds three 64 KB K/V stages instead of two.
    static constexpr bool kQInTmem = D == 256;
    static constexpr int kStages = D <= 128 ? 4 : 3;                    // K/V blocks in flight
    static constexpr int kQBytes = 128 * D * 2;                         // one Q tile: [halves][128 rows][128 B]
    static constexpr int kKBytes = kPfBlockN * D * 2;                   // K (or V) bytes of one block
    // A stage holds a block as eight "octets" of 8 keys, each [K half 0 ..][V half 0 ..] x [8 rows][128 B]: the image
    // of the 5-D box {64 elements, 8 rows, halves, 2 planes, 2 octets} that brings 16 keys.  The 8-row groups of any
    // one (plane, half) are then one octet apart throughout the block, which is what one stride field of an MMA
    // operand descriptor can express.
    static constexpr int kOctetBytes = 2 * kHalves * 1024;
    // shared memory: byte offsets from the 1024-aligned base
    static constexpr int q = 0;                                         // the tiles
    static constexpr int kv = q + (kQInTmem ? 0 : kTiles * kQBytes);    // stages x (K | V)
    static constexpr int pages = kv + kStages * 2 * kKBytes;            // int[kPfMaxTableSlice]
    static constexpr int holes = pages + kPfMaxTableSlice * 4;          // int[kStages]
    static constexpr int bars = holes + 16;                             // uint64[...]
    static constexpr int n_bars = 2 * kStages + 8 + 8 + 2;
    static constexpr int tmem = bars + n_bars * 8;                      // uint32 holder
    static constexpr int total = tmem + 16;
    // barrier indices
    static constexpr int BAR_KV_FULL = 0, BAR_KV_EMPTY = kStages, BAR_S_READY = 2 * kStages, BAR_S_FREE = BAR_S_READY + 2,
                         BAR_P_READY = BAR_S_FREE + 2, BAR_O_READY = BAR_P_READY + 2,
                         BAR_XU = BAR_O_READY + 2,   // [warp of the tile 0..3][tile]: that warp may run its exponentials
                         BAR_Q_READY = BAR_XU + 8;   // kQInTmem: the tile's Q rows are in tensor memory
    // tensor-memory columns: S of the tiles, O of the tiles, P (hi | lo) of the tiles
    static constexpr uint32_t kColS = 0, kColO = 2 * kPfBlockN, kColP = 2 * kPfBlockN + kTiles * D;
    // kQInTmem: dims [0, 128) of Q in columns 64..127 (beside S), dims [128, 256) in 448..511 (behind P)
    static constexpr uint32_t kColQ0 = kPfBlockN, kColQ1 = kColP + 64;
};


template <typename T, int D>
__global__ void __launch_bounds__(kPfThreads, 1)
attend_prefill_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ PrefillParams p) {
    using Sh = PfShape<D>;
    // CTA -> work unit (tile group, KV head, sequence) and, in the split tail of the launch, the piece of its keys
    int unit = blockIdx.x, piece = 0, pieces = 1;
    if (unit >= p.full_units) {
        const int tail = unit - p.full_units;
        pieces = p.tail_pieces;
        unit = p.full_units + tail / pieces;
        piece = tail - (tail / pieces) * pieces;
    }
    const int bx = unit % p.grid_x, by = (unit / p.grid_x) % p.grid_y, bz = unit / (p.grid_x * p.grid_y);
    // sequences with fewer tiles than grid_x leave their extra units idle
    const int p_m = p.m[bz], p_pos_start = p.pos_start[bz], p_row = p.row[bz];
    if (bx * Sh::kTiles * (128 / p.group) >= p_m) return;
    const void* const p_q = p.q[bz];
    void* const p_out = p.out[bz];
    float* const partial = pieces > 1 ? p.partials + (size_t)(blockIdx.x - p.full_units) * Sh::kTiles * 128 * (D + 4) : nullptr;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sbase = smem_u32(smem);
    int* s_pages = reinterpret_cast<int*>(smem + Sh::pages);
    volatile int* s_holes = reinterpret_cast<volatile int*>(smem + Sh::holes);
    const uint32_t bars = sbase + Sh::bars;
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + Sh::tmem);
    __shared__ int s_dead;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = p.group, kvh = by;
    const int tok_per_tile = 128 / g;
    const int rows_used = tok_per_tile * g;
    const int t0 = bx * Sh::kTiles * tok_per_tile;                      // first chunk token of tile A
    const int t_end = min(t0 + Sh::kTiles * tok_per_tile, p_m);         // one past the last token of the CTA
    const bool tile_b_active = Sh::kTiles == 2 && t0 + tok_per_tile < p_m;
    const int kv_hi = p_pos_start + t_end;                              // keys any row of this CTA may see
    const int n_blocks_all = (kv_hi + kPfBlockN - 1) / kPfBlockN;
    // this CTA's share of the key blocks: all of them, or piece `piece` of `pieces` (the last piece gets the diagonal)
    const int jb0 = (int)((long long)n_blocks_all * piece / pieces);
    const int n_blocks = (int)((long long)n_blocks_all * (piece + 1) / pieces) - jb0;
    if (n_blocks == 0) {
        // more pieces than key blocks: nothing to do here; the merge reads l = 0 for every row of this piece
        if (partial != nullptr && threadIdx.x < Sh::kTiles * 128) partial[(size_t)threadIdx.x * (D + 4) + D + 1] = 0.f;
        return;
    }
    const int n_groups = (kv_hi + 15) / 16;
    constexpr int fmt = Elem<T>::kUmmaFormat;
    const bool use_lo = kv_hi <= kPfLoTermMaxKeys;

    if (tid == 0) {
        s_dead = 0;
        for (int s = 0; s < Sh::kStages; s++) {
            mbar_init(bars + 8 * (Sh::BAR_KV_FULL + s), 1);
            mbar_init(bars + 8 * (Sh::BAR_KV_EMPTY + s), tile_b_active ? 2 : 1);   // one commit per issuing thread
        }
        for (int x = 0; x < 2; x++) {
            mbar_init(bars + 8 * (Sh::BAR_S_READY + x), 1);
            mbar_init(bars + 8 * (Sh::BAR_S_FREE + x), 4);       // one arrival per softmax warp of the tile
            mbar_init(bars + 8 * (Sh::BAR_P_READY + x), 4);
            mbar_init(bars + 8 * (Sh::BAR_O_READY + x), 1);
        }
        for (int i = 0; i < 8; i++) mbar_init(bars + 8 * (Sh::BAR_XU + i), 1);
        mbar_init(bars + 8 * Sh::BAR_Q_READY, 4);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap) : "memory");
    }
    if (warp == kPfMmaWarp) tmem_alloc(sbase + Sh::tmem, kPfTmemCols);
    pdl_wait();                                  // Q, the pool and the table may come from the preceding kernel
    pdl_launch_dependents();

    // block-table slice: one page id per 16 keys (staged when it fits)
    const bool pages_staged = n_groups <= kPfMaxTableSlice;
    if (pages_staged) {
        for (int gi = tid; gi < n_groups; gi += kPfThreads) {
            const int logical = (gi * 16) / p.page_size;
            int page = logical < p.table_stride ? p.tables[(int64_t)p_row * p.table_stride + logical] : -1;
            if (page >= p.max_pages) {
                page = -1;
                atomicExch(p.error_word, (int)KERR_BAD_PAGE);
            }
            s_pages[gi] = page;
        }
    }
    // Q tiles: row r = (token t0 + X * tok_per_tile + r / g, query head kvh * g + r % g), written in the
    // K-major 128-byte-swizzled layout the MMA descriptor expects; unused rows are zero.
    if (!Sh::kQInTmem && warp < kPfSoftmaxWarps) {
        const int x = warp >> 2, r = (warp & 3) * 32 + lane;
        const int t = t0 + x * tok_per_tile + r / g;
        const bool valid = r < rows_used && t < p_m;
        const T* src = reinterpret_cast<const T*>(p_q) + ((int64_t)t * p.num_q_heads + kvh * g + r % g) * D;
        uint8_t* dst = smem + Sh::q + x * Sh::kQBytes;
#pragma unroll
        for (int c = 0; c < D / 8; c++) {
            Vec16 v = {{0u, 0u, 0u, 0u}};
            if (valid) v = ldg16(src + 8 * c);
            *reinterpret_cast<Vec16*>(dst + (c >> 3) * (128 * 128) + swz(r, c & 7)) = v;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *s_tmem;

    if (warp == kPfProducerWarp) {
        // ------------------------------- TMA producer -------------------------------
        const int64_t rows_per_plane = (int64_t)p.num_kv_heads * p.page_size;
        for (int j = 0; j < n_blocks; j++) {
            const int s = j % Sh::kStages, u = j / Sh::kStages;
            bool ok = true;
            if (lane == 0) ok = mbar_wait(bars + 8 * (Sh::BAR_KV_EMPTY + s), (u & 1) ^ 1);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0) { atomicExch(p.error_word, (int)KERR_WAIT_EMPTY); s_dead = 1; }
                break;
            }
            uint8_t* stage = smem + Sh::kv + s * 2 * Sh::kKBytes;
            // One box per group of 16 keys: K and V rows, both 64-dim halves (8 KB), issued by lanes 0..3.
            const int my_gi = lane & 3;
            int page = -1;
            {
                const int grp = (jb0 + j) * 4 + my_gi;
                if (grp < n_groups) {
                    if (pages_staged) page = s_pages[grp];
                    else {
                        const int logical = (grp * 16) / p.page_size;
                        page = logical < p.table_stride ? __ldg(p.tables + (int64_t)p_row * p.table_stride + logical) : -1;
                        if (page >= p.max_pages) page = -1;
                    }
                }
            }
            const int holes = (int)(__ballot_sync(0xffffffffu, page < 0) & 0xfu);      // lanes 0..3 hold groups 0..3
            const uint32_t bytes = (uint32_t)(4 - __popc(holes)) * (2u * Sh::kKBytes / 4u);
            if (holes) {
                // nothing will be loaded there: give the MMAs zeros instead of stale shared memory
                for (int g4 = 0; g4 < 4; g4++) {
                    if (!((holes >> g4) & 1)) continue;
                    for (int i = lane; i < 2 * Sh::kOctetBytes / 16; i += 32)
                        *reinterpret_cast<Vec16*>(stage + g4 * 2 * Sh::kOctetBytes + 16 * i) = Vec16{{0u, 0u, 0u, 0u}};
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            __syncwarp();
            if (lane == 0) {
                s_holes[s] = holes;
                mbar_arrive_expect_tx(bars + 8 * (Sh::BAR_KV_FULL + s), bytes);
            }
            __syncwarp();
            if (lane < 4 && page >= 0) {
                const int tok = ((jb0 + j) * 4 + lane) * 16;
                // K-plane row of the group's first key, in octets of 8 rows (a multiple of 8: pages hold multiples of 16)
                const int64_t row = (((int64_t)p.layer * p.max_pages + page) * 2) * rows_per_plane +
                                    (int64_t)kvh * p.page_size + (tok % p.page_size);
                tma_load_5d(smem_u32(stage) + lane * 2 * Sh::kOctetBytes, &tmap, 0, 0, 0, 0, (int)(row >> 3),
                            bars + 8 * (Sh::BAR_KV_FULL + s));
            }
        }
    } else if (warp >= kPfMmaWarp) {
        // ------------------------------- MMA issuers -------------------------------
        // One thread per tile: warp kPfMmaWarp + x issues S = Q K^T and O += P V of tile x.  Each thread is
        // a serial stream of waits, a handful of instructions and commits; two of them keep the tensor pipe
        // fed while one waits for its softmax warps.
        const int x = warp - kPfMmaWarp;
        if (lane == 0 && (x == 0 || tile_b_active)) {
            constexpr uint32_t idesc_qk = umma_idesc_f16(fmt, 128, kPfBlockN, 0, 0);
            constexpr uint32_t idesc_pv = umma_idesc_f16(fmt, 128, D, 0, 1);
            bool dead = false;
            // Descriptors differ only in the start-address field of their low word (address >> 4 in bits
            // [0,14)): one add per MMA.  Between two MMAs the issuing thread executes nothing else: a run-time
            // predicate or branch per instruction costs this lone thread 20-80 cycles, more than the 32-64
            // cycles of tensor work an instruction carries.
            constexpr uint32_t kDescHiQ = (1024u >> 4) | (1u << 14) | (2u << 29);    // Q: 8-row groups 1 KB apart, version 1, 128-byte swizzle
            constexpr uint32_t kDescHi = ((uint32_t)Sh::kOctetBytes >> 4) | (1u << 14) | (2u << 29);   // K, V: 8-row groups one octet apart
            constexpr uint32_t kLboK = (16u >> 4) << 16;                            // K-major operands
            // V, MN-major: the next 64-dim run (the other half) is 1 KB on; 16 keys = two octets
            constexpr uint32_t kLboV = (1024u >> 4) << 16;
            constexpr uint32_t v_step = (2u * Sh::kOctetBytes) >> 4;                   // from one group of 16 keys to the next
            auto mk = [](uint32_t lo, uint32_t hi) -> uint64_t { return ((uint64_t)hi << 32) | lo; };
            const uint32_t qa = ((((sbase + Sh::q) & 0x3FFFFu) >> 4) | kLboK) + x * (Sh::kQBytes >> 4);
            const uint32_t kv_lo0 = ((sbase + Sh::kv) & 0x3FFFFu) >> 4;
            const uint32_t d_s = tmem_base + Sh::kColS + x * kPfBlockN;
            const uint32_t d_o = tmem_base + Sh::kColO + x * D;
            const uint32_t pa = tmem_base + Sh::kColP + x * 64;           // hi at +0, lo at +32; 8 columns per 16 keys
            auto issue_qk = [&](int s) {
                const uint32_t kb = (kv_lo0 + s * (2 * Sh::kKBytes >> 4)) | kLboK;
#pragma unroll
                for (int kk = 0; kk < D / 16; kk++) {
                    const uint32_t off_q = ((kk >> 2) * (128 * 128) + (kk & 3) * 32) >> 4;
                    const uint32_t off_k = ((kk >> 2) * 1024 + (kk & 3) * 32) >> 4;     // half, then 16 dims = 32 bytes
                    if (Sh::kQInTmem)       // A = Q in tensor memory: 16 dims are 8 packed columns
                        umma_f16_ts(d_s, tmem_base + (kk < 8 ? Sh::kColQ0 : Sh::kColQ1) + (kk & 7) * 8, mk(kb + off_k, kDescHi), idesc_qk, kk > 0);
                    else
                        umma_f16(d_s, mk(qa + off_q, kDescHiQ), mk(kb + off_k, kDescHi), idesc_qk, kk > 0);
                }
                umma_commit(bars + 8 * (Sh::BAR_S_READY + x));
            };
            auto issue_pv = [&](int s, bool first_block) {
                const uint32_t vb = (kv_lo0 + s * (2 * Sh::kKBytes >> 4) + ((Sh::kHalves * 1024u) >> 4)) | kLboV;   // V half 0 of octet 0
                const uint32_t acc0 = first_block ? 0u : 1u;
                if (!use_lo) {
                    umma_f16_ts(d_o, pa, mk(vb, kDescHi), idesc_pv, acc0);
                    umma_f16_ts(d_o, pa + 8, mk(vb + 1 * v_step, kDescHi), idesc_pv, 1u);
                    umma_f16_ts(d_o, pa + 16, mk(vb + 2 * v_step, kDescHi), idesc_pv, 1u);
                    umma_f16_ts(d_o, pa + 24, mk(vb + 3 * v_step, kDescHi), idesc_pv, 1u);
                } else {
#pragma unroll
                    for (int kk = 0; kk < kPfBlockN / 16; kk++) {
                        const uint64_t vdesc = mk(vb + kk * v_step, kDescHi);
                        umma_f16_ts(d_o, pa + kk * 8, vdesc, idesc_pv, kk == 0 ? acc0 : 1u);
                        umma_f16_ts(d_o, pa + 32 + kk * 8, vdesc, idesc_pv, 1u);
                    }
                }
                umma_commit(bars + 8 * (Sh::BAR_O_READY + x));
            };
            // S(0)
            if (!mbar_wait(bars + 8 * (Sh::BAR_KV_FULL + 0), 0)) dead = true;
            if (Sh::kQInTmem && !dead && !mbar_wait(bars + 8 * Sh::BAR_Q_READY, 0)) dead = true;
            if (!dead) {
                tcgen05_fence_after();
                issue_qk(0);
            }
            for (int j = 0; j < n_blocks && !dead; j++) {
                const int s = j % Sh::kStages;
                // S(j+1): as soon as the softmax warps have pulled S(j) out of tensor memory
                if (j + 1 < n_blocks) {
                    const int s1 = (j + 1) % Sh::kStages;
                    if (!mbar_wait(bars + 8 * (Sh::BAR_KV_FULL + s1), ((j + 1) / Sh::kStages) & 1)) { dead = true; break; }
                    if (!mbar_wait(bars + 8 * (Sh::BAR_S_FREE + x), j & 1)) { dead = true; break; }
                    tcgen05_fence_after();
                    issue_qk(s1);
                }
                // O += P(j) V(j)
                if (!mbar_wait(bars + 8 * (Sh::BAR_P_READY + x), j & 1)) { dead = true; break; }
                tcgen05_fence_after();
                issue_pv(s, j == 0);
                umma_commit(bars + 8 * (Sh::BAR_KV_EMPTY + s));        // this tile's MMAs that read the stage are done
            }
            if (dead) {
                atomicExch(p.error_word, (int)KERR_WAIT_FULL);
                s_dead = 1;
            }
        }
    } else {
        // ------------------------------- softmax / correction / epilogue -------------------------------
        const int x = warp >> 2;                                        // tile 0 / 1
        const int r = (warp & 3) * 32 + lane;                           // tile row = TMEM lane
        if (x == 0 || tile_b_active) {
            const int t = t0 + x * tok_per_tile + r / g;
            const bool valid = r < rows_used && t < p_m;
            const int limit = valid ? p_pos_start + t + 1 : 0;          // keys [0, limit) are visible to this row
            const int tile_min_limit = p_pos_start + t0 + x * tok_per_tile + 1;
            const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
            const uint32_t t_s = tmem_base + lane_base + Sh::kColS + x * kPfBlockN;
            const uint32_t t_o = tmem_base + lane_base + Sh::kColO + x * D;
            const uint32_t t_p = tmem_base + lane_base + Sh::kColP + x * 64;
            float m_used = kNegBigPf, l = 0.f;
            bool dead = false;
            const bool xu_turns = tile_b_active;
            if (Sh::kQInTmem) {
                // this thread's Q row into tensor memory, 64 dims (32 packed columns) at a time: column c holds dims
                // 2c and 2c + 1, as the MMA reads an A operand there; rows past the tile's tokens are zero
                const T* src = reinterpret_cast<const T*>(p_q) + ((int64_t)t * p.num_q_heads + kvh * g + r % g) * D;
#pragma unroll 1
                for (int piece = 0; piece < D / 64; piece++) {
                    uint32_t qw[32];
#pragma unroll
                    for (int c = 0; c < 8; c++) {
                        Vec16 v = {{0u, 0u, 0u, 0u}};
                        if (valid) v = ldg16(src + piece * 64 + 8 * c);
#pragma unroll
                        for (int e = 0; e < 4; e++) qw[4 * c + e] = v.w[e];
                    }
                    tmem_st32(tmem_base + lane_base + (piece < 2 ? Sh::kColQ0 : Sh::kColQ1) + (piece & 1) * 32, qw);
                }
                tmem_wait_st();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bars + 8 * Sh::BAR_Q_READY);
            }
            for (int j = 0; j < n_blocks; j++) {
                if (!mbar_wait(bars + 8 * (Sh::BAR_S_READY + x), j & 1)) { dead = true; break; }
                tcgen05_fence_after();
                float sv[2][32];
                tmem_ld32(t_s, sv[0]);
                tmem_ld32(t_s + 32, sv[1]);
                tmem_wait_ld();
                tcgen05_fence_before();
                __syncwarp();                                           // S(j+1) may overwrite the columns now
                if (lane == 0) mbar_arrive(bars + 8 * (Sh::BAR_S_FREE + x));
                const int key0 = (jb0 + j) * kPfBlockN;
                const int holes = s_holes[j % Sh::kStages];
                // Blocks left of the diagonal with all pages present need no mask: that is almost all of them.
                const bool unmasked = (key0 + kPfBlockN <= tile_min_limit) && holes == 0;
                if (!unmasked) {
#pragma unroll
                    for (int h = 0; h < 2; h++)
#pragma unroll
                        for (int c = 0; c < 32; c++) {
                            const int k = h * 32 + c;
                            if (key0 + k >= limit || ((holes >> (k >> 4)) & 1)) sv[h][c] = -INFINITY;
                        }
                }
                // row maximum of the raw scores: eight independent chains instead of one 64 deep
                // four independent chains of three-input maxima: 32 instructions for 64 scores
                float mx4[4];
#pragma unroll
                for (int i = 0; i < 4; i++) mx4[i] = fmaxf(sv[0][2 * i], sv[0][2 * i + 1]);
#pragma unroll
                for (int c = 8; c < 32; c += 2) mx4[(c >> 1) & 3] = fmax3(mx4[(c >> 1) & 3], sv[0][c], sv[0][c + 1]);
#pragma unroll
                for (int c = 0; c < 32; c += 2) mx4[(c >> 1) & 3] = fmax3(mx4[(c >> 1) & 3], sv[1][c], sv[1][c + 1]);
                float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                mx *= p.scale_log2;                                      // scale > 0: max commutes with it
                // Keep the scale in use unless the row maximum outgrew it by more than 2^8.
                float factor = 1.f;
                bool need = false;
                if (mx > m_used + kPfRescaleThreshold) {
                    factor = fast_exp2(m_used - mx);
                    l *= factor;
                    m_used = mx;
                    need = j > 0;
                }
                // The exponential unit delivers 16 results per clock and SM, which makes a block's exponentials as
                // long as its MMAs; warp k of tile 0 and warp k of tile 1 share a scheduler and its quarter of that
                // unit.  Left alone, both run their exponentials at the same time, each at half rate, and then leave
                // the unit idle together while they load, take maxima and store.  They take turns instead: a warp
                // starts its exponentials when its partner has finished the partner's, so that one's loads, maxima
                // and stores run under the other's exponentials.
                if (xu_turns) {
                    if (!mbar_wait(bars + 8 * (Sh::BAR_XU + 2 * (warp & 3) + x), (uint32_t)((j & 1) ^ (x ^ 1)))) { dead = true; break; }
                }
                // p = 2^(s * scale_log2 - m): one FMA and one EX2 per score
                const float neg_m = -m_used;
                float sum4[4] = {0.f, 0.f, 0.f, 0.f};                    // independent partial sums
                const unsigned long long scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
                const unsigned long long negm2 = pack_f32x2(neg_m, neg_m);
                unsigned long long sum2[4] = {0ull, 0ull, 0ull, 0ull};    // packed pairs of partial sums (+0.f, +0.f)
                uint32_t phi[32], plo[32];
                if (!use_lo) {
                    // two scores per multiply-add and per add (packed fp32 pairs), one exponential each, one
                    // conversion per pair
#pragma unroll
                    for (int h = 0; h < 2; h++) {
#pragma unroll
                        for (int c = 0; c < 32; c += 2) {
                            float a0, a1;
                            unpack_f32x2(fma_f32x2(pack_f32x2(sv[h][c], sv[h][c + 1]), scale2, negm2), a0, a1);
                            const float p0 = fast_exp2_ordered(a0), p1 = fast_exp2_ordered(a1);
                            sum2[(c >> 1) & 3] = add_f32x2(sum2[(c >> 1) & 3], pack_f32x2(p0, p1));
                            phi[h * 16 + (c >> 1)] = Elem<T>::pack2(p0, p1);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        float s0, s1;
                        unpack_f32x2(sum2[i], s0, s1);
                        sum4[i] = s0 + s1;
                    }
                } else {
#pragma unroll
                    for (int h = 0; h < 2; h++)
#pragma unroll
                        for (int c = 0; c < 32; c += 2) {
                            const float p0 = fast_exp2_ordered(fmaf(sv[h][c], p.scale_log2, neg_m));
                            const float p1 = fast_exp2_ordered(fmaf(sv[h][c + 1], p.scale_log2, neg_m));
                            sum4[(c >> 1) & 3] += p0 + p1;
                            const uint32_t hi = Elem<T>::pack2(p0, p1);
                            const float2 hf = Elem<T>::unpack2(hi);
                            phi[h * 16 + (c >> 1)] = hi;
                            plo[h * 16 + (c >> 1)] = Elem<T>::pack2(p0 - hf.x, p1 - hf.y);
                        }
                }
                if (xu_turns) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bars + 8 * (Sh::BAR_XU + 2 * (warp & 3) + (x ^ 1)));   // the partner's turn
                }
                l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
                if (j > 0) {
                    // PV(j-1) must have landed before O is touched or P is overwritten
                    if (!mbar_wait(bars + 8 * (Sh::BAR_O_READY + x), (j - 1) & 1)) { dead = true; break; }
                    tcgen05_fence_after();
                    if (__any_sync(0xffffffffu, need)) {
#pragma unroll 1
                        for (int c0 = 0; c0 < D; c0 += 32) {
                            float ov[32];
                            tmem_ld32(t_o + c0, ov);
                            tmem_wait_ld();
#pragma unroll
                            for (int c = 0; c < 32; c++) ov[c] *= factor;
                            tmem_st32(t_o + c0, ov);
                        }
                        tmem_wait_st();
                    }
                }
                // P(j) into tensor memory: 64 keys = 32 packed columns (hi), then the lo term
                tmem_st32(t_p, phi);
                if (use_lo) tmem_st32(t_p + 32, plo);
                tmem_wait_st();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bars + 8 * (Sh::BAR_P_READY + x));
            }
            if (!dead && !mbar_wait(bars + 8 * (Sh::BAR_O_READY + x), (n_blocks - 1) & 1)) dead = true;
            if (dead) {
                atomicExch(p.error_word, (int)KERR_WAIT_FULL);
                s_dead = 1;
            } else if (partial != nullptr) {
                // a piece of a split unit: the row's un-normalised O, its scale in use (log2 domain) and its sum
                tcgen05_fence_after();
                float* prow = partial + ((size_t)x * 128 + r) * (D + 4);
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    float ov[32];
                    tmem_ld32(t_o + c0, ov);
                    tmem_wait_ld();
                    if (valid && l > 0.f) {
#pragma unroll
                        for (int c = 0; c < 32; c += 4)
                            *reinterpret_cast<float4*>(prow + c0 + c) = make_float4(ov[c], ov[c + 1], ov[c + 2], ov[c + 3]);
                    }
                }
                prow[D] = m_used;
                prow[D + 1] = valid ? l : 0.f;
            } else {
                tcgen05_fence_after();
                const float inv = l > 0.f ? 1.f / l : 0.f;
                T* orow = reinterpret_cast<T*>(p_out) + ((int64_t)t * p.num_q_heads + kvh * g + r % g) * D;
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    float ov[32];
                    tmem_ld32(t_o + c0, ov);
                    tmem_wait_ld();
                    if (valid && l > 0.f) {
#pragma unroll
                        for (int c = 0; c < 32; c += 8) {
                            Vec16 v;
#pragma unroll
                            for (int e = 0; e < 4; e++) v.w[e] = Elem<T>::pack2(ov[c + 2 * e] * inv, ov[c + 2 * e + 1] * inv);
                            stg16(orow + c0 + c, v);
                        }
                    }
                }
            }
        }
    }
    // ------------------------------- teardown -------------------------------
    tcgen05_fence_before();
    __syncthreads();
    if (warp == kPfMmaWarp) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kPfTmemCols);
    }
}

}  // namespace


namespace {

// Merge of the pieces of the split tail: one warp per query row of a split unit.  out = sum_p o_p 2^(m_p - M) /
// sum_p l_p 2^(m_p - M) with M the largest scale among the pieces that saw a key; a row no piece saw a key for is
// left unwritten, as in the unsplit kernel.
template <typename T, int D>
__global__ void __launch_bounds__(128) prefill_merge_kernel(const __grid_constant__ PrefillParams p) {
    using Sh = PfShape<D>;
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int row_id = blockIdx.x * 4 + (threadIdx.x >> 5);            // (tail unit, tile, row)
    const int r = row_id % 128, x = (row_id / 128) % Sh::kTiles, tail_unit = row_id / (128 * Sh::kTiles);
    const int unit = p.full_units + tail_unit;
    if (unit >= p.n_units) return;
    const int bx = unit % p.grid_x, by = (unit / p.grid_x) % p.grid_y, bz = unit / (p.grid_x * p.grid_y);
    const int g = p.group, tok_per_tile = 128 / g;
    const int t = (bx * Sh::kTiles + x) * tok_per_tile + r / g;
    if (r >= tok_per_tile * g || t >= p.m[bz]) return;
    const float* base = p.partials + ((size_t)tail_unit * p.tail_pieces * Sh::kTiles + x) * 128 * (D + 4) + (size_t)r * (D + 4);
    const size_t piece_stride = (size_t)Sh::kTiles * 128 * (D + 4);
    float M = -INFINITY;
    for (int q = 0; q < p.tail_pieces; q++) {
        const float* pr = base + q * piece_stride;
        if (pr[D + 1] > 0.f) M = fmaxf(M, pr[D]);
    }
    if (M == -INFINITY) return;
    constexpr int PER = D / 32;                                        // dims per lane
    float acc[PER], L = 0.f;
#pragma unroll
    for (int i = 0; i < PER; i++) acc[i] = 0.f;
    for (int q = 0; q < p.tail_pieces; q++) {
        const float* pr = base + q * piece_stride;
        const float lq = pr[D + 1];
        if (!(lq > 0.f)) continue;
        const float w = fast_exp2(pr[D] - M);
        L += lq * w;
#pragma unroll
        for (int i = 0; i < PER; i++) acc[i] += pr[lane * PER + i] * w;
    }
    T* orow = reinterpret_cast<T*>(p.out[bz]) + ((int64_t)t * p.num_q_heads + by * g + r % g) * D + lane * PER;
    const float inv = 1.f / L;
#pragma unroll
    for (int i = 0; i < PER; i += 2) *reinterpret_cast<uint32_t*>(orow + i) = Elem<T>::pack2(acc[i] * inv, acc[i + 1] * inv);
}

}  // namespace

namespace {

// Pieces per unit of the tail (1: no split): the choice that makes the tail's CTAs fill whole waves of `sms` best,
// with a small charge per piece for its start-up, its partial and the merge.
int pick_tail_pieces(int tail_units, int sms) {
    if (tail_units <= 0) return 1;
    int best = 1;
    double best_cost = 1e30;
    for (int pc = 1; pc <= 8; pc++) {
        const int ctas = tail_units * pc;
        const double cost = (double)((ctas + sms - 1) / sms) / pc + (pc > 1 ? 0.03 + 0.01 * pc : 0.0);
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = pc;
        }
    }
    return best;
}

template <typename T, int D>
cudaError_t launch_prefill_d(const CUtensorMap& tmap, PrefillParams p, int max_m, int num_sms, float* scratch,
                             size_t scratch_bytes, cudaStream_t stream) {
    using Sh = PfShape<D>;
    constexpr size_t smem = 1024 + Sh::total;
    const int tok_per_cta = Sh::kTiles * (128 / p.group);
    p.grid_x = (max_m + tok_per_cta - 1) / tok_per_cta;
    p.grid_y = p.num_kv_heads;
    p.n_units = p.grid_x * p.grid_y * p.n_seq;
    // whole waves of one CTA per unit, then the remainder cut into pieces along the keys
    const int sms = num_sms > 0 ? num_sms : 1;
    int tail_units = p.n_units % sms;
    p.tail_pieces = scratch != nullptr ? pick_tail_pieces(tail_units, sms) : 1;
    const size_t per_cta = (size_t)Sh::kTiles * 128 * (D + 4) * sizeof(float);
    while (p.tail_pieces > 1 && (size_t)tail_units * p.tail_pieces * per_cta > scratch_bytes) p.tail_pieces--;
    if (p.tail_pieces <= 1) {
        p.tail_pieces = 1;
        tail_units = 0;
    }
    p.full_units = p.n_units - tail_units;
    p.partials = scratch;
    const int ctas = p.full_units + tail_units * p.tail_pieces;
    static std::atomic<bool> configured[64];      // per instantiation and device; any thread may be the first caller
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        e = cudaFuncSetAttribute(attend_prefill_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    e = launch_pdl(attend_prefill_kernel<T, D>, dim3(ctas), dim3(kPfThreads), smem, stream, tmap, p);
    if (e != cudaSuccess || tail_units == 0) return e;
    const int rows = tail_units * Sh::kTiles * 128;
    return launch_pdl(prefill_merge_kernel<T, D>, dim3((rows + 3) / 4), dim3(128), 0, stream, p);
}

}  // namespace

cudaError_t launch_attend_prefill(const CUtensorMap& tmap, const PrefillParams& p, int head_dim, int dtype, int num_sms,
                                  float* scratch, size_t scratch_bytes, cudaStream_t stream) {
    if (p.n_seq <= 0) return cudaSuccess;
    if (p.group < 1 || p.group > 16 || p.page_size % 16 != 0) return cudaErrorInvalidValue;
    int max_m = 0;
    for (int i = 0; i < p.n_seq; i++) max_m = p.m[i] > max_m ? p.m[i] : max_m;
    if (max_m <= 0 || p.n_seq > kMaxPrefillSeqs) return max_m <= 0 ? cudaSuccess : cudaErrorInvalidValue;
    const bool f16 = dtype == DRKV_DTYPE_F16;
#define DRKV_PF_CASE(DIM)                                                                                             \
    case DIM:                                                                                                          \
        return f16 ? launch_prefill_d<__half, DIM>(tmap, p, max_m, num_sms, scratch, scratch_bytes, stream)            \
                   : launch_prefill_d<__nv_bfloat16, DIM>(tmap, p, max_m, num_sms, scratch, scratch_bytes, stream);
    switch (head_dim) {
        DRKV_PF_CASE(64)
        DRKV_PF_CASE(128)
        DRKV_PF_CASE(256)
        default:
            return cudaErrorInvalidValue;
    }
#undef DRKV_PF_CASE
}

}  // namespace drkv
