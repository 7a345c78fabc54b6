// kernels.hpp — parameter blocks and launchers of the paged-KV kernels.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kv_common.cuh"

namespace drkv {

struct AppendParams {
    PoolLayout layout;
    void* pool;
    const int32_t* tables;   // [rows][table_stride]
    int table_stride;
    const int32_t* rows;     // per token table row, or nullptr: all tokens use `row`
    const int32_t* pos;      // per token position (rows != nullptr) or one device int (rows == nullptr)
    int row, pos_start;      // used when rows == nullptr (pos_start only if pos == nullptr)
    int layer;
    int rotary_dim;          // 0 = plain copy
    int wait_first;          // 1: read nothing before the programmatic-launch wait (positions and tables may come
                             // from the caller's kernel directly in front: the raw-pointer entry points)
    const float* inv_freq;   // [rotary_dim / 2] device
    const void* k_src;
    const void* v_src;
};

struct CowParams {
    PoolLayout layout;
    void* pool;
    int src_page, dst_page, n_slots;
};

// Flat [layer][K|V][token][kv_head][dim] <-> paged copy of tokens [start_token, start_token + num_tokens).
struct FlatCopyParams {
    PoolLayout layout;
    void* pool;
    void* flat;
    const int32_t* table;     // one sequence's row
    int table_stride;
    int start_token, num_tokens, num_layers;
};

// Split-KV decode attention.  One CTA handles (chunk of keys, KV head, sequence).
struct DecodeParams {
    const int32_t* tables;
    int table_stride;
    const int32_t* rows;      // [n_seq] table row per batch entry, nullptr = `row` for all
    const int32_t* kv_len;    // [n_seq] keys visible, nullptr = `kv_end` + batch index * `kv_step`
    int row, kv_begin, kv_end;
    int kv_step;              // kv_len == nullptr: entry b sees kv_end + b * kv_step keys (1: the tokens of a prefill chunk)
    const void* q;            // [n_seq][Hq][D]
    float* part_o;            // [n_seq][Hq][max_chunks][D]   un-normalised
    float* part_m;            // [n_seq][Hq][max_chunks]      natural-log domain
    float* part_l;            // [n_seq][Hq][max_chunks]
    int layer, max_pages, num_q_heads, num_kv_heads, group, page_size;
    int chunk_tokens, max_chunks;
    int tail_chunks, tail_split;   // last tail_chunks chunks of a sequence go as tail_split pieces each (0: off)
    int n_seq;
    int few_keys_possible;    // 0: the host knows that every row of the launch sees more than 1 024 keys; else 1
    // shared-prefix plan (all null / 0 without one): family block k covers chunks [0, fb_chunks[k]) of table
    // row fb_row[k] for the batch entries fb_members[16 k + i] (-1 = none); sequence b starts at chunk
    // seq_first_chunk[b].  rows_per_item: query rows a family block fills (members * group), else 0.
    int n_fb, rows_per_item;
    const int32_t* fb_row;
    const int32_t* fb_chunks;
    const int32_t* fb_members;
    const int32_t* seq_first_chunk;
    // tile masses for the importance scorer (null = off): tile_lse[(((seq * Hkv + kv_head) * max_tiles + tile) * group + head_in_group) * 4 + quarter]
    float* tile_lse;
    int max_tiles;
    int total_items;          // upper bound n_seq * num_kv_heads * max_chunks (sizes the grid)
    int* work_counter;        // device int, 0 at launch; the last warp to leave rewinds it
    int* exit_count;          // device int, 0 at launch: warps that have left
    float scale_log2;         // scale * log2(e)
    int* error_word;
    int wait_first;           // 1: read nothing before the programmatic-launch wait (raw-pointer entry points, whose
                              // block table may be written by the caller's kernel directly in front)
    // Fused append (all null / 0: off): the new token of batch entry b, at position kv_len[b] - 1, comes from
    // k_new / v_new [n_seq][Hkv][D] instead of the pool.  The work item that reaches that position rotates K,
    // puts both rows into its shared-memory tile and writes them to the pool page (head dims 64 and 128).
    const void* k_new;
    const void* v_new;
    void* pool;
    const float* inv_freq;    // [rotary_dim / 2]
    int rotary_dim;
};

// Chunked-prefill attention: for each of n_seq sequences, chunk tokens [0, m) at positions pos_start + t.
constexpr int kMaxPrefillSeqs = 16;   // sequences one launch can take (grid.z)
struct PrefillParams {
    const int32_t* tables;
    int table_stride;
    int n_seq;
    int row[kMaxPrefillSeqs], pos_start[kMaxPrefillSeqs], m[kMaxPrefillSeqs];
    const void* q[kMaxPrefillSeqs];   // [m][Hq][D]
    void* out[kMaxPrefillSeqs];       // [m][Hq][D]
    int layer, max_pages, num_q_heads, num_kv_heads, group, page_size;
    float scale_log2;
    int* error_word;
    // Work units are (tile group of tokens, KV head, sequence), numbered x fastest.  The launch has one CTA per unit
    // for the first full_units of them; each of the remaining ones (what would be a partly filled last wave of CTAs)
    // is cut along the keys into tail_pieces CTAs that write un-normalised partials, merged by a second kernel.
    int grid_x, grid_y, n_units, full_units, tail_pieces;
    float* partials;          // [(unit - full_units) * tail_pieces + piece][tile][128 rows][head_dim + 4]: o, m (log2), l, 2 unused (rows stay 16-byte aligned)
};

// Cross-GPU merge of one sequence's split-KV partials by peer stores, the tail of the merge kernel
// (exchange.cuh); world == 0: off.
constexpr int kMaxExchangeRanks = 16;
struct ExchangeParams {
    float2* peer_slots[kMaxExchangeRanks];      // every rank's area of {value, sequence number} words, as mapped into this process
    int world, rank, parity;
    uint32_t seq_no;
    unsigned long long wait_ns;                 // how long a rank waits for a peer's flag before it gives up
    int* error_word;
};

struct CombineParams {
    const float* part_o;
    const float* part_m;
    const float* part_l;
    const int32_t* kv_len;    // [n_seq] or nullptr
    int kv_begin, kv_end, kv_step;        // as in DecodeParams
    int num_q_heads, head_dim, chunk_tokens, max_chunks;
    int tail_chunks, tail_split;          // as in DecodeParams
    const int32_t* seq_first_chunk;       // shared-prefix plan's first own chunk per sequence, or nullptr
    void* out;                // storage type [n_seq][Hq][D] (normalised) ...
    float* out_partial;       // ... or fp32 partial [Hq*D | Hq m | Hq l] when non-null
    float* lse2_out;          // optional [n_seq][Hq]: log2 of the softmax denominator on the kernel's score scale
    ExchangeParams xchg;      // with xchg.world > 0 (one sequence): exchange with the peers, then write `out`
};

// Importance scorer: per-page attention mass from the decode kernel's tile values.
struct PageMassParams {
    const float* tile_lse;    // [(((seq * Hkv + kv_head) * max_tiles + tile) * group + head_in_group) * 4 + quarter]
    const float* lse2;        // [n_seq][Hq]
    const int32_t* rows;      // [n_seq] table rows
    const int32_t* kv_len;    // [n_seq]
    float* fresh;             // [max_seqs][table_stride] accumulator of new scores
    int num_q_heads, num_kv_heads, max_tiles, page_size, table_stride;
};
cudaError_t launch_page_mass(const PageMassParams& p, int n_seq, int max_kv_len, cudaStream_t stream);
cudaError_t launch_importance_update(float* scores, float* fresh, int64_t n, float decay, cudaStream_t stream);
cudaError_t launch_importance_add(float* scores, const float* new_scores, int n, float decay, cudaStream_t stream);


cudaError_t launch_append_rope(const AppendParams& p, int n_tokens, int dtype, cudaStream_t stream);
cudaError_t launch_cow_copy(const CowParams& p, int num_layers, cudaStream_t stream);
cudaError_t launch_flat_paged_copy(const FlatCopyParams& p, bool to_flat, int num_sms, cudaStream_t stream);

// The decode kernel's descriptor: 4-D view whose one box is 16 key rows x head_dim x (K, V).
bool make_pool_slot_tensor_map(CUtensorMap* out, const void* pool, int num_layers, int max_pages,
                               int num_kv_heads, int page_size, int head_dim, const char** err);

cudaError_t launch_attend_decode(const CUtensorMap& tmap, const DecodeParams& p, int num_sms, int head_dim,
                                 int dtype, cudaStream_t stream);
constexpr int kMaxDecodeSeqs = 2048;   // sequences one decode-attention launch can take
// warps of one decode CTA, each with its own queue of items; family_blocks: the pass has shared-prefix family blocks
int decode_warps_per_cta(int head_dim, bool family_blocks = false);
// The prefill kernel's descriptor (head_dim 128): 5-D view whose one box is 16 key rows x both 64-dim halves x (K, V),
// landing in 8-row groups of 128 bytes ordered [octet of 8 keys][plane][half].
bool make_pool_kv16_tensor_map(CUtensorMap* out, const void* pool, int num_layers, int max_pages,
                               int num_kv_heads, int page_size, int head_dim, const char** err);
// scratch / scratch_bytes: device memory for the partials of a split tail (none: no split); num_sms sizes the waves
cudaError_t launch_attend_prefill(const CUtensorMap& tmap, const PrefillParams& p, int head_dim, int dtype, int num_sms,
                                  float* scratch, size_t scratch_bytes, cudaStream_t stream);
cudaError_t launch_combine(const CombineParams& p, int n_seq, int dtype, cudaStream_t stream);

// Merges partials that already sit in the external layout (drkv_attend_partial).
cudaError_t launch_combine_external(int n_parts, const float* parts, int num_q_heads, int head_dim,
                                    void* out, int dtype, cudaStream_t stream);

}  // namespace drkv
