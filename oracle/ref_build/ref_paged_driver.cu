// C entry points over the reference's own paged K/V write, RoPE, decode- and prefill-attention kernels
// (src/machina/paged_attention.h:27-71, src/machina/layer.h apply_rope), its flat <-> paged copies
// (src/memoria/cache_kernels.h:44-74) and its bf16 split-K decode + merge (src/sensus/auditus/asr/asr_ops.h,
// invoke_causal_gqa_decode), compiled from the reference sources where they lie, for recording golden
// outputs on a GPU.  Test infrastructure only.
//
// The batched RoPE and the prefill attention kernels are `static` in the reference's translation unit
// (paged_attention.cu:412, 465) and otherwise reachable only through the whole attention layer with its
// weights, so that file is compiled as part of this one: the kernels are launched below with exactly the
// grids of the reference's own launch sites (paged_attention.cu:604-630).
#include "machina/paged_attention.cu"

#include "machina/layer.h"
#include "machina/model.h"
#include "machina/paged_attention.h"
#include "memoria/cache_kernels.h"
#include "memoria/importance_scorer.h"
#include "sensus/auditus/asr/asr_ops.h"
#include <cstdio>
#include <cstdlib>

namespace deusridet {
// The launchers read their shapes from these process-wide statics (paged_attention.cu:110-114, 276-281).
int ModelConfig::NUM_ATTN_HEADS = 24;
int ModelConfig::NUM_KV_HEADS = 4;
int ModelConfig::HEAD_DIM = 256;
int ModelConfig::NUM_KV_GROUPS = 6;
int ModelConfig::KV_PROJ_DIM = 1024;
int ModelConfig::ATTN_OUT_DIM = 6144;
int ModelConfig::ROTARY_DIM = 64;
float ModelConfig::ROPE_THETA = 1e7f;
float ModelConfig::RMS_EPS = 1e-6f;

// Reached only from the full-layer composites, which this driver never calls.
static void not_linked(const char* what) {
    std::fprintf(stderr, "reference checker: %s is not linked\n", what);
    std::abort();
}
void sigmoid_gate(const __half*, const __half*, __half*, int, cudaStream_t) { not_linked("sigmoid_gate"); }
void linear_forward(const __half*, const Linear&, __half*, int, cudaStream_t) { not_linked("linear_forward"); }
void fp16_gemv(const __half*, const __half*, __half*, int, int, cudaStream_t) { not_linked("fp16_gemv"); }
}  // namespace deusridet

// (no using-directive: the reference's `deusridet::log` namespace would collide with ::log in the headers
// nvcc appends to the translation unit)
using deusridet::ModelConfig;
using deusridet::ImportanceScorer;
using deusridet::apply_rope;
using deusridet::paged_kv_cache_write;
using deusridet::paged_kv_cache_write_batch;
using deusridet::paged_gqa_decode_attention;
using deusridet::paged_rope_batch_kernel;
using deusridet::paged_prefill_attention_kernel;
using deusridet::invoke_extract_kv_from_pages;
using deusridet::invoke_inject_kv_to_pages;
namespace asr_ops = deusridet::asr_ops;

extern "C" {

void refp_set_model(int hq, int hkv, int d, int rot, float theta) {
    ModelConfig::NUM_ATTN_HEADS = hq;
    ModelConfig::NUM_KV_HEADS = hkv;
    ModelConfig::HEAD_DIM = d;
    ModelConfig::NUM_KV_GROUPS = hq / hkv;
    ModelConfig::KV_PROJ_DIM = hkv * d;
    ModelConfig::ATTN_OUT_DIM = hq * d;
    ModelConfig::ROTARY_DIM = rot;
    ModelConfig::ROPE_THETA = theta;
}

void refp_apply_rope(void* q, void* k, const int* d_pos) {
    apply_rope((__half*)q, (__half*)k, ModelConfig::NUM_ATTN_HEADS, ModelConfig::NUM_KV_HEADS, ModelConfig::HEAD_DIM,
               ModelConfig::ROTARY_DIM, d_pos, ModelConfig::ROPE_THETA, 0);
}

void refp_cache_write(const void* k, const void* v, void* pool, const int* table, int layer, const int* d_pos,
                      int max_blocks, int block_size) {
    paged_kv_cache_write((const __half*)k, (const __half*)v, (__half*)pool, table, layer, d_pos, max_blocks,
                         block_size, 0);
}

void refp_cache_write_batch(const void* k, const void* v, void* pool, const int* table, int layer, int pos_start,
                            int m, int max_blocks, int block_size) {
    paged_kv_cache_write_batch((const __half*)k, (const __half*)v, (__half*)pool, table, layer, pos_start, m,
                               max_blocks, block_size, 0);
}

void refp_decode_attention(const void* q, void* pool, const int* table, void* out, int layer, int seq_len,
                           int max_blocks, int block_size, float scale) {
    paged_gqa_decode_attention((const __half*)q, (__half*)pool, table, (__half*)out, layer, seq_len, max_blocks,
                               block_size, scale, 0);
}

int refp_sync(void) { return (int)cudaDeviceSynchronize(); }

// paged_rope_batch_kernel with the grid of its only launch site (paged_attention.cu:604-613): q [m][Hq][D] and
// k [m][Hkv][D] rotated in place at positions pos_start + t.
void refp_rope_batch(void* q, void* k, int pos_start, int m) {
    const int hq = ModelConfig::NUM_ATTN_HEADS, hkv = ModelConfig::NUM_KV_HEADS;
    dim3 grid(hq > hkv ? hq : hkv, m);
    paged_rope_batch_kernel<<<grid, ModelConfig::ROTARY_DIM / 2, 0, 0>>>(
        (__half*)q, (__half*)k, hq, hkv, ModelConfig::HEAD_DIM, ModelConfig::ROTARY_DIM, pos_start, m,
        ModelConfig::ROPE_THETA);
}

// paged_prefill_attention_kernel with the grid of its only launch site (paged_attention.cu:621-630).
void refp_prefill_attention(const void* q, const void* pool, const int* table, void* out, int layer, int pos_start,
                            int m, int max_blocks, int block_size, float scale) {
    dim3 grid(ModelConfig::NUM_ATTN_HEADS, m);
    paged_prefill_attention_kernel<<<grid, ModelConfig::HEAD_DIM, 0, 0>>>(
        (const __half*)q, (const __half*)pool, table, (__half*)out, layer, pos_start, m, max_blocks, block_size,
        ModelConfig::HEAD_DIM, ModelConfig::NUM_KV_HEADS, ModelConfig::NUM_KV_GROUPS, scale);
}

// invoke_extract_kv_from_pages / invoke_inject_kv_to_pages (cache_kernels.cu:147-187); shapes from refp_set_model.
void refp_extract(void* dst, const void* pool, const int* table, int start_token, int num_tokens, int num_layers,
                  int block_size, int max_blocks) {
    invoke_extract_kv_from_pages((__half*)dst, (const __half*)pool, table, start_token, num_tokens, num_layers,
                                 ModelConfig::NUM_KV_HEADS, ModelConfig::HEAD_DIM, block_size, max_blocks, 0);
}
void refp_inject(void* pool, const void* src, const int* table, int start_token, int num_tokens, int num_layers,
                 int block_size, int max_blocks) {
    invoke_inject_kv_to_pages((__half*)pool, (const __half*)src, table, start_token, num_tokens, num_layers,
                              ModelConfig::NUM_KV_HEADS, ModelConfig::HEAD_DIM, block_size, max_blocks, 0);
}

// invoke_causal_gqa_decode (asr_ops_attn.cu:110-132): bf16, contiguous caches [seq][Hkv][D], 128-key partitions,
// head_dim 128 (four warps hard-wired, :59).  workspace: fp32 [Hq * max_parts * D] partial o, then
// [Hq * max_parts] m, then [Hq * max_parts] l; the kernels index partition p of head h at h * num_parts + p,
// num_parts = ceil(seq_len / 128).
void refp_split_k_decode(void* out, const void* q, const void* k_cache, const void* v_cache, int hq, int hkv, int d,
                         int seq_len, float* workspace, int max_parts) {
    asr_ops::invoke_causal_gqa_decode((__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
                                      (const __nv_bfloat16*)v_cache, 1, hq, hkv, d, seq_len, 0, workspace, max_parts);
}

// ImportanceScorer (src/memoria/importance_scorer.h:25-67): `steps` updates of n scores with the host
// arrays new_scores[step][n]; out[step][n] = the mirrored scores after each update.
int refp_importance_run(const float* new_scores, int steps, int n, float decay, float* out) {
    ImportanceScorer scorer;
    if (!scorer.init(n, decay)) return -1;
    float* d_new = nullptr;
    if (cudaMalloc(&d_new, sizeof(float) * n) != cudaSuccess) return -2;
    for (int s = 0; s < steps; s++) {
        cudaMemcpy(d_new, new_scores + (size_t)s * n, sizeof(float) * n, cudaMemcpyHostToDevice);
        cudaDeviceSynchronize();             // the scorer runs on its own stream
        scorer.update(d_new, n);
        scorer.sync_to_host();
        for (int i = 0; i < n; i++) out[(size_t)s * n + i] = scorer.score(i);
    }
    cudaFree(d_new);
    scorer.destroy();
    return (int)cudaGetLastError();
}

}  // extern "C"
