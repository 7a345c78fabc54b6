// C entry points over the reference's own paged K/V write, RoPE and decode-attention launchers
// (src/machina/paged_attention.h:27-71, src/machina/layer.h apply_rope), compiled from the reference
// sources where they lie, for recording golden outputs on a GPU.  Test infrastructure only.
#include "machina/layer.h"
#include "machina/model.h"
#include "machina/paged_attention.h"
#include "memoria/importance_scorer.h"
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

using namespace deusridet;

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
