// decode_noalloc.cu — decode attention for callers that cannot obtain device memory.
//
// The split-KV decode kernel needs a few hundred kilobytes of fp32 partials between its two
// launches.  The engine allocates that at creation and drkv_k_decode_attention borrows it from
// the caller, but some callers can do neither: a plug-in running inside a server that has
// already handed every byte of HBM to its own pool allocator, a decode thread with a latency
// budget that cannot absorb the device-wide synchronisation cudaMalloc/cudaFree imply, or a
// process that filled the GPU with KV pages on purpose and has nothing left to lend.  For
// them the library carries one fixed scratch area of its own, linked into the module as a
// __device__ array, and this file is the only place that touches it.
#include <mutex>

#include "../../include/drkv.h"
#include "kernels.hpp"
#include "stateless.hpp"

using namespace drkv;

namespace {

// Lives in the module image: every GPU that loads libdrkv.so holds these bytes until the
// process exits, whether or not the entry point below is ever called.
static __device__ __align__(256) unsigned char g_builtin_scratch[DRKV_NOALLOC_SCRATCH_BYTES];

// g_builtin_scratch is a host-side handle in host code, not a device address: the address the
// kernels need comes from cudaGetSymbolAddress, once per device, with that device current.
std::mutex g_setup_mu;
void* g_scratch_ptr[64] = {};

int builtin_scratch(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        set_last_error("decode_attention_noalloc: no usable CUDA device is current");
        return DRKV_ERR_NO_DEVICE;
    }
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t ce = cudaGetSymbolAddress(&p, g_builtin_scratch);
        if (ce != cudaSuccess || p == nullptr) {
            set_last_error("decode_attention_noalloc: cudaGetSymbolAddress on the built-in scratch failed");
            return DRKV_ERR_CUDA;
        }
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return DRKV_OK;
}

}  // namespace

namespace drkv {
int noalloc_scratch_for_current_device(void** out) { return builtin_scratch(out); }
}  // namespace drkv

extern "C" int drkv_k_decode_attention_noalloc(const drkv_geometry* g, const void* q, const void* kv_pool,
                                               const int32_t* d_block_table, void* out, int layer, int seq_len,
                                               int max_pages, float scale, void* stream) {
    if (!stateless_geometry_ok(g) || !q || !kv_pool || !d_block_table || !out || layer < 0 ||
        layer >= g->num_layers || max_pages <= 0 || seq_len < 0) {
        set_last_error("decode_attention_noalloc: bad argument");
        return DRKV_ERR_INVALID;
    }
    if (seq_len == 0) return DRKV_OK;   // no key: the output stays untouched, as in the other entry points
    void* scratch = nullptr;
    int rc = builtin_scratch(&scratch);
    if (rc != DRKV_OK) return rc;
    int dev = 0, num_sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    // Same chunking rule as the caller-scratch entry point; a longer sequence gets larger chunks
    // (fewer partials) until it fits, and is refused once even 4096-key chunks do not.
    int chunk = stateless_pick_chunk(g, seq_len, num_sms);
    while (stateless_scratch_bytes(g, seq_len, chunk) > DRKV_NOALLOC_SCRATCH_BYTES && chunk < 4096)
        chunk = chunk * 2 < 4096 ? chunk * 2 : 4096;
    if (stateless_scratch_bytes(g, seq_len, chunk) > DRKV_NOALLOC_SCRATCH_BYTES) {
        set_last_error("decode_attention_noalloc: seq_len x heads needs more than the built-in scratch "
                       "(DRKV_NOALLOC_SCRATCH_BYTES); use drkv_k_decode_attention with caller memory");
        return DRKV_ERR_CAPACITY;
    }
    // stateless_decode() zeroes the header (queue head, error word) on the stream before the
    // launches; every partial the merge reads is rewritten by this call, so nothing else of the
    // previous call's contents matters.
    return stateless_decode(g, q, kv_pool, d_block_table, out, layer, seq_len, max_pages, scale, scratch, chunk,
                            (cudaStream_t)stream);
}
