// stateless.hpp — helpers shared by the entry points that take raw pointers instead of an engine.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/drkv.h"

namespace drkv {

constexpr size_t kStatelessHeaderBytes = 256;   // [0] queue head, [1] error word, [2] exit count, rest padding

bool stateless_geometry_ok(const drkv_geometry* g);
int stateless_pick_chunk(const drkv_geometry* g, int seq_len, int num_sms);
size_t stateless_scratch_bytes(const drkv_geometry* g, int seq_len, int chunk);
int stateless_decode(const drkv_geometry* g, const void* q, const void* kv_pool, const int32_t* d_block_table,
                     void* out, int layer, int seq_len, int max_pages, float scale, void* scratch, int chunk,
                     cudaStream_t stream);
// Address of the library's built-in decode scratch on the current device (decode_noalloc.cu).
int noalloc_scratch_for_current_device(void** out);
void set_last_error(const char* msg);   // the text drkv_last_error() returns on this thread

}  // namespace drkv
