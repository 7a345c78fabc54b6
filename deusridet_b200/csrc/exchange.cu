// exchange.cu — merge of split-KV partials across GPUs without a library collective.
//
// One sequence whose pages are split by key range over `world` GPUs: every rank has an un-normalised
// partial (m, l, o) per query head (the contiguous_split_k layout of
// src/sensus/auditus/asr/asr_ops_attn.cu:29-86) and needs the merged output (asr_ops_attn.cu:88-108).
// The payload is Hq * (D + 2) floats per rank (33 KB at 64 heads): latency, not bandwidth.  Instead of an
// all-gather followed by a merge kernel, ONE kernel per rank pushes its partial into every rank's exchange
// area with ordinary peer stores over NVLink, raises a per-(rank, head) flag, waits — bounded — for the
// peers' flags of the same head and merges.  No multicast, no kernel of this GPU waits for another kernel
// of this GPU; a peer that never arrives makes the wait give up after its limit and set the engine's
// error word (the context stays usable).
//
// Area of one rank (device memory of that rank, mapped into every peer by CUDA IPC):
//   slots  float [2 parities][world][Hq * (D + 2)]     written by rank r at index r
//   flags  uint32 [world][Hq]                           sequence number of the last push of (r, head)
// Two parities are enough: a rank finishes call s + 1 only after every peer has pushed for s + 1, which a
// peer does only after it has finished merging call s.
#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/drkv.h"
#include "kernels.hpp"
#include "kv_common.cuh"
#include "sm100_primitives.cuh"

namespace drkv {

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <typename T>
__global__ void __launch_bounds__(128) exchange_merge_kernel(const ExchangeParams p) {
    const int h = blockIdx.x, tid = threadIdx.x;
    const int D = p.head_dim, hq = p.num_q_heads;
    const int64_t per_rank = (int64_t)hq * (D + 2);
    __shared__ int s_ok;
    pdl_wait();                                          // the local partial comes from the preceding kernel
    pdl_launch_dependents();
    // ---- push this rank's (o, m, l) of head h into slot `rank` of every rank's area ----
    const float* mine = p.local_partial;
    for (int r = 0; r < p.world; r++) {
        float* dst = p.peer_slots[r] + ((int64_t)p.parity * p.world + p.rank) * per_rank;
        for (int d = tid; d < D; d += blockDim.x) dst[(int64_t)h * D + d] = mine[(int64_t)h * D + d];
        if (tid == 0) {
            dst[(int64_t)hq * D + h] = mine[(int64_t)hq * D + h];
            dst[(int64_t)hq * (D + 1) + h] = mine[(int64_t)hq * (D + 1) + h];
        }
    }
    __threadfence_system();                              // the data before the flags, system-wide
    __syncthreads();
    if (tid < p.world) st_release_sys(p.peer_flags[tid] + (int64_t)p.rank * hq + h, p.seq_no);
    // ---- wait for every rank's flag of this head (bounded) ----
    if (tid == 0) s_ok = 1;
    __syncthreads();
    if (tid < p.world) {
        const uint32_t* f = p.peer_flags[p.rank] + (int64_t)tid * hq + h;
        const unsigned long long t0 = global_timer();
        uint32_t spins = 0;
        // sequence numbers only grow; the signed difference copes with wrap-around
        while ((int32_t)(ld_acquire_sys(f) - p.seq_no) < 0) {
            if ((++spins & 63u) == 0 && global_timer() - t0 > kWaitLimitNs) {
                s_ok = 0;
                break;
            }
        }
    }
    __syncthreads();
    if (!s_ok) {
        if (tid == 0) atomicExch(p.error_word, (int)KERR_WAIT_PEER);
        return;
    }
    // ---- merge in rank order with the running-max update of asr_ops_attn.cu:94-107 ----
    const float* slots = p.peer_slots[p.rank] + (int64_t)p.parity * p.world * per_rank;
    const float kLog2e = 1.4426950408889634f;
    for (int d = tid; d < D; d += blockDim.x) {
        float m = -1.0e20f, l = 0.f, acc = 0.f;
        for (int r = 0; r < p.world; r++) {
            const float* base = slots + r * per_rank;
            const float pm = __ldcg(base + (int64_t)hq * D + h), pl = __ldcg(base + (int64_t)hq * (D + 1) + h);
            const float pv = __ldcg(base + (int64_t)h * D + d);
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
        if (l > 0.f) reinterpret_cast<T*>(p.out)[(int64_t)h * D + d] = Elem<T>::from_f(acc / l);
    }
}

}  // namespace

cudaError_t launch_exchange_merge(const ExchangeParams& p, int dtype, cudaStream_t stream) {
    if (p.world < 1 || p.world > kMaxExchangeRanks || p.num_q_heads <= 0) return cudaErrorInvalidValue;
    if (dtype == DRKV_DTYPE_F16)
        return launch_pdl(exchange_merge_kernel<__half>, dim3(p.num_q_heads), dim3(128), 0, stream, p);
    return launch_pdl(exchange_merge_kernel<__nv_bfloat16>, dim3(p.num_q_heads), dim3(128), 0, stream, p);
}

}  // namespace drkv
