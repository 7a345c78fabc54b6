// exchange.cuh — merge of split-KV partials across GPUs without a library collective: the tail of the
// chunk-merge kernel.
//
// One sequence whose pages are split by key range over `world` GPUs: every rank has an un-normalised
// partial (m, l, o) per query head (the contiguous_split_k layout of
// src/sensus/auditus/asr/asr_ops_attn.cu:29-86) and needs the merged output (asr_ops_attn.cu:88-108).
// The payload is Hq * (D + 2) floats per rank (33 KB at 64 heads): latency, not bandwidth.  The CTA that has
// just merged this rank's chunks of head h pushes (o, m, l) of that head into every rank's exchange area
// with ordinary peer stores over NVLink, raises a per-(rank, head) flag, waits — bounded — for the peers'
// flags of the same head and merges.  No multicast, no kernel of this GPU waits for another kernel of this
// GPU; a peer that never arrives makes the wait give up after its limit and set the engine's error word
// (the context stays usable).
//
// Area of one rank (device memory of that rank, mapped into every peer by CUDA IPC):
//   slots  float [2 parities][world][Hq * (D + 2)]     written by rank r at index r
//   flags  uint32 [world][Hq]                           sequence number of the last push of (r, head)
// Two parities are enough: a rank finishes call s + 1 only after every peer has pushed for s + 1, which a
// peer does only after it has finished merging call s.
#pragma once

#include <cstdint>

#include "kernels.hpp"
#include "kv_common.cuh"
#include "sm100_primitives.cuh"

namespace drkv {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Called by every thread of the CTA that owns head h.  Thread d < D holds o[d] (un-normalised, on the scale
// of m); m and l are CTA-uniform.  Writes out[h][0..D) in the storage type when any key was visible.
template <typename T>
__device__ void exchange_and_merge(const ExchangeParams& x, int h, int hq, int D, float o_d, float m, float l, void* out,
                                   int* s_ok) {
    const int tid = threadIdx.x;
    const int64_t per_rank = (int64_t)hq * (D + 2);
    for (int r = 0; r < x.world; r++) {
        float* dst = x.peer_slots[r] + ((int64_t)x.parity * x.world + x.rank) * per_rank;
        if (tid < D) dst[(int64_t)h * D + tid] = o_d;
        if (tid == 0) {
            dst[(int64_t)hq * D + h] = m;
            dst[(int64_t)hq * (D + 1) + h] = l;
        }
    }
    if (tid == 0) *s_ok = 1;
    __syncthreads();
    if (tid < x.world) {
        // the barrier made the CTA's stores visible to this thread; its system-scope fence orders them, for
        // every observer, before the flag
        __threadfence_system();
        st_release_sys(x.peer_flags[tid] + (int64_t)x.rank * hq + h, x.seq_no);
        const uint32_t* f = x.peer_flags[x.rank] + (int64_t)tid * hq + h;
        const unsigned long long t0 = global_timer();
        uint32_t spins = 0;
        // sequence numbers only grow; the signed difference copes with wrap-around
        while ((int32_t)(ld_acquire_sys(f) - x.seq_no) < 0) {
            if ((++spins & 63u) == 0 && global_timer() - t0 > x.wait_ns) {
                *s_ok = 0;
                break;
            }
        }
    }
    __syncthreads();
    if (!*s_ok) {
        if (tid == 0) atomicExch(x.error_word, (int)KERR_WAIT_PEER);
        return;
    }
    // merge in rank order with the running-max update of asr_ops_attn.cu:94-107
    if (tid < D) {
        const float* slots = x.peer_slots[x.rank] + (int64_t)x.parity * x.world * per_rank;
        const float kLog2e = 1.4426950408889634f;
        float mm = -1.0e20f, ll = 0.f, acc = 0.f;
        for (int r = 0; r < x.world; r++) {
            const float* base = slots + r * per_rank;
            const float pm = __ldcg(base + (int64_t)hq * D + h), pl = __ldcg(base + (int64_t)hq * (D + 1) + h);
            const float pv = __ldcg(base + (int64_t)h * D + tid);
            if (pm > mm) {
                const float f = fast_exp2((mm - pm) * kLog2e);
                acc = acc * f + pv;
                ll = ll * f + pl;
                mm = pm;
            } else {
                const float f = fast_exp2((pm - mm) * kLog2e);
                acc += pv * f;
                ll += pl * f;
            }
        }
        if (ll > 0.f) reinterpret_cast<T*>(out)[(int64_t)h * D + tid] = Elem<T>::from_f(acc / ll);
    }
}

}  // namespace drkv
