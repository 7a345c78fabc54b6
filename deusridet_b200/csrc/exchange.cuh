// exchange.cuh — merge of split-KV partials across GPUs without a library collective: the tail of the
// chunk-merge kernel.
//
// One sequence whose pages are split by key range over `world` GPUs: every rank has an un-normalised
// partial (m, l, o) per query head (the contiguous_split_k layout of
// src/sensus/auditus/asr/asr_ops_attn.cu:29-86) and needs the merged output (asr_ops_attn.cu:88-108).
// The payload is Hq * (D + 2) floats per rank (33 KB at 64 heads): latency, not bandwidth.  The CTA that has
// just merged this rank's chunks of head h pushes (o, m, l) of that head into every rank's exchange area
// with ordinary peer stores over NVLink and merges what the peers have pushed for the same head.  Every value
// travels as one 8-byte store {value, sequence number of the call}: an aligned 8-byte store arrives whole, so a
// word whose second half carries this call's number holds this call's value, and the receiver polls the words
// themselves — bounded — instead of a flag.  No fence and no flag round trip sit between the push and the
// peers' reads: a system-scope fence after the stores (to order them before a flag) costs a round trip over
// NVLink for every head, which was most of the 10 us per layer that two GPUs added to one.  No multicast, no
// kernel of this GPU waits for another kernel of this GPU; a peer that never arrives makes the wait give up after
// its limit and set the engine's error word (the context stays usable).
//
// Area of one rank (device memory of that rank, mapped into every peer by CUDA IPC or given by pointer):
//   words  {float value, uint32 sequence number} [2 parities][world][Hq * (D + 2)]     written by rank r at index r
// Two parities are enough: a rank finishes call s + 1 only after every peer has pushed for s + 1, which a
// peer does only after it has finished merging call s.  The area starts zeroed and sequence numbers start at 1.
#pragma once

#include <cstdint>

#include "kernels.hpp"
#include "kv_common.cuh"
#include "sm100_primitives.cuh"

namespace drkv {

// One scalar 64-bit access each (value in the low half, sequence number in the high half): a naturally aligned
// scalar access is single-copy atomic, which is what makes the number vouch for the value.
__device__ __forceinline__ void st_word_sys(float2* p, float value, uint32_t seq) {
    const unsigned long long w = ((unsigned long long)seq << 32) | __float_as_uint(value);
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void ld_word_sys(const float2* p, float& value, uint32_t& seq) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    value = __uint_as_float((uint32_t)w);
    seq = (uint32_t)(w >> 32);
}

// Called by every thread of the CTA that owns head h.  Thread d < D holds o[d] (un-normalised, on the scale
// of m); m and l are CTA-uniform.  Writes out[h][0..D) in the storage type when any key was visible.
template <typename T>
__device__ void exchange_and_merge(const ExchangeParams& x, int h, int hq, int D, float o_d, float m, float l, void* out,
                                   int* s_ok) {
    const int tid = threadIdx.x;
    const int64_t per_rank = (int64_t)hq * (D + 2);
    // push: word (rank, head, d) of every rank's area; threads 0 and 1 also carry m and l of the head
    for (int r = 0; r < x.world; r++) {
        float2* dst = x.peer_slots[r] + ((int64_t)x.parity * x.world + x.rank) * per_rank;
        if (tid < D) st_word_sys(dst + (int64_t)h * D + tid, o_d, x.seq_no);
        if (tid == 0) st_word_sys(dst + (int64_t)hq * D + h, m, x.seq_no);
        if (tid == 1) st_word_sys(dst + (int64_t)hq * (D + 1) + h, l, x.seq_no);
    }
    if (tid == 0) *s_ok = 1;
    __syncthreads();
    // pull: the same word of every rank's slot in this rank's own area, polled until it carries this call's number
    const float2* slots = x.peer_slots[x.rank] + (int64_t)x.parity * x.world * per_rank;
    const float kLog2e = 1.4426950408889634f;
    float mm = -1.0e20f, ll = 0.f, acc = 0.f;
    bool ok = true;
    if (tid < D) {
        const unsigned long long t0 = global_timer();
        for (int r = 0; r < x.world && ok; r++) {
            const float2* base = slots + r * per_rank;
            float pv = 0.f, pm = 0.f, pl = 0.f;
            uint32_t s0 = 0, s1 = 0, s2 = 0, spins = 0;
            for (;;) {                                  // three words of rank r: o[d], m, l of this head
                if (s0 != x.seq_no) ld_word_sys(base + (int64_t)h * D + tid, pv, s0);
                if (s1 != x.seq_no) ld_word_sys(base + (int64_t)hq * D + h, pm, s1);
                if (s2 != x.seq_no) ld_word_sys(base + (int64_t)hq * (D + 1) + h, pl, s2);
                if (s0 == x.seq_no && s1 == x.seq_no && s2 == x.seq_no) break;
                if ((++spins & 63u) == 0 && global_timer() - t0 > x.wait_ns) {
                    ok = false;
                    break;
                }
            }
            if (!ok) break;
            // merge in rank order with the running-max update of asr_ops_attn.cu:94-107
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
        if (!ok) *s_ok = 0;
    }
    __syncthreads();
    if (!*s_ok) {                                       // all or nothing: no head is written from a partial set of ranks
        if (tid == 0) atomicExch(x.error_word, (int)KERR_WAIT_PEER);
        return;
    }
    if (tid < D && ll > 0.f) reinterpret_cast<T*>(out)[(int64_t)h * D + tid] = Elem<T>::from_f(acc / ll);
}

}  // namespace drkv
