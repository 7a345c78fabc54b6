// attend_decode.cu — split-KV paged GQA decode attention for sm_100a, plus the LSE combine.
//
// Replaces paged_gqa_decode_attention_kernel (src/machina/paged_attention.cu:179-269): one
// CTA per query head walking every key with two block barriers per key.  Here:
//   * grid = (key chunks, KV heads, sequences): the keys of one sequence are split into
//     chunks, each CTA produces an un-normalised partial (m, l, o) per query head of the
//     GQA group, a second small kernel merges the partials (same arithmetic as
//     contiguous_split_k_merge_kernel, src/sensus/auditus/asr/asr_ops_attn.cu:88-108);
//   * every K/V byte is read from HBM once per KV head: the query heads of a group share
//     the tile (the reference re-reads it once per query head);
//   * pages are gathered by TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//     into a 3-stage shared-memory ring guarded by mbarriers, issued by a producer warp
//     from a shared-memory copy of the block-table slice;
//   * QK^T and PV run as m16n8k16 tensor-core tiles with fp32 accumulation: the 4..16
//     query rows of a GQA group are far from a dense contraction (the tensor pipe stays
//     under 10 % busy), they only keep the SM's issue slots free so that the kernel stays
//     HBM-bound; softmax statistics are reduced with warp shuffles in fp32.  P is fed to
//     the PV product as a two-term (hi + lo) split so that it carries ~16 significant bits.
// Holes (table entry < 0) contribute nothing.  All waits are bounded; a wait that gives
// up records a code in the engine's error word and the CTA retires without trapping.
#include "kernels.hpp"
#include "kv_common.cuh"

namespace drkv {

namespace {

constexpr int kConsumerWarps = 4;
constexpr int kDecodeThreads = (kConsumerWarps + 1) * 32;
constexpr int kGroupTokens = 16;                               // keys per warp per stage
constexpr int kStageTokens = kConsumerWarps * kGroupTokens;    // 64
constexpr int kStages = 3;
constexpr int kMaxChunkGroups = 256;                           // chunk_tokens <= 4096
constexpr float kNegBig = -1.0e30f;                            // "no key seen yet" in the log2 domain
constexpr unsigned long long kWaitLimitNs = 2000000000ull;     // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false after kWaitLimitNs without completion.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0 && global_timer() - t0 > kWaitLimitNs) return false;
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

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

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Byte offset inside a 16-row x 128-byte sub-tile written by TMA with 128-byte swizzle:
// the 16-byte chunk index is XORed with the row index modulo 8 (tile base 1024-aligned).
__device__ __forceinline__ uint32_t swz(int row, int chunk16) {
    return (uint32_t)(row * 128 + ((chunk16 ^ (row & 7)) << 4));
}

// Two-term split of a pair of probabilities into the storage type: hi = rn(p), lo = rn(p - hi).
template <typename T>
__device__ __forceinline__ void split_pack(float p0, float p1, uint32_t& hi, uint32_t& lo) {
    hi = Elem<T>::pack2(p0, p1);
    float2 h = Elem<T>::unpack2(hi);
    lo = Elem<T>::pack2(p0 - h.x, p1 - h.y);
}

// HI: the GQA group has more than 8 query heads, so rows 8..15 of the 16-row tile are live.
template <typename T, int D, bool HI>
__global__ void __launch_bounds__(kDecodeThreads, 2)
attend_decode_kernel(const __grid_constant__ CUtensorMap tmap, const DecodeParams p) {
    constexpr int NH = D / 64;                       // 128-byte sub-rows per head row
    constexpr int KSTEPS = D / 16;
    constexpr int NT = D / 8;
    constexpr int TILE_BYTES = NH * 2048;            // 16 keys of K (or V)
    constexpr int STAGE_BYTES = 2 * kConsumerWarps * TILE_BYTES;
    constexpr int OROW = D + 8;                      // padded fp32 row of the merge buffer
    constexpr int NR = HI ? 2 : 1;

    const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int trow = p.rows != nullptr ? p.rows[b] : p.row;
    const int kv_end = p.kv_len != nullptr ? p.kv_len[b] : p.kv_end;
    const int kv_begin = p.kv_begin;
    const int tok_lo = (kv_begin / kGroupTokens) * kGroupTokens + chunk * p.chunk_tokens;
    if (tok_lo >= kv_end) return;                    // uniform over the CTA, before any barrier exists
    const int tok_hi = min(tok_lo + p.chunk_tokens, kv_end);
    const int n_groups = (tok_hi - tok_lo + kGroupTokens - 1) / kGroupTokens;
    const int n_iters = (n_groups + kConsumerWarps - 1) / kConsumerWarps;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_tile = smem + kStages * STAGE_BYTES;
    int* s_pages = reinterpret_cast<int*>(q_tile + TILE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_pages + kMaxChunkGroups);
    __shared__ int s_dead;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kStages);

    if (tid == 0) {
        s_dead = 0;
        for (int s = 0; s < kStages; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, kConsumerWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap) : "memory");
    }
    // Block-table slice of this chunk: one page id per 16-key group.
    for (int gi = tid; gi < n_groups; gi += kDecodeThreads) {
        const int logical = (tok_lo + gi * kGroupTokens) / p.page_size;
        int page = -1;
        if (logical < p.table_stride) page = p.tables[(int64_t)trow * p.table_stride + logical];
        if (page >= p.max_pages) {
            page = -1;
            atomicExch(p.error_word, (int)KERR_BAD_PAGE);
        }
        s_pages[gi] = page;
    }
    // Query rows of the group, swizzled like a K tile; rows beyond the group are zero.
    {
        const T* qb = reinterpret_cast<const T*>(p.q) + ((int64_t)b * p.num_q_heads + (int64_t)kvh * p.group) * D;
        for (int i = tid; i < 16 * (D / 8); i += kDecodeThreads) {
            const int r = i / (D / 8), c = i - r * (D / 8);
            Vec16 v = {{0u, 0u, 0u, 0u}};
            if (r < p.group) v = ldg16(qb + (int64_t)r * D + c * 8);
            *reinterpret_cast<Vec16*>(q_tile + (c >> 3) * 2048 + swz(r, c & 7)) = v;
        }
    }
    __syncthreads();

    float m2[2] = {kNegBig, kNegBig};
    float lsum[2] = {0.f, 0.f};
    float o[NT][2 * NR];
#pragma unroll
    for (int i = 0; i < NT; i++)
#pragma unroll
        for (int j = 0; j < 2 * NR; j++) o[i][j] = 0.f;

    if (warp == kConsumerWarps) {
        // ---------------- producer: one lane issues the TMA gathers ----------------
        if (lane == 0) {
            const int64_t rows_per_plane = (int64_t)p.num_kv_heads * p.page_size;
            for (int it = 0; it < n_iters; it++) {
                const int s = it % kStages, u = it / kStages;
                if (!mbar_wait(bar_empty + 8 * s, (u & 1) ^ 1)) {
                    atomicExch(p.error_word, (int)KERR_WAIT_EMPTY);
                    s_dead = 1;
                    break;
                }
                uint32_t bytes = 0;
#pragma unroll
                for (int g = 0; g < kConsumerWarps; g++) {
                    const int gi = it * kConsumerWarps + g;
                    if (gi < n_groups && s_pages[gi] >= 0) bytes += 2 * TILE_BYTES;
                }
                mbar_arrive_expect_tx(bar_full + 8 * s, bytes);
                const uint32_t stage = smem_u32(smem + s * STAGE_BYTES);
#pragma unroll
                for (int g = 0; g < kConsumerWarps; g++) {
                    const int gi = it * kConsumerWarps + g;
                    if (gi >= n_groups) break;
                    const int page = s_pages[gi];
                    if (page < 0) continue;
                    const int tok = tok_lo + gi * kGroupTokens;
                    const int slot = tok % p.page_size;
                    const int64_t rk = (((int64_t)p.layer * p.max_pages + page) * 2) * rows_per_plane +
                                       (int64_t)kvh * p.page_size + slot;
                    const int64_t rv = rk + rows_per_plane;
#pragma unroll
                    for (int h = 0; h < NH; h++) {
                        tma_load_2d(stage + g * TILE_BYTES + h * 2048, &tmap, h * 64, (int)rk, bar_full + 8 * s);
                        tma_load_2d(stage + (kConsumerWarps + g) * TILE_BYTES + h * 2048, &tmap, h * 64, (int)rv,
                                    bar_full + 8 * s);
                    }
                }
            }
        }
    } else {
        // ---------------- consumers: warp w owns key group w of every stage ----------------
        uint32_t qf[KSTEPS][4];
        {
            const int mi = lane >> 3;
            const int r = (mi & 1) * 8 + (lane & 7);
            const uint32_t qbase = smem_u32(q_tile);
#pragma unroll
            for (int kk = 0; kk < KSTEPS; kk++) {
                const int c = 2 * kk + (mi >> 1);
                ldmatrix_x4(qf[kk], qbase + (c >> 3) * 2048 + swz(r, c & 7));
                if (!HI) { qf[kk][1] = 0u; qf[kk][3] = 0u; }
            }
        }
        const int col = (lane & 3) * 2;
        for (int it = 0; it < n_iters; it++) {
            const int s = it % kStages, u = it / kStages;
            if (!mbar_wait(bar_full + 8 * s, u & 1)) {
                atomicExch(p.error_word, (int)KERR_WAIT_FULL);
                s_dead = 1;
                break;
            }
            const int gi = it * kConsumerWarps + warp;
            if (gi < n_groups && s_pages[gi] >= 0) {
                const int tok0 = tok_lo + gi * kGroupTokens;
                const int v_hi = min(kGroupTokens, kv_end - tok0);   // keys [v_lo, v_hi) of the group are visible
                const int v_lo = max(0, kv_begin - tok0);
                uint8_t* kt = smem + s * STAGE_BYTES + warp * TILE_BYTES;
                uint8_t* vt = kt + kConsumerWarps * TILE_BYTES;
                if (v_hi < kGroupTokens || v_lo > 0) {
                    // Slots outside the visible range may hold anything (stale pages): give the
                    // PV product zeros there so that 0 * garbage cannot produce a NaN.
                    for (int i = lane; i < kGroupTokens * NH * 8; i += 32) {
                        const int r = i / (NH * 8), c = i - r * (NH * 8);
                        if (r >= v_hi || r < v_lo)
                            *reinterpret_cast<Vec16*>(vt + (c >> 3) * 2048 + swz(r, c & 7)) = Vec16{{0u, 0u, 0u, 0u}};
                    }
                    __syncwarp();
                }
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
                        ldmatrix_x4(kb, kbase + (c >> 3) * 2048 + swz(key, c & 7));
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
                    split_pack<T>(p0, p1, phi[r], plo[r]);          // a0 (r=0) / a1 (r=1)
                    split_pack<T>(p8, p9, phi[2 + r], plo[2 + r]);  // a2 / a3
                }
                if (!HI) { phi[1] = phi[3] = plo[1] = plo[3] = 0u; }
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
                        ldmatrix_x4_trans(vb, vbase + (c >> 3) * 2048 + swz(key, c & 7));
                        if (HI) {
                            Mma<T>::run(o[j][0], o[j][1], o[j][2 * NR - 2], o[j][2 * NR - 1], phi[0], phi[1], phi[2], phi[3], vb[0], vb[1]);
                            Mma<T>::run(o[j][0], o[j][1], o[j][2 * NR - 2], o[j][2 * NR - 1], plo[0], plo[1], plo[2], plo[3], vb[0], vb[1]);
                            Mma<T>::run(o[j + 1][0], o[j + 1][1], o[j + 1][2 * NR - 2], o[j + 1][2 * NR - 1], phi[0], phi[1], phi[2], phi[3], vb[2], vb[3]);
                            Mma<T>::run(o[j + 1][0], o[j + 1][1], o[j + 1][2 * NR - 2], o[j + 1][2 * NR - 1], plo[0], plo[1], plo[2], plo[3], vb[2], vb[3]);
                        } else {
                            float z0 = 0.f, z1 = 0.f;   // rows 8..15 are padding: their sums are discarded
                            Mma<T>::run(o[j][0], o[j][1], z0, z1, phi[0], 0u, phi[2], 0u, vb[0], vb[1]);
                            Mma<T>::run(o[j][0], o[j][1], z0, z1, plo[0], 0u, plo[2], 0u, vb[0], vb[1]);
                            Mma<T>::run(o[j + 1][0], o[j + 1][1], z0, z1, phi[0], 0u, phi[2], 0u, vb[2], vb[3]);
                            Mma<T>::run(o[j + 1][0], o[j + 1][1], z0, z1, plo[0], 0u, plo[2], 0u, vb[2], vb[3]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);
        }
        // row sums live split over the 4 lanes of a quad
#pragma unroll
        for (int r = 0; r < NR; r++) {
            lsum[r] += __shfl_xor_sync(0xffffffffu, lsum[r], 1);
            lsum[r] += __shfl_xor_sync(0xffffffffu, lsum[r], 2);
        }
    }

    // ---------------- merge the four warps' partials, write the chunk partial ----------------
    __syncthreads();   // every issued TMA has been waited for by every consumer: the ring is quiescent
    if (s_dead) return;
    float* mo = reinterpret_cast<float*>(smem);                       // [4][16][OROW]
    float* mm = mo + kConsumerWarps * 16 * OROW;                      // [4][16]
    float* ml = mm + kConsumerWarps * 16;                             // [4][16]
    if (warp < kConsumerWarps) {
        const int r0 = lane >> 2;
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const int row = r0 + 8 * r;
            float* dst = mo + (warp * 16 + row) * OROW + (lane & 3) * 2;
#pragma unroll
            for (int i = 0; i < NT; i++)
                *reinterpret_cast<float2*>(dst + 8 * i) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
            if ((lane & 3) == 0) {
                mm[warp * 16 + row] = m2[r];
                ml[warp * 16 + row] = lsum[r];
            }
        }
    }
    __syncthreads();
    const float kLn2 = 0.6931471805599453f;
    for (int i = tid; i < p.group * D; i += kDecodeThreads) {
        const int row = i / D, d = i - row * D;
        float mmax = kNegBig;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; w++) mmax = fmaxf(mmax, mm[w * 16 + row]);
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; w++) {
            const float f = fast_exp2(mm[w * 16 + row] - mmax);
            acc += f * mo[(w * 16 + row) * OROW + d];
            l += f * ml[w * 16 + row];
        }
        const int64_t slot = ((int64_t)b * p.num_q_heads + (int64_t)kvh * p.group + row) * p.max_chunks + chunk;
        const bool empty = !(l > 0.f);
        p.part_o[slot * D + d] = empty ? 0.f : acc;
        if (d == 0) {
            p.part_m[slot] = empty ? -1.0e20f : mmax * kLn2;
            p.part_l[slot] = empty ? 0.f : l;
        }
    }
}

// Merge of chunk partials: m = max m_c, weights exp(m_c - m); out = sum w_c o_c / sum w_c l_c.
// Left unwritten when no key was visible (paged_attention.cu:266-268).
template <typename T>
__global__ void __launch_bounds__(128) combine_kernel(const CombineParams p) {
    const int h = blockIdx.x, b = blockIdx.y;
    const int kv_end = p.kv_len != nullptr ? p.kv_len[b] : p.kv_end;
    const int base = (p.kv_begin / kGroupTokens) * kGroupTokens;
    int nchunks = kv_end > base ? (kv_end - base + p.chunk_tokens - 1) / p.chunk_tokens : 0;
    nchunks = min(nchunks, p.max_chunks);
    const int64_t slot0 = ((int64_t)b * p.num_q_heads + h) * p.max_chunks;
    const int D = p.head_dim;
    const float kLog2e = 1.4426950408889634f;

    float mmax = -1.0e20f;
    for (int c = 0; c < nchunks; c++) mmax = fmaxf(mmax, p.part_m[slot0 + c]);
    float l = 0.f;
    for (int c = 0; c < nchunks; c++)
        l += p.part_l[slot0 + c] * fast_exp2((p.part_m[slot0 + c] - mmax) * kLog2e);

    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f;
        for (int c = 0; c < nchunks; c++)
            acc += p.part_o[(slot0 + c) * D + d] * fast_exp2((p.part_m[slot0 + c] - mmax) * kLog2e);
        if (p.out_partial != nullptr) {
            p.out_partial[(int64_t)h * D + d] = l > 0.f ? acc : 0.f;
        } else if (l > 0.f) {
            reinterpret_cast<T*>(p.out)[((int64_t)b * p.num_q_heads + h) * D + d] = Elem<T>::from_f(acc / l);
        }
    }
    if (p.out_partial != nullptr && threadIdx.x == 0) {
        p.out_partial[(int64_t)p.num_q_heads * D + h] = l > 0.f ? mmax : -1.0e20f;
        p.out_partial[(int64_t)p.num_q_heads * (D + 1) + h] = l > 0.f ? l : 0.f;
    }
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

template <typename T, int D>
cudaError_t launch_decode_t(const CUtensorMap& tmap, const DecodeParams& p, int n_seq, cudaStream_t stream) {
    constexpr int NH = D / 64;
    constexpr size_t smem = 1024 + (size_t)kStages * 2 * kConsumerWarps * NH * 2048 + NH * 2048 +
                            kMaxChunkGroups * sizeof(int) + 2 * kStages * sizeof(uint64_t);
    dim3 grid(p.max_chunks, p.num_kv_heads, n_seq);
    cudaError_t e;
    if (p.group > 8) {
        e = cudaFuncSetAttribute(attend_decode_kernel<T, D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attend_decode_kernel<T, D, true><<<grid, kDecodeThreads, smem, stream>>>(tmap, p);
    } else {
        e = cudaFuncSetAttribute(attend_decode_kernel<T, D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attend_decode_kernel<T, D, false><<<grid, kDecodeThreads, smem, stream>>>(tmap, p);
    }
    return cudaGetLastError();
}

}  // namespace

bool make_pool_tensor_map(CUtensorMap* out, const void* pool, int num_layers, int max_pages, int num_kv_heads,
                          int page_size, int head_dim, const char** err) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            fn == nullptr) {
            if (err) *err = "cuTensorMapEncodeTiled is not available from this driver";
            return false;
        }
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const uint64_t rows = (uint64_t)num_layers * max_pages * 2 * num_kv_heads * page_size;
    if (rows >= (1ull << 31)) {
        if (err) *err = "pool has more than 2^31 head rows: not addressable by one TMA descriptor";
        return false;
    }
    cuuint64_t gdim[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)head_dim * 2};
    cuuint32_t box[2] = {64, 16};
    cuuint32_t estride[2] = {1, 1};
    CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(pool), gdim, gstride, box, estride,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (err) *err = "cuTensorMapEncodeTiled failed";
        return false;
    }
    return true;
}

cudaError_t launch_attend_decode(const CUtensorMap& tmap, const DecodeParams& p, int n_seq, int head_dim, int dtype,
                                 cudaStream_t stream) {
    if (n_seq <= 0 || p.max_chunks <= 0) return cudaSuccess;
    if (p.chunk_tokens % kStageTokens != 0 || p.chunk_tokens / kGroupTokens > kMaxChunkGroups || p.group > 16 ||
        p.page_size % kGroupTokens != 0)
        return cudaErrorInvalidValue;
    const bool f16 = dtype == DRKV_DTYPE_F16;
    switch (head_dim) {
        case 64:
            return f16 ? launch_decode_t<__half, 64>(tmap, p, n_seq, stream)
                       : launch_decode_t<__nv_bfloat16, 64>(tmap, p, n_seq, stream);
        case 128:
            return f16 ? launch_decode_t<__half, 128>(tmap, p, n_seq, stream)
                       : launch_decode_t<__nv_bfloat16, 128>(tmap, p, n_seq, stream);
        case 256:
            return f16 ? launch_decode_t<__half, 256>(tmap, p, n_seq, stream)
                       : launch_decode_t<__nv_bfloat16, 256>(tmap, p, n_seq, stream);
        default:
            return cudaErrorInvalidValue;
    }
}

cudaError_t launch_combine(const CombineParams& p, int n_seq, int dtype, cudaStream_t stream) {
    if (n_seq <= 0) return cudaSuccess;
    dim3 grid(p.num_q_heads, n_seq);
    if (dtype == DRKV_DTYPE_F16)
        combine_kernel<__half><<<grid, 128, 0, stream>>>(p);
    else
        combine_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(p);
    return cudaGetLastError();
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
