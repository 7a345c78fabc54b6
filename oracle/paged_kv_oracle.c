/*
 * paged_kv_oracle.c — CPU restatement of the DeusRidet reference's paged KV-cache arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA kernels and the timed
 * CPU baseline; nothing in the product links, imports or falls back to it.
 *
 * Each function follows the reference lines it cites (paths relative to the reference tree).  The
 * reference ships no test, golden vector or fixture for this path.  Pinning, by running the reference
 * itself:
 *   - pool addressing, page ids, tables, eviction order: against the reference's compiled Memoria
 *     objects (oracle/ref_build/, tests/test_bookkeeping_vs_reference.py);
 *   - fp16 K/V write (single and batched), RoPE and decode attention: against outputs of the reference's
 *     own CUDA kernels recorded on a B200 (tests/golden/paged_attention_reference.npz, written by
 *     tests/golden/make_paged_attention_golden.py; tests/test_oracle_vs_reference_kernels.py) - writes
 *     bit-exact, RoPE within the error of the reference's fast-math intrinsics, attention within 2e-3;
 *   - bf16, batches of sequences, holes, prefill attention (its reference kernel is `static` and only
 *     reachable through the full layer), split-KV partials and their merge, extract/inject: "parity
 *     unpinned" - they restate the cited kernels with the same building blocks as the pinned functions,
 *     but no reference execution pins them.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).  Contraction
 * is off so that every rounding below is the one written.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define OKV_F16 0
#define OKV_BF16 1

typedef struct okv_geom {
    int32_t num_layers, num_q_heads, num_kv_heads, head_dim, page_size, dtype, rotary_dim;
    float rope_theta;
} okv_geom;

/* ---------------------------------------------------------------------------------------
 * storage types: IEEE binary16 and bfloat16, round-to-nearest-even (what __float2half and
 * __float2bfloat16 do in the reference kernels)
 * ------------------------------------------------------------------------------------- */
static inline float bits_f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float bf16_to_f(uint16_t b) { return bits_f((uint32_t)b << 16); }
static inline uint16_t f_to_bf16(float f) {
    uint32_t u = f_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;          /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static inline float f16_to_f(uint16_t h) {
    uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    if (e == 0) {
        if (m == 0) return bits_f(s);
        float v = (float)m * 5.9604644775390625e-08f;             /* m * 2^-24 */
        return s ? -v : v;
    }
    if (e == 31) return bits_f(s | 0x7f800000u | (m << 13));
    return bits_f(s | ((e + 112u) << 23) | (m << 13));
}
static inline uint16_t f_to_f16(float f) {
    uint32_t u = f_bits(f), s = (u >> 16) & 0x8000u, a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(s | 0x7fffu);
    if (a >= 0x477ff000u) return (uint16_t)(s | 0x7c00u);         /* >= 65520 rounds to inf */
    if (a < 0x33000001u) return (uint16_t)s;                      /* <= 2^-25 rounds to 0 */
    if (a < 0x38800000u) {                                        /* subnormal half */
        uint32_t m = (a & 0x7fffffu) | 0x800000u;
        int shift = 126 - (int)(a >> 23);                         /* 14..24 */
        uint32_t r = m >> shift, rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (r & 1u))) r++;
        return (uint16_t)(s | r);
    }
    uint32_t r = a - 0x38000000u;                                 /* rebias 127 -> 15 */
    r += 0xfffu + ((r >> 13) & 1u);
    return (uint16_t)(s | (r >> 13));
}
static inline float st_to_f(uint16_t x, int dtype) { return dtype == OKV_F16 ? f16_to_f(x) : bf16_to_f(x); }
static inline uint16_t f_to_st(float f, int dtype) { return dtype == OKV_F16 ? f_to_f16(f) : f_to_bf16(f); }

void okv_to_float(const uint16_t* src, float* dst, int64_t n, int dtype) {
    for (int64_t i = 0; i < n; i++) dst[i] = st_to_f(src[i], dtype);
}
void okv_from_float(const float* src, uint16_t* dst, int64_t n, int dtype) {
    for (int64_t i = 0; i < n; i++) dst[i] = f_to_st(src[i], dtype);
}

/* ---------------------------------------------------------------------------------------
 * pool addressing — src/machina/paged_attention.cu:36-64, src/memoria/block_pool.cpp:81-95
 * ------------------------------------------------------------------------------------- */
static inline int64_t pool_row(const okv_geom* g, int max_pages, int layer, int page, int kv, int head, int slot) {
    int64_t kv_plane = (int64_t)g->num_kv_heads * g->page_size * g->head_dim;
    int64_t block_stride = 2 * kv_plane;
    int64_t layer_stride = (int64_t)max_pages * block_stride;
    return (int64_t)layer * layer_stride + (int64_t)page * block_stride + (int64_t)kv * kv_plane +
           (int64_t)head * g->page_size * g->head_dim + (int64_t)slot * g->head_dim;
}
int64_t okv_pool_elem(const okv_geom* g, int max_pages, int layer, int page, int kv, int head, int slot) {
    return pool_row(g, max_pages, layer, page, kv, head, slot);
}

/* ---------------------------------------------------------------------------------------
 * RoPE — src/machina/layer_attention.cu:32-69, src/machina/paged_attention.cu:412-451
 *   freq_i = 1 / theta^(2i/rot) (fp32), angle = pos * freq_i (fp32), pairs (i, i + rot/2),
 *   x0' = x0 cos - x1 sin, x1' = x1 cos + x0 sin, rounded to the storage type.
 * The reference takes cosf/sinf of the fp32 angle on the device; their bits depend on the
 * math library and on --use_fast_math.  The contract here: sin/cos are the fp32 rounding of
 * an fp64 evaluation made only of IEEE add/mul/fma (below), and the rotation is
 *   x0' = fma(x0, c, -(x1*s)),  x1' = fma(x1, c, x0*s)   in fp32.
 * ------------------------------------------------------------------------------------- */
void okv_inv_freq(float theta, int rot, float* out) {
    for (int i = 0; i < rot / 2; i++) out[i] = 1.0f / powf(theta, (2.0f * (float)i) / (float)rot);
}

void okv_sincos(float angle, float* s, float* c) {
    const double two_over_pi = 0.63661977236758134308;
    const double magic = 6755399441055744.0;           /* 1.5 * 2^52 */
    const double pio2_hi = 1.57079632673412561417;
    const double pio2_lo = 6.07710050650619224932e-11;
    double x = (double)angle;
    double t = fma(x, two_over_pi, magic);
    uint64_t tb;
    memcpy(&tb, &t, 8);
    int k = (int)(uint32_t)tb;                          /* low word = nearest integer */
    double kd = t + (-magic);
    double r = fma(-kd, pio2_hi, x);
    r = fma(-kd, pio2_lo, r);
    double z = r * r;
    double ps = 1.0 / 355687428096000.0;
    ps = fma(ps, z, -1.0 / 1307674368000.0);
    ps = fma(ps, z, 1.0 / 6227020800.0);
    ps = fma(ps, z, -1.0 / 39916800.0);
    ps = fma(ps, z, 1.0 / 362880.0);
    ps = fma(ps, z, -1.0 / 5040.0);
    ps = fma(ps, z, 1.0 / 120.0);
    ps = fma(ps, z, -1.0 / 6.0);
    double rz = r * z;
    double sn = fma(rz, ps, r);
    double pc = -1.0 / 6402373705728000.0;
    pc = fma(pc, z, 1.0 / 20922789888000.0);
    pc = fma(pc, z, -1.0 / 87178291200.0);
    pc = fma(pc, z, 1.0 / 479001600.0);
    pc = fma(pc, z, -1.0 / 3628800.0);
    pc = fma(pc, z, 1.0 / 40320.0);
    pc = fma(pc, z, -1.0 / 720.0);
    pc = fma(pc, z, 1.0 / 24.0);
    pc = fma(pc, z, -0.5);
    double cs = fma(z, pc, 1.0);
    float fs = (float)sn, fc = (float)cs;
    switch (k & 3) {
        case 0: *s = fs; *c = fc; break;
        case 1: *s = fc; *c = -fs; break;
        case 2: *s = -fs; *c = -fc; break;
        default: *s = -fc; *c = fs; break;
    }
}

/* Rotates one head row [head_dim] in place. */
static void rope_row(uint16_t* row, const okv_geom* g, int pos, const float* inv_freq) {
    int half = g->rotary_dim / 2;
    for (int i = 0; i < half; i++) {
        float angle = (float)pos * inv_freq[i];
        float s, c;
        okv_sincos(angle, &s, &c);
        float x0 = st_to_f(row[i], g->dtype), x1 = st_to_f(row[i + half], g->dtype);
        float y0 = fmaf(x0, c, -(x1 * s));
        float y1 = fmaf(x1, c, x0 * s);
        row[i] = f_to_st(y0, g->dtype);
        row[i + half] = f_to_st(y1, g->dtype);
    }
}
void okv_rope_rows(uint16_t* rows, int n_rows, const okv_geom* g, int pos) {
    float inv_freq[256];
    okv_inv_freq(g->rope_theta, g->rotary_dim, inv_freq);
    for (int r = 0; r < n_rows; r++) rope_row(rows + (int64_t)r * g->head_dim, g, pos, inv_freq);
}

/* ---------------------------------------------------------------------------------------
 * append — src/machina/paged_attention.cu:73-102 (one token) and :123-153 (m tokens):
 * logical = pos / P, slot = pos % P, page = table[logical], rows copied verbatim.  The
 * reference rotates K before this call (paged_attention.cu:353-361, 604-619); rope != 0
 * does the same here first.  A table entry < 0 writes nothing.
 * ------------------------------------------------------------------------------------- */
void okv_append(const okv_geom* g, uint16_t* pool, int max_pages, const int32_t* table, int layer, int pos_start,
                int m, const uint16_t* k_src, const uint16_t* v_src, int rope) {
    int D = g->head_dim, H = g->num_kv_heads, P = g->page_size;
    float inv_freq[256];
    if (rope && g->rotary_dim > 0) okv_inv_freq(g->rope_theta, g->rotary_dim, inv_freq);
    uint16_t krow[256];
    for (int t = 0; t < m; t++) {
        int pos = pos_start + t;
        int page = table[pos / P], slot = pos % P;
        if (page < 0) continue;
        for (int h = 0; h < H; h++) {
            memcpy(krow, k_src + ((int64_t)t * H + h) * D, (size_t)D * 2);
            if (rope && g->rotary_dim > 0) rope_row(krow, g, pos, inv_freq);
            memcpy(pool + pool_row(g, max_pages, layer, page, 0, h, slot), krow, (size_t)D * 2);
            memcpy(pool + pool_row(g, max_pages, layer, page, 1, h, slot), v_src + ((int64_t)t * H + h) * D,
                   (size_t)D * 2);
        }
    }
}

/* ---------------------------------------------------------------------------------------
 * attention core — src/machina/paged_attention.cu:179-269: for one query head, keys visited
 * in logical order; s = scale * sum_d q_d k_d (fp32); m' = max(m, s); alpha = exp(m - m');
 * p = exp(s - m'); o = o*alpha + v*p; l = l*alpha + p; start m = -FLT_MAX, l = 0, o = 0.
 * Keys [kv_begin, kv_end); table entries < 0 are skipped.  Returns the un-normalised state.
 * ------------------------------------------------------------------------------------- */
static void attend_head(const okv_geom* g, const uint16_t* pool, int max_pages, const int32_t* table, int layer,
                        int kv_head, int kv_begin, int kv_end, const uint16_t* q_row, float scale, float* o,
                        float* m_out, float* l_out) {
    int D = g->head_dim, P = g->page_size, dt = g->dtype;
    float q[256];
    for (int d = 0; d < D; d++) q[d] = st_to_f(q_row[d], dt);
    float m = -3.402823466e+38f, l = 0.0f;
    for (int d = 0; d < D; d++) o[d] = 0.0f;
    float kf[256], vf[256];
    for (int t = kv_begin; t < kv_end; t++) {
        int page = table[t / P];
        if (page < 0) continue;
        const uint16_t* k = pool + pool_row(g, max_pages, layer, page, 0, kv_head, t % P);
        const uint16_t* v = pool + pool_row(g, max_pages, layer, page, 1, kv_head, t % P);
        for (int d = 0; d < D; d++) kf[d] = st_to_f(k[d], dt);
        /* The reference sums one product per lane with an xor-shuffle tree and then the warp
         * sums in order (paged_attention.cu:236-249); eight strided partial sums joined by a
         * tree keep that shape and let the compiler use vector registers. */
        float a8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int d = 0; d < D; d += 8)
            for (int j = 0; j < 8; j++) a8[j] += q[d + j] * kf[d + j];
        float dot = ((a8[0] + a8[4]) + (a8[2] + a8[6])) + ((a8[1] + a8[5]) + (a8[3] + a8[7]));
        float s = dot * scale;
        float m_new = s > m ? s : m;
        float alpha = expf(m - m_new);
        float p = expf(s - m_new);
        for (int d = 0; d < D; d++) vf[d] = st_to_f(v[d], dt);
        for (int d = 0; d < D; d++) o[d] = o[d] * alpha + vf[d] * p;
        l = l * alpha + p;
        m = m_new;
    }
    *m_out = m;
    *l_out = l;
}

/* Decode attention for a batch: q/out [n_seq][Hq][D] storage type; sequence i uses table row
 * rows[i] (table_stride entries per row) and sees kv_len[i] keys.  Output rows with l == 0
 * are left unwritten (paged_attention.cu:266-268). */
void okv_attend_decode(const okv_geom* g, const uint16_t* pool, int max_pages, const int32_t* tables,
                       int table_stride, const int32_t* rows, const int32_t* kv_len, int n_seq, int layer,
                       const uint16_t* q, uint16_t* out, float scale) {
    int Hq = g->num_q_heads, D = g->head_dim, group = g->num_q_heads / g->num_kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < n_seq; b++) {
        for (int h = 0; h < Hq; h++) {
            float o[256], m, l;
            const int32_t* table = tables + (int64_t)rows[b] * table_stride;
            attend_head(g, pool, max_pages, table, layer, h / group, 0, kv_len[b], q + ((int64_t)b * Hq + h) * D,
                        scale, o, &m, &l);
            if (l > 0.0f)
                for (int d = 0; d < D; d++) out[((int64_t)b * Hq + h) * D + d] = f_to_st(o[d] / l, g->dtype);
        }
    }
}

/* Same result before rounding to the storage type, from an order-independent fp64 softmax:
 * a bound on what any summation order may legitimately return.  out_f [n_seq][Hq][D] fp32. */
void okv_attend_decode_f64(const okv_geom* g, const uint16_t* pool, int max_pages, const int32_t* tables,
                           int table_stride, const int32_t* rows, const int32_t* kv_len, int n_seq, int layer,
                           const uint16_t* q, float* out_f, float scale) {
    int Hq = g->num_q_heads, D = g->head_dim, group = g->num_q_heads / g->num_kv_heads, P = g->page_size;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < n_seq; b++) {
        for (int h = 0; h < Hq; h++) {
            const int32_t* table = tables + (int64_t)rows[b] * table_stride;
            const uint16_t* qr = q + ((int64_t)b * Hq + h) * D;
            int n = kv_len[b], kvh = h / group;
            double* s = (double*)malloc(sizeof(double) * (size_t)(n > 0 ? n : 1));
            double mx = -1e300;
            for (int t = 0; t < n; t++) {
                int page = table[t / P];
                if (page < 0) { s[t] = -1e300; continue; }
                const uint16_t* k = pool + pool_row(g, max_pages, layer, page, 0, kvh, t % P);
                double dot = 0;
                for (int d = 0; d < D; d++) dot += (double)st_to_f(qr[d], g->dtype) * (double)st_to_f(k[d], g->dtype);
                s[t] = dot * (double)scale;
                if (s[t] > mx) mx = s[t];
            }
            double acc[256], l = 0;
            for (int d = 0; d < D; d++) acc[d] = 0;
            for (int t = 0; t < n; t++) {
                int page = table[t / P];
                if (page < 0) continue;
                double p = exp(s[t] - mx);
                const uint16_t* v = pool + pool_row(g, max_pages, layer, page, 1, kvh, t % P);
                for (int d = 0; d < D; d++) acc[d] += p * (double)st_to_f(v[d], g->dtype);
                l += p;
            }
            for (int d = 0; d < D; d++) out_f[((int64_t)b * Hq + h) * D + d] = l > 0 ? (float)(acc[d] / l) : 0.0f;
            free(s);
        }
    }
}

/* Attention mass per logical page, the input the importance scorer is declared for
 * (src/memoria/importance_scorer.h:8-15: per-block attention weights accumulated across layers; the
 * reference has no producer, so the definition is this build's): mass[b][j] += sum over query heads h
 * and keys t of page j of softmax_t(scale * q_h . k_t), in fp64.  mass [n_seq][mass_stride], added to. */
void okv_page_mass(const okv_geom* g, const uint16_t* pool, int max_pages, const int32_t* tables, int table_stride,
                   const int32_t* rows, const int32_t* kv_len, int n_seq, int layer, const uint16_t* q,
                   double* mass, int mass_stride, float scale) {
    int Hq = g->num_q_heads, D = g->head_dim, group = g->num_q_heads / g->num_kv_heads, P = g->page_size;
#pragma omp parallel for schedule(dynamic, 1)
    for (int b = 0; b < n_seq; b++) {
        const int32_t* table = tables + (int64_t)rows[b] * table_stride;
        int n = kv_len[b];
        double* s = (double*)malloc(sizeof(double) * (size_t)(n > 0 ? n : 1));
        for (int h = 0; h < Hq; h++) {
            const uint16_t* qr = q + ((int64_t)b * Hq + h) * D;
            int kvh = h / group;
            double mx = -1e300, l = 0;
            for (int t = 0; t < n; t++) {
                int page = table[t / P];
                if (page < 0) { s[t] = -1e300; continue; }
                const uint16_t* k = pool + pool_row(g, max_pages, layer, page, 0, kvh, t % P);
                double dot = 0;
                for (int d = 0; d < D; d++) dot += (double)st_to_f(qr[d], g->dtype) * (double)st_to_f(k[d], g->dtype);
                s[t] = dot * (double)scale;
                if (s[t] > mx) mx = s[t];
            }
            for (int t = 0; t < n; t++)
                if (table[t / P] >= 0) l += exp(s[t] - mx);
            if (!(l > 0)) continue;
            for (int t = 0; t < n; t++)
                if (table[t / P] >= 0) mass[(int64_t)b * mass_stride + t / P] += exp(s[t] - mx) / l;
        }
        free(s);
    }
}

/* ImportanceScorer::update's arithmetic (src/memoria/importance_scorer.cu:27-37): the device compiler
 * contracts scores[b] * decay + new_scores[b] into one fused multiply-add. */
void okv_importance_update(float* scores, const float* fresh, int n, float decay) {
    for (int i = 0; i < n; i++) scores[i] = fmaf(scores[i], decay, fresh[i]);
}

/* Chunked-prefill attention — src/machina/paged_attention.cu:465-554: q/out [m][Hq][D]; token t
 * of the chunk sees causal_len = pos_start + t + 1 keys; same recurrence. */
void okv_attend_prefill(const okv_geom* g, const uint16_t* pool, int max_pages, const int32_t* table, int layer,
                        int pos_start, int m, const uint16_t* q, uint16_t* out, float scale) {
    int Hq = g->num_q_heads, D = g->head_dim, group = g->num_q_heads / g->num_kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int t = 0; t < m; t++) {
        for (int h = 0; h < Hq; h++) {
            float o[256], mm, l;
            attend_head(g, pool, max_pages, table, layer, h / group, 0, pos_start + t + 1,
                        q + ((int64_t)t * Hq + h) * D, scale, o, &mm, &l);
            if (l > 0.0f)
                for (int d = 0; d < D; d++) out[((int64_t)t * Hq + h) * D + d] = f_to_st(o[d] / l, g->dtype);
        }
    }
}

/* Split-KV partial over keys [kv_begin, kv_end) of one sequence — the decode recurrence above
 * with the (m, l, o) convention of contiguous_split_k_decode_kernel
 * (src/sensus/auditus/asr/asr_ops_attn.cu:29-86): o un-normalised, empty range m = -1e20, l = 0.
 * part = [Hq*D o | Hq m | Hq l] fp32. */
void okv_attend_partial(const okv_geom* g, const uint16_t* pool, int max_pages, const int32_t* table, int layer,
                        int kv_begin, int kv_end, const uint16_t* q, float* part, float scale) {
    int Hq = g->num_q_heads, D = g->head_dim, group = g->num_q_heads / g->num_kv_heads;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < Hq; h++) {
        float o[256], m, l;
        attend_head(g, pool, max_pages, table, layer, h / group, kv_begin, kv_end, q + (int64_t)h * D, scale, o, &m, &l);
        if (!(l > 0.0f)) {
            m = -1e20f;
            l = 0.0f;
            for (int d = 0; d < D; d++) o[d] = 0.0f;
        }
        memcpy(part + (int64_t)h * D, o, sizeof(float) * (size_t)D);
        part[(int64_t)Hq * D + h] = m;
        part[(int64_t)Hq * (D + 1) + h] = l;
    }
}

/* Merge of partials — src/sensus/auditus/asr/asr_ops_attn.cu:88-108: running max with rescale,
 * result acc / l, 0 if l == 0 (here: left unwritten, as the paged kernel does). */
void okv_combine(const okv_geom* g, int n_parts, const float* parts, uint16_t* out) {
    int Hq = g->num_q_heads, D = g->head_dim;
    int64_t stride = (int64_t)Hq * (D + 2);
    for (int h = 0; h < Hq; h++) {
        for (int d = 0; d < D; d++) {
            float m = -1e20f, l = 0.0f, acc = 0.0f;
            for (int p = 0; p < n_parts; p++) {
                const float* base = parts + p * stride;
                float pm = base[(int64_t)Hq * D + h], pl = base[(int64_t)Hq * (D + 1) + h], pv = base[(int64_t)h * D + d];
                if (pm > m) {
                    float sc = expf(m - pm);
                    acc = acc * sc + pv;
                    l = l * sc + pl;
                    m = pm;
                } else {
                    float sc = expf(pm - m);
                    acc += pv * sc;
                    l += pl * sc;
                }
            }
            if (l > 0.0f) out[(int64_t)h * D + d] = f_to_st(acc / l, g->dtype);
        }
    }
}

/* Copy-on-write of a page's first n_slots slots, all layers and heads (specified by this
 * build; the reference has no fork). */
void okv_cow_copy(const okv_geom* g, uint16_t* pool, int max_pages, int src_page, int dst_page, int n_slots) {
    for (int layer = 0; layer < g->num_layers; layer++)
        for (int kv = 0; kv < 2; kv++)
            for (int h = 0; h < g->num_kv_heads; h++)
                memcpy(pool + pool_row(g, max_pages, layer, dst_page, kv, h, 0),
                       pool + pool_row(g, max_pages, layer, src_page, kv, h, 0),
                       (size_t)n_slots * g->head_dim * 2);
}

/* Flat <-> paged copies — src/memoria/cache_kernels.cu:30-87 (extract: a token whose table entry is
 * negative reads as zeros) and :93-141 (inject: such a token is skipped).  Flat layout
 * [layer][K|V][token][kv_head][dim], src/memoria/cache_kernels.h:29. */
void okv_extract(const okv_geom* g, uint16_t* dst, const uint16_t* pool, int max_pages, const int32_t* table,
                 int start_token, int num_tokens) {
    int D = g->head_dim, H = g->num_kv_heads, P = g->page_size;
    for (int layer = 0; layer < g->num_layers; layer++)
        for (int kv = 0; kv < 2; kv++)
            for (int t = 0; t < num_tokens; t++) {
                int pos = start_token + t, page = table[pos / P];
                for (int h = 0; h < H; h++) {
                    uint16_t* out = dst + ((((int64_t)layer * 2 + kv) * num_tokens + t) * H + h) * D;
                    if (page < 0) memset(out, 0, (size_t)D * 2);
                    else memcpy(out, pool + pool_row(g, max_pages, layer, page, kv, h, pos % P), (size_t)D * 2);
                }
            }
}
void okv_inject(const okv_geom* g, uint16_t* pool, const uint16_t* src, int max_pages, const int32_t* table,
                int start_token, int num_tokens) {
    int D = g->head_dim, H = g->num_kv_heads, P = g->page_size;
    for (int layer = 0; layer < g->num_layers; layer++)
        for (int kv = 0; kv < 2; kv++)
            for (int t = 0; t < num_tokens; t++) {
                int pos = start_token + t, page = table[pos / P];
                if (page < 0) continue;
                for (int h = 0; h < H; h++)
                    memcpy(pool + pool_row(g, max_pages, layer, page, kv, h, pos % P),
                           src + ((((int64_t)layer * 2 + kv) * num_tokens + t) * H + h) * D, (size_t)D * 2);
            }
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; a timed baseline asks for the host's cores itself. */
void okv_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int okv_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
