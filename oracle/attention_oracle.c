/*
 * CPU oracle for the fusor attention path.  TEST INFRASTRUCTURE ONLY: this file is
 * the checker the CUDA library is compared against and the timed CPU baseline; the
 * product library never links, loads or calls it.
 *
 * It restates, in plain C, the arithmetic of the reference's CPU attention:
 *   fusor-ml/fusor/src/composite/flash_attention.rs:77-200  (the composite)
 * on the primitive semantics of
 *   fusor-ml/cpu/src/matmul.rs:200-326   (one f32 gemm per (batch, head))
 *   fusor-ml/cpu/src/reduce.rs:700-764   (sequential max / sum, identities -inf / 0)
 *   fusor-ml/cpu/src/elementwise.rs:120-157 (libm expf per lane)
 *   fusor-ml/cpu/src/pairwise.rs:48-81   (sub / add / true division)
 *
 * Parity status: the matmuls of the reference run inside the third-party `gemm`
 * crate 0.18.2 (Cargo.lock:3241-3244), which is not vendored and whose accumulation
 * order is unspecified, and no Rust toolchain exists to run the reference itself.
 * Bit-level parity is therefore UNPINNED.  What is pinned: every known-answer the
 * reference's own tests hold for this path (tests/test_oracle_pins.py):
 *   fusor-ml/fusor/src/composite/flash_attention.rs:208-359,
 *   fusor-ml/core/src/composite/flash_attention.rs:561-673,
 *   fusor-ml/fusor/src/cache/attention_mask.rs:84-111, mask_cache.rs:119-176.
 *
 * Each output element of both products accumulates over the contraction index in
 * ascending order (what a gemm micro-kernel does per C element); the loops are laid
 * out so that the compiler vectorises across independent output elements only.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_MASK_NONE 0
#define ORACLE_MASK_QK 1        /* additive [Sq, Skv]      (MaskKind::QKMask,       flash_attention.rs:151-162) */
#define ORACLE_MASK_BATCH_KEY 2 /* additive [B, Skv]       (MaskKind::BatchKeyMask, flash_attention.rs:163-174) */
#define ORACLE_MASK_CAUSAL 3    /* analytic: 0 if k <= q + causal_offset else -inf; equals
                                   AttentionMask::causal (attention_mask.rs:26-46) left-padded with
                                   `causal_offset` zero columns by MaskCache::get_mask (mask_cache.rs:73-82) */

int oracle_abi_version(void) { return 1; }

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* A launcher may have exported OMP_NUM_THREADS=1 (torchrun does); the timed CPU baseline sets its thread count itself. */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* K^T for one (batch, kv head): kt[d * Skv + j] = k[j * D + d].
 * (k.transpose(2,3) is made contiguous before the gemm, cpu/src/tensor.rs:1063-1072.) */
static void transpose_k(const float* k, float* kt, int Skv, int D) {
#pragma omp parallel for schedule(static)
    for (int d = 0; d < D; ++d)
        for (int j = 0; j < Skv; ++j) kt[(size_t)d * Skv + j] = k[(size_t)j * D + d];
}

/* One output row of the composite.  `s` is a scratch row of Skv floats.
 * n_cols <= Skv: columns >= n_cols are known to carry a -inf mask and are skipped
 * (adds exact zeros in the reference, so the result is bit-identical); pass Skv for
 * the literal dense evaluation. */
static void composite_row(const float* qrow, const float* kt, const float* v, const float* mask_row,
                          int causal_last, float* s, float* out, int Skv, int n_cols, int D, float scale) {
    /* scores = q @ k^T           (flash_attention.rs:141-142) */
    for (int j = 0; j < n_cols; ++j) s[j] = 0.0f;
    for (int d = 0; d < D; ++d) {
        const float qd = qrow[d];
        const float* kr = kt + (size_t)d * Skv;
        for (int j = 0; j < n_cols; ++j) s[j] += qd * kr[j];
    }
    /* * scale, after the product (flash_attention.rs:145) */
    for (int j = 0; j < n_cols; ++j) s[j] = s[j] * scale;
    /* + mask                     (flash_attention.rs:148-180) */
    if (mask_row)
        for (int j = 0; j < n_cols; ++j) s[j] = s[j] + mask_row[j];
    if (causal_last >= -1)
        for (int j = causal_last + 1; j < n_cols; ++j) s[j] = s[j] + (-INFINITY);
    /* max over the last dim, sequential from -inf (reduce.rs:178,754-758) */
    float mx = -INFINITY;
    for (int j = 0; j < n_cols; ++j) mx = s[j] > mx ? s[j] : mx;
    /* exp(scores - max)          (flash_attention.rs:189-191) */
    for (int j = 0; j < n_cols; ++j) s[j] = expf(s[j] - mx);
    /* sum, sequential ascending  (reduce.rs:182,754-758) */
    float sum = 0.0f;
    for (int j = 0; j < n_cols; ++j) sum += s[j];
    /* true division              (flash_attention.rs:196) */
    for (int j = 0; j < n_cols; ++j) s[j] = s[j] / sum;
    /* weights @ v                (flash_attention.rs:199) */
    for (int d = 0; d < D; ++d) out[d] = 0.0f;
    for (int j = 0; j < n_cols; ++j) {
        const float w = s[j];
        const float* vr = v + (size_t)j * D;
        for (int d = 0; d < D; ++d) out[d] += w * vr[d];
    }
}

/*
 * Composite attention, f32, contiguous [B,H,S,D] tensors.
 *   q [B,Hq,Sq,D]   k,v [B,Hkv,Skv,D]   out [B,Hq,Sq,D]  (or [n_rows, D] when `rows` is given)
 *   GQA: query head h reads kv head h / (Hq/Hkv)          (flash_attention.rs:101-138)
 *   rows: optional list of flat row ids ((b*Hq + h)*Sq + q), sorted ascending; NULL = all rows.
 *   skip_masked: with ORACLE_MASK_CAUSAL only, do not evaluate columns whose mask is -inf.
 * Returns 0, or a negative code for an argument the reference would assert on.
 */
int oracle_attention_f32(const float* q, const float* k, const float* v, const float* mask, int mask_kind,
                         int64_t causal_offset, float* out, int B, int Hq, int Hkv, int Sq, int Skv, int D,
                         float scale, const int64_t* rows, int64_t n_rows, int skip_masked) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || D <= 0) return -1;
    if (Hq % Hkv != 0) return -2; /* flash_attention.rs:94-99 */
    if ((mask_kind == ORACLE_MASK_QK || mask_kind == ORACLE_MASK_BATCH_KEY) && !mask) return -3;
    const int g = Hq / Hkv;
    float* kt = (float*)malloc((size_t)D * Skv * sizeof(float));
    if (!kt) return -4;
    int nthreads = oracle_num_threads();
    float* scratch = (float*)malloc((size_t)nthreads * Skv * sizeof(float));
    if (!scratch) { free(kt); return -4; }

    int64_t row_cursor = 0;
    for (int b = 0; b < B; ++b) {
        for (int hk = 0; hk < Hkv; ++hk) {
            const int64_t first_row = ((int64_t)b * Hq + (int64_t)hk * g) * Sq;
            const int64_t end_row = first_row + (int64_t)g * Sq;
            int64_t lo = 0, hi = (int64_t)g * Sq;
            if (rows) {
                lo = row_cursor;
                while (row_cursor < n_rows && rows[row_cursor] < end_row) ++row_cursor;
                hi = row_cursor;
                if (lo == hi) continue;
            }
            const float* kb = k + ((size_t)b * Hkv + hk) * (size_t)Skv * D;
            const float* vb = v + ((size_t)b * Hkv + hk) * (size_t)Skv * D;
            transpose_k(kb, kt, Skv, D);
#pragma omp parallel for schedule(dynamic, 8)
            for (int64_t it = lo; it < hi; ++it) {
#ifdef _OPENMP
                float* s = scratch + (size_t)omp_get_thread_num() * Skv;
#else
                float* s = scratch;
#endif
                const int64_t flat = rows ? rows[it] : first_row + it;
                const int qi = (int)(flat % Sq);
                const float* qrow = q + (size_t)flat * D;
                float* orow = out + (size_t)(rows ? it : flat) * D;
                const float* mrow = NULL;
                int causal_last = -2, n_cols = Skv;
                if (mask_kind == ORACLE_MASK_QK) mrow = mask + (size_t)qi * Skv;
                else if (mask_kind == ORACLE_MASK_BATCH_KEY) mrow = mask + (size_t)b * Skv;
                else if (mask_kind == ORACLE_MASK_CAUSAL) {
                    int64_t last = (int64_t)qi + causal_offset;
                    if (last >= Skv) last = Skv - 1;
                    if (last < -1) last = -1;
                    causal_last = (int)last;
                    if (skip_masked && causal_last >= 0) n_cols = causal_last + 1;
                }
                composite_row(qrow, kt, vb, mrow, causal_last, s, orow, Skv, n_cols, D, scale);
            }
        }
    }
    free(scratch);
    free(kt);
    return 0;
}

/*
 * Diagnostic second oracle: the arithmetic ORDER of the reference's fused GPU kernel
 * (fusor-ml/core/src/composite/flash_attention.rs:147-331): one 32-lane subgroup per
 * output row, lane owns dims lane + i*32, keys visited serially with an online
 * (m, d, acc) update; m starts at -3.40282e38 (min_for_dtype, core/src/reduce.rs:825-831).
 * The subgroupAdd order is unspecified in WGSL; lanes are summed ascending here.
 */
int oracle_attention_online_f32(const float* q, const float* k, const float* v, const float* mask,
                                float* out, int B, int Hq, int Hkv, int Sq, int Skv, int D, float scale) {
    if (Hq % Hkv != 0) return -2;
    const int g = Hq / Hkv;
    const int64_t n = (int64_t)B * Hq * Sq;
#pragma omp parallel for schedule(dynamic, 16)
    for (int64_t flat = 0; flat < n; ++flat) {
        const int qi = (int)(flat % Sq);
        const int h = (int)((flat / Sq) % Hq);
        const int b = (int)(flat / ((int64_t)Sq * Hq));
        const float* qrow = q + (size_t)flat * D;
        const float* kb = k + ((size_t)b * Hkv + h / g) * (size_t)Skv * D;
        const float* vb = v + ((size_t)b * Hkv + h / g) * (size_t)Skv * D;
        float m = -3.40282e38f, dsum = 0.0f;
        float acc[1024];
        if (D > 1024) continue;
        for (int d = 0; d < D; ++d) acc[d] = 0.0f;
        for (int j = 0; j < Skv; ++j) {
            float lane_partial[32];
            for (int l = 0; l < 32; ++l) {
                float p = 0.0f;
                for (int d = l; d < D; d += 32) p += qrow[d] * kb[(size_t)j * D + d];
                lane_partial[l] = p;
            }
            float dot = 0.0f;
            for (int l = 0; l < 32; ++l) dot += lane_partial[l];
            float score = dot * scale;
            if (mask) score = score + mask[(size_t)qi * Skv + j];
            const float old_m = m;
            m = score > m ? score : m;
            const float e_old = expf(old_m - m);
            const float e_s = expf(score - m);
            dsum = dsum * e_old + e_s;
            for (int d = 0; d < D; ++d) acc[d] = acc[d] * e_old + e_s * vb[(size_t)j * D + d];
        }
        for (int d = 0; d < D; ++d) out[(size_t)flat * D + d] = acc[d] / dsum;
    }
    return 0;
}

/* AttentionMask::causal (fusor-ml/fusor/src/cache/attention_mask.rs:26-46): [S,S], -inf where j > i. */
void oracle_causal_mask(float* mask, int S) {
    for (int i = 0; i < S; ++i)
        for (int j = 0; j < S; ++j) mask[(size_t)i * S + j] = j > i ? -INFINITY : 0.0f;
}

/* MaskCache::create_sliding_window_mask (mask_cache.rs:88-116): -inf where i < j or j + w <= i. */
void oracle_sliding_window_mask(float* mask, int S, int window) {
    for (int i = 0; i < S; ++i)
        for (int j = 0; j < S; ++j)
            mask[(size_t)i * S + j] = (i < j || j + window <= i) ? -INFINITY : 0.0f;
}

/*
 * Log-sum-exp merge of split-KV partials (same rule as the (m, d) combine of the
 * reference softmax kernel, fusor-ml/core/src/composite/softmax.rs:59-82):
 *   part[p][row] = { m, l, O[D] } with O un-normalised;  M = max m_p,
 *   L = sum l_p e^{m_p - M},  out = sum O_p e^{m_p - M} / L.
 * A part with m = -inf and l = 0 contributes nothing.
 */
void oracle_lse_combine(const float* parts, int n_parts, int64_t n_rows, int D, float* out) {
    const size_t rec = (size_t)D + 2;
    for (int64_t r = 0; r < n_rows; ++r) {
        float M = -INFINITY;
        for (int p = 0; p < n_parts; ++p) {
            const float m = parts[((size_t)p * n_rows + r) * rec];
            M = m > M ? m : M;
        }
        float L = 0.0f;
        for (int d = 0; d < D; ++d) out[(size_t)r * D + d] = 0.0f;
        for (int p = 0; p < n_parts; ++p) {
            const float* pr = parts + ((size_t)p * n_rows + r) * rec;
            if (pr[1] == 0.0f) continue;
            const float w = expf(pr[0] - M);
            L += pr[1] * w;
            for (int d = 0; d < D; ++d) out[(size_t)r * D + d] += pr[2 + d] * w;
        }
        /* a row whose parts are all empty attends to no key: zeros (the merge has no reference counterpart; this is
           the rule the library documents) */
        for (int d = 0; d < D; ++d) out[(size_t)r * D + d] = L > 0.0f ? out[(size_t)r * D + d] / L : 0.0f;
    }
}

/* Split-KV partial of one key range [k0, k1) in the units oracle_lse_combine merges. */
int oracle_attention_partial_f32(const float* q, const float* k, const float* v, float* part, int B, int Hq,
                                 int Hkv, int Sq, int Skv, int D, float scale, int k0, int k1) {
    if (Hq % Hkv != 0) return -2;
    const int g = Hq / Hkv;
    const int64_t n = (int64_t)B * Hq * Sq;
    const size_t rec = (size_t)D + 2;
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t flat = 0; flat < n; ++flat) {
        const int h = (int)((flat / Sq) % Hq);
        const int b = (int)(flat / ((int64_t)Sq * Hq));
        const float* qrow = q + (size_t)flat * D;
        const float* kb = k + ((size_t)b * Hkv + h / g) * (size_t)Skv * D;
        const float* vb = v + ((size_t)b * Hkv + h / g) * (size_t)Skv * D;
        float* pr = part + (size_t)flat * rec;
        float m = -INFINITY;
        for (int j = k0; j < k1; ++j) {
            float dot = 0.0f;
            for (int d = 0; d < D; ++d) dot += qrow[d] * kb[(size_t)j * D + d];
            dot *= scale;
            m = dot > m ? dot : m;
        }
        float l = 0.0f;
        for (int d = 0; d < D; ++d) pr[2 + d] = 0.0f;
        for (int j = k0; j < k1; ++j) {
            float dot = 0.0f;
            for (int d = 0; d < D; ++d) dot += qrow[d] * kb[(size_t)j * D + d];
            const float e = expf(dot * scale - m);
            l += e;
            for (int d = 0; d < D; ++d) pr[2 + d] += e * vb[(size_t)j * D + d];
        }
        pr[0] = m;
        pr[1] = l;
    }
    return 0;
}

/*
 * Rotary position embedding as the reference's CPU composites compute it, f32, contiguous [B,H,S,D]:
 *   interleaved = 0: Tensor::rope            (fusor-ml/fusor/src/composite/rope.rs:38-68, rotate_half :8-19):
 *                    out = x * cos + rotate_half(x) * sin, halves (i, i + D/2) share cos/sin[pos][i]
 *   interleaved = 1: Tensor::rope_interleaved (rope.rs:70-118): pairs (2i, 2i+1):
 *                    y0 = x0 * c - x1 * s,  y1 = x0 * s + x1 * c
 * cos, sin: [context_length][D/2]; row start_pos + t is used for sequence position t
 * (RopeCache::forward narrows the tables at start_pos, rope.rs:232-246).
 * Each product is rounded before the add / subtract (separate mul_ and add_ ops): contraction is switched off.
 */
__attribute__((optimize("fp-contract=off"))) int oracle_rope_f32(const float* x, const float* cos_t, const float* sin_t,
                                                                 float* out, int B, int H, int S, int D, int start_pos,
                                                                 int interleaved) {
    if (D % 2 != 0) return -1;
    const int half = D / 2;
    for (long long bh = 0; bh < (long long)B * H; ++bh)
        for (int t = 0; t < S; ++t) {
            const float* xr = x + ((size_t)bh * S + t) * D;
            float* orow = out + ((size_t)bh * S + t) * D;
            const float* c = cos_t + (size_t)(start_pos + t) * half;
            const float* s = sin_t + (size_t)(start_pos + t) * half;
            for (int i = 0; i < half; ++i) {
                if (interleaved) {
                    const float x0 = xr[2 * i], x1 = xr[2 * i + 1];
                    const float a = x0 * c[i], b = x1 * s[i];
                    const float e = x0 * s[i], f = x1 * c[i];
                    orow[2 * i] = a - b;
                    orow[2 * i + 1] = e + f;
                } else {
                    const float x1 = xr[i], x2 = xr[i + half];
                    const float a = x1 * c[i], b = (-x2) * s[i];
                    const float e = x2 * c[i], f = x1 * s[i];
                    orow[i] = a + b;
                    orow[i + half] = e + f;
                }
            }
        }
    return 0;
}

/*
 * Output projection after attention, f32:
 *   out[b, s, n] = sum_k x[b, s, k] * w[n, k] + bias[n],   x[b, s, h * D + d] = attn[b, h, s, d]
 * (attn_output.transpose(1, 2).reshape([b, q_len, hidden]) then Linear::forward: matmul with the weight, bias added
 * afterwards; models/kalosm-llama/src/raw/attention_layer.rs:450-454, fusor-ml/fusor/src/layers/linear.rs:72-115.  The
 * reference's weight is a GGUF-quantised QMatrix; the oracle takes its dense values.)  Each output element accumulates
 * over k in ascending order.  attn [B,Hq,S,D], w [N, Hq*D], bias [N] or NULL, out [B,S,N], all contiguous.
 */
int oracle_out_proj_f32(const float* attn, const float* w, const float* bias, float* out, int B, int Hq, int S, int D,
                        int N) {
    if (B <= 0 || Hq <= 0 || S <= 0 || D <= 0 || N <= 0) return -1;
    const int K = Hq * D;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int s = 0; s < S; ++s) {
            float* x = (float*)malloc((size_t)K * sizeof(float));
            for (int h = 0; h < Hq; ++h)
                memcpy(x + (size_t)h * D, attn + (((size_t)b * Hq + h) * S + s) * D, (size_t)D * sizeof(float));
            float* o = out + ((size_t)b * S + s) * N;
            for (int n = 0; n < N; ++n) {
                const float* wr = w + (size_t)n * K;
                float acc = 0.0f;
                for (int k = 0; k < K; ++k) acc += x[k] * wr[k];
                o[n] = bias ? acc + bias[n] : acc;
            }
            free(x);
        }
    return 0;
}
