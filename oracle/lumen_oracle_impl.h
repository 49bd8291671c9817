/*
 * TEST INFRASTRUCTURE — CPU restatement of the Lumen (chen-197/Lumen) Llama inference path.
 *
 * This file is included twice by lumen_oracle.c: once with REAL=float (the reference's
 * arithmetic: IEEE f32, the reference's operation order, no FMA contraction) and once with
 * REAL=double (a shadow that bounds the rounding error of both the f32 oracle and the GPU
 * path).  Weights and inputs are always f32 arrays; REAL is the type of every intermediate,
 * accumulator and output.
 *
 * PARITY UNPINNED: the reference ships no tests, golden vectors or fixtures and cannot be
 * compiled where this was written (it is Rust; no rustc/cargo), so nothing but the source
 * text pins these functions.  Each function cites the reference lines it restates.
 * Third-party arithmetic the reference delegates (ndarray 0.15 `general_mat_mul` ->
 * the `matrixmultiply` crate, version unpinned because the reference has no Cargo.lock;
 * Rust std `powf/cos/sin/exp/sqrt` -> platform libm) is restated as a k-ordered triple loop
 * and glibc libm.
 *
 * Parallel axes are the ones Rayon uses in the reference (output elements, (b,h) rows), so
 * every output element is computed by one thread in a fixed order: results do not depend
 * on the thread count.
 */

#ifndef REAL
#error "include from lumen_oracle.c with REAL and SFX defined"
#endif

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SFX)

/* ---- libm in the working precision ------------------------------------------------- */
static inline REAL FN(r_exp)(REAL x) { return sizeof(REAL) == 4 ? (REAL)expf((float)x) : (REAL)exp((double)x); }
static inline REAL FN(r_sqrt)(REAL x) { return sizeof(REAL) == 4 ? (REAL)sqrtf((float)x) : (REAL)sqrt((double)x); }

/*
 * ops::matmul::matmul — src/ops/matmul.rs:10-103.
 * a[M,K] (row-major, M = product of leading dims), w[N,K] row-major ("[out,in]"),
 * out[M,N] = a . w^T.
 * M == 1 branch (matmul.rs:42-69): parallel over n, `sum = 0; for k: sum += w*x` in k order.
 * M > 1 branch (matmul.rs:70-92) calls general_mat_mul whose blocking is third-party and
 * unpinned; restated with the same k-ordered dot per output element.
 */
void FN(lo_matmul)(const float *a, long m, long k, const float *w, long n, REAL *out) {
#pragma omp parallel for collapse(2) schedule(static)
    for (long i = 0; i < m; ++i) {
        for (long j = 0; j < n; ++j) {
            const float *row = w + j * k;
            const float *x = a + i * k;
            REAL sum = 0;
            for (long t = 0; t < k; ++t) {
                REAL p = (REAL)row[t] * (REAL)x[t];
                sum += p;
            }
            out[i * n + j] = sum;
        }
    }
}

/* Same product with an activation already held in REAL (model-internal use). */
static void FN(matmul_rr)(const REAL *a, long m, long k, const float *w, long n, REAL *out) {
#pragma omp parallel for collapse(2) schedule(static)
    for (long i = 0; i < m; ++i) {
        for (long j = 0; j < n; ++j) {
            const float *row = w + j * k;
            const REAL *x = a + i * k;
            REAL sum = 0;
            for (long t = 0; t < k; ++t) {
                REAL p = (REAL)row[t] * x[t];
                sum += p;
            }
            out[i * n + j] = sum;
        }
    }
}

/*
 * RMSNorm::forward — src/layers/norm/rms_norm.rs:24-62 (math :49-56):
 * ss = fold(0, acc + v*v) in order; rms = sqrt(ss/dim + eps); inv = 1/rms; o = (x*inv)*w.
 */
static void FN(rmsnorm_rr)(const REAL *x, long rows, long dim, const float *w, float eps, REAL *out) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r) {
        const REAL *xr = x + r * dim;
        REAL ss = 0;
        for (long i = 0; i < dim; ++i) {
            REAL sq = xr[i] * xr[i];
            ss = ss + sq;
        }
        REAL rms = FN(r_sqrt)(ss / (REAL)dim + (REAL)eps);
        REAL inv = (REAL)1 / rms;
        for (long i = 0; i < dim; ++i) {
            REAL t = xr[i] * inv;
            out[r * dim + i] = t * (REAL)w[i];
        }
    }
}

void FN(lo_rmsnorm)(const float *x, long rows, long dim, const float *w, float eps, REAL *out) {
    REAL *tmp = (REAL *)malloc(sizeof(REAL) * (size_t)(rows * dim));
    for (long i = 0; i < rows * dim; ++i) tmp[i] = (REAL)x[i];
    FN(rmsnorm_rr)(tmp, rows, dim, w, eps, out);
    free(tmp);
}

/*
 * RotaryEmbedding::precompute_freqs_cis — src/layers/attention/encoding.rs:29-54.
 * freq = 1.0 / theta.powf((j*2)/dim); val = pos*freq; cos/sin written at columns j and
 * j+dim/2.  The tables are f32 in the reference; the f64 shadow evaluates them in double.
 * Output tables are [max_seq, dim].
 */
void FN(lo_rope_table)(long dim, long max_seq, float theta, REAL *cos_t, REAL *sin_t) {
    long half = dim / 2;
    for (long i = 0; i < max_seq; ++i) {
        for (long j = 0; j < half; ++j) {
            REAL c, s;
            if (sizeof(REAL) == 4) {
                float pos = (float)i;
                float freq = 1.0f / powf(theta, ((float)j * 2.0f) / (float)dim);
                float val = pos * freq;
                c = (REAL)cosf(val);
                s = (REAL)sinf(val);
            } else {
                double freq = 1.0 / pow((double)theta, ((double)j * 2.0) / (double)dim);
                double val = (double)i * freq;
                c = (REAL)cos(val);
                s = (REAL)sin(val);
            }
            cos_t[i * dim + j] = c;
            cos_t[i * dim + j + half] = c;
            sin_t[i * dim + j] = s;
            sin_t[i * dim + j + half] = s;
        }
    }
}

/*
 * RotaryEmbedding::rope_1token_copy — encoding.rs:173-204 (rotation :195-203) and the inline
 * q rotation of the decode path, self_attention.rs:220-227:
 * dst[j] = x1*c - x2*s; dst[j+half] = x2*c + x1*s.  Returns -1 when pos >= max_seq (the
 * reference panics, encoding.rs:176-181).
 */
static int FN(rope_1token_rr)(const REAL *src, REAL *dst, long d, long pos, long max_seq,
                              const REAL *cos_t, const REAL *sin_t) {
    if (pos >= max_seq) return -1;
    long half = d / 2;
    const REAL *c = cos_t + pos * d, *s = sin_t + pos * d;
    for (long j = 0; j < half; ++j) {
        REAL x1 = src[j], x2 = src[j + half];
        REAL a = x1 * c[j], b = x2 * s[j];
        REAL e = x2 * c[j], f = x1 * s[j];
        dst[j] = a - b;
        dst[j + half] = e + f;
    }
    return 0;
}

/*
 * RotaryEmbedding::forward — encoding.rs:56-123: x[B,H,S,D] rotated at positions
 * offset..offset+S.  Returns -1 when offset+S > max_seq (panic at :62-68).
 */
static int FN(rope_forward_rr)(const REAL *x, long b, long h, long s, long d, long offset, long max_seq,
                               const REAL *cos_t, const REAL *sin_t, REAL *out) {
    if (offset + s > max_seq) return -1;
#pragma omp parallel for collapse(2) schedule(static)
    for (long bb = 0; bb < b; ++bb)
        for (long hh = 0; hh < h; ++hh)
            for (long ss = 0; ss < s; ++ss) {
                const REAL *src = x + ((bb * h + hh) * s + ss) * d;
                REAL *dst = out + ((bb * h + hh) * s + ss) * d;
                FN(rope_1token_rr)(src, dst, d, offset + ss, max_seq, cos_t, sin_t);
            }
    return 0;
}

int FN(lo_rope_forward)(const float *x, long b, long h, long s, long d, long offset, long max_seq,
                        float theta, REAL *out) {
    long n = b * h * s * d;
    REAL *xr = (REAL *)malloc(sizeof(REAL) * (size_t)n);
    REAL *ct = (REAL *)malloc(sizeof(REAL) * (size_t)(max_seq * d));
    REAL *st = (REAL *)malloc(sizeof(REAL) * (size_t)(max_seq * d));
    for (long i = 0; i < n; ++i) xr[i] = (REAL)x[i];
    FN(lo_rope_table)(d, max_seq, theta, ct, st);
    int rc = FN(rope_forward_rr)(xr, b, h, s, d, offset, max_seq, ct, st, out);
    free(xr); free(ct); free(st);
    return rc;
}

/* SiLU::forward — src/layers/activation.rs:139-147: sig = 1/(1+exp(-x)); x*sig. */
static inline REAL FN(silu1)(REAL x) {
    REAL sig = (REAL)1 / ((REAL)1 + FN(r_exp)(-x));
    return x * sig;
}

void FN(lo_silu)(const float *x, long n, REAL *out) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; ++i) out[i] = FN(silu1)((REAL)x[i]);
}

/* Tensor * Tensor, Tensor + Tensor (same shape) — src/ops/arithmetic.rs:105-109, :48-52. */
void FN(lo_mul)(const float *a, const float *b, long n, REAL *out) {
    for (long i = 0; i < n; ++i) out[i] = (REAL)a[i] * (REAL)b[i];
}
void FN(lo_add)(const float *a, const float *b, long n, REAL *out) {
    for (long i = 0; i < n; ++i) out[i] = (REAL)a[i] + (REAL)b[i];
}

/*
 * Embedding::forward — src/layers/basic/embedding.rs:21-57: ids are f32, cast `as usize`
 * (:50; a negative or NaN id saturates to 0 in Rust); id >= vocab panics (:55) -> returns -1.
 */
int FN(lo_embedding)(const float *ids, long n, const float *table, long vocab, long dim, REAL *out) {
    for (long i = 0; i < n; ++i) {
        float f = ids[i];
        long idx = (f != f || f <= 0.0f) ? 0 : (f >= 9.2e18f ? vocab : (long)f);
        if (idx >= vocab) return -1;
        for (long j = 0; j < dim; ++j) out[i * dim + j] = (REAL)table[idx * dim + j];
    }
    return 0;
}

/*
 * ops::fused::fused_softmax forward — src/ops/fused.rs:39-83.  x[B,H,Q,K]; mask j>i only if
 * causal && Q>1 (no past offset); max over unmasked of x*scale; exp(x*scale-max); masked -> 0;
 * times 1/(sum + 1e-10).
 */
void FN(lo_fused_softmax)(const float *x, long b, long h, long q, long k, float scale, int causal, REAL *out) {
#pragma omp parallel for schedule(static)
    for (long bh = 0; bh < b * h; ++bh) {
        for (long i = 0; i < q; ++i) {
            const float *row = x + (bh * q + i) * k;
            REAL *o = out + (bh * q + i) * k;
            int masking = causal && q > 1;
            REAL mx = -INFINITY;
            for (long j = 0; j < k; ++j) {
                if (masking && j > i) continue;
                REAL v = (REAL)row[j] * (REAL)scale;
                if (v > mx) mx = v;
            }
            REAL sum = 0;
            for (long j = 0; j < k; ++j) {
                if (masking && j > i) { o[j] = 0; continue; }
                REAL v = FN(r_exp)((REAL)row[j] * (REAL)scale - mx);
                o[j] = v;
                sum += v;
            }
            /* `1e-10` is an f64 literal narrowed to the f32 element type in the reference. */
            REAL inv = (REAL)1 / (sum + (sizeof(REAL) == 4 ? (REAL)1e-10f : (REAL)1e-10));
            for (long j = 0; j < k; ++j) o[j] *= inv;
        }
    }
}

/* ---- KV cache (KVCacheInner — src/layers/attention/self_attention.rs:24-44) ----------- */
typedef struct {
    long b, h_kv, max_seq, d, len;
    REAL *k, *v; /* [B,Hkv,max_seq,D], zero-initialised (:35-36) */
} FN(lo_kv);

FN(lo_kv) *FN(lo_kv_new)(long b, long h_kv, long max_seq, long d) {
    FN(lo_kv) *c = (FN(lo_kv) *)calloc(1, sizeof(*c));
    c->b = b; c->h_kv = h_kv; c->max_seq = max_seq; c->d = d; c->len = 0;
    size_t n = (size_t)(b * h_kv * max_seq * d);
    c->k = (REAL *)calloc(n, sizeof(REAL));
    c->v = (REAL *)calloc(n, sizeof(REAL));
    return c;
}
void FN(lo_kv_free)(FN(lo_kv) *c) { if (c) { free(c->k); free(c->v); free(c); } }
void FN(lo_kv_reset)(FN(lo_kv) *c) { c->len = 0; } /* :41-43: len only, contents kept */
long FN(lo_kv_len)(const FN(lo_kv) *c) { return c->len; }
void FN(lo_kv_set_len)(FN(lo_kv) *c, long n) { c->len = n; } /* `len` is a pub field (:27) */
REAL *FN(lo_kv_k)(FN(lo_kv) *c) { return c->k; }
REAL *FN(lo_kv_v)(FN(lo_kv) *c) { return c->v; }

/* Optional per-head RMSNorm over head_dim applied to q/k before RoPE (Qwen3 placement).
 * Not in the reference; uses the rms_norm.rs:49-56 formula over D. */
static void FN(head_norm)(REAL *x, long heads, long d, const float *w, float eps) {
    if (!w) return;
    FN(rmsnorm_rr)(x, heads, d, w, eps, x);
}

/*
 * Decode step of SelfAttention::forward, S == 1 — self_attention.rs:125-297.
 * q[B,Hq*D], k_new/v_new[B,Hkv*D] (projection outputs).  Writes RoPE(k_new) and v_new into
 * cache row past_len (:141-180), then per (b,h) row (:199-293): RoPE(q) at past_len, one
 * pass over j = 0..=past_len with the branching online softmax (:252-285), out = ctx *
 * (1/(l + 1e-9)) (:287-290).  out is [B,Hq,D] == [B,1,Hq*D].  Returns -2 on cache overflow
 * (assert at :144-149), -1 on RoPE range.
 */
static int FN(attn_decode_rr)(const REAL *q, const REAL *k_new, const REAL *v_new, FN(lo_kv) *c,
                              long hq, float scale, int causal, const REAL *cos_t, const REAL *sin_t,
                              long rope_max, REAL *out) {
    long b = c->b, hkv = c->h_kv, d = c->d, max_seq = c->max_seq;
    long past = c->len, total = past + 1, n_rep = hq / hkv;
    if (total > max_seq) return -2;
    if (past >= rope_max) return -1;
    for (long bb = 0; bb < b; ++bb)
        for (long hk = 0; hk < hkv; ++hk) {
            REAL *dk = c->k + ((bb * hkv + hk) * max_seq + past) * d;
            REAL *dv = c->v + ((bb * hkv + hk) * max_seq + past) * d;
            FN(rope_1token_rr)(k_new + (bb * hkv + hk) * d, dk, d, past, rope_max, cos_t, sin_t);
            memcpy(dv, v_new + (bb * hkv + hk) * d, sizeof(REAL) * (size_t)d);
        }
    c->len = total;
#pragma omp parallel for schedule(static)
    for (long row = 0; row < b * hq; ++row) {
        long bb = row / hq, hh = row % hq, hk = hh / n_rep;
        REAL qbuf[512], ctx[512];
        FN(rope_1token_rr)(q + row * d, qbuf, d, past, rope_max, cos_t, sin_t);
        const REAL *ks = c->k + (bb * hkv + hk) * max_seq * d;
        const REAL *vs = c->v + (bb * hkv + hk) * max_seq * d;
        for (long i = 0; i < d; ++i) ctx[i] = 0;
        REAL m = -INFINITY, l = 0;
        for (long j = 0; j < total; ++j) {
            if (causal && j > past) break;
            const REAL *kr = ks + j * d, *vr = vs + j * d;
            REAL dot = 0;
            for (long i = 0; i < d; ++i) { REAL p = qbuf[i] * kr[i]; dot += p; }
            REAL score = dot * (REAL)scale;
            if (score > m) {
                REAL s = FN(r_exp)(m - score);
                for (long i = 0; i < d; ++i) ctx[i] *= s;
                l *= s;
                m = score;
                for (long i = 0; i < d; ++i) ctx[i] += vr[i];
                l += (REAL)1;
            } else {
                REAL w = FN(r_exp)(score - m);
                for (long i = 0; i < d; ++i) { REAL p = w * vr[i]; ctx[i] += p; }
                l += w;
            }
        }
        REAL inv = (REAL)1 / (l + (sizeof(REAL) == 4 ? (REAL)1e-9f : (REAL)1e-9));
        for (long i = 0; i < d; ++i) out[row * d + i] = ctx[i] * inv;
    }
    return 0;
}

/*
 * Prefill branch, S > 1 — self_attention.rs:308-426 with gqa_attention_no_repeat_bshd_view
 * (:519-641) and softmax_inplace_view (:643-678).  q[B,S,Hq*D], k/v[B,S,Hkv*D].
 * RoPE on q,k at positions past..past+S (:334-335), slab write (:397-400), then per (b,head):
 * scores = Q K^T (k-ordered dot; third-party GEMM in the reference), *scale, mask
 * j > past+i -> -inf, max, exp, sum, * 1/(sum + 1e-9), ctx = P V (j-ordered, masked terms are
 * exact zeros).  out is [B,S,Hq,D].
 */
static int FN(attn_prefill_rr)(const REAL *q, const REAL *k, const REAL *v, long s, FN(lo_kv) *c, long hq,
                               float scale, int causal, const REAL *cos_t, const REAL *sin_t,
                               long rope_max, REAL *out) {
    long b = c->b, hkv = c->h_kv, d = c->d, max_seq = c->max_seq;
    long past = c->len, total = past + s, n_rep = hq / hkv;
    if (past + s > rope_max) return -1; /* rope.forward runs first (:334) */
    if (total > max_seq) return -2;
    REAL *qrot = (REAL *)malloc(sizeof(REAL) * (size_t)(b * s * hq * d)); /* [B,S,Hq,D] */
#pragma omp parallel for collapse(2) schedule(static)
    for (long bb = 0; bb < b; ++bb)
        for (long ss = 0; ss < s; ++ss) {
            for (long hh = 0; hh < hq; ++hh)
                FN(rope_1token_rr)(q + ((bb * s + ss) * hq + hh) * d, qrot + ((bb * s + ss) * hq + hh) * d, d,
                                   past + ss, rope_max, cos_t, sin_t);
            for (long hk = 0; hk < hkv; ++hk) {
                REAL *dk = c->k + ((bb * hkv + hk) * max_seq + past + ss) * d;
                REAL *dv = c->v + ((bb * hkv + hk) * max_seq + past + ss) * d;
                FN(rope_1token_rr)(k + ((bb * s + ss) * hkv + hk) * d, dk, d, past + ss, rope_max, cos_t, sin_t);
                memcpy(dv, v + ((bb * s + ss) * hkv + hk) * d, sizeof(REAL) * (size_t)d);
            }
        }
    c->len = total;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (long hh = 0; hh < hq; ++hh)
        for (long bb = 0; bb < b; ++bb) {
            long hk = hh / n_rep;
            const REAL *ks = c->k + (bb * hkv + hk) * max_seq * d;
            const REAL *vs = c->v + (bb * hkv + hk) * max_seq * d;
            REAL *sc = (REAL *)malloc(sizeof(REAL) * (size_t)total);
            for (long i = 0; i < s; ++i) {
                const REAL *qr = qrot + ((bb * s + i) * hq + hh) * d;
                long q_abs = past + i;
                for (long j = 0; j < total; ++j) {
                    REAL dot = 0;
                    for (long t = 0; t < d; ++t) { REAL p = qr[t] * ks[j * d + t]; dot += p; }
                    REAL val = dot * (REAL)scale;
                    if (causal && j > q_abs) val = -INFINITY;
                    sc[j] = val;
                }
                REAL mx = -INFINITY;
                for (long j = 0; j < total; ++j) if (sc[j] > mx) mx = sc[j];
                REAL sum = 0;
                for (long j = 0; j < total; ++j) { REAL e = FN(r_exp)(sc[j] - mx); sc[j] = e; sum += e; }
                REAL inv = (REAL)1 / (sum + (sizeof(REAL) == 4 ? (REAL)1e-9f : (REAL)1e-9));
                for (long j = 0; j < total; ++j) sc[j] *= inv;
                REAL *o = out + ((bb * s + i) * hq + hh) * d;
                for (long t = 0; t < d; ++t) {
                    REAL acc = 0;
                    for (long j = 0; j < total; ++j) { REAL p = sc[j] * vs[j * d + t]; acc += p; }
                    o[t] = acc;
                }
            }
            free(sc);
        }
    free(qrot);
    return 0;
}

/*
 * Standalone attention entry for tests: q[B,S,Hq*D], k/v[B,S,Hkv*D] as f32; dispatches like
 * SelfAttention::forward after the projections (S==1 -> decode path, else prefill path).
 * q_norm/k_norm may be NULL.
 */
int FN(lo_attention)(const float *q, const float *k, const float *v, long s, FN(lo_kv) *c, long hq,
                     float theta, long rope_max, int causal, const float *q_norm, const float *k_norm,
                     float norm_eps, REAL *out) {
    long b = c->b, hkv = c->h_kv, d = c->d;
    long nq = b * s * hq * d, nk = b * s * hkv * d;
    REAL *qr = (REAL *)malloc(sizeof(REAL) * (size_t)nq);
    REAL *kr = (REAL *)malloc(sizeof(REAL) * (size_t)nk);
    REAL *vr = (REAL *)malloc(sizeof(REAL) * (size_t)nk);
    REAL *ct = (REAL *)malloc(sizeof(REAL) * (size_t)(rope_max * d));
    REAL *st = (REAL *)malloc(sizeof(REAL) * (size_t)(rope_max * d));
    for (long i = 0; i < nq; ++i) qr[i] = (REAL)q[i];
    for (long i = 0; i < nk; ++i) { kr[i] = (REAL)k[i]; vr[i] = (REAL)v[i]; }
    FN(head_norm)(qr, b * s * hq, d, q_norm, norm_eps);
    FN(head_norm)(kr, b * s * hkv, d, k_norm, norm_eps);
    FN(lo_rope_table)(d, rope_max, theta, ct, st);
    float scale = 1.0f / sqrtf((float)d); /* (head_dim as f32).sqrt().recip(), self_attention.rs:89 */
    int rc = (s == 1) ? FN(attn_decode_rr)(qr, kr, vr, c, hq, scale, causal, ct, st, rope_max, out)
                      : FN(attn_prefill_rr)(qr, kr, vr, s, c, hq, scale, causal, ct, st, rope_max, out);
    free(qr); free(kr); free(vr); free(ct); free(st);
    return rc;
}

/* ---- model (src/models/llama.rs) ------------------------------------------------------ */
typedef struct {
    lo_config cfg;
    long head_dim;
    const float *embed, *final_norm, *lm_head;
    const float **wq, **wk, **wv, **wo, **wgate, **wup, **wdown, **norm1, **norm2, **qn, **kn;
    REAL *cos_t, *sin_t;
} FN(lo_llama);

FN(lo_llama) *FN(lo_llama_new)(const lo_config *cfg) {
    FN(lo_llama) *m = (FN(lo_llama) *)calloc(1, sizeof(*m));
    m->cfg = *cfg;
    /* head_dim = hidden/heads (llama.rs:162, self_attention.rs:75) unless overridden (Qwen3). */
    m->head_dim = cfg->head_dim > 0 ? cfg->head_dim : cfg->hidden / cfg->heads;
    long L = cfg->layers;
    const float ***arr[] = {&m->wq, &m->wk, &m->wv, &m->wo, &m->wgate, &m->wup, &m->wdown,
                            &m->norm1, &m->norm2, &m->qn, &m->kn};
    for (unsigned i = 0; i < sizeof(arr) / sizeof(arr[0]); ++i) *arr[i] = (const float **)calloc((size_t)L, sizeof(float *));
    m->cos_t = (REAL *)malloc(sizeof(REAL) * (size_t)(cfg->max_seq * m->head_dim));
    m->sin_t = (REAL *)malloc(sizeof(REAL) * (size_t)(cfg->max_seq * m->head_dim));
    FN(lo_rope_table)(m->head_dim, cfg->max_seq, cfg->theta, m->cos_t, m->sin_t);
    return m;
}

void FN(lo_llama_free)(FN(lo_llama) *m) {
    if (!m) return;
    free(m->wq); free(m->wk); free(m->wv); free(m->wo); free(m->wgate); free(m->wup); free(m->wdown);
    free(m->norm1); free(m->norm2); free(m->qn); free(m->kn); free(m->cos_t); free(m->sin_t); free(m);
}

/* Parameter names are the Hugging Face names of LlamaModel::named_parameters, llama.rs:218-279
 * (+ self_attn.q_norm / k_norm for the Qwen3 variant).  The pointer is borrowed. */
int FN(lo_llama_set_param)(FN(lo_llama) *m, const char *name, const float *p) {
    if (!strcmp(name, "model.embed_tokens.weight")) { m->embed = p; return 0; }
    if (!strcmp(name, "model.norm.weight")) { m->final_norm = p; return 0; }
    if (!strcmp(name, "lm_head.weight")) { m->lm_head = p; return 0; }
    long li; char rest[128];
    if (sscanf(name, "model.layers.%ld.%127s", &li, rest) != 2 || li < 0 || li >= m->cfg.layers) return -1;
    struct { const char *n; const float **a; } tab[] = {
        {"self_attn.q_proj.weight", m->wq}, {"self_attn.k_proj.weight", m->wk},
        {"self_attn.v_proj.weight", m->wv}, {"self_attn.o_proj.weight", m->wo},
        {"mlp.gate_proj.weight", m->wgate}, {"mlp.up_proj.weight", m->wup},
        {"mlp.down_proj.weight", m->wdown}, {"input_layernorm.weight", m->norm1},
        {"post_attention_layernorm.weight", m->norm2}, {"self_attn.q_norm.weight", m->qn},
        {"self_attn.k_norm.weight", m->kn}};
    for (unsigned i = 0; i < sizeof(tab) / sizeof(tab[0]); ++i)
        if (!strcmp(rest, tab[i].n)) { tab[i].a[li] = p; return 0; }
    return -1;
}

/*
 * LlamaModel::forward — llama.rs:181-206; layer = LlamaDecoderLayer::forward_infer
 * (:104-116); MLP = LlamaMLP::forward (:59-65).  ids[B,S] are f32 token ids; caches is an
 * array of `layers` KV caches; logits[B,S,V] (lm_head on every position, :202-205).
 * Returns 0, -1 (RoPE range), -2 (KV overflow), -3 (embedding id out of range).
 */
int FN(lo_llama_forward)(FN(lo_llama) *m, const float *ids, long b, long s, FN(lo_kv) **caches, REAL *logits) {
    const lo_config *cf = &m->cfg;
    long H = cf->hidden, I = cf->inter, hq = cf->heads, hkv = cf->kv_heads, d = m->head_dim;
    long M = b * s, qd = hq * d, kvd = hkv * d;
    float scale = 1.0f / sqrtf((float)d);
    REAL *x = (REAL *)malloc(sizeof(REAL) * (size_t)(M * H));
    REAL *nx = (REAL *)malloc(sizeof(REAL) * (size_t)(M * H));
    REAL *q = (REAL *)malloc(sizeof(REAL) * (size_t)(M * qd));
    REAL *k = (REAL *)malloc(sizeof(REAL) * (size_t)(M * kvd));
    REAL *v = (REAL *)malloc(sizeof(REAL) * (size_t)(M * kvd));
    REAL *att = (REAL *)malloc(sizeof(REAL) * (size_t)(M * qd));
    REAL *proj = (REAL *)malloc(sizeof(REAL) * (size_t)(M * H));
    REAL *gate = (REAL *)malloc(sizeof(REAL) * (size_t)(M * I));
    REAL *up = (REAL *)malloc(sizeof(REAL) * (size_t)(M * I));
    int rc = FN(lo_embedding)(ids, M, m->embed, cf->vocab, H, x) ? -3 : 0;
    for (long l = 0; rc == 0 && l < cf->layers; ++l) {
        FN(rmsnorm_rr)(x, M, H, m->norm1[l], cf->eps, nx);
        FN(matmul_rr)(nx, M, H, m->wq[l], qd, q);
        FN(matmul_rr)(nx, M, H, m->wk[l], kvd, k);
        FN(matmul_rr)(nx, M, H, m->wv[l], kvd, v);
        if (cf->qk_norm) {
            FN(head_norm)(q, M * hq, d, m->qn[l], cf->eps);
            FN(head_norm)(k, M * hkv, d, m->kn[l], cf->eps);
        }
        rc = (s == 1) ? FN(attn_decode_rr)(q, k, v, caches[l], hq, scale, 1, m->cos_t, m->sin_t, cf->max_seq, att)
                      : FN(attn_prefill_rr)(q, k, v, s, caches[l], hq, scale, 1, m->cos_t, m->sin_t, cf->max_seq, att);
        if (rc) break;
        FN(matmul_rr)(att, M, qd, m->wo[l], H, proj);
        for (long i = 0; i < M * H; ++i) x[i] = x[i] + proj[i];            /* llama.rs:110 */
        FN(rmsnorm_rr)(x, M, H, m->norm2[l], cf->eps, nx);                 /* :113 */
        FN(matmul_rr)(nx, M, H, m->wgate[l], I, gate);
        FN(matmul_rr)(nx, M, H, m->wup[l], I, up);
#pragma omp parallel for schedule(static)
        for (long i = 0; i < M * I; ++i) gate[i] = FN(silu1)(gate[i]) * up[i]; /* llama.rs:61-63 */
        FN(matmul_rr)(gate, M, I, m->wdown[l], H, proj);
        for (long i = 0; i < M * H; ++i) x[i] = x[i] + proj[i];            /* :115 */
    }
    if (rc == 0) {
        FN(rmsnorm_rr)(x, M, H, m->final_norm, cf->eps, nx);
        FN(matmul_rr)(nx, M, H, m->lm_head, cf->vocab, logits);
    }
    free(x); free(nx); free(q); free(k); free(v); free(att); free(proj); free(gate); free(up);
    return rc;
}

#undef FN
#undef CAT
#undef CAT_
