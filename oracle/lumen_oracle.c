/*
 * TEST INFRASTRUCTURE — not part of the shipped library.
 *
 * CPU restatement (plain C + OpenMP) of the inference path of chen-197/Lumen, used only as
 * the parity checker by the test-suite, by the GPU smoke test and as the timed CPU baseline
 * of the benchmark.  Nothing in the product library links or calls it.
 *
 * PARITY UNPINNED: the reference has no tests, golden vectors or fixtures, and it cannot be
 * built where this was written (Rust, no toolchain), so these functions are pinned by the
 * reference's source text only; see lumen_oracle_impl.h for the per-function citations.
 *
 * Build (see Makefile): gcc -O2 -fopenmp -ffp-contract=off -fno-fast-math.
 * -ffp-contract=off matters: Rust never fuses `sum += w * x` into an FMA, and GCC would.
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* The nine fields of LlamaConfig (src/models/llama.rs:11-21) plus two the reference lacks:
 * head_dim (0 = hidden/heads) and qk_norm (Qwen3 per-head q/k RMSNorm). */
typedef struct {
    long vocab, hidden, inter, layers, heads, kv_heads;
    float eps;
    long max_seq;
    float theta;
    long head_dim;
    int qk_norm;
} lo_config;

#define REAL float
#define SFX _f32
#include "lumen_oracle_impl.h"
#undef REAL
#undef SFX

#define REAL double
#define SFX _f64
#include "lumen_oracle_impl.h"
#undef REAL
#undef SFX

/*
 * LlamaKVCache — src/kv_cache.rs:5-59.  [1,Hkv,max_seq,D] f32 slabs.
 * update (:31-49): copies k,v [1,Hkv,S,D] into rows start_pos..start_pos+S, panics on
 * overflow (:34-36) -> returns -2.  get_view (:51-59): owned copies of the first n rows.
 */
typedef struct {
    long head_num, max_seq_len, dim;
    float *k, *v;
} lo_llama_kv;

lo_llama_kv *lo_llama_kv_new(long kv_heads, long max_seq, long head_dim) {
    lo_llama_kv *c = (lo_llama_kv *)calloc(1, sizeof(*c));
    c->head_num = kv_heads; c->max_seq_len = max_seq; c->dim = head_dim;
    c->k = (float *)calloc((size_t)(kv_heads * max_seq * head_dim), sizeof(float));
    c->v = (float *)calloc((size_t)(kv_heads * max_seq * head_dim), sizeof(float));
    return c;
}
void lo_llama_kv_free(lo_llama_kv *c) { if (c) { free(c->k); free(c->v); free(c); } }

int lo_llama_kv_update(lo_llama_kv *c, const float *k, const float *v, long s, long start_pos) {
    long end = start_pos + s;
    if (end > c->max_seq_len) return -2;
    for (long h = 0; h < c->head_num; ++h) {
        memcpy(c->k + (h * c->max_seq_len + start_pos) * c->dim, k + h * s * c->dim, sizeof(float) * (size_t)(s * c->dim));
        memcpy(c->v + (h * c->max_seq_len + start_pos) * c->dim, v + h * s * c->dim, sizeof(float) * (size_t)(s * c->dim));
    }
    return 0;
}

void lo_llama_kv_get_view(const lo_llama_kv *c, long n, float *k_out, float *v_out) {
    for (long h = 0; h < c->head_num; ++h) {
        memcpy(k_out + h * n * c->dim, c->k + h * c->max_seq_len * c->dim, sizeof(float) * (size_t)(n * c->dim));
        memcpy(v_out + h * n * c->dim, c->v + h * c->max_seq_len * c->dim, sizeof(float) * (size_t)(n * c->dim));
    }
}

/* Round-to-nearest-even f32 -> bf16 -> f32, the value a bf16 safetensors weight takes after
 * the loader's upcast (src/loader.rs:50-64 upcasts; the rounding is how such a file is made). */
void lo_round_bf16(const float *x, long n, float *out) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; ++i) {
        unsigned u; memcpy(&u, &x[i], 4);
        if ((u & 0x7fffffffu) > 0x7f800000u) { u |= 0x00400000u; u &= 0xffff0000u; }
        else { u += 0x7fffu + ((u >> 16) & 1u); u &= 0xffff0000u; }
        memcpy(&out[i], &u, 4);
    }
}

/* sample_top_p (src/main.rs:74-137) with the uniform draw `r` passed in (the reference draws it from its
 * thread RNG, :69-72): repetition penalty over the recent tokens (one division per occurrence), temperature
 * (floored at 1e-5), softmax with sequential f32 sums and 1/(sum + 1e-9), stable descending sort, nucleus cut
 * at the first rank where the sequential cumulative sum reaches top_p (clamped to [1e-6, 1]), then the
 * inverse-CDF walk over probs[i] / cumulative. */
typedef struct { float p; long i; } lo_pi;
static int lo_pi_cmp(const void *a, const void *b) {
    const lo_pi *x = (const lo_pi *)a, *y = (const lo_pi *)b;
    if (x->p > y->p) return -1;
    if (x->p < y->p) return 1;
    return (x->i > y->i) - (x->i < y->i); /* stable: ties keep index order */
}
long lo_sample_top_p(const float *logits, long n, float temperature, float top_p, float repetition_penalty,
                     const long *recent, long n_recent, float r) {
    float *adj = (float *)malloc(sizeof(float) * (size_t)n);
    lo_pi *idx = (lo_pi *)malloc(sizeof(lo_pi) * (size_t)n);
    for (long i = 0; i < n; ++i) adj[i] = logits[i];
    if (repetition_penalty > 1.0f)
        for (long k = 0; k < n_recent; ++k)
            if (recent[k] >= 0 && recent[k] < n) adj[recent[k]] /= repetition_penalty;
    const float temp = temperature > 1e-5f ? temperature : 1e-5f;
    float maxv = -INFINITY;
    for (long i = 0; i < n; ++i) { adj[i] /= temp; if (adj[i] > maxv) maxv = adj[i]; }
    float sum = 0.0f;
    for (long i = 0; i < n; ++i) { adj[i] = expf(adj[i] - maxv); sum += adj[i]; }
    const float inv = 1.0f / (sum + 1e-9f);
    for (long i = 0; i < n; ++i) { adj[i] *= inv; idx[i].p = adj[i]; idx[i].i = i; }
    qsort(idx, (size_t)n, sizeof(lo_pi), lo_pi_cmp);
    float target = top_p < 0.0f ? 0.0f : (top_p > 1.0f ? 1.0f : top_p);
    if (target < 1e-6f) target = 1e-6f;
    float cumulative = 0.0f;
    long cut = 0;
    for (long k = 0; k < n; ++k) {
        cumulative += idx[k].p;
        cut = k + 1;
        if (cumulative >= target) break;
    }
    if (cut < 1) cut = 1;
    float acc = 0.0f;
    long out = idx[cut - 1].i;
    for (long k = 0; k < cut; ++k) {
        acc += idx[k].p / cumulative;
        if (r <= acc) { out = idx[k].i; break; }
    }
    free(adj);
    free(idx);
    return out;
}

int lo_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp single
        n = omp_get_num_threads();
    }
#endif
    return n;
}

/* Thread count of every later parallel loop, independent of OMP_NUM_THREADS (launchers such as
 * torchrun export OMP_NUM_THREADS=1 to their children); n <= 0 leaves it unchanged. */
void lo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
