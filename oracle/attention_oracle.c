/* attention_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C CPU restatement of scaled-dot-product attention exactly as it is
 * composed today from the reference's public operators on its C CPU backend:
 *
 *     O = softmax((Q @ K^T) * scale [+ mask], axis=-1) @ V
 *
 * Each step below names the reference code whose arithmetic it follows
 * (paths are relative to the reference project):
 *
 *   batched matmul, naive ijk with a DOUBLE accumulator, result cast to float
 *       src/tensor/operators_cpu.c:47-60 (matmul), :62-67 (matmul_batched)
 *   scalar multiply in fp32                src/tensor/operators.def:54
 *   broadcast add of a {0,-inf} mask       src/tensor/operators.def:65
 *   row max with fmaxf, left to right      src/tensor/operators_cpu.c:107-120
 *   broadcast subtract / divide            src/tensor/operators.def:66,68
 *   expf                                   src/tensor/operators.def:72
 *   row sum in fp32, left to right         src/tensor/operators_cpu.c:92-105
 *   softmax sequencing                     ember/tensor/tensor.py:430-437
 *
 * The reference has no attention operator, no log-sum-exp output and no
 * backward; the backward here is the manual-backward composition the
 * reference's layers use (ember/nn/layers.py:50-56 for the matmul pattern,
 * ember/loss/losses.py:53-56 for the softmax gradient):
 *
 *     dV = P^T @ dO ; dP = dO @ V^T ; delta = sum(dP * P, axis=-1)
 *     dS = (P * (dP - delta)) * scale ; dQ = dS @ K ; dK = dS^T @ Q
 *
 * Parity pin: this file is checked bit-for-bit against the reference's own
 * compiled C operators (oracle/_ref, built from the reference sources by the
 * Makefile beside this file) and against the committed golden vectors that
 * the reference's Python front-end produced (tests/golden/).
 *
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may link
 * or call this file. The shipped library never does.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>

static int g_threads = 1;

void oracle_set_threads(int n) { g_threads = n > 0 ? n : 1; }
int oracle_get_threads(void) { return g_threads; }

/* The reference is single-threaded. Slices (one per batch*head) are
 * independent, so the harness may spread them over host threads; the
 * arithmetic inside a slice is untouched. */
typedef void (*slice_fn)(int b, void *ctx);
typedef struct {
    slice_fn fn;
    void *ctx;
    int n;
    int next;
    pthread_mutex_t mu;
} pool_t;

static void *pool_worker(void *arg)
{
    pool_t *p = (pool_t *)arg;
    for (;;) {
        pthread_mutex_lock(&p->mu);
        int b = p->next++;
        pthread_mutex_unlock(&p->mu);
        if (b >= p->n) break;
        p->fn(b, p->ctx);
    }
    return NULL;
}

static void for_each_slice(int n, slice_fn fn, void *ctx)
{
    int nt = g_threads < n ? g_threads : n;
    if (nt <= 1) {
        for (int b = 0; b < n; b++) fn(b, ctx);
        return;
    }
    pool_t p = {fn, ctx, n, 0, PTHREAD_MUTEX_INITIALIZER};
    pthread_t *th = (pthread_t *)malloc((size_t)nt * sizeof(pthread_t));
    for (int t = 0; t < nt; t++) pthread_create(&th[t], NULL, pool_worker, &p);
    for (int t = 0; t < nt; t++) pthread_join(th[t], NULL);
    free(th);
}

/* out(n x m) = a(n x k) @ b(k x m); double accumulator, fp32 result.
 * Mirrors src/tensor/operators_cpu.c:47-60. */
static void mm(const float *a, const float *b, float *out, int n, int m, int k)
{
    for (int i = 0; i < n; i++) {
        for (int j = 0; j < m; j++) {
            double acc = 0.0;
            for (int l = 0; l < k; l++) acc += (double)a[(size_t)i * k + l] * (double)b[(size_t)l * m + j];
            out[(size_t)i * m + j] = (float)acc;
        }
    }
}

/* out(m x n) = a(n x m)^T. The reference transposes on the host (NumPy)
 * because its transpose is 2-D only (ember/tensor/tensor.py:376-384). */
static void tr(const float *a, float *out, int n, int m)
{
    for (int i = 0; i < n; i++)
        for (int j = 0; j < m; j++) out[(size_t)j * n + i] = a[(size_t)i * m + j];
}

/* Softmax probabilities of one (b,h) slice; s is overwritten by P.
 * mask semantics: key j is visible to query i iff j <= i + (lk - lq)
 * (lower-triangular, aligned to the bottom-right corner). */
static void scores_to_probs(float *s, float *row_max, float *row_sum, int lq, int lk, float scale,
                            int causal)
{
    const size_t n = (size_t)lq * lk;
    for (size_t i = 0; i < n; i++) s[i] = s[i] * scale; /* operators.def:54 */
    if (causal) {                                       /* operators.def:65 */
        const int off = lk - lq;
        for (int i = 0; i < lq; i++)
            for (int j = 0; j < lk; j++) {
                float mask = (j > i + off) ? -INFINITY : 0.0f;
                s[(size_t)i * lk + j] = s[(size_t)i * lk + j] + mask;
            }
    }
    for (int i = 0; i < lq; i++) {
        float *r = s + (size_t)i * lk;
        float m = r[0]; /* operators_cpu.c:107-120 */
        for (int j = 1; j < lk; j++) m = fmaxf(m, r[j]);
        for (int j = 0; j < lk; j++) r[j] = r[j] - m; /* operators.def:66 */
        for (int j = 0; j < lk; j++) r[j] = expf(r[j]); /* operators.def:72 */
        float sum = 0.0f; /* operators_cpu.c:92-105 */
        for (int j = 0; j < lk; j++) sum += r[j];
        for (int j = 0; j < lk; j++) r[j] = r[j] / sum; /* operators.def:68 */
        row_max[i] = m;
        row_sum[i] = sum;
    }
}

static void fwd_slice(const float *q, const float *k, const float *v, float *out, float *lse,
                      float *p_out, int lq, int lk, int d, float scale, int causal)
{
    float *kt = (float *)malloc((size_t)d * lk * sizeof(float));
    float *s = p_out ? p_out : (float *)malloc((size_t)lq * lk * sizeof(float));
    float *rm = (float *)malloc((size_t)lq * sizeof(float));
    float *rs = (float *)malloc((size_t)lq * sizeof(float));
    tr(k, kt, lk, d);
    mm(q, kt, s, lq, lk, d);
    scores_to_probs(s, rm, rs, lq, lk, scale, causal);
    mm(s, v, out, lq, d, lk);
    if (lse)
        for (int i = 0; i < lq; i++) lse[i] = (float)((double)rm[i] + log((double)rs[i]));
    free(kt);
    if (!p_out) free(s);
    free(rm);
    free(rs);
}

/* q: (bh, lq, d)  k,v: (bh, lk, d)  out: (bh, lq, d)  lse: (bh, lq) or NULL
 * p_out: (bh, lq, lk) or NULL. All contiguous row-major fp32. */
typedef struct {
    const float *q, *k, *v, *dout;
    float *out, *lse, *p_out, *dq, *dk, *dv;
    int lq, lk, d, causal;
    float scale;
} args_t;

static void fwd_one(int b, void *ctx)
{
    args_t *a = (args_t *)ctx;
    const int lq = a->lq, lk = a->lk, d = a->d;
    fwd_slice(a->q + (size_t)b * lq * d, a->k + (size_t)b * lk * d, a->v + (size_t)b * lk * d,
              a->out + (size_t)b * lq * d, a->lse ? a->lse + (size_t)b * lq : NULL,
              a->p_out ? a->p_out + (size_t)b * lq * lk : NULL, lq, lk, d, a->scale, a->causal);
}

void oracle_attention_fwd(const float *q, const float *k, const float *v, float *out, float *lse,
                          float *p_out, int bh, int lq, int lk, int d, float scale, int causal)
{
    args_t a = {q, k, v, NULL, out, lse, p_out, NULL, NULL, NULL, lq, lk, d, causal, scale};
    for_each_slice(bh, fwd_one, &a);
}

static void bwd_slice(const float *q, const float *k, const float *v, const float *dout, float *dq,
                      float *dk, float *dv, int lq, int lk, int d, float scale, int causal)
{
    const size_t nS = (size_t)lq * lk;
    float *kt = (float *)malloc((size_t)d * lk * sizeof(float));
    float *vt = (float *)malloc((size_t)d * lk * sizeof(float));
    float *p = (float *)malloc(nS * sizeof(float));
    float *pt = (float *)malloc(nS * sizeof(float));
    float *dp = (float *)malloc(nS * sizeof(float));
    float *rm = (float *)malloc((size_t)lq * sizeof(float));
    float *rs = (float *)malloc((size_t)lq * sizeof(float));

    /* forward recompute of P */
    tr(k, kt, lk, d);
    mm(q, kt, p, lq, lk, d);
    scores_to_probs(p, rm, rs, lq, lk, scale, causal);

    /* dV = P^T @ dO */
    tr(p, pt, lq, lk);
    mm(pt, dout, dv, lk, d, lq);

    /* dP = dO @ V^T */
    tr(v, vt, lk, d);
    mm(dout, vt, dp, lq, lk, d);

    /* delta = sum(dP * P, axis=-1); dS = (P * (dP - delta)) * scale */
    for (int i = 0; i < lq; i++) {
        float *pr = p + (size_t)i * lk, *dpr = dp + (size_t)i * lk;
        float delta = 0.0f;
        for (int j = 0; j < lk; j++) {
            float prod = dpr[j] * pr[j]; /* operators.def:42 */
            delta += prod;               /* operators_cpu.c:92-105 */
        }
        for (int j = 0; j < lk; j++) {
            float t = dpr[j] - delta; /* operators.def:66 */
            t = pr[j] * t;            /* operators.def:42 */
            dpr[j] = t * scale;       /* operators.def:54 */
        }
    }

    /* dQ = dS @ K ; dK = dS^T @ Q */
    mm(dp, k, dq, lq, d, lk);
    tr(dp, pt, lq, lk);
    mm(pt, q, dk, lk, d, lq);

    free(kt);
    free(vt);
    free(p);
    free(pt);
    free(dp);
    free(rm);
    free(rs);
}

static void bwd_one(int b, void *ctx)
{
    args_t *a = (args_t *)ctx;
    const int lq = a->lq, lk = a->lk, d = a->d;
    bwd_slice(a->q + (size_t)b * lq * d, a->k + (size_t)b * lk * d, a->v + (size_t)b * lk * d,
              a->dout + (size_t)b * lq * d, a->dq + (size_t)b * lq * d, a->dk + (size_t)b * lk * d,
              a->dv + (size_t)b * lk * d, lq, lk, d, a->scale, a->causal);
}

void oracle_attention_bwd(const float *q, const float *k, const float *v, const float *dout,
                          float *dq, float *dk, float *dv, int bh, int lq, int lk, int d,
                          float scale, int causal)
{
    args_t a = {q, k, v, dout, NULL, NULL, NULL, dq, dk, dv, lq, lk, d, causal, scale};
    for_each_slice(bh, bwd_one, &a);
}

/* ------------------------------------------------------------------------
 * The layer either side of attention: the reference's Linear
 * (ember/nn/layers.py:45-56).
 *
 *     forward   y      = b + x @ w             x (m,k), w (k,n), b (n)
 *     backward  grad_w = x^T @ grad_y          transpose on the host, then matmul
 *               grad_b = sum(grad_y, axis=0)   fp32, rows added top to bottom
 *               grad_x = grad_y @ w^T
 *
 * matmul: src/tensor/operators_cpu.c:47-60 (double accumulator); broadcast add:
 * src/tensor/operators.def:65; sum over axis 0: src/tensor/operators_cpu.c:92-105.
 * Rows of the result are independent, so the worker pool splits them in blocks.
 * ------------------------------------------------------------------------ */
typedef struct {
    const float *a, *b, *bias;
    float *out;
    int n, m, k, rows_per_block;
} mm_args_t;

static void mm_block(int blk, void *ctx)
{
    const mm_args_t *g = (const mm_args_t *)ctx;
    const int r0 = blk * g->rows_per_block;
    const int r1 = r0 + g->rows_per_block < g->n ? r0 + g->rows_per_block : g->n;
    mm(g->a + (size_t)r0 * g->k, g->b, g->out + (size_t)r0 * g->m, r1 - r0, g->m, g->k);
    if (g->bias)
        for (int i = r0; i < r1; i++)
            for (int j = 0; j < g->m; j++) g->out[(size_t)i * g->m + j] = g->bias[j] + g->out[(size_t)i * g->m + j];
}

static void mm_threaded(const float *a, const float *b, const float *bias, float *out, int n, int m, int k)
{
    mm_args_t g = {a, b, bias, out, n, m, k, 8};
    for_each_slice((n + g.rows_per_block - 1) / g.rows_per_block, mm_block, &g);
}

void oracle_linear_fwd(const float *x, const float *w, const float *b, float *y, int m, int n, int k)
{
    mm_threaded(x, w, b, y, m, n, k);
}

void oracle_linear_bwd(const float *x, const float *w, const float *dy, float *dx, float *dw, float *db,
                       int m, int n, int k)
{
    float *xt = (float *)malloc((size_t)m * k * sizeof(float));
    float *wt = (float *)malloc((size_t)k * n * sizeof(float));
    tr(x, xt, m, k);                      /* (k, m) */
    tr(w, wt, k, n);                      /* (n, k) */
    mm_threaded(xt, dy, NULL, dw, k, n, m);
    for (int j = 0; j < n; j++) {
        float s = 0.0f;
        for (int r = 0; r < m; r++) s += dy[(size_t)r * n + j];
        db[j] = s;
    }
    mm_threaded(dy, wt, NULL, dx, m, k, n);
    free(xt);
    free(wt);
}

/* ------------------------------------------------------------------------
 * Softmax over the last axis and the softmax cross-entropy loss, as the
 * reference composes them from its operators.
 *
 *   softmax (ember/tensor/tensor.py:430-437):
 *       shifted = a - amax(a, -1, keepdims) ; e = exp(shifted) ; e / sum(e, -1, keepdims)
 *   CrossEntropyLoss.forward (ember/loss/losses.py:42-51):
 *       shifted   = pred - amax(pred, -1, keepdims)
 *       log_probs = shifted - log(sum(exp(shifted), -1, keepdims))
 *       probs     = exp(log_probs)
 *       loss      = -sum(target * log_probs) / n          n = rows; sum() over ALL elements
 *   CrossEntropyLoss.backward (losses.py:53-56):  (probs - target) / n
 *
 * amax: fmaxf left to right (src/tensor/operators_cpu.c:107-120); row sums fp32
 * left to right (:92-105); the loss sum is the flat fp32 sum (:78-83), negated
 * and divided in Python floats (double); "/ n" in backward is a float divide by
 * (float)n (src/tensor/operators.def:58).
 * ------------------------------------------------------------------------ */
void oracle_softmax(const float *x, float *y, int rows, int cols)
{
    for (int r = 0; r < rows; r++) {
        const float *a = x + (size_t)r * cols;
        float *o = y + (size_t)r * cols;
        float m = a[0];
        for (int j = 1; j < cols; j++) m = fmaxf(m, a[j]);
        float s = 0.0f;
        for (int j = 0; j < cols; j++) {
            o[j] = expf(a[j] - m);
            s += o[j];
        }
        for (int j = 0; j < cols; j++) o[j] = o[j] / s;
    }
}

double oracle_cross_entropy_fwd(const float *pred, const float *target, float *probs, int rows, int cols)
{
    float total = 0.0f;
    for (int r = 0; r < rows; r++) {
        const float *a = pred + (size_t)r * cols, *t = target + (size_t)r * cols;
        float *p = probs + (size_t)r * cols;
        float m = a[0];
        for (int j = 1; j < cols; j++) m = fmaxf(m, a[j]);
        float s = 0.0f;
        for (int j = 0; j < cols; j++) s += expf(a[j] - m);
        const float lg = logf(s);
        for (int j = 0; j < cols; j++) {
            const float lp = (a[j] - m) - lg;
            p[j] = expf(lp);
            total += t[j] * lp;
        }
    }
    return -(double)total / (double)rows;
}

void oracle_cross_entropy_bwd(const float *probs, const float *target, float *grad, int rows, int cols)
{
    const float n = (float)rows;
    const size_t total = (size_t)rows * cols;
    for (size_t i = 0; i < total; i++) grad[i] = (probs[i] - target[i]) / n;
}
