/* ref_driver.c -- times the REFERENCE's own CPU functions on the MoE-FFN decode
 * path.  TEST / BASELINE INFRASTRUCTURE ONLY; never part of the shipped library.
 *
 * This file contains no arithmetic of its own on the projection path: it calls
 * the functions of oracle/_ref/libsalt_ref.so (the reference sources compiled
 * unmodified) in the order the reference adapter does for one decode step
 * (models/gemma4-26b-a4b/src/gemma4_text.c:8344-8363 and 7908-8064):
 *   salt_gemma4_router_input -> salt_router_scores -> salt_gemma4_router_topk
 *   -> ascending-expert sort -> per selected expert: salt_simd_q4_matvec
 *   (gate, up) -> salt_gemma4_gelu_tanh(gate)*up -> salt_simd_q4_matvec (down)
 *   -> output += expert_output * weight.
 * Rows of each projection are partitioned over a persistent pthread pool; the
 * reference states that row partitioning changes ownership only, never the
 * order of operations (src/kernels.c:289-290).
 */
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* reference prototypes (include/salt/simd.h:60-62, kernels.h, gemma4.h) */
void salt_simd_q4_matvec(const uint32_t *vals, const uint16_t *scales, const uint16_t *biases, int R, int C,
                         const float *x, float *y, int r0, int r1);
void salt_router_scores(const float *W, const float *bias, int E, int H, const float *x, float *scores);
int salt_gemma4_router_input(float *out, const float *state, const float *scale, int hidden, float eps);
int salt_gemma4_router_topk(const float *logits, const float *per_expert_scale, int n_experts, int topk,
                            int *selected, float *weights);
float salt_gemma4_gelu_tanh(float x);
int salt_gemma4_rmsnorm(float *out, const float *x, const float *weight, int n, float eps, int with_scale);

typedef struct {
    int hidden, inter, n_experts, topk;
    float eps;
    const float *router_w, *router_scale, *per_expert_scale;
    const uint8_t *pool;
    size_t expert_stride;
} RefLayer;

typedef struct {
    const uint32_t *vals;
    const uint16_t *scales, *biases;
    int R, C;
    const float *x;
    float *y;
} RefTask;

/* ---- a small persistent pool: workers take row chunks of a task list ---- */
typedef struct {
    pthread_t *threads;
    int n;
    pthread_mutex_t mu;
    pthread_cond_t go, done;
    const RefTask *tasks;
    int ntasks, chunk_rows;
    int next_chunk, total_chunks, finished, generation, stop;
    int *chunk_task, *chunk_r0;
} RefPool;

static RefPool g_pool;

static void run_chunk(const RefPool *p, int c) {
    const RefTask *t = &p->tasks[p->chunk_task[c]];
    int r0 = p->chunk_r0[c], r1 = r0 + p->chunk_rows;
    if (r1 > t->R) r1 = t->R;
    salt_simd_q4_matvec(t->vals, t->scales, t->biases, t->R, t->C, t->x, t->y, r0, r1);
}

static void *worker(void *arg) {
    RefPool *p = (RefPool *)arg;
    int seen = 0;
    pthread_mutex_lock(&p->mu);
    for (;;) {
        while (!p->stop && p->generation == seen) pthread_cond_wait(&p->go, &p->mu);
        if (p->stop) break;
        seen = p->generation;
        while (p->next_chunk < p->total_chunks) {
            int c = p->next_chunk++;
            pthread_mutex_unlock(&p->mu);
            run_chunk(p, c);
            pthread_mutex_lock(&p->mu);
            if (++p->finished == p->total_chunks) pthread_cond_signal(&p->done);
        }
    }
    pthread_mutex_unlock(&p->mu);
    return NULL;
}

int refdrv_pool_start(int threads) {
    RefPool *p = &g_pool;
    if (p->threads) return p->n;
    if (threads < 1) threads = 1;
    memset(p, 0, sizeof *p);
    pthread_mutex_init(&p->mu, NULL);
    pthread_cond_init(&p->go, NULL);
    pthread_cond_init(&p->done, NULL);
    p->threads = (pthread_t *)calloc((size_t)threads, sizeof(pthread_t));
    p->chunk_task = (int *)malloc(sizeof(int) * 65536);
    p->chunk_r0 = (int *)malloc(sizeof(int) * 65536);
    for (int i = 0; i < threads - 1; i++)   /* the caller is the last worker */
        if (pthread_create(&p->threads[p->n], NULL, worker, p) == 0) p->n++;
    p->n += 1;
    return p->n;
}

void refdrv_pool_stop(void) {
    RefPool *p = &g_pool;
    if (!p->threads) return;
    pthread_mutex_lock(&p->mu);
    p->stop = 1;
    pthread_cond_broadcast(&p->go);
    pthread_mutex_unlock(&p->mu);
    for (int i = 0; i < p->n - 1; i++) pthread_join(p->threads[i], NULL);
    free(p->threads); free(p->chunk_task); free(p->chunk_r0);
    memset(p, 0, sizeof *p);
}

static void run_tasks(const RefTask *tasks, int ntasks) {
    RefPool *p = &g_pool;
    int total_rows = 0, chunks = 0;
    for (int i = 0; i < ntasks; i++) total_rows += tasks[i].R;
    int chunk_rows = total_rows / (p->n * 4) + 1;
    if (chunk_rows < 8) chunk_rows = 8;
    for (int i = 0; i < ntasks; i++)
        for (int r = 0; r < tasks[i].R && chunks < 65536; r += chunk_rows) {
            p->chunk_task[chunks] = i;
            p->chunk_r0[chunks++] = r;
        }
    pthread_mutex_lock(&p->mu);
    p->tasks = tasks; p->ntasks = ntasks; p->chunk_rows = chunk_rows;
    p->next_chunk = 0; p->total_chunks = chunks; p->finished = 0;
    p->generation++;
    pthread_cond_broadcast(&p->go);
    while (p->next_chunk < p->total_chunks) {
        int c = p->next_chunk++;
        pthread_mutex_unlock(&p->mu);
        run_chunk(p, c);
        pthread_mutex_lock(&p->mu);
        ++p->finished;
    }
    while (p->finished < p->total_chunks) pthread_cond_wait(&p->done, &p->mu);
    pthread_mutex_unlock(&p->mu);
}

static void expert_tensor(const RefLayer *L, int e, int which, RefTask *t) {
    size_t elems = (size_t)L->hidden * (size_t)L->inter;
    size_t vb = elems / 2, gb = elems / 64 * 2;
    const uint8_t *base = L->pool + (size_t)e * L->expert_stride + (size_t)which * (vb + 2 * gb);
    t->vals = (const uint32_t *)(const void *)base;
    t->scales = (const uint16_t *)(const void *)(base + vb);
    t->biases = (const uint16_t *)(const void *)(base + vb + gb);
}

/* One MoE-FFN layer for B tokens; scratch is allocated per call (not timed
 * separately: it is a few hundred KB).  Returns 0, or -1 if a reference
 * function rejects its input. */
int refdrv_moe_layer_q4(const RefLayer *L, const float *x, int B, float *y, int *selected_out,
                        float *weights_out) {
    const int H = L->hidden, M = L->inter, E = L->n_experts, K = L->topk;
    const int jobs = B * K;
    int *sel = (int *)malloc(sizeof(int) * (size_t)jobs);
    float *w = (float *)malloc(sizeof(float) * (size_t)jobs);
    float *rin = (float *)malloc(sizeof(float) * (size_t)(H + E));
    float *gate = (float *)malloc(sizeof(float) * (size_t)jobs * (size_t)M * 2);
    float *up = gate + (size_t)jobs * M;
    float *down = (float *)malloc(sizeof(float) * (size_t)jobs * (size_t)H);
    RefTask *tasks = (RefTask *)malloc(sizeof(RefTask) * (size_t)jobs * 2);
    int rc = -1;
    if (!sel || !w || !rin || !gate || !down || !tasks) goto out;
    if (!g_pool.threads) refdrv_pool_start(1);
    for (int t = 0; t < B; t++) {
        int *s = sel + (size_t)t * K;
        float *wt = w + (size_t)t * K;
        if (salt_gemma4_router_input(rin, x + (size_t)t * H, L->router_scale, H, L->eps) != 0) goto out;
        salt_router_scores(L->router_w, NULL, E, H, rin, rin + H);
        if (salt_gemma4_router_topk(rin + H, L->per_expert_scale, E, K, s, wt) != 0) goto out;
        for (int a = 0; a < K; a++)            /* gemma4_text.c:8541-8550 */
            for (int b = a + 1; b < K; b++)
                if (s[b] < s[a]) {
                    int id = s[a]; s[a] = s[b]; s[b] = id;
                    float ww = wt[a]; wt[a] = wt[b]; wt[b] = ww;
                }
    }
    for (int j = 0; j < jobs; j++) {
        const float *xt = x + (size_t)(j / K) * H;
        expert_tensor(L, sel[j], 0, &tasks[2 * j]);
        tasks[2 * j].R = M; tasks[2 * j].C = H; tasks[2 * j].x = xt; tasks[2 * j].y = gate + (size_t)j * M;
        expert_tensor(L, sel[j], 1, &tasks[2 * j + 1]);
        tasks[2 * j + 1].R = M; tasks[2 * j + 1].C = H; tasks[2 * j + 1].x = xt;
        tasks[2 * j + 1].y = up + (size_t)j * M;
    }
    run_tasks(tasks, 2 * jobs);
    for (size_t i = 0; i < (size_t)jobs * M; i++) gate[i] = salt_gemma4_gelu_tanh(gate[i]) * up[i];
    for (int j = 0; j < jobs; j++) {
        expert_tensor(L, sel[j], 2, &tasks[j]);
        tasks[j].R = H; tasks[j].C = M; tasks[j].x = gate + (size_t)j * M; tasks[j].y = down + (size_t)j * H;
    }
    run_tasks(tasks, jobs);
    for (int t = 0; t < B; t++) {
        float *yt = y + (size_t)t * H;
        memset(yt, 0, sizeof(float) * (size_t)H);
        for (int k = 0; k < K; k++) {          /* gemma4_text.c:8060-8064 */
            const float *o = down + ((size_t)t * K + k) * H;
            float weight = w[(size_t)t * K + k];
            for (int d = 0; d < H; d++) yt[d] += o[d] * weight;
        }
    }
    if (selected_out) memcpy(selected_out, sel, sizeof(int) * (size_t)jobs);
    if (weights_out) memcpy(weights_out, w, sizeof(float) * (size_t)jobs);
    rc = 0;
out:
    free(sel); free(w); free(rin); free(gate); free(down); free(tasks);
    return rc;
}

/* RMSNorm between layers of the stacked configuration (gemma4.c:85-101). */
int refdrv_rmsnorm_rows(float *out, const float *x, const float *weight, int rows, int n, float eps) {
    for (int r = 0; r < rows; r++)
        if (salt_gemma4_rmsnorm(out + (size_t)r * n, x + (size_t)r * n, weight, n, eps, 1) != 0) return -1;
    return 0;
}
