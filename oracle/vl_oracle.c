/*
 * CPU oracle for the VectorLink ANN hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the reference's algorithm
 * (vectorlink_gpu/kernels.py, queue.py, utils.py, ann.py).  It is the checker
 * the CUDA path is compared with; the product never links or calls it.  Only
 * the test-suite, the smoke check and the CPU-baseline leg of the benchmark
 * may load the library built from this file.
 *
 * Parity status: pinned.  The kernel restatements below are checked against
 * outputs of the reference's own Numba kernels executed under the Numba CUDA
 * simulator, and the driver restatements against the reference's own
 * queue.py / utils.py / ann.py executed on CPU; both sets of outputs are
 * committed as fixtures under tests/golden/ with the script that made them.
 * The squared-L2 metric does not exist in the reference: for it parity is
 * unpinned and the oracle is the same summation tree applied to (a-b)^2.
 *
 * Every function cites the reference lines it follows.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define VLO_MAXINT 2147483647            /* constants.py:5 */
static const float VLO_MAXFLOAT = 3.4028e37f; /* constants.py:6 (rounded to fp32) */

#define VLO_COSINE 0
#define VLO_SQL2 1

/* ------------------------------------------------------------------------
 * Distance arithmetic: kernels.py:85-114 (cosine_distance), 38-72 (sum),
 * 27-35 (warp_reduce).
 *
 * Products are stored one per slot of a shared buffer (so no FMA can form),
 * slots 1024*k+t are folded onto slot t in increasing k (kernels.py:43-47),
 * then slot t is added to slot t+h for h = 512, 256, ..., 1.  Slots at or
 * beyond the vector dimension hold zero (the reference reads them
 * uninitialised when dim < 1024; zero is the only well-defined reading), so
 * the halving tree can start at the first power of two >= min(dim,1024)
 * without changing a single bit of the result.
 * The result is (1 - sum) / 2 clamped to [0, 1] (kernels.py:107-113).
 * ---------------------------------------------------------------------- */
static float tree_sum(float *buf, int dim)
{
    int top = dim < 1024 ? dim : 1024;
    for (int k = 1; 1024 * k < dim; ++k) {
        int lim = dim - 1024 * k;
        if (lim > 1024) lim = 1024;
        for (int t = 0; t < lim; ++t) buf[t] = buf[t] + buf[1024 * k + t];
    }
    int p = 1;
    while (p < top) p <<= 1;
    for (int t = top; t < p; ++t) buf[t] = 0.0f;
    for (int h = p >> 1; h >= 1; h >>= 1)
        for (int t = 0; t < h; ++t) buf[t] = buf[t] + buf[t + h];
    return buf[0];
}

static float pair_distance(const float *a, const float *b, int dim, int metric, float *buf)
{
    if (metric == VLO_COSINE) {
        for (int i = 0; i < dim; ++i) buf[i] = a[i] * b[i];
        float c = tree_sum(buf, dim);
        float r = (1.0f - c) / 2.0f;
        if (r < 0.0f) r = 0.0f; else if (r > 1.0f) r = 1.0f;
        return r;
    }
    for (int i = 0; i < dim; ++i) { float d = a[i] - b[i]; buf[i] = d * d; }
    return tree_sum(buf, dim);
}

static int scratch_len(int dim)
{
    int n = dim < 1024 ? 1024 : dim;
    return n + 16;
}

float vlo_pair_distance(const float *a, const float *b, int dim, int metric)
{
    float *buf = (float *)malloc(sizeof(float) * scratch_len(dim));
    float r = pair_distance(a, b, dim, metric, buf);
    free(buf);
    return r;
}

/* kernels.py:130-171 / 174-201: out[i,j] = dist(vectors[i], vectors[beams[i,j]]),
 * MAXFLOAT where beams[i,j] == MAXINT. */
void vlo_calculate_distances(const float *vectors, int64_t n, int dim, const int32_t *beams,
                             int w, float *out, int metric)
{
#pragma omp parallel
    {
        float *buf = (float *)malloc(sizeof(float) * scratch_len(dim));
#pragma omp for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            for (int j = 0; j < w; ++j) {
                int32_t nb = beams[i * w + j];
                out[i * w + j] = (nb == VLO_MAXINT)
                                     ? VLO_MAXFLOAT
                                     : pair_distance(vectors + i * (int64_t)dim,
                                                     vectors + (int64_t)nb * dim, dim, metric, buf);
            }
        }
        free(buf);
    }
}

/* kernels.py:204-257 / 260-311: for query b, visited node v, slot j:
 * id = beams[visit[b,v], j]; idx_out[b, v*W+j] = id; dist_out = dist(vectors[id], q[b]);
 * sentinels when visit[b,v] == MAXINT.  A MAXINT neighbour id is unguarded in the
 * reference (it would index vectors out of range); the well-defined reading,
 * used here, is to emit the sentinels. */
void vlo_search_from_seeds(const float *queries, int64_t b_count, const int32_t *visit, int v_count,
                           const int32_t *beams, int w, const float *vectors, int64_t n, int dim,
                           int32_t *idx_out, float *dist_out, int metric)
{
    (void)n;
#pragma omp parallel
    {
        float *buf = (float *)malloc(sizeof(float) * scratch_len(dim));
#pragma omp for schedule(dynamic, 4)
        for (int64_t b = 0; b < b_count; ++b) {
            for (int v = 0; v < v_count; ++v) {
                int32_t node = visit[b * v_count + v];
                for (int j = 0; j < w; ++j) {
                    int64_t o = b * (int64_t)v_count * w + (int64_t)v * w + j;
                    int32_t nb = node == VLO_MAXINT ? VLO_MAXINT : beams[(int64_t)node * w + j];
                    if (nb == VLO_MAXINT) {
                        idx_out[o] = VLO_MAXINT;
                        dist_out[o] = VLO_MAXFLOAT;
                    } else {
                        idx_out[o] = nb;
                        dist_out[o] = pair_distance(vectors + (int64_t)nb * dim,
                                                    queries + b * (int64_t)dim, dim, metric, buf);
                    }
                }
            }
        }
        free(buf);
    }
}

/* kernels.py:471-488: every slot of the (possibly strided) view whose id occurs in the row's
 * exclusion list, scanned up to its first MAXINT, becomes MAXINT / MAXFLOAT. */
static void punchout_excluded_row(int32_t *ids, float *dist, int q, const int32_t *excl, int e)
{
    for (int s = 0; s < q; ++s) {
        int32_t v = ids[s];
        for (int i = 0; i < e; ++i) {
            int32_t x = excl[i];
            if (x == VLO_MAXINT) break;
            if (v == x) { ids[s] = VLO_MAXINT; dist[s] = VLO_MAXFLOAT; }
        }
    }
}

void vlo_punchout_excluded(int32_t *ids, float *dist, int64_t ld, int64_t b_count, int q,
                           const int32_t *excl, int e)
{
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < b_count; ++b)
        punchout_excluded_row(ids + b * ld, dist + b * ld, q, excl + b * (int64_t)e, e);
}

typedef struct { float d; int32_t id; } pair_t;

static int cmp_pair(const void *pa, const void *pb)
{
    const pair_t *a = (const pair_t *)pa, *b = (const pair_t *)pb;
    if (a->d < b->d) return -1;
    if (a->d > b->d) return 1;
    if (a->id < b->id) return -1;
    if (a->id > b->id) return 1;
    return 0;
}

static int cmp_i32(const void *pa, const void *pb)
{
    int32_t a = *(const int32_t *)pa, b = *(const int32_t *)pb;
    return a < b ? -1 : (a > b ? 1 : 0);
}

/* queue.py:15-18 -> utils.py:44-53 (index_sort: sort by id, then stable sort by distance,
 * i.e. order (distance, id)) -> kernels.py:400-406 (punchout_duplicates_: mark_kernel
 * 314-330 sets bit 30 of ids[q+1] when ids[q] == ids[q+1] with bit 30 masked off;
 * punchout_pair_kernel 333-349 turns flagged entries into sentinels; a last sort by
 * distance moves them to the end).  The last sort keeps the (distance, id) order of the
 * survivors. */
static void queue_sort_row(int32_t *ids, float *dist, int cap, pair_t *tmp, uint8_t *flag)
{
    for (int i = 0; i < cap; ++i) { tmp[i].d = dist[i]; tmp[i].id = ids[i]; }
    qsort(tmp, cap, sizeof(pair_t), cmp_pair);
    const int32_t mask = ~(1 << 30);
    flag[0] = 0;
    for (int i = 0; i + 1 < cap; ++i) flag[i + 1] = ((tmp[i].id & mask) == (tmp[i + 1].id & mask));
    for (int i = 0; i < cap; ++i)
        if (flag[i] || (tmp[i].id & (1 << 30))) { tmp[i].id = VLO_MAXINT; tmp[i].d = VLO_MAXFLOAT; }
    /* stable sort by distance only == stable partition here, because survivors are in order
     * and every punched entry carries the largest distance */
    int o = 0;
    for (int i = 0; i < cap; ++i)
        if (!(tmp[i].d >= VLO_MAXFLOAT)) { ids[o] = tmp[i].id; dist[o] = tmp[i].d; ++o; }
    /* entries with distance >= MAXFLOAT keep their relative order after the real ones */
    for (int i = 0; i < cap; ++i)
        if (tmp[i].d >= VLO_MAXFLOAT) { ids[o] = tmp[i].id; dist[o] = tmp[i].d; ++o; }
}

void vlo_queue_sort(int32_t *ids, float *dist, int64_t b_count, int cap)
{
#pragma omp parallel
    {
        pair_t *tmp = (pair_t *)malloc(sizeof(pair_t) * (cap + 1));
        uint8_t *flag = (uint8_t *)malloc(cap + 1);
#pragma omp for schedule(static)
        for (int64_t b = 0; b < b_count; ++b)
            queue_sort_row(ids + b * (int64_t)cap, dist + b * (int64_t)cap, cap, tmp, flag);
        free(tmp);
        free(flag);
    }
}

/* queue.py:37-61 (Queue.insert): copy the candidates into columns [length, length+m),
 * punch out excluded ids in that tail view, queue_sort the whole row; optionally report
 * head != old head per column. */
void vlo_queue_insert(int32_t *ids, float *dist, int64_t b_count, int cap, int length,
                      const int32_t *cand_ids, const float *cand_dist, int m,
                      const int32_t *excl, int e, uint8_t *changed)
{
#pragma omp parallel
    {
        pair_t *tmp = (pair_t *)malloc(sizeof(pair_t) * (cap + 1));
        uint8_t *flag = (uint8_t *)malloc(cap + 1);
        int32_t *old = (int32_t *)malloc(sizeof(int32_t) * (length + 1));
#pragma omp for schedule(static)
        for (int64_t b = 0; b < b_count; ++b) {
            int32_t *ri = ids + b * (int64_t)cap;
            float *rd = dist + b * (int64_t)cap;
            if (changed) memcpy(old, ri, sizeof(int32_t) * length);
            memcpy(ri + length, cand_ids + b * (int64_t)m, sizeof(int32_t) * m);
            memcpy(rd + length, cand_dist + b * (int64_t)m, sizeof(float) * m);
            if (excl) punchout_excluded_row(ri + length, rd + length, m, excl + b * (int64_t)e, e);
            queue_sort_row(ri, rd, cap, tmp, flag);
            if (changed)
                for (int i = 0; i < length; ++i) changed[b * (int64_t)length + i] = (ri[i] != old[i]);
        }
        free(tmp);
        free(flag);
        free(old);
    }
}

/* queue.py:87-95 (pop_n_ids): copy the first min(length, n) ids, overwrite those slots
 * with sentinels, do not re-sort. */
int vlo_queue_pop(int32_t *ids, float *dist, int64_t b_count, int cap, int length, int n,
                  int32_t *out)
{
    int take = length < n ? length : n;
    for (int64_t b = 0; b < b_count; ++b)
        for (int i = 0; i < take; ++i) {
            out[b * take + i] = ids[b * (int64_t)cap + i];
            ids[b * (int64_t)cap + i] = VLO_MAXINT;
            dist[b * (int64_t)cap + i] = VLO_MAXFLOAT;
        }
    return take;
}

/* utils.py:85-89 (dedup_sort) with kernels.py:370-380 (dedup_tensor_: mark_kernel +
 * punchout_kernel 352-367): sort ids, punch adjacent repeats, sort again. */
static void dedup_sort_row(int32_t *ids, int e, uint8_t *flag)
{
    qsort(ids, e, sizeof(int32_t), cmp_i32);
    const int32_t mask = ~(1 << 30);
    flag[0] = 0;
    for (int i = 0; i + 1 < e; ++i) flag[i + 1] = ((ids[i] & mask) == (ids[i + 1] & mask));
    for (int i = 0; i < e; ++i)
        if (flag[i] || (ids[i] & (1 << 30))) ids[i] = VLO_MAXINT;
    qsort(ids, e, sizeof(int32_t), cmp_i32);
}

void vlo_dedup_sort(int32_t *ids, int64_t b_count, int e)
{
    uint8_t *flag = (uint8_t *)malloc(e + 1);
    for (int64_t b = 0; b < b_count; ++b) dedup_sort_row(ids + b * (int64_t)e, e, flag);
    free(flag);
}

/* utils.py:61-82 (add_new_to_seen_): find the first column that is MAXINT in every row;
 * none -> report "None" (return 0).  Otherwise copy the first min(remaining, v) visited
 * ids there and dedup_sort every row (return 1). */
int vlo_add_new_to_seen(int32_t *seen, int64_t b_count, int e, const int32_t *visit, int v)
{
    int first = -1;
    for (int c = 0; c < e && first < 0; ++c) {
        int all = 1;
        for (int64_t b = 0; b < b_count; ++b)
            if (seen[b * (int64_t)e + c] != VLO_MAXINT) { all = 0; break; }
        if (all) first = c;
    }
    if (first < 0) return 0;
    int ncopy = e - first < v ? e - first : v;
    if (ncopy == 0) return 1;
#pragma omp parallel
    {
        uint8_t *flag = (uint8_t *)malloc(e + 1);
#pragma omp for schedule(static)
        for (int64_t b = 0; b < b_count; ++b) {
            memcpy(seen + b * (int64_t)e + first, visit + b * (int64_t)v, sizeof(int32_t) * ncopy);
            dedup_sort_row(seen + b * (int64_t)e, e, flag);
        }
        free(flag);
    }
    return 1;
}

/* ann.py:37-93 (closest_vectors).  search queue rows are updated in place.
 * Returns the number of loop iterations executed.  `beam_size_cfg` is config["beam_size"],
 * `w` the width of `beams` (beams.size()[1]). */
int vlo_closest_vectors(const float *queries, int64_t b_count, int32_t *sq_ids, float *sq_dist,
                        int sq_len, int sq_cap, const float *vectors, int64_t n, int dim,
                        const int32_t *beams, int w, int beam_size_cfg, int pvc, int vqf, int ef,
                        int readahead, const int32_t *excl, int excl_w, int metric)
{
    int extra = w * pvc;                         /* ann.py:48 */
    int vq_len = vqf * beam_size_cfg;            /* ann.py:50 */
    int vq_cap = vq_len + extra;                 /* ann.py:51 */
    int e = ef * vq_len;                         /* ann.py:54 */
    int32_t *vq_ids = (int32_t *)malloc(sizeof(int32_t) * b_count * vq_cap);
    float *vq_dist = (float *)malloc(sizeof(float) * b_count * vq_cap);
    for (int64_t i = 0; i < b_count * vq_cap; ++i) { vq_ids[i] = VLO_MAXINT; vq_dist[i] = VLO_MAXFLOAT; }
    int head = sq_len < vq_len ? sq_len : vq_len; /* queue.py:30-35 */
    for (int64_t b = 0; b < b_count; ++b)
        for (int i = 0; i < head; ++i) {
            vq_ids[b * vq_cap + i] = sq_ids[b * (int64_t)sq_cap + i];
            vq_dist[b * vq_cap + i] = sq_dist[b * (int64_t)sq_cap + i];
        }
    int32_t *seen = (int32_t *)malloc(sizeof(int32_t) * (b_count * e + 1));
    for (int64_t i = 0; i < b_count * e; ++i) seen[i] = VLO_MAXINT;
    int seen_live = 1;
    int take = vq_len < pvc ? vq_len : pvc;
    int m = take * w;
    int32_t *visit = (int32_t *)malloc(sizeof(int32_t) * (b_count * take + 1));
    int32_t *c_ids = (int32_t *)malloc(sizeof(int32_t) * (b_count * m + 1));
    float *c_dist = (float *)malloc(sizeof(float) * (b_count * m + 1));
    uint8_t *changed = (uint8_t *)malloc(b_count * sq_len + 1);
    int progressing = 1, count = 0;
    while (progressing) {
        ++count;
        int checking = (count % readahead) == 0;
        vlo_queue_pop(vq_ids, vq_dist, b_count, vq_cap, vq_len, pvc, visit);
        vlo_search_from_seeds(queries, b_count, visit, take, beams, w, vectors, n, dim, c_ids, c_dist,
                              metric);
        vlo_queue_insert(sq_ids, sq_dist, b_count, sq_cap, sq_len, c_ids, c_dist, m, excl, excl_w,
                         checking ? changed : NULL);
        if (seen_live) seen_live = vlo_add_new_to_seen(seen, b_count, e, visit, take);
        if (seen_live)
            vlo_queue_insert(vq_ids, vq_dist, b_count, vq_cap, vq_len, c_ids, c_dist, m, seen, e, NULL);
        if (checking) {
            progressing = 0;
            for (int64_t i = 0; i < b_count * sq_len; ++i)
                if (changed[i]) { progressing = 1; break; }
        }
    }
    free(vq_ids); free(vq_dist); free(seen); free(visit); free(c_ids); free(c_dist); free(changed);
    return count;
}

/* kernels.py:409-438 (prune_kernel).  The kernel is launched with block (W,1,1) but reads
 * threadIdx.y, so z is always beams[y, 0].  It edits beams/distances in place; blocks are
 * taken here in increasing (x, slot) order, which is the order the Numba simulator runs
 * them in and one of the schedules a GPU may produce.  Rows of other nodes are only read at
 * slot 0, which is never punched in a row sorted by distance (the precondition here), so
 * rows can be processed independently. */
void vlo_prune_punch(int32_t *beams, float *dist, int64_t n, int w)
{
    int32_t *z0 = (int32_t *)malloc(sizeof(int32_t) * (n + 1));
    float *d0 = (float *)malloc(sizeof(float) * (n + 1));
    for (int64_t x = 0; x < n; ++x) { z0[x] = beams[x * w]; d0[x] = dist[x * w]; }
#pragma omp parallel for schedule(static)
    for (int64_t x = 0; x < n; ++x) {
        int32_t *rb = beams + x * w;
        float *rd = dist + x * w;
        for (int s = 0; s < w; ++s) {
            int32_t y = rb[s];
            if (y == VLO_MAXINT) continue;
            int32_t z = (y == x) ? rb[0] : z0[y];
            float dyz = (y == x) ? rd[0] : d0[y];
            if (z == VLO_MAXINT) continue;
            int xi = -1;
            for (int i = 0; i < w; ++i) if (rb[i] == z) xi = i;
            if (xi < 0) continue;
            if (rd[xi] > rd[s] && rd[xi] > dyz) { rb[xi] = VLO_MAXINT; rd[xi] = VLO_MAXFLOAT; }
        }
    }
    free(z0);
    free(d0);
}

/* kernels.py:441-468 (prune_): the punch pass, then each row sorted by distance and the ids
 * gathered.  Order among equal distances is unspecified in the reference (non-stable sort);
 * (distance, id) is used here. */
void vlo_prune(int32_t *beams, float *dist, int64_t n, int w)
{
    vlo_prune_punch(beams, dist, n, w);
#pragma omp parallel
    {
        pair_t *tmp = (pair_t *)malloc(sizeof(pair_t) * (w + 1));
#pragma omp for schedule(static)
        for (int64_t x = 0; x < n; ++x) {
            int32_t *rb = beams + x * w;
            float *rd = dist + x * w;
            for (int i = 0; i < w; ++i) { tmp[i].d = rd[i]; tmp[i].id = rb[i]; }
            qsort(tmp, w, sizeof(pair_t), cmp_pair);
            for (int i = 0; i < w; ++i) { rd[i] = tmp[i].d; rb[i] = tmp[i].id; }
        }
        free(tmp);
    }
}

/* utils.py:35-41 (generate_circulant_beams) and 26-32 (generate_queue_circulants):
 * row i holds sort_j(i + p_j) mod count_mod. */
void vlo_circulants(int64_t rows, int64_t row0, int64_t modulus, const int32_t *primes, int w,
                    int32_t *out)
{
    int32_t *sp = (int32_t *)malloc(sizeof(int32_t) * (w + 1));
    memcpy(sp, primes, sizeof(int32_t) * w);
    qsort(sp, w, sizeof(int32_t), cmp_i32);   /* adding i keeps the order of the sorted primes */
    for (int64_t i = 0; i < rows; ++i)
        for (int j = 0; j < w; ++j)
            out[i * w + j] = (int32_t)(((int64_t)(i + row0) + sp[j]) % modulus);
    free(sp);
}

/* ann.py:196-208 (initial_queue) + ann.py:235-259 (ann_calculate_recall): self-recall of the
 * first `sample` rows; returns the number of rows whose best hit is themselves. */
int64_t vlo_self_recall(const float *vectors, int64_t n, int dim, const int32_t *beams, int w,
                        int64_t sample, int beam_size_cfg, int pvc, int vqf, int ef, int rsqf,
                        int readahead, const int32_t *primes, int metric)
{
    int q = rsqf * beam_size_cfg;
    int extra = q > pvc * beam_size_cfg ? q : pvc * beam_size_cfg;
    int cap = q + extra;
    int32_t *ids = (int32_t *)malloc(sizeof(int32_t) * sample * cap);
    float *dist = (float *)malloc(sizeof(float) * sample * cap);
    for (int64_t i = 0; i < sample * cap; ++i) { ids[i] = VLO_MAXINT; dist[i] = VLO_MAXFLOAT; }
    int32_t *seeds = (int32_t *)malloc(sizeof(int32_t) * sample * q);
    float *sd = (float *)malloc(sizeof(float) * sample * q);
    vlo_circulants(sample, 0, sample, primes, q, seeds);
    vlo_calculate_distances(vectors, sample, dim, seeds, q, sd, metric);
    vlo_queue_insert(ids, dist, sample, cap, q, seeds, sd, q, NULL, 0, NULL);
    vlo_closest_vectors(vectors, sample, ids, dist, q, cap, vectors, n, dim, beams, w, beam_size_cfg,
                        pvc, vqf, ef, readahead, NULL, 0, metric);
    int64_t found = 0;
    for (int64_t i = 0; i < sample; ++i) found += (ids[i * cap] == (int32_t)i);
    free(ids); free(dist); free(seeds); free(sd);
    return found;
}

/* ann.py:109-193 (generate_ann).  Two documented departures from the reference, both where
 * the reference's own result is accidental: the distances carried into the next loop and
 * returned are those of the pruned neighbour lists (the reference keeps the initial
 * circulant distances because it assigns prune_'s result to an unused name, ann.py:172),
 * and a MAXINT neighbour produces sentinels instead of an out-of-range read.
 * out_beams/out_dist are [n, beam_size]; full_beams/full_dist (optional) [n, W].
 * Returns the number of optimisation loops run; *recall_found gets the last self-recall. */
int vlo_generate_ann(const float *vectors, int64_t n, int dim, int beam_size, int bqf, int pvc,
                     int vqf, int ef, int loops, int64_t batch_size, int rsqf, int readahead,
                     int do_prune, const int32_t *primes, int metric, int32_t *out_beams,
                     float *out_dist, int32_t *full_beams, float *full_dist, int64_t *recall_found)
{
    int w = beam_size * bqf;
    int cap = w + w * pvc;
    int32_t *beams = (int32_t *)malloc(sizeof(int32_t) * n * w);
    float *bd = (float *)malloc(sizeof(float) * n * w);
    int32_t *nb = (int32_t *)malloc(sizeof(int32_t) * n * w);
    float *nd = (float *)malloc(sizeof(float) * n * w);
    vlo_circulants(n, 0, n, primes, w, beams);
    vlo_calculate_distances(vectors, n, dim, beams, w, bd, metric);
    int done = 0;
    int64_t found = 0;
    for (int loop = 0; loop < loops; ++loop) {
        for (int64_t start = 0; start < n; start += batch_size) {
            int64_t batch = n - start < batch_size ? n - start : batch_size;
            int32_t *excl = (int32_t *)malloc(sizeof(int32_t) * batch);
            for (int64_t i = 0; i < batch; ++i) excl[i] = (int32_t)(start + i);  /* ann.py:315-320 */
            int32_t *qi = (int32_t *)malloc(sizeof(int32_t) * batch * cap);
            float *qd = (float *)malloc(sizeof(float) * batch * cap);
            for (int64_t i = 0; i < batch * cap; ++i) { qi[i] = VLO_MAXINT; qd[i] = VLO_MAXFLOAT; }
            vlo_queue_insert(qi, qd, batch, cap, w, beams + start * w, bd + start * w, w, NULL, 0, NULL);
            vlo_closest_vectors(vectors + start * dim, batch, qi, qd, w, cap, vectors, n, dim, beams, w,
                                beam_size, pvc, vqf, ef, readahead, excl, 1, metric);
            for (int64_t i = 0; i < batch; ++i) {
                memcpy(nb + (start + i) * w, qi + i * cap, sizeof(int32_t) * w);
                memcpy(nd + (start + i) * w, qd + i * cap, sizeof(float) * w);
            }
            free(excl); free(qi); free(qd);
        }
        if (do_prune) vlo_prune(nb, nd, n, w);
        memcpy(beams, nb, sizeof(int32_t) * n * w);
        memcpy(bd, nd, sizeof(float) * n * w);
        ++done;
        int64_t sample = n < 1000 ? n : 1000;
        int32_t *narrow = (int32_t *)malloc(sizeof(int32_t) * n * beam_size);
        for (int64_t i = 0; i < n; ++i) memcpy(narrow + i * beam_size, beams + i * w, sizeof(int32_t) * beam_size);
        found = vlo_self_recall(vectors, n, dim, narrow, beam_size, sample, beam_size, pvc, vqf, ef, rsqf,
                                readahead, primes, metric);
        free(narrow);
        if (found == sample) break;
    }
    for (int64_t i = 0; i < n; ++i) {
        memcpy(out_beams + i * beam_size, beams + i * w, sizeof(int32_t) * beam_size);
        memcpy(out_dist + i * beam_size, bd + i * w, sizeof(float) * beam_size);
    }
    if (full_beams) memcpy(full_beams, beams, sizeof(int32_t) * n * w);
    if (full_dist) memcpy(full_dist, bd, sizeof(float) * n * w);
    if (recall_found) *recall_found = found;
    free(beams); free(bd); free(nb); free(nd);
    return done;
}

/* Exact brute-force k nearest neighbours in double precision (ground truth for recall;
 * not part of the reference).  exclude_self: skip id == query row index + self_base. */
void vlo_bruteforce_knn(const float *vectors, int64_t n, int dim, const float *queries, int64_t b_count,
                        int k, int metric, int exclude_self, int64_t self_base, int32_t *out_ids)
{
#pragma omp parallel
    {
        double *bd = (double *)malloc(sizeof(double) * k);
        int32_t *bi = (int32_t *)malloc(sizeof(int32_t) * k);
#pragma omp for schedule(dynamic, 1)
        for (int64_t b = 0; b < b_count; ++b) {
            int cnt = 0;
            const float *q = queries + b * (int64_t)dim;
            for (int64_t i = 0; i < n; ++i) {
                if (exclude_self && i == b + self_base) continue;
                const float *v = vectors + i * (int64_t)dim;
                double s = 0.0;
                if (metric == VLO_COSINE) { for (int t = 0; t < dim; ++t) s += (double)q[t] * v[t]; s = (1.0 - s) / 2.0; }
                else { for (int t = 0; t < dim; ++t) { double d = (double)q[t] - v[t]; s += d * d; } }
                if (cnt < k || s < bd[cnt - 1]) {
                    int p = cnt < k ? cnt : k - 1;
                    while (p > 0 && bd[p - 1] > s) { bd[p] = bd[p - 1]; bi[p] = bi[p - 1]; --p; }
                    bd[p] = s; bi[p] = (int32_t)i;
                    if (cnt < k) ++cnt;
                }
            }
            for (int t = 0; t < k; ++t) out_ids[b * k + t] = t < cnt ? bi[t] : VLO_MAXINT;
        }
        free(bd); free(bi);
    }
}

static int32_t vlo_uf_find(int32_t *parent, int32_t v)
{
    int32_t r = v;
    while (parent[r] != r) r = parent[r];
    while (parent[v] != r) { int32_t nx = parent[v]; parent[v] = r; v = nx; }
    return r;
}

/* Connected components of a thresholded neighbour graph (not in the reference, whose
 * ANN.clusters is a stub, ann.py:466-467): sequential union-find, always hooking the larger
 * root under the smaller, so labels[x] = smallest id of x's component.  dist may be NULL.
 * Returns the number of ids outside [0, n) that are not MAXINT (they are skipped). */
int64_t vlo_connected_components(const int32_t *ids, const float *dist, int64_t n, int w, float threshold,
                                 int32_t *labels)
{
    int64_t bad = 0;
    for (int64_t i = 0; i < n; ++i) labels[i] = (int32_t)i;
    for (int64_t x = 0; x < n; ++x)
        for (int s = 0; s < w; ++s) {
            int32_t y = ids[x * w + s];
            if (y == VLO_MAXINT) continue;
            if (y < 0 || y >= n) { ++bad; continue; }
            if (dist && !(dist[x * w + s] <= threshold)) continue;
            int32_t a = vlo_uf_find(labels, (int32_t)x), b = vlo_uf_find(labels, y);
            if (a < b) labels[b] = a;
            else if (b < a) labels[a] = b;
        }
    for (int64_t i = 0; i < n; ++i) labels[i] = vlo_uf_find(labels, (int32_t)i);
    return bad;
}

int vlo_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Threads for the parallel loops from here on (a launcher may have exported OMP_NUM_THREADS=1
 * for its worker processes; a timing run wants the host's cores regardless). */
void vlo_set_num_threads(int threads)
{
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
}
