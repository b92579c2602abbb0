/*
 * libvlgpu - C ABI of the B200 (sm_100a) kernels behind the VectorLink ANN graph builder
 * and beam searcher.
 *
 * The reference (vectorlink-ai/vectorlink-gpu) has no FFI layer: its device code is Numba
 * kernels called from Python operators.  Each entry point below therefore replaces one of
 * those Python operators (cited as file:line of the reference package `vectorlink_gpu/`),
 * and the Python drop-in package binds them with ctypes.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer borrowed for the call (never kept, never freed);
 *     ids are int32, distances fp32, rows are contiguous unless a leading dimension is given;
 *   - `stream` is a cudaStream_t passed as void*; calls are asynchronous on it;
 *   - return value: 0 = enqueued, negative = rejected (see vl_last_error());
 *   - `status` points to one device int that kernels OR VL_STATUS_* bits into instead of
 *     trapping (an id outside [0,N) that is not MAXINT is skipped and reported there);
 *   - sentinels are the reference's (constants.py:5-6): VL_MAXINT / VL_MAXFLOAT;
 *   - metric 0 = cosine distance on unit vectors, (1 - <a,b>)/2 clamped to [0,1]
 *     (kernels.py:85-114), summed in the reference's fixed order; metric 1 = squared
 *     Euclidean distance summed in the same order (not in the reference).
 */
#ifndef VLGPU_H
#define VLGPU_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VL_MAXINT 2147483647
#define VL_MAXFLOAT 3.4028e37f
#define VL_METRIC_COSINE 0
#define VL_METRIC_SQL2 1
#define VL_STATUS_BAD_ID 1
#define VL_STATUS_OVERFLOW 2
#define VL_STATUS_TIMEOUT 4   /* a bounded in-kernel wait ran out; the launch's results are not valid */

/* Text of the last rejected call on this host thread. */
const char* vl_last_error(void);

/* Version of this ABI (bumped when a signature or the layout of an output changes). */
int vl_abi_version(void);

/* calculate_distances (kernels.py:174-201, kernel 130-171), generalised to a separate query
 * matrix: dist_out[r, j] = distance(queries[r], vectors[ids[r, j]]), MAXFLOAT where
 * ids[r, j] == MAXINT.  The reference's call is queries == vectors, rows == n. */
int vl_calculate_distances(const float* vectors, int64_t n, int dim, const float* queries, int64_t rows,
                           const int32_t* ids, int w, float* dist_out, int metric, int* status, void* stream);

/* search_from_seeds (kernels.py:260-311, kernel 204-257): for query b, visited node
 * visit[b, v] and slot j: idx_out[b, v*w + j] = graph[visit[b, v], j] and dist_out the distance
 * of that vector to queries[b]; sentinels where visit[b, v] (or the neighbour) is MAXINT. */
int vl_search_from_seeds(const float* queries, int64_t b, const int32_t* visit, int v, const int32_t* graph, int w,
                         const float* vectors, int64_t n, int dim, int32_t* idx_out, float* dist_out, int metric,
                         int* status, void* stream);

/* Queue.insert (queue.py:37-61): rows [b, cap] of ids/dist in place.  The m candidates go to
 * columns [length, length+m), ids found in the row's exclusion list excl[b, 0..e) (scanned up
 * to its first MAXINT; kernels.py:471-488) become sentinels, then the whole row is ordered by
 * (distance, id), repeated ids are punched and the sentinels moved last (queue.py:15-18,
 * utils.py:44-53, kernels.py:400-406).  changed (optional, [b, length] bytes) receives
 * head != previous head.  cap <= 4096. */
int vl_queue_insert(int32_t* ids, float* dist, int64_t b, int cap, int length, const int32_t* cand_ids,
                    const float* cand_dist, int m, const int32_t* excl, int e, uint8_t* changed, void* stream);

/* Queue.pop_n_ids (queue.py:87-95): out[b, 0..take) = first take = min(length, n) ids of each
 * row; those slots become sentinels; rows are not re-sorted. */
int vl_queue_pop(int32_t* ids, float* dist, int64_t b, int cap, int length, int n, int32_t* out, void* stream);

/* punchout_excluded_ (kernels.py:491-501) on views with leading dimensions ld_ids / ld_dist. */
int vl_punchout_excluded(int32_t* ids, float* dist, int64_t ld_ids, int64_t ld_dist, int64_t b, int q,
                         const int32_t* excl, int e, void* stream);

/* dedup_tensor_pair_ (kernels.py:383-397) and, with dist == NULL, dedup_tensor_ (370-380):
 * an id equal to the id before it in its row becomes MAXINT (/MAXFLOAT); rows are not sorted. */
int vl_dedup_adjacent(int32_t* ids, float* dist, int64_t b, int cap, void* stream);

/* index_sort (utils.py:44-53) when dedup == 0: rows ordered by (distance, id);
 * queue_sort (queue.py:15-18) when dedup != 0: additionally repeated ids punched, sentinels last. */
int vl_sort_pairs(int32_t* ids, float* dist, int64_t b, int cap, int dedup, void* stream);

/* dedup_sort (utils.py:85-89) over rows of ids. */
int vl_dedup_sort_ids(int32_t* ids, int64_t b, int e, void* stream);

/* add_new_to_seen_ (utils.py:61-82): *first_out (device int) = first column of `seen` [b, e]
 * holding MAXINT in every row, or -1 (the reference then returns None and nothing is
 * written); otherwise the first min(e - first, v) ids of visit [b, v] are stored there and
 * every row goes through dedup_sort.  scratch: e device ints. */
int vl_seen_add(int32_t* seen, int64_t b, int e, const int32_t* visit, int v, int* scratch, int* first_out,
                void* stream);

/* No counterpart in the reference: vl_seen_add for callers that cannot provide (or allocate)
 * the scratch buffer - a process whose framework reserved all device memory up front, a plugin
 * that may not allocate after start-up, a loop that must never reach cudaMalloc.  The column
 * flags live in a fixed 16 KB device array inside the library (one per GPU, held until exit),
 * so e <= VL_SEEN_NOALLOC_MAX_WIDTH; wider lists are rejected with an error.  Calls nothing
 * that allocates.  Same results as vl_seen_add.  All calls on a GPU share the array: calls
 * that overlap on the GPU race, keep them stream-ordered.  The first call on a device looks up
 * the array's address and should happen before any stream capture begins.  The address is kept
 * per device for the life of the process: after a cudaDeviceReset (or any teardown of the
 * device's primary context) it is stale and this entry point must not be used again in that
 * process. */
#define VL_SEEN_NOALLOC_MAX_WIDTH 4096
int vl_seen_add_noalloc(int32_t* seen, int64_t b, int e, const int32_t* visit, int v, int* first_out, void* stream);

/* prune_ (kernels.py:441-468, kernel 409-438) followed by the cut to the first out_cols
 * columns (ann.py:190-193): rows of beams/dist [n, w], sorted by distance on entry, lose the
 * links x->z that have a detour over y's first neighbour (do_punch == 1; do_punch == 2 scans every
 * neighbour of y, the scan the reference's comment describes but its launch shape never ran), are ordered by
 * (distance, id) with sentinels last, and their first out_cols columns are written to the
 * outputs [n, out_cols].  Inputs are not modified.  w <= 2048. */
int vl_prune(const int32_t* beams, const float* dist, int64_t n, int w, int do_punch, int32_t* beams_out,
             float* dist_out, int out_cols, int* status, void* stream);

/* vl_prune over the rows [row_lo, row_hi) only: rows outside the range are still read (a row's
 * detour witnesses live in its neighbours' rows) but only rows of the range are written, at
 * their own row index of the [n, out_cols] outputs.  A build whose rows are split across
 * several GPUs prunes each GPU's share with it (the reference is single-device: constants.py:7). */
int vl_prune_rows(const int32_t* beams, const float* dist, int64_t n, int w, int64_t row_lo, int64_t row_hi,
                  int do_punch, int32_t* beams_out, float* dist_out, int out_cols, int* status, void* stream);

/* Reverse edges (the reference only sketches them: symmetrize_beams, kernels.py:503-550, is dead
 * code): out[y, 0..keep) = the nodes x that list y among the first `scan` columns of beams [n, d],
 * ordered by (rank of y in x's list, x), MAXINT-padded.  Two calls: phase 0 adds every node's
 * in-degree to deg [n] (zeroed by the caller); the caller turns deg into exclusive prefix sums
 * `offsets` [n] (int64) and provides a zeroed cursor [n] and keys [sum(deg)]; phase 1 fills and selects. */
int vl_reverse_edges(const int32_t* beams, int64_t n, int d, int scan, int phase, int32_t* deg, const int64_t* offsets,
                     int32_t* cursor, unsigned long long* keys, int keep, int32_t* out, int* status, void* stream);

/* Cluster extraction, announced by the reference on top of "all search queues" (README.md:24) but
 * left as an empty stub (ANN.clusters, ann.py:466-467): connected components of the neighbour
 * lists ids/dist [n, w] (row stride ld elements).  x and y = ids[x, s] are linked, in both
 * directions, when y != MAXINT and dist[x, s] <= threshold (every real id when dist == NULL).
 * labels[x] (int32 [n]) = the smallest node id of x's component. */
int vl_connected_components(const int32_t* ids, const float* dist, int64_t n, int w, int64_t ld, float threshold,
                            int32_t* labels, int* status, void* stream);

/* Initial-kNN tile pass (not in the reference, which starts every build from the circulant graph
 * of utils.py:35-41 / ann.py:116-118): tensor-core proposals of near neighbours for an opt-in
 * start graph.  Two steps.
 *
 * vl_knn_prepare: bf16 copy of the rows, zero-padded to dim_pad columns (a multiple of 64), and
 * |row|^2 in fp32 (sqnorm_out, may be NULL).
 *
 * vl_knn_tile: proposals for every row in [row_lo, row_hi).  The candidate range
 * [cand_lo, cand_hi) is cut into `segments` equal parts (each a multiple of 256 candidates, the
 * tile width), and a part's candidates fall into VL_KNN_TILE_LISTS = 4 classes by their position
 * in their tile: class k takes the 64 candidates [64 k, 64 k + 64) of every 256-candidate tile,
 * i.e. candidate c of a part that starts at c0 belongs to class ((c - c0) / 64) % 4.  There is one
 * list per class, and it holds the ids of the VL_KNN_TILE_K candidates of the class with the
 * smallest approximate score - bf16 inner
 * products accumulated in fp32 on the tensor cores (tcgen05.mma, operands staged by TMA), score =
 * sqnorm[c] - 2<q, c> (squared L2) or -2<q, c> when sqnorm == NULL (cosine).  The row itself is
 * never proposed.  out_ids [row_hi - row_lo, segments, VL_KNN_TILE_LISTS, VL_KNN_TILE_K], best
 * first within a list, MAXINT-padded.  The ids are PROPOSALS: the caller re-evaluates them with
 * vl_calculate_distances and orders them with vl_sort_pairs, so no bf16 value reaches a graph.
 * A wait inside the kernel that runs out sets VL_STATUS_TIMEOUT in *status. */
#define VL_KNN_TILE_K 16
#define VL_KNN_TILE_LISTS 4
int vl_knn_prepare(const float* vectors, int64_t n, int dim, uint16_t* bf16_out, int dim_pad, float* sqnorm_out,
                   void* stream);
int vl_knn_tile(const uint16_t* rows_bf16, int64_t n, int dim_pad, const float* sqnorm, int64_t row_lo, int64_t row_hi,
                int64_t cand_lo, int64_t cand_hi, int segments, int32_t* out_ids, int* status, void* stream);

/* closest_vectors (ann.py:37-93) as one kernel: the whole budgeted beam search of every query
 * row, with the search queue, the visit queue and the visited set of a row held on chip by
 * one warp.  Replaces, per iteration, pop_n_ids + search_from_seeds + two Queue.insert +
 * add_new_to_seen_.  The caller (the Python driver) checks the two flag arrays afterwards to
 * learn whether the reference's batch-wide loop would have stopped earlier. */
typedef struct vl_beam_params {
    const float* vectors;      /* [n, dim] */
    int64_t n;
    int32_t dim;               /* multiple of 4, rows 16-byte aligned */
    int32_t metric;
    const int32_t* graph;      /* [n, graph_w]  (`beams` of the reference) */
    int32_t graph_w;
    int32_t pvc;               /* config["parallel_visit_count"], <= 32 */
    const float* queries;      /* [rows, dim] */
    int64_t rows;
    const int32_t* seed_ids;   /* [rows, seed_ld]: seed_cols entries per row, inserted into an */
    const float* seed_dist;    /*   empty queue (= Queue.insert of ann.py:147 / the head of a Queue) */
    int64_t seed_ld;
    int32_t seed_cols;
    int32_t sq_len;            /* search queue length, <= 1024 */
    int32_t vq_len;            /* visit queue length = visit_queue_factor * beam_size, >= pvc */
    int32_t seen_cap;          /* exclude_factor * vq_len */
    int32_t* out_ids;          /* [rows, out_ld]: out_cols columns written per row: the head, then */
    float* out_dist;           /*   sentinels (or the raw last candidates when dump_last) */
    int64_t out_ld;
    int32_t out_cols;
    int32_t n_iters;           /* iterations of the reference loop to run */
    int32_t readahead;         /* config["speculative_readahead"] */
    int32_t dump_last;         /* != 0: the last iteration's insert is left to vl_sort_pairs: the row
                                  gets head + that iteration's candidates, unsorted (out_cols = capacity) */
    int32_t exclude_w;         /* columns of `exclude` (0 = none) */
    const int32_t* exclude;    /* [rows, exclude_w] per-row exclusion lists for the search queue */
    int64_t self_base;         /* >= 0: also exclude id self_base + row (ann.py:315-320); -1: no */
    int64_t group_rows;        /* rows per batch of the reference's host loop (flags are per batch) */
    uint32_t* changed_flags;   /* [groups, n_checks]: OR of "head changed" at iteration (c+1)*readahead */
    int32_t n_checks;
    int32_t memo_entries;      /* entries of the distance memo per row in flight: a power of two >= 2, or 0 = no memo */
    uint32_t* group_full;      /* [groups]: set when some row of the batch never popped a MAXINT */
    int32_t* status;
    unsigned long long* memo;  /* [memo_slots, memo_entries] scratch, any contents (see vl_beam_search_plan) */
    int64_t memo_slots;        /* rows in flight the scratch was sized for: >= blocks * warps_per_block of the plan */
    unsigned long long* stats; /* optional [16] counters (added to): [1] gathered candidates, [2] search-queue merges,
                                  [3] visit-queue merges, [4] class-A candidates, [5] class-B rounds, [6] rows, [7] iterations, [8..13] warp cycles spent in: pop +
                                  neighbour ids, memo probe, gather, memo update, search-queue merge, visit-queue merge */
    int32_t flags;             /* bit 0: also accumulate the per-phase cycle counters of `stats` */
    int32_t reserved;
    unsigned long long* row_ticket; /* optional device counter, zero at launch: warps then draw their next row from it
                                  (rows that take unequal time no longer wait for a fixed partner); NULL = fixed stride */
    int64_t group_row0;        /* row 0 of this launch sits at this position of the reference's host loop: its batch
                                  (the row of both flag arrays) is (group_row0 + row) / group_rows.  0 for a launch
                                  that starts on a batch boundary */
} vl_beam_params;

int vl_beam_search(const vl_beam_params* params, void* stream);

/* Bytes of shared memory one warp (= one query row in flight) of vl_beam_search needs for the
 * given shape, the warps per CTA and the CTAs it will launch.  blocks * warps_per_block is the
 * number of rows in flight, i.e. the memo_slots a distance memo must provide.
 *
 * The memo: during one row's search the same candidate id comes back many times (neighbour
 * lists of nearby nodes overlap; the reference recomputes its distance every time).  With a
 * memo the kernel keeps id -> distance of the row's recent candidates in a 2-way table in
 * global memory (L2-resident) and gathers only the ids it has not met: same bits, a fraction
 * of the gathers. */
int vl_beam_search_plan(const vl_beam_params* params, int* smem_per_warp, int* warps_per_block, int* blocks);

#ifdef __cplusplus
}
#endif
#endif /* VLGPU_H */
