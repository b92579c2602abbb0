// Gathered fp32 distance kernels: the operator-level replacements of the reference's
// cuda_distances_kernel (vectorlink_gpu/kernels.py:130-171) and
// cuda_search_from_seeds_kernel (kernels.py:204-257).
//
// The reference launches one CTA per (row, neighbour) pair and re-reads the query row for
// every pair.  Here one warp owns a (query row, segment of candidates) task: the query row
// is loaded once into registers, and the warp walks its candidates 32/LPR at a time, each
// candidate row fetched by LPR lanes with 128-bit loads (a contiguous LPR*16-byte span per
// load instruction).  The kernels are bound by the HBM gather of candidate rows:
// 4*dim + 12 bytes per evaluated pair.
#include "vl_common.cuh"
#include "vlgpu.h"

namespace {

constexpr int kWarpsPerBlock = 4;

// One task = (query row r, segment s).  Candidate m of the task is slot s*seg_len + m of
// the row's output.  Its id comes either from `ids` (self mode: ids[r, slot]) or from the
// graph (seed mode: graph[visit[r, s], m], MAXINT when the visited id is MAXINT).
template <int LPR, int JP, int METRIC, bool ALIGNED>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
gather_distance_kernel(const float* __restrict__ vectors, int64_t n, int dim,
                       const float* __restrict__ queries, int64_t rows, int segs, int seg_len,
                       const int32_t* __restrict__ ids,      // [rows, segs*seg_len] or null
                       const int32_t* __restrict__ visit,    // [rows, segs] or null
                       const int32_t* __restrict__ graph,    // [n, seg_len] when visit != null
                       int32_t* __restrict__ idx_out,        // [rows, segs*seg_len] or null
                       float* __restrict__ dist_out,         // [rows, segs*seg_len]
                       int* __restrict__ status)
{
    constexpr int G = 32 / LPR;  // candidates per warp step
    const int lane = threadIdx.x & 31;
    const int g = lane / LPR, lg = lane % LPR;
    const int64_t total = rows * segs;
    const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
    for (int64_t task = warp0; task < total; task += nwarps) {
        const int64_t r = task / segs;
        const int s = (int)(task - r * segs);
        const float* q = queries + r * (int64_t)dim;
        float4 qr[JP];
        vl_load_query<LPR, JP, ALIGNED>(q, dim, lg, qr);
        int32_t node = 0;
        if (visit) {
            node = __ldg(visit + r * segs + s);
            if (node != VL_MAXINT && (node < 0 || (int64_t)node >= n)) {
                if (lane == 0) atomicOr(status, VL_STATUS_BAD_ID);
                node = VL_MAXINT;
            }
        }
        const int64_t out0 = r * (int64_t)segs * seg_len + (int64_t)s * seg_len;
        for (int m0 = 0; m0 < seg_len; m0 += G) {
            const int m = m0 + g;
            int32_t id = VL_MAXINT;
            if (m < seg_len) {
                if (visit) id = (node == VL_MAXINT) ? VL_MAXINT : __ldg(graph + (int64_t)node * seg_len + m);
                else id = __ldg(ids + out0 + m);
            }
            bool live = (id != VL_MAXINT);
            if (live && (id < 0 || (int64_t)id >= n)) {
                live = false;
                if (lg == 0) atomicOr(status, VL_STATUS_BAD_ID);
            }
            const float* row = vectors + (int64_t)(live ? id : 0) * dim;
            float4 xr[JP];
            vl_load_row<LPR, JP, ALIGNED>(row, dim, lg, live, xr);
            float d = vl_row_distance<LPR, JP, METRIC, ALIGNED>(xr, qr, row, q, dim, lg, live);
            if (lg == 0 && m < seg_len) {
                dist_out[out0 + m] = live ? d : VL_MAXFLOAT;
                if (idx_out) idx_out[out0 + m] = live ? id : VL_MAXINT;
            }
        }
    }
}

template <int METRIC>
int launch_gather(const float* vectors, int64_t n, int dim, const float* queries, int64_t rows, int segs,
                  int seg_len, const int32_t* ids, const int32_t* visit, const int32_t* graph, int32_t* idx_out,
                  float* dist_out, int* status, cudaStream_t stream)
{
    const int64_t total = rows * segs;
    if (total == 0 || seg_len == 0) return 0;
    int64_t blocks = (total + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const int64_t cap = (int64_t)vl_sm_count() * 64;  // grid-stride beyond that
    if (blocks > cap) blocks = cap;
    const bool aligned = (dim % 4 == 0) && (((uintptr_t)vectors | (uintptr_t)queries) % 16 == 0);
    VlShape shape = vl_pick_shape(dim);
    VL_DISPATCH_SHAPE(shape, {
        if (aligned)
            gather_distance_kernel<LPR, JP, METRIC, true><<<(unsigned)blocks, kWarpsPerBlock * 32, 0, stream>>>(
                vectors, n, dim, queries, rows, segs, seg_len, ids, visit, graph, idx_out, dist_out, status);
        else
            gather_distance_kernel<LPR, JP, METRIC, false><<<(unsigned)blocks, kWarpsPerBlock * 32, 0, stream>>>(
                vectors, n, dim, queries, rows, segs, seg_len, ids, visit, graph, idx_out, dist_out, status);
    });
    VL_CHECK_LAUNCH("gather_distance_kernel");
    return 0;
}

}  // namespace

extern "C" int vl_calculate_distances(const float* vectors, int64_t n, int dim, const float* queries,
                                      int64_t rows, const int32_t* ids, int w, float* dist_out, int metric,
                                      int* status, void* stream)
{
    VL_CHECK_ARG(dim > 0 && w >= 0 && rows >= 0 && n >= 0, "vl_calculate_distances: bad size");
    if (rows == 0 || w == 0) return 0;
    VL_CHECK_ARG(vectors && queries && ids && dist_out && status, "vl_calculate_distances: null pointer");
    VL_CHECK_ARG(metric == VL_METRIC_COSINE || metric == VL_METRIC_SQL2, "vl_calculate_distances: unknown metric %d", metric);
    cudaStream_t st = (cudaStream_t)stream;
    if (metric == VL_METRIC_COSINE)
        return launch_gather<VL_METRIC_COSINE>(vectors, n, dim, queries, rows, 1, w, ids, nullptr, nullptr, nullptr, dist_out, status, st);
    return launch_gather<VL_METRIC_SQL2>(vectors, n, dim, queries, rows, 1, w, ids, nullptr, nullptr, nullptr, dist_out, status, st);
}

extern "C" int vl_search_from_seeds(const float* queries, int64_t b, const int32_t* visit, int v,
                                    const int32_t* graph, int w, const float* vectors, int64_t n, int dim,
                                    int32_t* idx_out, float* dist_out, int metric, int* status, void* stream)
{
    VL_CHECK_ARG(dim > 0 && w >= 0 && v >= 0 && b >= 0 && n >= 0, "vl_search_from_seeds: bad size");
    if (b == 0 || v == 0 || w == 0) return 0;
    VL_CHECK_ARG(vectors && queries && visit && graph && idx_out && dist_out && status, "vl_search_from_seeds: null pointer");
    VL_CHECK_ARG(metric == VL_METRIC_COSINE || metric == VL_METRIC_SQL2, "vl_search_from_seeds: unknown metric %d", metric);
    cudaStream_t st = (cudaStream_t)stream;
    if (metric == VL_METRIC_COSINE)
        return launch_gather<VL_METRIC_COSINE>(vectors, n, dim, queries, b, v, w, nullptr, visit, graph, idx_out, dist_out, status, st);
    return launch_gather<VL_METRIC_SQL2>(vectors, n, dim, queries, b, v, w, nullptr, visit, graph, idx_out, dist_out, status, st);
}
