// Connected components of a thresholded neighbour graph: the cluster extraction that the
// reference announces on top of "all search queues" (README.md:24) and leaves as an empty
// stub (ANN.clusters, vectorlink_gpu/ann.py:466-467).
//
// Node x and node y = ids[x, s] are linked when y is a real id and dist[x, s] <= threshold;
// links are undirected.  labels[x] = the smallest node id of x's component, which makes the
// result independent of the order in which edges are processed.
//
// Method: a lock-free union-find in the output array itself.  parent[v] <= v always holds: a
// root is only ever hooked under a SMALLER root (compare-and-swap on the root's own slot), and
// path halving only replaces a parent by one of its ancestors.  Every chase therefore walks a
// strictly decreasing chain and ends, whatever other threads do meanwhile, and a stale read is
// still an ancestor.  Three passes on the stream: init, one pass over the edges (coalesced
// reads of ids and dist, one thread per slot), flatten.
#include "vl_common.cuh"

namespace {

constexpr int kRetryLimit = 1 << 20;  // hooks one edge can lose to other threads before it gives up

__device__ __forceinline__ int32_t ld_parent(const int32_t* parent, int32_t v)
{
    return *reinterpret_cast<const volatile int32_t*>(parent + v);
}

// root of v, halving the path on the way
__device__ __forceinline__ int32_t find_root(int32_t* parent, int32_t v)
{
    int32_t cur = ld_parent(parent, v);
    if (cur != v) {
        int32_t prev = v, next;
        while (cur > (next = ld_parent(parent, cur))) {
            parent[prev] = next;
            prev = cur;
            cur = next;
        }
    }
    return cur;
}

__global__ void init_labels_kernel(int32_t* __restrict__ parent, int64_t n)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        parent[i] = (int32_t)i;
}

__global__ void hook_edges_kernel(const int32_t* __restrict__ ids, const float* __restrict__ dist, int64_t n, int w,
                                  int64_t ld, float threshold, int32_t* parent, int* __restrict__ status)
{
    const int64_t total = n * w;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t x = t / w;
        const int s = (int)(t - x * w);
        const int32_t y = ids[x * ld + s];
        if (y == VL_MAXINT) continue;
        if (y < 0 || (int64_t)y >= n) { atomicOr(status, VL_STATUS_BAD_ID); continue; }
        if (dist && !(dist[x * ld + s] <= threshold)) continue;
        int32_t a = find_root(parent, (int32_t)x), b = find_root(parent, y);
        int tries = 0;
        while (a != b) {
            if (a < b) { int32_t c = a; a = b; b = c; }      // a > b: hook a under b
            const int32_t old = atomicCAS(&parent[a], a, b);
            if (old == a) break;
            if (++tries > kRetryLimit) { atomicOr(status, VL_STATUS_OVERFLOW); break; }
            a = find_root(parent, old);                        // a was hooked meanwhile: go on from its new root
            b = find_root(parent, b);
        }
    }
}

__global__ void flatten_kernel(int32_t* parent, int64_t n)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int32_t r = ld_parent(parent, (int32_t)i);
        int32_t next;
        while (r > (next = ld_parent(parent, r))) r = next;
        parent[i] = r;       // r is a root and stays one: concurrent chases through i stay correct
    }
}

unsigned grid_for(int64_t items, int threads)
{
    int64_t blocks = (items + threads - 1) / threads;
    const int64_t cap = (int64_t)vl_sm_count() * 16;           // 16 CTAs of 256 threads fill an SM
    if (blocks > cap) blocks = cap;
    return (unsigned)(blocks < 1 ? 1 : blocks);
}

}  // namespace

extern "C" int vl_connected_components(const int32_t* ids, const float* dist, int64_t n, int w, int64_t ld,
                                       float threshold, int32_t* labels, int* status, void* stream)
{
    VL_CHECK_ARG(n >= 0 && n < ((int64_t)1 << 31) - 1, "vl_connected_components: %lld nodes do not fit int32 ids",
                 (long long)n);
    VL_CHECK_ARG(w >= 0 && ld >= w, "vl_connected_components: bad shape (w %d, ld %lld)", w, (long long)ld);
    if (n == 0) return 0;
    VL_CHECK_ARG(labels && status, "vl_connected_components: null pointer");
    VL_CHECK_ARG(w == 0 || ids, "vl_connected_components: null ids");
    cudaStream_t st = (cudaStream_t)stream;
    init_labels_kernel<<<grid_for(n, 256), 256, 0, st>>>(labels, n);
    VL_CHECK_LAUNCH("init_labels_kernel");
    if (w > 0) {
        hook_edges_kernel<<<grid_for(n * w, 256), 256, 0, st>>>(ids, dist, n, w, ld, threshold, labels, status);
        VL_CHECK_LAUNCH("hook_edges_kernel");
        flatten_kernel<<<grid_for(n, 256), 256, 0, st>>>(labels, n);
        VL_CHECK_LAUNCH("flatten_kernel");
    }
    return 0;
}
