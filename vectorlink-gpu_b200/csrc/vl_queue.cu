// Operator-level queue kernels: the replacements of the reference's Queue.insert chain
// (vectorlink_gpu/queue.py:37-61 -> utils.py:44-53 -> kernels.py:400-406), pop_n_ids
// (queue.py:87-95), punchout_excluded_ (kernels.py:471-501), dedup_tensor_[pair_]
// (kernels.py:370-397) and add_new_to_seen_ / dedup_sort (utils.py:61-89).
//
// The reference spends three torch.sort calls, three gathers and three small kernels per
// insert.  Here one CTA owns one queue row: the row is packed into 64-bit (distance, id)
// keys in shared memory, sorted once with a bitonic network, adjacent equal ids are turned
// into sentinels, and a second pass of the network moves the sentinels to the end.
#include "vl_common.cuh"
#include "vlgpu.h"

namespace {

constexpr int kSortThreads = 256;
constexpr int kMaxSortWidth = 4096;  // 32 KB of keys

__device__ __forceinline__ void bitonic_sort_smem(vl_key_t* keys, int p)
{
    for (int k = 2; k <= p; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = threadIdx.x; t < p / 2; t += blockDim.x) {
                int lo = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                int hi = lo | j;
                bool up = ((lo & k) == 0);
                vl_key_t a = keys[lo], b = keys[hi];
                if ((a > b) == up) { keys[lo] = b; keys[hi] = a; }
            }
            __syncthreads();
        }
    }
}

// kernels.py:314-349: after the sort, an entry whose id equals the id right before it
// (bit 30 ignored in the comparison) becomes the sentinel pair.
__device__ __forceinline__ void punch_adjacent(vl_key_t* keys, int p)
{
    const int32_t mask = ~VL_ID_FLAG;
    bool hit[kMaxSortWidth / kSortThreads];
    int c = 0;
    for (int i = threadIdx.x; i < p; i += blockDim.x, ++c)
        hit[c] = (i > 0) && ((vl_key_id(keys[i]) & mask) == (vl_key_id(keys[i - 1]) & mask));
    __syncthreads();
    c = 0;
    for (int i = threadIdx.x; i < p; i += blockDim.x, ++c)
        if (hit[c]) keys[i] = vl_sentinel_key();
    __syncthreads();
}

__device__ __forceinline__ bool excluded(int32_t id, const int32_t* __restrict__ excl, int e)
{
    // kernels.py:478-488: scan the row's list up to its first MAXINT
    for (int i = 0; i < e; ++i) {
        int32_t x = excl[i];
        if (x == VL_MAXINT) break;
        if (x == id) return true;
    }
    return false;
}

// Queue.insert for one row per CTA.  ids/dist: [b, cap] updated in place.
__global__ void __launch_bounds__(kSortThreads)
queue_insert_kernel(int32_t* __restrict__ ids, float* __restrict__ dist, int cap, int length,
                    const int32_t* __restrict__ cand_ids, const float* __restrict__ cand_dist, int m,
                    const int32_t* __restrict__ excl, int e, uint8_t* __restrict__ changed, int p)
{
    extern __shared__ vl_key_t keys[];
    int32_t* old_head = reinterpret_cast<int32_t*>(keys + p);
    const int64_t b = blockIdx.x;
    int32_t* ri = ids + b * cap;
    float* rd = dist + b * cap;
    for (int i = threadIdx.x; i < p; i += blockDim.x) {
        vl_key_t k = vl_sentinel_key();
        if (i < cap) {
            int32_t id;
            float d;
            if (i >= length && i < length + m) {
                id = cand_ids[b * m + (i - length)];
                d = cand_dist[b * m + (i - length)];
                if (excl && excluded(id, excl + b * e, e)) id = VL_MAXINT;
            } else {
                id = ri[i];
                d = rd[i];
            }
            k = vl_entry_key(d, id);
            if (changed && i < length) old_head[i] = id;
        }
        keys[i] = k;
    }
    __syncthreads();
    bitonic_sort_smem(keys, p);
    punch_adjacent(keys, p);
    bitonic_sort_smem(keys, p);
    for (int i = threadIdx.x; i < cap; i += blockDim.x) {
        vl_key_t k = keys[i];
        ri[i] = vl_key_id(k);
        rd[i] = vl_key_dist(k);
        if (changed && i < length) changed[b * length + i] = (vl_key_id(k) != old_head[i]);
    }
}

// punchout_excluded_ on a strided view (kernels.py:491-501)
__global__ void punchout_excluded_kernel(int32_t* __restrict__ ids, float* __restrict__ dist, int64_t ld_ids,
                                         int64_t ld_dist, int64_t b_count, int q,
                                         const int32_t* __restrict__ excl, int e)
{
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= b_count * q) return;
    int64_t b = t / q;
    int s = (int)(t - b * q);
    int32_t id = ids[b * ld_ids + s];
    if (excluded(id, excl + b * e, e)) {
        ids[b * ld_ids + s] = VL_MAXINT;
        dist[b * ld_dist + s] = VL_MAXFLOAT;
    }
}

// dedup_tensor_pair_ / dedup_tensor_ (kernels.py:370-397): mark + punch on rows as they are
__global__ void dedup_adjacent_kernel(int32_t* __restrict__ ids, float* __restrict__ dist, int64_t b_count, int cap)
{
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= b_count * cap) return;
    int64_t b = t / cap;
    int i = (int)(t - b * cap);
    const int32_t mask = ~VL_ID_FLAG;
    int32_t id = ids[t];
    bool hit = (id & VL_ID_FLAG) != 0;
    if (i > 0 && ((ids[t - 1] & mask) == (id & mask))) hit = true;
    // all threads of the grid read before any writes: the write below is deferred to a
    // second launch (see vl_dedup_adjacent), this kernel only records the decision
    if (hit) ids[t] = id | VL_ID_FLAG;
}
__global__ void punch_flagged_kernel(int32_t* __restrict__ ids, float* __restrict__ dist, int64_t count)
{
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= count) return;
    if (ids[t] & VL_ID_FLAG) {
        ids[t] = VL_MAXINT;
        if (dist) dist[t] = VL_MAXFLOAT;
    }
}

// sort rows of (id, dist) pairs by (distance, id); mode 1 also punches adjacent equal ids and
// re-sorts (= queue_sort, queue.py:15-18); mode 0 is the plain order (index_sort, utils.py:44-53)
__global__ void __launch_bounds__(kSortThreads)
sort_pairs_kernel(int32_t* __restrict__ ids, float* __restrict__ dist, int cap, int dedup, int p)
{
    extern __shared__ vl_key_t keys[];
    const int64_t b = blockIdx.x;
    for (int i = threadIdx.x; i < p; i += blockDim.x)
        keys[i] = i < cap ? (dedup ? vl_entry_key(dist[b * cap + i], ids[b * cap + i])
                                   : vl_make_key(dist[b * cap + i], ids[b * cap + i]))
                          : ~0ull;
    __syncthreads();
    bitonic_sort_smem(keys, p);
    if (dedup) {
        punch_adjacent(keys, p);
        bitonic_sort_smem(keys, p);
    }
    for (int i = threadIdx.x; i < cap; i += blockDim.x) {
        ids[b * cap + i] = vl_key_id(keys[i]);
        dist[b * cap + i] = vl_key_dist(keys[i]);
    }
}

// dedup_sort over id rows (utils.py:85-89): sort, punch adjacent repeats, sort
__global__ void __launch_bounds__(kSortThreads)
dedup_sort_ids_kernel(int32_t* __restrict__ ids, int e, int p, const int32_t* __restrict__ append,
                      int append_w, const int* __restrict__ first_col)
{
    extern __shared__ vl_key_t keys[];
    const int64_t b = blockIdx.x;
    int first = first_col ? *first_col : -1;
    if (first_col && first < 0) return;          // no empty column: the list is left as it is
    int ncopy = 0;
    if (first_col) ncopy = min(e - first, append_w);
    for (int i = threadIdx.x; i < p; i += blockDim.x) {
        vl_key_t k = ~0ull;
        if (i < e) {
            int32_t id = ids[b * e + i];
            if (first_col && i >= first && i < first + ncopy) id = append[b * append_w + (i - first)];
            k = (vl_key_t)(uint32_t)id;          // ids are non-negative: unsigned order == signed order
        }
        keys[i] = k;
    }
    __syncthreads();
    bitonic_sort_smem(keys, p);
    {
        const int32_t mask = ~VL_ID_FLAG;
        bool hit[kMaxSortWidth / kSortThreads];
        int c = 0;
        for (int i = threadIdx.x; i < e; i += blockDim.x, ++c) {
            int32_t id = (int32_t)keys[i];
            hit[c] = (id & VL_ID_FLAG) || (i > 0 && (((int32_t)keys[i - 1] & mask) == (id & mask)));
        }
        __syncthreads();
        c = 0;
        for (int i = threadIdx.x; i < e; i += blockDim.x, ++c)
            if (hit[c]) keys[i] = (vl_key_t)(uint32_t)VL_MAXINT;
        __syncthreads();
    }
    bitonic_sort_smem(keys, p);
    for (int i = threadIdx.x; i < e; i += blockDim.x) ids[b * e + i] = (int32_t)keys[i];
}

// add_new_to_seen_ step 1 (utils.py:62-66): which columns hold MAXINT in every row
__global__ void column_used_kernel(const int32_t* __restrict__ seen, int64_t count, int e, int* __restrict__ used)
{
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= count) return;
    if (seen[t] != VL_MAXINT) used[t % e] = 1;
}
__global__ void first_free_column_kernel(const int* __restrict__ used, int e, int* __restrict__ first)
{
    __shared__ int best;
    if (threadIdx.x == 0) best = 0x7fffffff;
    __syncthreads();
    for (int c = threadIdx.x; c < e; c += blockDim.x)
        if (!used[c]) atomicMin(&best, c);
    __syncthreads();
    if (threadIdx.x == 0) *first = (best == 0x7fffffff) ? -1 : best;
}

__global__ void queue_pop_kernel(int32_t* __restrict__ ids, float* __restrict__ dist, int64_t b_count, int cap,
                                 int take, int32_t* __restrict__ out)
{
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= b_count * take) return;
    int64_t b = t / take;
    int i = (int)(t - b * take);
    out[t] = ids[b * cap + i];
    ids[b * cap + i] = VL_MAXINT;
    dist[b * cap + i] = VL_MAXFLOAT;
}

int pow2_at_least(int v)
{
    int p = 2;
    while (p < v) p <<= 1;
    return p;
}

unsigned blocks_for(int64_t count, int threads) { return (unsigned)((count + threads - 1) / threads); }

}  // namespace

extern "C" int vl_queue_insert(int32_t* ids, float* dist, int64_t b, int cap, int length,
                               const int32_t* cand_ids, const float* cand_dist, int m,
                               const int32_t* excl, int e, uint8_t* changed, void* stream)
{
    VL_CHECK_ARG(ids && dist && (m == 0 || (cand_ids && cand_dist)), "vl_queue_insert: null pointer");
    VL_CHECK_ARG(cap > 0 && cap <= kMaxSortWidth, "vl_queue_insert: capacity %d outside 1..%d", cap, kMaxSortWidth);
    VL_CHECK_ARG(length >= 0 && m >= 0 && m <= cap - length, "vl_queue_insert: %d candidates do not fit behind %d of %d columns", m, length, cap);
    VL_CHECK_ARG(excl || e == 0, "vl_queue_insert: exclusion width without a list");
    if (b == 0) return 0;
    int p = pow2_at_least(cap);
    size_t smem = sizeof(vl_key_t) * p + sizeof(int32_t) * (changed ? length : 0);
    queue_insert_kernel<<<(unsigned)b, kSortThreads, smem, (cudaStream_t)stream>>>(ids, dist, cap, length, cand_ids, cand_dist, m,
                                                                                 excl, e, changed, p);
    VL_CHECK_LAUNCH("queue_insert_kernel");
    return 0;
}

extern "C" int vl_queue_pop(int32_t* ids, float* dist, int64_t b, int cap, int length, int n, int32_t* out,
                            void* stream)
{
    VL_CHECK_ARG(ids && dist && out, "vl_queue_pop: null pointer");
    int take = length < n ? length : n;
    VL_CHECK_ARG(take >= 0 && take <= cap, "vl_queue_pop: bad sizes");
    if (b == 0 || take == 0) return 0;
    queue_pop_kernel<<<blocks_for(b * take, 256), 256, 0, (cudaStream_t)stream>>>(ids, dist, b, cap, take, out);
    VL_CHECK_LAUNCH("queue_pop_kernel");
    return 0;
}

extern "C" int vl_punchout_excluded(int32_t* ids, float* dist, int64_t ld_ids, int64_t ld_dist, int64_t b, int q,
                                    const int32_t* excl, int e, void* stream)
{
    VL_CHECK_ARG(ids && dist && excl, "vl_punchout_excluded: null pointer");
    if (b == 0 || q == 0 || e == 0) return 0;
    punchout_excluded_kernel<<<blocks_for(b * q, 256), 256, 0, (cudaStream_t)stream>>>(ids, dist, ld_ids, ld_dist, b, q, excl, e);
    VL_CHECK_LAUNCH("punchout_excluded_kernel");
    return 0;
}

extern "C" int vl_dedup_adjacent(int32_t* ids, float* dist, int64_t b, int cap, void* stream)
{
    VL_CHECK_ARG(ids, "vl_dedup_adjacent: null pointer");
    if (b == 0 || cap == 0) return 0;
    // two launches: every comparison of the first reads ids with bit 30 masked off, so the
    // flags it sets cannot disturb a neighbour's comparison (same as kernels.py:314-330)
    dedup_adjacent_kernel<<<blocks_for(b * cap, 256), 256, 0, (cudaStream_t)stream>>>(ids, dist, b, cap);
    VL_CHECK_LAUNCH("dedup_adjacent_kernel");
    punch_flagged_kernel<<<blocks_for(b * cap, 256), 256, 0, (cudaStream_t)stream>>>(ids, dist, b * cap);
    VL_CHECK_LAUNCH("punch_flagged_kernel");
    return 0;
}

extern "C" int vl_sort_pairs(int32_t* ids, float* dist, int64_t b, int cap, int dedup, void* stream)
{
    VL_CHECK_ARG(ids && dist, "vl_sort_pairs: null pointer");
    VL_CHECK_ARG(cap > 0 && cap <= kMaxSortWidth, "vl_sort_pairs: width %d outside 1..%d", cap, kMaxSortWidth);
    if (b == 0) return 0;
    int p = pow2_at_least(cap);
    sort_pairs_kernel<<<(unsigned)b, kSortThreads, sizeof(vl_key_t) * p, (cudaStream_t)stream>>>(ids, dist, cap, dedup, p);
    VL_CHECK_LAUNCH("sort_pairs_kernel");
    return 0;
}

extern "C" int vl_dedup_sort_ids(int32_t* ids, int64_t b, int e, void* stream)
{
    VL_CHECK_ARG(ids, "vl_dedup_sort_ids: null pointer");
    VL_CHECK_ARG(e > 0 && e <= kMaxSortWidth, "vl_dedup_sort_ids: width %d outside 1..%d", e, kMaxSortWidth);
    if (b == 0) return 0;
    int p = pow2_at_least(e);
    dedup_sort_ids_kernel<<<(unsigned)b, kSortThreads, sizeof(vl_key_t) * p, (cudaStream_t)stream>>>(ids, e, p, nullptr, 0, nullptr);
    VL_CHECK_LAUNCH("dedup_sort_ids_kernel");
    return 0;
}

extern "C" int vl_seen_add(int32_t* seen, int64_t b, int e, const int32_t* visit, int v, int* scratch,
                           int* first_out, void* stream)
{
    VL_CHECK_ARG(seen && visit && scratch && first_out, "vl_seen_add: null pointer");
    VL_CHECK_ARG(e >= 0 && e <= kMaxSortWidth, "vl_seen_add: width %d outside 0..%d", e, kMaxSortWidth);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t ce;
    if (e == 0 || b == 0) {  // utils.py:67-69: no column at all -> None; -1 is four 0xFF bytes
        ce = cudaMemsetAsync(first_out, 0xFF, sizeof(int), st);
        VL_CHECK_ARG(ce == cudaSuccess, "vl_seen_add: cudaMemsetAsync: %s", cudaGetErrorString(ce));
        return 0;
    }
    ce = cudaMemsetAsync(scratch, 0, sizeof(int) * e, st);
    VL_CHECK_ARG(ce == cudaSuccess, "vl_seen_add: cudaMemsetAsync: %s", cudaGetErrorString(ce));
    column_used_kernel<<<blocks_for(b * e, 256), 256, 0, st>>>(seen, b * e, e, scratch);
    VL_CHECK_LAUNCH("column_used_kernel");
    first_free_column_kernel<<<1, 256, 0, st>>>(scratch, e, first_out);
    VL_CHECK_LAUNCH("first_free_column_kernel");
    int p = pow2_at_least(e);
    dedup_sort_ids_kernel<<<(unsigned)b, kSortThreads, sizeof(vl_key_t) * p, st>>>(seen, e, p, visit, v, first_out);
    VL_CHECK_LAUNCH("dedup_sort_ids_kernel");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// vl_seen_add_noalloc: the visited-list update of vl_seen_add for callers that cannot give it
// scratch memory.  Some hosts of this library own no allocator at the point of the call: a
// serving process whose framework reserved all of HBM up front and hands out nothing later, a
// plugin that is forbidden to allocate after initialisation, or a latency-critical loop in
// which cudaMalloc (which synchronises the whole device) must never run.  For them the per-
// column "is this column used" flags live in the fixed array below instead of a caller buffer.
//
// The array is file-scope device memory: every GPU that loads this library holds one copy of
// it (16 KB) until the process exits.  Its name is a host-side handle, not a device address,
// so host code must not pass it to a kernel; the address is taken once per device with
// cudaGetSymbolAddress while that device is current, and that pointer is what the kernels get.
// All calls on a device share the array and it keeps whatever the previous call left, so each
// call first clears the part it uses; two calls that overlap on the GPU (different streams)
// would race on it - keep calls on one stream or otherwise ordered.
// The first call on a device performs the address look-up; make that first call outside of
// any stream capture.
// ---------------------------------------------------------------------------------------------
#include <mutex>

// VL_SEEN_NOALLOC_MAX_WIDTH (vlgpu.h): most columns (`e`) the fixed scratch can serve
static __device__ __align__(256) int g_seen_scratch[VL_SEEN_NOALLOC_MAX_WIDTH];
// the kernels that consume the flags are sized for rows of at most kMaxSortWidth columns
static_assert(VL_SEEN_NOALLOC_MAX_WIDTH <= kMaxSortWidth, "the fixed scratch must not be wider than a sortable row");

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
int* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of g_seen_scratch on the current device (looked up once per device).
int seen_scratch_address(int** out)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    VL_CHECK_ARG(e == cudaSuccess, "vl_seen_add_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    VL_CHECK_ARG(dev >= 0 && dev < kMaxDevices, "vl_seen_add_noalloc: device %d outside 0..%d", dev, kMaxDevices - 1);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_seen_scratch);
        VL_CHECK_ARG(e == cudaSuccess && p, "vl_seen_add_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_scratch_addr[dev] = static_cast<int*>(p);
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace

extern "C" int vl_seen_add_noalloc(int32_t* seen, int64_t b, int e, const int32_t* visit, int v, int* first_out,
                                   void* stream)
{
    VL_CHECK_ARG(seen && visit && first_out, "vl_seen_add_noalloc: null pointer");
    VL_CHECK_ARG(e >= 0 && e <= VL_SEEN_NOALLOC_MAX_WIDTH,
                 "vl_seen_add_noalloc: list width %d exceeds the fixed scratch of %d columns; use vl_seen_add with a "
                 "caller-provided scratch buffer", e, VL_SEEN_NOALLOC_MAX_WIDTH);
    cudaStream_t st = (cudaStream_t)stream;
    if (e == 0 || b == 0) {   // -1 is four 0xFF bytes: no host buffer involved
        cudaError_t ze = cudaMemsetAsync(first_out, 0xFF, sizeof(int), st);
        VL_CHECK_ARG(ze == cudaSuccess, "vl_seen_add_noalloc: cudaMemsetAsync: %s", cudaGetErrorString(ze));
        return 0;
    }
    int* scratch = nullptr;
    int rc = seen_scratch_address(&scratch);
    if (rc) return rc;
    // the array still holds the previous call's flags: clear the e entries this call reads
    cudaError_t ce = cudaMemsetAsync(scratch, 0, sizeof(int) * e, st);
    VL_CHECK_ARG(ce == cudaSuccess, "vl_seen_add_noalloc: cudaMemsetAsync: %s", cudaGetErrorString(ce));
    column_used_kernel<<<blocks_for(b * e, 256), 256, 0, st>>>(seen, b * e, e, scratch);
    VL_CHECK_LAUNCH("column_used_kernel");
    first_free_column_kernel<<<1, 256, 0, st>>>(scratch, e, first_out);
    VL_CHECK_LAUNCH("first_free_column_kernel");
    int p = pow2_at_least(e);
    dedup_sort_ids_kernel<<<(unsigned)b, kSortThreads, sizeof(vl_key_t) * p, st>>>(seen, e, p, visit, v, first_out);
    VL_CHECK_LAUNCH("dedup_sort_ids_kernel");
    return 0;
}
