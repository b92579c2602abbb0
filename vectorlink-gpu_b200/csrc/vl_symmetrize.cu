// Reverse-edge lists of a neighbour graph: for every node y the nodes x that list y among
// their first `scan` neighbours, best-ranked first.  The reference only sketches this step
// (symmetrize_beams_kernel, vectorlink_gpu/kernels.py:503-550, is dead code inside a string
// literal: an O(N^2) scan with a racy shared counter); here it is three linear passes over the
// edges: in-degree count, CSR fill, and a per-node selection of the `keep` smallest
// (rank of y in x's list, x) keys - which makes the result independent of the order in which
// the atomics of the fill pass happen to land.
#include "vl_common.cuh"

namespace {

__global__ void indegree_kernel(const int32_t* __restrict__ beams, int64_t n, int d, int scan, int32_t* __restrict__ deg,
                                int* __restrict__ status)
{
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n * scan) return;
    int64_t x = t / scan;
    int r = (int)(t - x * scan);
    int32_t y = beams[x * d + r];
    if (y == VL_MAXINT) return;
    if (y < 0 || (int64_t)y >= n) { atomicOr(status, VL_STATUS_BAD_ID); return; }
    atomicAdd(&deg[y], 1);
}

__global__ void fill_kernel(const int32_t* __restrict__ beams, int64_t n, int d, int scan,
                            const int64_t* __restrict__ offsets, int32_t* __restrict__ cursor,
                            vl_key_t* __restrict__ keys)
{
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n * scan) return;
    int64_t x = t / scan;
    int r = (int)(t - x * scan);
    int32_t y = beams[x * d + r];
    if (y == VL_MAXINT || y < 0 || (int64_t)y >= n) return;
    int slot = atomicAdd(&cursor[y], 1);
    keys[offsets[y] + slot] = ((vl_key_t)(uint32_t)r << 32) | (uint32_t)x;
}

// one warp per node: the `keep` smallest keys of its segment, in rising order
__global__ void select_kernel(const vl_key_t* __restrict__ keys, const int64_t* __restrict__ offsets,
                              const int32_t* __restrict__ deg, int64_t n, int keep, int32_t* __restrict__ out)
{
    const int lane = threadIdx.x & 31;
    int64_t y = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (y >= n) return;
    const vl_key_t* seg = keys + offsets[y];
    const int count = deg[y];
    vl_key_t last = 0;
    bool first = true;
    for (int i = 0; i < keep; ++i) {
        vl_key_t best = ~0ull;
        for (int c = lane; c < count; c += 32) {
            vl_key_t k = seg[c];
            if ((first || k > last) && k < best) best = k;
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            vl_key_t o = __shfl_xor_sync(0xffffffffu, best, off);
            best = o < best ? o : best;
        }
        if (lane == 0) out[y * keep + i] = best == ~0ull ? VL_MAXINT : (int32_t)(uint32_t)best;
        if (best == ~0ull) {
            for (int j = i + 1 + lane; j < keep; j += 32) out[y * keep + j] = VL_MAXINT;
            break;
        }
        last = best;
        first = false;
    }
}

}  // namespace

extern "C" int vl_reverse_edges(const int32_t* beams, int64_t n, int d, int scan, int phase, int32_t* deg,
                                const int64_t* offsets, int32_t* cursor, unsigned long long* keys, int keep,
                                int32_t* out, int* status, void* stream)
{
    VL_CHECK_ARG(beams && deg && status, "vl_reverse_edges: null pointer");
    VL_CHECK_ARG(n >= 0 && d > 0 && scan > 0 && scan <= d, "vl_reverse_edges: bad shape");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned blocks = (unsigned)((n * scan + 255) / 256);
    if (phase == 0) {
        indegree_kernel<<<blocks, 256, 0, st>>>(beams, n, d, scan, deg, status);
        VL_CHECK_LAUNCH("indegree_kernel");
        return 0;
    }
    VL_CHECK_ARG(phase == 1, "vl_reverse_edges: phase %d is neither 0 (count) nor 1 (fill + select)", phase);
    VL_CHECK_ARG(offsets && cursor && keys && out && keep > 0, "vl_reverse_edges: null pointer");
    fill_kernel<<<blocks, 256, 0, st>>>(beams, n, d, scan, offsets, cursor, keys);
    VL_CHECK_LAUNCH("fill_kernel");
    select_kernel<<<(unsigned)((n + 3) / 4), 128, 0, st>>>(keys, offsets, deg, n, keep, out);
    VL_CHECK_LAUNCH("select_kernel");
    return 0;
}
