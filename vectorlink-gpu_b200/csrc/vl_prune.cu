// Detour prune + per-row sort + top-degree cut: the replacement of the reference's
// prune_kernel / prune_ (vectorlink_gpu/kernels.py:409-468) and of the narrow to the first
// `beam_size` columns that generate_ann applies afterwards (ann.py:190-193).
//
// Reference semantics kept: the kernel is launched with block (W,1,1) but indexes
// threadIdx.y, so the detour witness z is always y's FIRST neighbour; x->z is punched when
// d(x,z) > d(x,y) and d(x,z) > d(y,z).  The reference edits rows in place with one CTA per
// (x, slot); here one warp owns row x and walks its slots in rising order, seeing its own
// earlier punches - the order in which the reference's blocks are numbered, and the one the
// Numba simulator executes.  Other rows are read only at slot 0, which a row sorted by
// distance never loses, so rows are independent and the result is deterministic.
#include "vl_common.cuh"
#include "vlgpu.h"

namespace {

constexpr int kPruneWarps = 4;

__device__ __forceinline__ void warp_bitonic_sort(vl_key_t* keys, int p, int lane)
{
    for (int k = 2; k <= p; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = lane; t < p / 2; t += 32) {
                int lo = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                int hi = lo | j;
                bool up = ((lo & k) == 0);
                vl_key_t a = keys[lo], b = keys[hi];
                if ((a > b) == up) { keys[lo] = b; keys[hi] = a; }
            }
            __syncwarp();
        }
    }
}

__global__ void __launch_bounds__(kPruneWarps * 32)
prune_kernel(const int32_t* __restrict__ beams, const float* __restrict__ dist, int64_t n, int64_t x0, int64_t x1, int w,
             int do_punch, int32_t* __restrict__ beams_out, float* __restrict__ dist_out, int out_cols, int p,
             int* __restrict__ status)
{
    extern __shared__ vl_key_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // per warp: keys[p] | ids[w] | d[w] | z[w] | dyz[w]
    const size_t per_warp = (size_t)p + 2 * (size_t)((w + 1) / 2) * 2;
    vl_key_t* keys = smem + warp * per_warp;
    int32_t* ids = reinterpret_cast<int32_t*>(keys + p);
    float* d = reinterpret_cast<float*>(ids + w);
    int32_t* zs = reinterpret_cast<int32_t*>(d + w);
    float* dyz = reinterpret_cast<float*>(zs + w);

    for (int64_t x = x0 + (int64_t)blockIdx.x * kPruneWarps + warp; x < x1; x += (int64_t)gridDim.x * kPruneWarps) {
        for (int s = lane; s < w; s += 32) {
            int32_t y = beams[x * w + s];
            float dxy = dist[x * w + s];
            ids[s] = y;
            d[s] = dxy;
            int32_t z = VL_MAXINT;
            float dz = VL_MAXFLOAT;
            if (do_punch == 1 && y != VL_MAXINT) {
                if (y < 0 || (int64_t)y >= n) atomicOr(status, VL_STATUS_BAD_ID);
                else { z = beams[(int64_t)y * w]; dz = dist[(int64_t)y * w]; }
            }
            zs[s] = z;
            dyz[s] = dz;
        }
        __syncwarp();
        if (do_punch == 2) {
            // The scan the authors describe (kernels.py:441-457) but never ran: every neighbour z
            // of y is a possible detour witness, not only y's first one.  Rows of y come from the
            // input buffers; row x sees its own earlier punches, slots in rising order.
            for (int s = 0; s < w; ++s) {
                const int32_t y = ids[s];
                if (y == VL_MAXINT || y < 0 || (int64_t)y >= n) continue;
                const float dxy = d[s];
                for (int j0 = 0; j0 < w; j0 += 32) {
                    const int j = j0 + lane;
                    int32_t z = VL_MAXINT;
                    float dz = VL_MAXFLOAT;
                    if (j < w) { z = beams[(int64_t)y * w + j]; dz = dist[(int64_t)y * w + j]; }
                    // each lane looks its z up in row x (last matching slot), then punches
                    int xi = -1;
                    if (z != VL_MAXINT)
                        for (int i = 0; i < w; ++i) if (ids[i] == z) xi = i;
                    const bool hit = xi >= 0 && d[xi] > dxy && d[xi] > dz;
                    __syncwarp();
                    if (hit) { ids[xi] = VL_MAXINT; d[xi] = VL_MAXFLOAT; }
                    __syncwarp();
                }
            }
        } else if (do_punch) {
            for (int s = 0; s < w; ++s) {
                if (ids[s] == VL_MAXINT) continue;       // warp-uniform: shared reads
                int32_t z = zs[s];
                if (z == VL_MAXINT) continue;
                int xi = -1;                              // kernels.py:424-427: the LAST matching slot
                for (int base = ((w - 1) / 32) * 32; base >= 0 && xi < 0; base -= 32) {
                    int i = base + lane;
                    unsigned hit = __ballot_sync(0xffffffffu, i < w && ids[i] == z);
                    if (hit) xi = base + 31 - __clz(hit);
                }
                if (xi < 0) continue;
                float dxz = d[xi];
                if (dxz > d[s] && dxz > dyz[s]) {
                    __syncwarp();
                    if (lane == 0) { ids[xi] = VL_MAXINT; d[xi] = VL_MAXFLOAT; }
                    __syncwarp();
                }
            }
        }
        for (int i = lane; i < p; i += 32) keys[i] = i < w ? vl_make_key(d[i], ids[i]) : ~0ull;
        __syncwarp();
        warp_bitonic_sort(keys, p, lane);
        for (int i = lane; i < out_cols; i += 32) {
            beams_out[x * out_cols + i] = vl_key_id(keys[i]);
            dist_out[x * out_cols + i] = vl_key_dist(keys[i]);
        }
        __syncwarp();
    }
}

}  // namespace

extern "C" int vl_prune_rows(const int32_t* beams, const float* dist, int64_t n, int w, int64_t row_lo, int64_t row_hi,
                             int do_punch, int32_t* beams_out, float* dist_out, int out_cols, int* status, void* stream)
{
    VL_CHECK_ARG(beams && dist && beams_out && dist_out && status, "vl_prune: null pointer");
    VL_CHECK_ARG(w > 0 && w <= 2048, "vl_prune: row width %d outside 1..2048", w);
    VL_CHECK_ARG(out_cols > 0 && out_cols <= w, "vl_prune: cannot keep %d of %d columns", out_cols, w);
    VL_CHECK_ARG(beams != beams_out && dist != dist_out, "vl_prune: output must not alias input");
    VL_CHECK_ARG(0 <= row_lo && row_lo <= row_hi && row_hi <= n, "vl_prune: rows [%lld, %lld) outside [0, %lld)",
                 (long long)row_lo, (long long)row_hi, (long long)n);
    if (row_hi == row_lo) return 0;
    int p = 2;
    while (p < w) p <<= 1;
    size_t per_warp = (size_t)p + 2 * (size_t)((w + 1) / 2) * 2;
    size_t smem = per_warp * sizeof(vl_key_t) * kPruneWarps;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(prune_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        VL_CHECK_ARG(e == cudaSuccess, "vl_prune: %s", cudaGetErrorString(e));
    }
    int64_t blocks = (row_hi - row_lo + kPruneWarps - 1) / kPruneWarps;
    const int64_t cap = (int64_t)vl_sm_count() * 32;
    if (blocks > cap) blocks = cap;
    prune_kernel<<<(unsigned)blocks, kPruneWarps * 32, smem, (cudaStream_t)stream>>>(beams, dist, n, row_lo, row_hi, w, do_punch,
                                                                                   beams_out, dist_out, out_cols, p, status);
    VL_CHECK_LAUNCH("prune_kernel");
    return 0;
}

extern "C" int vl_prune(const int32_t* beams, const float* dist, int64_t n, int w, int do_punch,
                        int32_t* beams_out, float* dist_out, int out_cols, int* status, void* stream)
{
    VL_CHECK_ARG(n >= 0, "vl_prune: negative row count");
    return vl_prune_rows(beams, dist, n, w, 0, n, do_punch, beams_out, dist_out, out_cols, status, stream);
}
