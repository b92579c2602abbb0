// Initial-kNN tile pass: a tensor-core proposal of near neighbours for the start graph of the
// build, as an opt-in replacement of the circulant start graph the reference uses
// (vectorlink_gpu/utils.py:35-41, called at ann.py:116-118).  Not in the reference.
//
// The pass only PROPOSES candidates: bf16 inner products of a tile of 128 rows against tiles
// of 128 candidate rows on the 5th-generation tensor cores, a per-row running top-k of the
// approximate score (|c|^2 - 2<q,c> for squared L2, -2<q,c> for cosine).  The caller then
// re-evaluates every proposed pair with the exact fp32 summation tree (vl_calculate_distances)
// and orders them with vl_sort_pairs, so the lists that enter the graph carry the same exact
// distances as everything else; bf16 only decides which pairs get that exact evaluation.
//
// Shape of the kernel (one CTA per SM, persistent over work items = row tile x candidate segment):
//   warp 0, one lane : TMA producer - cp.async.bulk.tensor 2D loads of the row tile's and the
//                      candidate tile's 64-column k-block (128 B rows, 128B swizzle) into a
//                      4-stage shared-memory ring, completion on an mbarrier per stage;
//   warp 1, one lane : issues tcgen05.mma (kind::f16, bf16 x bf16 -> fp32, M=128, N=128, K=16)
//                      from shared-memory descriptors into one of two TMEM accumulators
//                      (128 columns each), tcgen05.commit releases the stage / publishes the tile;
//   warps 2..5       : read their quarter of the accumulator's 128 lanes with tcgen05.ld (one
//                      row per thread), turn inner products into scores and keep the row's
//                      32 best (score, id) keys in registers; the accumulator is handed back as
//                      soon as it is read, so the next tile's MMAs overlap the selection.
// No load uses cluster multicast, no thread-block cluster is launched.
//
// Every wait (mbarrier phases) is bounded by wall time: when a wait runs out the kernel sets
// VL_STATUS_TIMEOUT in the status word, raises a CTA-wide abort flag that ends all roles, waits
// (bounded again) for its own copies and MMAs in flight, frees its TMEM columns and returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include "vl_common.cuh"

namespace {

constexpr int kTileRows = 128;                 // M of the MMA: rows of the row tile
constexpr int kTileCands = 128;                // N of the MMA: candidates per tile
constexpr int kBlockK = 64;                    // bf16 elements per k-block = one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kTopK = VL_KNN_TILE_K;           // keys kept per row and segment
constexpr int kThreads = 192;                  // warp 0 producer, warp 1 MMA, warps 2-5 selection
constexpr uint32_t kTileBytes = kTileRows * kBlockK * 2;              // 16 KB per operand per stage
constexpr uint32_t kStageBytes = 2 * kTileBytes;
constexpr uint32_t kTmemCols = 2 * kTileCands;                         // two accumulators
constexpr unsigned long long kWaitLimitNs = 2000000000ull;             // 2 s per wait

// shared-memory layout behind the 1024-byte aligned base
constexpr uint32_t kOffBars = kStages * kStageBytes;                   // full[4] empty[4] tfull[2] tempty[2] drain[1]
constexpr uint32_t kOffSlot = kOffBars + 8 * (2 * kStages + 5);        // TMEM base address written by tcgen05.alloc
constexpr uint32_t kOffAbort = kOffSlot + 4;
constexpr uint32_t kOffBias = (kOffAbort + 4 + 127) & ~127u;           // [4 warps][2 buffers][128] floats
constexpr uint32_t kOffPend = kOffBias + 4 * 2 * kTileCands * 4;      // [32 slots][128 rows] keys waiting for insertion
constexpr uint32_t kSmemBytes = kOffPend + 32 * kTileRows * 8 + 1024;  // + slack for the alignment

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long now_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Waits for the phase of `bar` with the given parity.  False when another role raised the abort
// flag or when the wait ran out of time (it then raises the flag itself and records the timeout).
__device__ __noinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status)
{
    if (mbar_test(bar, parity)) return true;
    const unsigned long long t0 = now_ns();
#pragma unroll 1
    for (uint32_t spin = 0;; ++spin) {
        if (mbar_test(bar, parity)) return true;
        if ((spin & 31u) == 31u) {
            if (*abort_flag) return false;
            if (now_ns() - t0 > kWaitLimitNs) {
                *abort_flag = 1;
                atomicOr(status, VL_STATUS_TIMEOUT);
                return false;
            }
            __nanosleep(40);
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, bf16 inputs, fp32 accumulate, M=128 N=128 K=16
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive accumulator columns of this thread's TMEM lane
__device__ __forceinline__ void tc_load32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major bf16 tile stored as 128-byte rows under the 128B
// swizzle (what the TMA box {64, 128} with CU_TENSOR_MAP_SWIZZLE_128B writes): start address and
// offsets in 16-byte units, 8-row groups 1024 bytes apart, descriptor version 1 (sm_100),
// layout type 2 = 128-byte swizzle.  The tile base is 1024-byte aligned (base offset 0).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr)
{
    return (uint64_t)((addr & 0x3ffffu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// kind::f16 instruction descriptor: D fp32, A and B bf16, both K-major, N=128, M=128
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTileCands >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);

struct KnnArgs {
    const float* bias;        // |c|^2 per candidate row (squared L2) or nullptr (cosine)
    int64_t n;                // rows of the bf16 matrix
    int kblocks;              // padded dimension / 64
    int64_t row_lo, row_hi;   // rows that get lists
    int64_t cand_lo, cand_hi; // candidates offered to every row
    int segments;             // the candidate range is cut into this many parts, each with its own top-k
    int64_t seg_len;          // candidates per part (a multiple of 128)
    int32_t* out_ids;         // [row_hi - row_lo, segments * kTopK]
    int* status;
};

__global__ void __launch_bounds__(kThreads, 1)
knn_tile_kernel(const __grid_constant__ CUtensorMap tmap, const KnnArgs a)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - raw);
    const uint32_t bar_full = base + kOffBars;                    // + 8 * stage
    const uint32_t bar_empty = bar_full + 8 * kStages;
    const uint32_t bar_tfull = bar_empty + 8 * kStages;           // + 8 * accumulator
    const uint32_t bar_tempty = bar_tfull + 16;
    const uint32_t bar_drain = bar_tempty + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + kOffSlot);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + kOffAbort);
    float* bias_smem = reinterpret_cast<float*>(base_ptr + kOffBias);
    vl_key_t* pend_smem = reinterpret_cast<vl_key_t*>(base_ptr + kOffPend);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, 4); }
        mbar_init(bar_drain, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void*)tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t row_tiles = (a.row_hi - a.row_lo + kTileRows - 1) / kTileRows;
    const int64_t items = row_tiles * a.segments;

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        uint32_t it = 0;
        bool ok = true;
#pragma unroll 1
        for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
            const int64_t rt = item / a.segments, seg = item % a.segments;
            const int64_t row0 = a.row_lo + rt * kTileRows;
            const int64_t c_begin = a.cand_lo + seg * a.seg_len;
            const int64_t c_end = (c_begin + a.seg_len < a.cand_hi) ? c_begin + a.seg_len : a.cand_hi;
#pragma unroll 1
            for (int64_t c0 = c_begin; c0 < c_end && ok; c0 += kTileCands) {
#pragma unroll 1
                for (int kb = 0; kb < a.kblocks; ++kb, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, a.status);
                    if (!ok) break;
                    mbar_expect_tx(bar_full + 8 * s, kStageBytes);
                    tma_load_2d(base + s * kStageBytes, &tmap, kb * kBlockK, (int)row0, bar_full + 8 * s);
                    tma_load_2d(base + s * kStageBytes + kTileBytes, &tmap, kb * kBlockK, (int)c0, bar_full + 8 * s);
                }
            }
        }
        if (!ok) {
            // leaving early: the copies already issued still land in shared memory; wait for them
            const uint32_t issued = it < kStages ? it : kStages;
            for (uint32_t j = 0; j < issued; ++j) {
                const uint32_t last = it - 1 - j;
                const unsigned long long t0 = now_ns();
                while (!mbar_test(bar_full + 8 * (last % kStages), (last / kStages) & 1u) && now_ns() - t0 < kWaitLimitNs) __nanosleep(100);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        uint32_t it = 0, tile = 0;
        bool ok = true;
#pragma unroll 1
        for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
            const int64_t seg = item % a.segments;
            const int64_t c_begin = a.cand_lo + seg * a.seg_len;
            const int64_t c_end = (c_begin + a.seg_len < a.cand_hi) ? c_begin + a.seg_len : a.cand_hi;
#pragma unroll 1
            for (int64_t c0 = c_begin; c0 < c_end && ok; c0 += kTileCands, ++tile) {
                const uint32_t buf = tile & 1u, tph = (tile >> 1) & 1u;
                ok = mbar_wait(bar_tempty + 8 * buf, tph ^ 1u, abort_flag, a.status);   // accumulator drained?
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * kTileCands;
#pragma unroll 1
                for (int kb = 0; kb < a.kblocks; ++kb, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, a.status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t a_desc = smem_desc_sw128(base + s * kStageBytes);
                    const uint64_t b_desc = smem_desc_sw128(base + s * kStageBytes + kTileBytes);
#pragma unroll
                    for (int kk = 0; kk < kBlockK / 16; ++kk)      // 16 bf16 = 32 bytes = 2 descriptor units per step
                        tc_mma_bf16(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, kIdesc, (kb | kk) != 0);
                    tc_commit(bar_empty + 8 * s);                  // stage reusable once these MMAs have read it
                }
                if (ok) tc_commit(bar_tfull + 8 * buf);            // accumulator complete
            }
        }
        // every MMA issued above must have finished before the TMEM columns are given back
        tc_commit(bar_drain);
        {
            const unsigned long long t0 = now_ns();
            while (!mbar_test(bar_drain, 0) && now_ns() - t0 < kWaitLimitNs) __nanosleep(100);
        }
    } else if (warp >= 2) {
        // ---------------- selection: one row of the tile per thread ----------------
        const int quarter = warp & 3;                              // the TMEM lanes this warp may read
        const int row_in_tile = quarter * 32 + lane;
        float* my_bias = bias_smem + (warp - 2) * 2 * kTileCands;
        uint32_t tile = 0;
        bool ok = true;
#pragma unroll 1
        for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
            const int64_t rt = item / a.segments, seg = item % a.segments;
            const int64_t row = a.row_lo + rt * kTileRows + row_in_tile;
            const int64_t c_begin = a.cand_lo + seg * a.seg_len;
            const int64_t c_end = (c_begin + a.seg_len < a.cand_hi) ? c_begin + a.seg_len : a.cand_hi;
            // the row's best keys so far, ascending, in registers; `worst` = score of the last one
            vl_key_t top[kTopK];
#pragma unroll
            for (int j = 0; j < kTopK; ++j) top[j] = ~0ull;
            float worst = __int_as_float(0x7f800000);             // +inf until the list is full
            vl_key_t* pend = pend_smem + row_in_tile;              // slot p of this row at pend[p * kTileRows]
#pragma unroll 1
            for (int64_t c0 = c_begin; c0 < c_end; c0 += kTileCands, ++tile) {
                const uint32_t buf = tile & 1u, tph = (tile >> 1) & 1u;
                // this warp's copy of the tile's score offsets: |c|^2 (squared L2) or 0 (cosine), +inf past the
                // segment's end so that such a column never qualifies (warp-local: this role uses no CTA-wide barrier)
                __syncwarp();
#pragma unroll
                for (int j = lane; j < kTileCands; j += 32)
                    my_bias[buf * kTileCands + j] = (c0 + j < c_end) ? (a.bias ? __ldg(a.bias + c0 + j) : 0.0f)
                                                                     : __int_as_float(0x7f800000);
                __syncwarp();
                ok = mbar_wait(bar_tfull + 8 * buf, tph, abort_flag, a.status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * kTileCands;
#pragma unroll 1
                for (int ch = 0; ch < kTileCands / 32; ++ch) {
                    uint32_t v[32];
                    __syncwarp();                                   // the loads below are warp-collective
                    tc_load32(taddr + ch * 32, v);
                    tc_wait_ld();
                    // pass 1 (unrolled, a few instructions per column): which columns beat the row's worst key
                    int n_pend = 0;
                    const float* bias_ch = my_bias + buf * kTileCands + ch * 32;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float score = fmaf(-2.0f, __uint_as_float(v[j]), bias_ch[j]);
                        if (score < worst) {
                            pend[n_pend * kTileRows] = ((vl_key_t)vl_ord(score) << 32) | (uint32_t)(c0 + ch * 32 + j);
                            ++n_pend;
                        }
                    }
                    // pass 2 (rare after the first tiles): sorted insertion, one copy of the code
#pragma unroll 1
                    for (int p = 0; p < n_pend; ++p) {
                        const vl_key_t key = pend[p * kTileRows];
                        if ((int64_t)(uint32_t)key == row || !(key < top[kTopK - 1])) continue;
                        top[kTopK - 1] = key;            // replace the worst, then let it sink to its place
#pragma unroll
                        for (int t = kTopK - 1; t > 0; --t) {
                            const vl_key_t lo = top[t - 1], hi = top[t];
                            const bool sw = hi < lo;
                            top[t - 1] = sw ? hi : lo;
                            top[t] = sw ? lo : hi;
                        }
                        if (top[kTopK - 1] != ~0ull) worst = vl_unord((uint32_t)(top[kTopK - 1] >> 32));
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);  // 4 warps -> accumulator free again
            }
            if (ok && row < a.row_hi) {
                int32_t* out = a.out_ids + ((row - a.row_lo) * a.segments + seg) * kTopK;
#pragma unroll
                for (int j = 0; j < kTopK; ++j) out[j] = top[j] == ~0ull ? VL_MAXINT : (int32_t)(uint32_t)top[j];
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// fp32 rows -> bf16 rows padded with zeros to dim_pad columns, and |row|^2 in fp32
__global__ void knn_prepare_kernel(const float* __restrict__ vectors, int64_t n, int dim, __nv_bfloat16* __restrict__ out,
                                   int dim_pad, float* __restrict__ sqnorm)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp0; r < n; r += nwarps) {
        float acc = 0.0f;
        for (int c = lane; c < dim_pad; c += 32) {
            const float x = c < dim ? __ldg(vectors + r * dim + c) : 0.0f;
            out[r * dim_pad + c] = __float2bfloat16_rn(x);
            acc = fmaf(x, x, acc);
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (sqnorm && lane == 0) sqnorm[r] = acc;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

extern "C" int vl_knn_prepare(const float* vectors, int64_t n, int dim, uint16_t* bf16_out, int dim_pad, float* sqnorm_out,
                              void* stream)
{
    VL_CHECK_ARG(vectors && bf16_out, "vl_knn_prepare: null pointer");
    VL_CHECK_ARG(n >= 0 && dim > 0 && dim_pad >= dim && dim_pad % kBlockK == 0,
                 "vl_knn_prepare: dim_pad %d must be a multiple of %d not below dim %d", dim_pad, kBlockK, dim);
    if (n == 0) return 0;
    int64_t blocks = (n + 7) / 8;
    const int64_t cap = (int64_t)vl_sm_count() * 16;
    if (blocks > cap) blocks = cap;
    knn_prepare_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(vectors, n, dim, reinterpret_cast<__nv_bfloat16*>(bf16_out),
                                                                         dim_pad, sqnorm_out);
    VL_CHECK_LAUNCH("knn_prepare_kernel");
    return 0;
}

extern "C" int vl_knn_tile(const uint16_t* rows_bf16, int64_t n, int dim_pad, const float* sqnorm, int64_t row_lo,
                           int64_t row_hi, int64_t cand_lo, int64_t cand_hi, int segments, int32_t* out_ids, int* status,
                           void* stream)
{
    VL_CHECK_ARG(rows_bf16 && out_ids && status, "vl_knn_tile: null pointer");
    VL_CHECK_ARG(n > 0 && n < (1ll << 31), "vl_knn_tile: row count %lld outside int32", (long long)n);
    VL_CHECK_ARG(dim_pad > 0 && dim_pad % kBlockK == 0, "vl_knn_tile: padded dimension %d is not a multiple of %d", dim_pad, kBlockK);
    VL_CHECK_ARG((uintptr_t)rows_bf16 % 16 == 0, "vl_knn_tile: the bf16 matrix must be 16-byte aligned");
    VL_CHECK_ARG(0 <= row_lo && row_lo <= row_hi && row_hi <= n, "vl_knn_tile: bad row range");
    VL_CHECK_ARG(0 <= cand_lo && cand_lo <= cand_hi && cand_hi <= n, "vl_knn_tile: bad candidate range");
    VL_CHECK_ARG(segments >= 1 && segments <= 64, "vl_knn_tile: segments %d outside 1..64", segments);
    if (row_hi == row_lo) return 0;

    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        VL_CHECK_ARG(e == cudaSuccess && q == cudaDriverEntryPointSuccess && fn, "vl_knn_tile: cuTensorMapEncodeTiled is not available");
        encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    CUtensorMap tmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)dim_pad, (cuuint64_t)n};
    const cuuint64_t gstride[1] = {(cuuint64_t)dim_pad * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)kTileRows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(rows_bf16), gdim, gstride, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    VL_CHECK_ARG(cr == CUDA_SUCCESS, "vl_knn_tile: cuTensorMapEncodeTiled failed (%d)", (int)cr);

    KnnArgs a;
    a.bias = sqnorm;
    a.n = n;
    a.kblocks = dim_pad / kBlockK;
    a.row_lo = row_lo; a.row_hi = row_hi;
    a.cand_lo = cand_lo; a.cand_hi = cand_hi;
    a.segments = segments;
    const int64_t span = cand_hi - cand_lo;
    int64_t seg_len = (span + segments - 1) / segments;
    seg_len = (seg_len + kTileCands - 1) / kTileCands * kTileCands;
    a.seg_len = seg_len > 0 ? seg_len : kTileCands;
    a.out_ids = out_ids;
    a.status = status;

    cudaError_t e = cudaFuncSetAttribute(knn_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    VL_CHECK_ARG(e == cudaSuccess, "vl_knn_tile: %s", cudaGetErrorString(e));
    const int64_t items = ((row_hi - row_lo + kTileRows - 1) / kTileRows) * segments;
    const int sms = vl_sm_count();
    const unsigned grid = (unsigned)(items < sms ? items : sms);
    knn_tile_kernel<<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(tmap, a);
    VL_CHECK_LAUNCH("knn_tile_kernel");
    return 0;
}
