// Initial-kNN tile pass: a tensor-core proposal of near neighbours for the start graph of the
// build, as an opt-in replacement of the circulant start graph the reference uses
// (vectorlink_gpu/utils.py:35-41, called at ann.py:116-118).  Not in the reference.
//
// The pass only PROPOSES candidates: bf16 inner products of a tile of 128 rows against tiles
// of 256 candidate rows on the 5th-generation tensor cores, a per-row running top-k of the
// approximate score (|c|^2 - 2<q,c> for squared L2, -2<q,c> for cosine).  The caller then
// re-evaluates every proposed pair with the exact fp32 summation tree (vl_calculate_distances)
// and orders them with vl_sort_pairs, so the lists that enter the graph carry the same exact
// distances as everything else; bf16 only decides which pairs get that exact evaluation.
//
// Shape of the kernel (one CTA per SM, persistent over work items = row tile x candidate segment):
//   warp 0, one lane : TMA producer - cp.async.bulk.tensor 2D loads of 64-column k-blocks (128 B
//                      rows, 128B swizzle) into a shared-memory ring, completion on an mbarrier
//                      per stage.  Rows of at most 128 padded columns keep the row tile resident
//                      (loaded once per work item) and stream only candidate tiles (3 stages of
//                      32 KB); longer rows stream both operands (3 stages of 48 KB);
//   warp 1, one lane : issues tcgen05.mma (kind::f16, bf16 x bf16 -> fp32, M=128, N=256, K=16)
//                      from shared-memory descriptors into one of two TMEM accumulators
//                      (256 columns each: all of TMEM), tcgen05.commit releases the stage /
//                      publishes the tile.  (N=128 tiles measured 17 % slower: the row operand is
//                      fetched from shared memory once per instruction whatever N is);
//   warps 2..17      : selection, one warp per (quarter of the tile's rows, column class).  Class c is
//                      columns [64 c, 64 c + 64) of every tile, so all sixteen warps examine a tile at
//                      once while the MMAs of the next tile fill the other accumulator, and a row
//                      ends up with four lists per segment (the 16 best of each class).  A warp
//                      reads its quarter of the accumulator's 128 lanes with tcgen05.ld (one row per
//                      thread, 32 columns per instruction), turns inner products into scores
//                      and keeps each row's 16 best (score, id) keys in shared memory, one key per
//                      lane.  The common path costs one instruction per column: two scores per packed
//                      FMA, the minimum of eight scores by 3-input min, one compare; only groups of
//                      eight columns in which some row beats its worst key are looked at column by
//                      column, and each such (row, column) is inserted by the warp with one ballot
//                      and one shuffle.  The accumulator is handed back as soon as the tile's last
//                      columns are in registers.  (Measured on 1M x 128 rows: two groups of four warps
//                      that own one accumulator each, i.e. alternate tiles: 0.48 s; eight warps on
//                      every tile, two classes: 0.42 s; sixteen warps, four classes: 0.36 s; with the
//                      packed / min3 common path: 0.33 s; the MMA and TMA side alone: 0.21 s.)
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
constexpr int kTileCands = 256;                // N of the MMA: candidates per tile
constexpr int kBlockK = 64;                    // bf16 elements per k-block = one 128-byte swizzle row
constexpr int kMaxStages = 4;                  // barrier slots (3 stages in use)
constexpr int kResidentKBlocks = 2;            // row tiles of up to 2 k-blocks (128 columns) stay in shared memory
constexpr int kTopK = VL_KNN_TILE_K;           // keys per list
constexpr int kLists = VL_KNN_TILE_LISTS;      // lists per row and segment: one per column class of a tile
constexpr int kSelCols = kTileCands / kLists;  // class c = columns [c * kSelCols, (c + 1) * kSelCols) of every tile
constexpr int kSelWarps = 4 * kLists;          // one selection warp per (quarter of the rows, column class)
constexpr int kThreads = 64 + 32 * kSelWarps;  // warp 0 producer, warp 1 MMA, warps 2-17 selection
constexpr uint32_t kTileBytes = kTileRows * kBlockK * 2;              // 16 KB: one k-block of the row tile
constexpr uint32_t kCandBytes = kTileCands * kBlockK * 2;             // 32 KB: one k-block of a candidate tile
// operand region, 144 KB: resident mode = 3 candidate stages of 32 KB + the row tile's 2 k-blocks;
// streaming mode = 3 stages of (candidates 32 KB + rows 16 KB)
constexpr uint32_t kOperandBytes = 3 * (kCandBytes + kTileBytes);
constexpr uint32_t kOffRowTile = 3 * kCandBytes;
constexpr uint32_t kTmemCols = 2 * kTileCands;                         // two accumulators
constexpr unsigned long long kWaitLimitNs = 2000000000ull;             // 2 s per wait

// shared-memory layout behind the 1024-byte aligned base
constexpr uint32_t kOffBars = kOperandBytes;
// full[4] empty[4] tfull[2] tempty[2] drain rows_full rows_empty
constexpr uint32_t kOffSlot = kOffBars + 8 * (2 * kMaxStages + 7);     // TMEM base address written by tcgen05.alloc
constexpr uint32_t kOffAbort = kOffSlot + 4;
constexpr uint32_t kOffBias = (kOffAbort + 4 + 127) & ~127u;           // [16 warps][64] floats: score offsets of a warp's columns of the current tile
constexpr uint32_t kOffLists = kOffBias + kSelWarps * kSelCols * 4;    // [4 classes][128 rows][16] best keys of the work item
constexpr uint32_t kSmemBytes = kOffLists + kLists * kTileRows * kTopK * 8 + 1024;   // + slack for the alignment
static_assert(kTopK == 16 && kLists == 4, "a row's list is held one key per lane of a half warp; 64 columns per class");
static_assert(kSelCols % 32 == 0, "a selection warp examines whole chunks of 32 columns");
static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA");

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
// D[tmem] (+)= A[smem] * B[smem]^T, bf16 inputs, fp32 accumulate, M=128 N=256 K=16
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

// kind::f16 instruction descriptor: D fp32, A and B bf16, both K-major, N=256, M=128
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTileCands >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);

#ifdef VL_KNN_STATS
#define VL_T0() const long long t_begin__ = clock64()
#define VL_T1(slot) do { if (a.stats) atomicAdd(a.stats + (slot), (unsigned long long)(clock64() - t_begin__)); } while (0)
#else
#define VL_T0() do {} while (0)
#define VL_T1(slot) do {} while (0)
#endif

struct KnnArgs {
    const float* bias;        // |c|^2 per candidate row (squared L2) or nullptr (cosine)
    int64_t n;                // rows of the bf16 matrix
    int kblocks;              // padded dimension / 64
    int64_t row_lo, row_hi;   // rows that get lists
    int64_t cand_lo, cand_hi; // candidates offered to every row
    int segments;             // the candidate range is cut into this many parts, each with its own top-k
    int64_t seg_len;          // candidates per part (a multiple of 256)
    int32_t* out_ids;         // [row_hi - row_lo, segments, kLists, kTopK]
    int* status;
    unsigned long long* stats; // cycle counters of a profiling build (-DVL_KNN_STATS), else unused
};

// v[j] for a j that is the same in every lane of the warp: a jump on j (register arrays cannot be
// indexed at run time; the branch is uniform, so it costs one case, not thirty-two)
__device__ __forceinline__ uint32_t pick32(const uint32_t (&v)[32], int j)
{
    uint32_t x = 0;
    switch (j) {
#define VL_PICK(i) case i: x = v[i]; break;
        VL_PICK(0) VL_PICK(1) VL_PICK(2) VL_PICK(3) VL_PICK(4) VL_PICK(5) VL_PICK(6) VL_PICK(7)
        VL_PICK(8) VL_PICK(9) VL_PICK(10) VL_PICK(11) VL_PICK(12) VL_PICK(13) VL_PICK(14) VL_PICK(15)
        VL_PICK(16) VL_PICK(17) VL_PICK(18) VL_PICK(19) VL_PICK(20) VL_PICK(21) VL_PICK(22) VL_PICK(23)
        VL_PICK(24) VL_PICK(25) VL_PICK(26) VL_PICK(27) VL_PICK(28) VL_PICK(29) VL_PICK(30) VL_PICK(31)
#undef VL_PICK
    }
    return x;
}

// two scores at once: {b0, b1} - 2 * {v0, v1}, each half an ordinary fp32 fma
__device__ __forceinline__ void score2(uint32_t v0, uint32_t v1, float b0, float b1, float& s0, float& s1)
{
    asm("{\n\t.reg .b64 A, B, C, D;\n\tmov.b64 A, {%2, %3};\n\tmov.b64 B, {%4, %4};\n\tmov.b64 C, {%5, %6};\n\t"
        "fma.rn.f32x2 D, A, B, C;\n\tmov.b64 {%0, %1}, D;\n\t}"
        : "=f"(s0), "=f"(s1) : "r"(v0), "r"(v1), "f"(-2.0f), "f"(b0), "f"(b1));
}
__device__ __forceinline__ float min3f(float a, float b, float c)
{
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// RESIDENT: the row tile (all its k-blocks) is loaded once per work item and only candidate
// tiles go through the ring; otherwise a ring stage holds one k-block of both operands.
template <bool RESIDENT>
__global__ void __launch_bounds__(kThreads, 1)
knn_tile_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap_cand, const KnnArgs a)
{
    constexpr uint32_t kStages = 3;
    constexpr uint32_t kStageBytes = RESIDENT ? kCandBytes : kCandBytes + kTileBytes;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - raw);
    const uint32_t bar_full = base + kOffBars;                    // + 8 * stage
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;
    const uint32_t bar_tfull = bar_empty + 8 * kMaxStages;        // + 8 * accumulator
    const uint32_t bar_tempty = bar_tfull + 16;
    const uint32_t bar_drain = bar_tempty + 16;
    const uint32_t bar_rows_full = bar_drain + 8;                 // resident row tile landed
    const uint32_t bar_rows_empty = bar_rows_full + 8;            // every MMA that reads it has finished
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + kOffSlot);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + kOffAbort);
    float* bias_smem = reinterpret_cast<float*>(base_ptr + kOffBias);
    vl_key_t* lists_smem = reinterpret_cast<vl_key_t*>(base_ptr + kOffLists);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, kSelWarps); }
        mbar_init(bar_drain, 1);
        mbar_init(bar_rows_full, 1);
        mbar_init(bar_rows_empty, 1);
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
        uint32_t it = 0, nres = 0;                                  // nres: work items with a non-empty candidate range so far
        bool ok = true;
#pragma unroll 1
        for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
            const int64_t rt = item / a.segments, seg = item % a.segments;
            const int64_t row0 = a.row_lo + rt * kTileRows;
            const int64_t c_begin = a.cand_lo + seg * a.seg_len;
            const int64_t c_end = (c_begin + a.seg_len < a.cand_hi) ? c_begin + a.seg_len : a.cand_hi;
            if (RESIDENT && c_begin < c_end) {
                // the previous item's MMAs must be done with the row tile before it is overwritten
                ok = mbar_wait(bar_rows_empty, (nres & 1u) ^ 1u, abort_flag, a.status);
                if (!ok) break;
                ++nres;
                mbar_expect_tx(bar_rows_full, a.kblocks * kTileBytes);
                for (int kb = 0; kb < a.kblocks; ++kb)
                    tma_load_2d(base + kOffRowTile + kb * kTileBytes, &tmap, kb * kBlockK, (int)row0, bar_rows_full);
            }
#pragma unroll 1
            for (int64_t c0 = c_begin; c0 < c_end && ok; c0 += kTileCands) {
#pragma unroll 1
                for (int kb = 0; kb < a.kblocks; ++kb, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    { VL_T0(); ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, a.status); VL_T1(0); }
                    if (!ok) break;
                    mbar_expect_tx(bar_full + 8 * s, kStageBytes);
                    if (!RESIDENT) tma_load_2d(base + s * kStageBytes + kCandBytes, &tmap, kb * kBlockK, (int)row0, bar_full + 8 * s);
                    tma_load_2d(base + s * kStageBytes, &tmap_cand, kb * kBlockK, (int)c0, bar_full + 8 * s);
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
        uint32_t it = 0, nres = 0, used0 = 0, used1 = 0;            // tiles accumulator 0 / 1 has held so far
        bool ok = true;
#pragma unroll 1
        for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
            const int64_t seg = item % a.segments;
            const int64_t c_begin = a.cand_lo + seg * a.seg_len;
            const int64_t c_end = (c_begin + a.seg_len < a.cand_hi) ? c_begin + a.seg_len : a.cand_hi;
            if (RESIDENT && c_begin < c_end) {
                ok = mbar_wait(bar_rows_full, nres & 1u, abort_flag, a.status);
                if (!ok) break;
                ++nres;
                tc_fence_after();
            }
            uint32_t lt = 0;                                        // tile index within the segment: its parity picks the accumulator
#pragma unroll 1
            for (int64_t c0 = c_begin; c0 < c_end && ok; c0 += kTileCands, ++lt) {
                const uint32_t buf = lt & 1u;
                const uint32_t tph = (buf ? used1 : used0) & 1u;
                if (buf) ++used1; else ++used0;
                { VL_T0(); ok = mbar_wait(bar_tempty + 8 * buf, tph ^ 1u, abort_flag, a.status); VL_T1(1); }   // accumulator drained?
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * kTileCands;
#pragma unroll 1
                for (int kb = 0; kb < a.kblocks; ++kb, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    { VL_T0(); ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, a.status); VL_T1(2); }
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t a_desc = smem_desc_sw128(RESIDENT ? base + kOffRowTile + kb * kTileBytes
                                                                     : base + s * kStageBytes + kCandBytes);
                    const uint64_t b_desc = smem_desc_sw128(base + s * kStageBytes);
#pragma unroll
                    for (int kk = 0; kk < kBlockK / 16; ++kk)      // 16 bf16 = 32 bytes = 2 descriptor units per step
                        tc_mma_bf16(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, kIdesc, (kb | kk) != 0);
                    tc_commit(bar_empty + 8 * s);                  // stage reusable once these MMAs have read it
                }
                if (ok) tc_commit(bar_tfull + 8 * buf);            // accumulator complete
            }
            if (RESIDENT && ok && c_begin < c_end) tc_commit(bar_rows_empty);   // row tile free once this item's MMAs are done
        }
        // every MMA issued above must have finished before the TMEM columns are given back
        tc_commit(bar_drain);
        {
            const unsigned long long t0 = now_ns();
            while (!mbar_test(bar_drain, 0) && now_ns() - t0 < kWaitLimitNs) __nanosleep(100);
        }
    } else if (warp >= 2) {
        // ---------------- selection: one row of the tile per thread ----------------
        const int cls = (warp - 2) >> 2;                           // this warp's column class
        const int quarter = warp & 3;                              // the TMEM lanes this warp may read
        const int row_in_tile = quarter * 32 + lane;
        float* bias_tile = bias_smem + (warp - 2) * kSelCols;
        const float kInf = __int_as_float(0x7f800000);
        uint32_t used0 = 0, used1 = 0;                             // tiles accumulator 0 / 1 has held so far
        bool ok = true;
#pragma unroll 1
        for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
            const int64_t rt = item / a.segments, seg = item % a.segments;
            const int64_t row = a.row_lo + rt * kTileRows + row_in_tile;
            const int64_t c_begin = a.cand_lo + seg * a.seg_len;
            const int64_t c_end = (c_begin + a.seg_len < a.cand_hi) ? c_begin + a.seg_len : a.cand_hi;
            // The kTopK best keys of each of this warp's 32 rows, ascending, in shared memory: row r's list is
            // warp_lists[r * kTopK + lane], one key per lane, so that an insertion is a warp-wide shift (a few
            // instructions) instead of a register sort by the one lane that owns the row.  Each lane keeps
            // `worst`, the score of its own row's last key (+inf until the list is full).
            vl_key_t* warp_lists = lists_smem + ((size_t)cls * kTileRows + quarter * 32) * kTopK;
            __syncwarp();
#pragma unroll
            for (int i = 0; i < kTopK; ++i) warp_lists[i * 32 + lane] = ~0ull;
            __syncwarp();
            float worst = kInf;

            // Examines 32 accumulator columns.  Common path, one instruction per column: per group of 8 columns
            // four packed FMAs make the scores, 3-input minima reduce them to the smallest, one compare tells
            // whether this row has anything below its worst key there.  Only the groups in which some row of
            // the warp has (usually none or one) are looked at column by column, and every (row, column)
            // that qualifies is inserted into its row's list by the whole warp.
            auto examine = [&](const uint32_t (&v)[32], const float* bias32, int64_t col0) {
                uint32_t sub = 0;
#pragma unroll
                for (int s8 = 0; s8 < 4; ++s8) {
                    const float4 c0 = *reinterpret_cast<const float4*>(bias32 + 8 * s8);
                    const float4 c1 = *reinterpret_cast<const float4*>(bias32 + 8 * s8 + 4);
                    float s0, s1, s2, s3, s4, s5, s6, s7;
                    score2(v[8 * s8 + 0], v[8 * s8 + 1], c0.x, c0.y, s0, s1);
                    score2(v[8 * s8 + 2], v[8 * s8 + 3], c0.z, c0.w, s2, s3);
                    score2(v[8 * s8 + 4], v[8 * s8 + 5], c1.x, c1.y, s4, s5);
                    score2(v[8 * s8 + 6], v[8 * s8 + 7], c1.z, c1.w, s6, s7);
                    const float m = fminf(min3f(min3f(s0, s1, s2), min3f(s3, s4, s5), s6), s7);
                    sub |= (m < worst) ? (1u << s8) : 0u;
                }
                uint32_t any = __reduce_or_sync(0xffffffffu, sub);
#pragma unroll 1
                while (any) {
                    const int s8 = __ffs(any) - 1;                  // the same for every lane
                    any &= any - 1;
                    uint32_t mk = 0;
#define VL_MARKS8(B) { \
                        const float4 c0 = *reinterpret_cast<const float4*>(bias32 + (B)); \
                        const float4 c1 = *reinterpret_cast<const float4*>(bias32 + (B) + 4); \
                        mk |= (fmaf(-2.0f, __uint_as_float(v[(B) + 0]), c0.x) < worst) ? 1u : 0u; \
                        mk |= (fmaf(-2.0f, __uint_as_float(v[(B) + 1]), c0.y) < worst) ? 2u : 0u; \
                        mk |= (fmaf(-2.0f, __uint_as_float(v[(B) + 2]), c0.z) < worst) ? 4u : 0u; \
                        mk |= (fmaf(-2.0f, __uint_as_float(v[(B) + 3]), c0.w) < worst) ? 8u : 0u; \
                        mk |= (fmaf(-2.0f, __uint_as_float(v[(B) + 4]), c1.x) < worst) ? 16u : 0u; \
                        mk |= (fmaf(-2.0f, __uint_as_float(v[(B) + 5]), c1.y) < worst) ? 32u : 0u; \
                        mk |= (fmaf(-2.0f, __uint_as_float(v[(B) + 6]), c1.z) < worst) ? 64u : 0u; \
                        mk |= (fmaf(-2.0f, __uint_as_float(v[(B) + 7]), c1.w) < worst) ? 128u : 0u; }
                    switch (s8) {
                        case 0: VL_MARKS8(0) break;
                        case 1: VL_MARKS8(8) break;
                        case 2: VL_MARKS8(16) break;
                        default: VL_MARKS8(24) break;
                    }
#undef VL_MARKS8
                    uint32_t cols = __reduce_or_sync(0xffffffffu, mk);
#pragma unroll 1
                    while (cols) {
                        const int jj = __ffs(cols) - 1;
                        cols &= cols - 1;
                        const int j = 8 * s8 + jj;
                        const float score = fmaf(-2.0f, __uint_as_float(pick32(v, j)), bias32[j]);
                        const vl_key_t my_key = ((vl_key_t)vl_ord(score) << 32) | (uint32_t)(col0 + j);
                        unsigned live = __ballot_sync(0xffffffffu, ((mk >> jj) & 1u) && score < worst && col0 + j != row);
#pragma unroll 1
                        while (live) {
                            const int owner = __ffs(live) - 1;
                            live &= live - 1;
                            const vl_key_t key = __shfl_sync(0xffffffffu, my_key, owner);
                            vl_key_t* lst = warp_lists + owner * kTopK;
                            const vl_key_t e = lane < kTopK ? lst[lane] : ~0ull;
                            const int pos = __popc(__ballot_sync(0xffffffffu, e < key));
                            const vl_key_t prev = __shfl_up_sync(0xffffffffu, e, 1);
                            const vl_key_t ne = lane < pos ? e : (lane == pos ? key : prev);
                            if (lane < kTopK) lst[lane] = ne;
                            const vl_key_t tail = __shfl_sync(0xffffffffu, ne, kTopK - 1);
                            if (lane == owner && tail != ~0ull) worst = vl_unord((uint32_t)(tail >> 32));
                            __syncwarp();
                        }
                    }
                }
            };
            // score offsets of this warp's columns of a tile: |c|^2 (squared L2) or 0 (cosine), +inf past the
            // segment's end so that such a column never qualifies
            auto load_bias = [&](int64_t c0, float (&b)[kSelCols / 32]) {
#pragma unroll
                for (int q = 0; q < kSelCols / 32; ++q) {
                    const int64_t c = c0 + lane + 32 * q;
                    b[q] = (c < c_end) ? (a.bias ? __ldg(a.bias + c) : 0.0f) : kInf;
                }
            };
            float next_bias[kSelCols / 32];
            const int64_t c_off = (int64_t)cls * kSelCols;
            if (c_begin < c_end) load_bias(c_begin + c_off, next_bias);
            uint32_t lt = 0;
#pragma unroll 1
            for (int64_t c0 = c_begin; c0 < c_end; c0 += kTileCands, ++lt) {
                // this warp's own copy of the offsets (warp-local: this role uses no CTA-wide barrier); the
                // next tile's offsets are requested now and stored when this tile is done
                __syncwarp();
#pragma unroll
                for (int q = 0; q < kSelCols / 32; ++q) bias_tile[lane + 32 * q] = next_bias[q];
                __syncwarp();
                if (c0 + kTileCands < c_end) load_bias(c0 + kTileCands + c_off, next_bias);
                const uint32_t buf = lt & 1u;
                const uint32_t tph = (buf ? used1 : used0) & 1u;
                if (buf) ++used1; else ++used0;
                { VL_T0(); ok = mbar_wait(bar_tfull + 8 * buf, tph, abort_flag, a.status); if (lane == 0 && warp == 2) VL_T1(3); }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * kTileCands + cls * kSelCols;
                VL_T0();
                {
                    // four warps per scheduler hide each other's latencies: one chunk of 32 columns at a time
                    uint32_t v0[32];
#pragma unroll 1
                    for (int ch = 0; ch < kSelCols / 32; ++ch) {
                        __syncwarp();
                        tc_load32(taddr + ch * 32, v0);
                        tc_wait_ld();
                        if (ch + 1 == kSelCols / 32) {
                            // the tile's last columns are in registers: hand the accumulator back now, the
                            // next tile's MMAs run while this chunk is examined
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
                        }
                        examine(v0, bias_tile + ch * 32, c0 + c_off + ch * 32);
                    }
                    __syncwarp();
                }
                if (lane == 0 && warp == 2) { VL_T1(5); if (a.stats) atomicAdd(a.stats + 6, 1ull); }
            }
            if (ok) {      // the warp writes its rows' lists, 32 ids = 128 bytes per step
                __syncwarp();
                const int64_t first_row = a.row_lo + rt * kTileRows + quarter * 32;
                constexpr int kRowsPerStep = 32 / kTopK;
#pragma unroll 1
                for (int r0 = 0; r0 < 32; r0 += kRowsPerStep) {
                    const int r = r0 + lane / kTopK, kk = lane % kTopK;
                    if (first_row + r < a.row_hi) {
                        const vl_key_t k = warp_lists[r * kTopK + kk];
                        a.out_ids[(((first_row + r - a.row_lo) * a.segments + seg) * kLists + cls) * kTopK + kk] =
                            k == ~0ull ? VL_MAXINT : (int32_t)(uint32_t)k;
                    }
                }
                __syncwarp();
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

#ifdef VL_KNN_STATS
static unsigned long long* g_knn_stats = nullptr;
extern "C" void vl_knn_debug_stats(unsigned long long* device_counters) { g_knn_stats = device_counters; }
#endif

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
    CUtensorMap tmap_cand;
    const cuuint32_t box_cand[2] = {(cuuint32_t)kBlockK, (cuuint32_t)kTileCands};
    cr = encode(&tmap_cand, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(rows_bf16), gdim, gstride, box_cand, estr,
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
    a.stats = nullptr;
#ifdef VL_KNN_STATS
    a.stats = g_knn_stats;
#endif

    const bool resident = a.kblocks <= kResidentKBlocks;
    auto kernel = resident ? knn_tile_kernel<true> : knn_tile_kernel<false>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    VL_CHECK_ARG(e == cudaSuccess, "vl_knn_tile: %s", cudaGetErrorString(e));
    const int64_t items = ((row_hi - row_lo + kTileRows - 1) / kTileRows) * segments;
    const int sms = vl_sm_count();
    const unsigned grid = (unsigned)(items < sms ? items : sms);
    kernel<<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(tmap, tmap_cand, a);
    VL_CHECK_LAUNCH("knn_tile_kernel");
    return 0;
}
