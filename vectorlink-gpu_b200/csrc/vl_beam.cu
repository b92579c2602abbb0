// Fused beam search: the reference's closest_vectors loop (vectorlink_gpu/ann.py:37-93) as
// ONE kernel.  Per iteration the reference launches pop_n_ids (queue.py:87-95),
// search_from_seeds (kernels.py:204-311), two Queue.insert chains (queue.py:37-61: three
// torch.sort + gathers + dedup kernels each), add_new_to_seen_ (utils.py:61-82) and syncs
// the host; queue state makes a round trip through HBM every time.
//
// Here one warp owns one query row for the whole search:
//   * the query row lives in registers (the lane layout of vl_common.cuh);
//   * the search queue head, the visit queue and the visited set live in shared memory
//     (two sorted arrays of 64-bit (distance,id) keys and an open-addressing hash set);
//   * per iteration the warp pops `pvc` ids, reads their graph rows, gathers the candidate
//     vectors with 128-bit loads (32/LPR rows per step, two steps in flight), and merges the
//     candidates into both queues.
// The only HBM traffic that scales with the work is the gather: 4*dim bytes per candidate
// row + 4 bytes per neighbour id; that is the roofline this kernel is measured against.
//
// Queue semantics reproduced exactly (for capacity == length + candidates per iteration,
// which every queue the reference's drivers create satisfies): after an insert the queue is
// the `length` smallest distinct (distance,id) keys of old head + new candidates minus the
// excluded ids.  "Smallest `length` of a union" can be taken in any grouping, so candidates
// are merged 32 at a time and only those below the current cut-off key are looked at.
// The visited list `seen` (utils.py:61-89) is a set here: a candidate is kept out of the
// visit queue iff its id was popped while the list still had room, and the list's fill level
// (pvc ids per iteration, as for a batch in which at least one row always pops real ids)
// ends the feeding of the visit queue after ceil(E/pvc) iterations, like the reference.
// The two batch-wide decisions of the reference's host loop - "did any row's head change at a
// check iteration" and "was some row's pop always full" - are written to flag arrays for the
// caller, which re-runs a batch with a smaller n_iters or through the operator-level
// path when the reference would have taken a different course.
#include "vl_common.cuh"

namespace {

constexpr int kBeamWarps = 4;             // most warps (= rows in flight) per CTA
constexpr int32_t kHashEmpty = -1;

struct BeamSmem {      // per-warp carve-up, in bytes from the warp's base
    int cand, sq_a, sq_b, vq_a, vq_b, hash, pop, mpos, total;
    int hash_slots, hash_shift;
};

__host__ __device__ inline BeamSmem beam_smem_layout(int m, int sq_len, int vq_len, int seen_cap)
{
    BeamSmem s;
    int off = 0;
    s.cand = off; off += 8 * m;
    s.sq_a = off; off += 8 * sq_len;
    s.sq_b = off; off += 8 * sq_len;
    s.vq_a = off; off += 8 * vq_len;
    s.vq_b = off; off += 8 * vq_len;
    int slots = 32, shift = 27;
    while (slots < seen_cap + seen_cap / 2 + 1) { slots <<= 1; --shift; }
    s.hash_slots = slots;
    s.hash_shift = shift;
    s.hash = off; off += 4 * slots;
    s.pop = off; off += 4 * 32;
    s.mpos = off; off += 4 * 32;
    s.total = (off + 15) & ~15;
    return s;
}

__device__ __forceinline__ unsigned hash_slot(int32_t id, int shift) { return ((uint32_t)id * 2654435761u) >> shift; }

__device__ __forceinline__ void hash_insert(int32_t* table, int slots, int shift, int32_t id, int* status)
{
    unsigned s = hash_slot(id, shift);
    for (int probe = 0; probe < slots; ++probe) {
        int32_t prev = atomicCAS(&table[s], kHashEmpty, id);
        if (prev == kHashEmpty || prev == id) return;
        s = (s + 1) & (slots - 1);
    }
    atomicOr(status, VL_STATUS_OVERFLOW);
}

__device__ __forceinline__ bool hash_contains(const int32_t* table, int slots, int shift, int32_t id)
{
    unsigned s = hash_slot(id, shift);
    for (int probe = 0; probe < slots; ++probe) {
        int32_t v = table[s];
        if (v == id) return true;
        if (v == kHashEmpty) return false;
        s = (s + 1) & (slots - 1);
    }
    return false;
}

// ascending sort of one 64-bit key per lane across the warp (bitonic network on shuffles)
__device__ __forceinline__ vl_key_t warp_sort32(vl_key_t k, int lane)
{
#pragma unroll
    for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
        for (int j = size >> 1; j > 0; j >>= 1) {
            vl_key_t o = __shfl_xor_sync(0xffffffffu, k, j);
            bool up = ((lane & size) == 0);
            bool lower = ((lane & j) == 0);
            bool take_min = (up == lower);
            k = take_min ? (k < o ? k : o) : (k < o ? o : k);
        }
    }
    return k;
}

// Merge the keys of the lanes flagged `want` into the sorted list `cur` (length len, sentinels
// last), dropping keys already present and repeats; result in `nxt`, cut at len, and the two
// pointers swapped.  `mpos` is a 32-int scratch of the warp.  Every `want` key is below
// cur[len-1], so the smallest new distinct key always enters: returns true iff one did.
// All 32 lanes call this.
__device__ __forceinline__ bool merge_chunk(vl_key_t*& cur, vl_key_t*& nxt, int len, vl_key_t key, bool want,
                                            int lane, int* mpos)
{
    const vl_key_t kNone = ~0ull;
    const unsigned wmask = __ballot_sync(0xffffffffu, want);
    vl_key_t k;
    if (__popc(wmask) == 1) {
        vl_key_t k0 = __shfl_sync(0xffffffffu, key, __ffs(wmask) - 1);
        k = lane == 0 ? k0 : kNone;
    } else {
        k = warp_sort32(want ? key : kNone, lane);
    }
    bool valid = (k != kNone);
    const vl_key_t prev = __shfl_up_sync(0xffffffffu, k, 1);
    if (lane > 0 && prev == k) valid = false;
    int lo = 0;
    if (valid) {   // lo = number of list keys below k
        int hi = len;
        while (lo < hi) {
            int mid = (lo + hi) >> 1;
            if (cur[mid] < k) lo = mid + 1; else hi = mid;
        }
        if (lo < len && cur[lo] == k) valid = false;
    }
    const unsigned vmask = __ballot_sync(0xffffffffu, valid);
    if (!vmask) return false;
    const int rank = __popc(vmask & ((1u << lane) - 1u));
    const int nv = __popc(vmask);
    if (valid) mpos[rank] = lo;
    __syncwarp();
    // a list element moves down by the number of entering keys below it (those with pos <= j)
    for (int jb = 0; jb < len; jb += 32) {
        const int j = jb + lane;
        if (j < len) {
            const vl_key_t e = cur[j];
            int shift = 0;
            for (int s = 0; s < nv; ++s) shift += (mpos[s] <= j);
            if (j + shift < len) nxt[j + shift] = e;
        }
    }
    if (valid && lo + rank < len) nxt[lo + rank] = k;
    __syncwarp();
    vl_key_t* t = cur; cur = nxt; nxt = t;
    return true;
}

// JU > 0: exact-fit rows (dim == 4*LPR*JU, see vl_load_exact); JU == 0: any dim % 4 == 0.
template <int LPR, int JP, int JU, int METRIC>
__global__ void __launch_bounds__(kBeamWarps * 32)
beam_search_kernel(const vl_beam_params p, const BeamSmem lay)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int G = 32 / LPR;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane / LPR, lg = lane % LPR;
    unsigned char* base = smem_raw + (size_t)warp * lay.total;
    uint2* cand = reinterpret_cast<uint2*>(base + lay.cand);
    vl_key_t* candk = reinterpret_cast<vl_key_t*>(base + lay.cand);
    int32_t* hash = reinterpret_cast<int32_t*>(base + lay.hash);
    int32_t* pop = reinterpret_cast<int32_t*>(base + lay.pop);
    int* mpos = reinterpret_cast<int*>(base + lay.mpos);

    const int wb = p.graph_w, pvc = p.pvc, m_total = p.pvc * p.graph_w;
    const int sq_len = p.sq_len, vq_len = p.vq_len, e_cap = p.seen_cap;
    const int k_none = (e_cap + pvc - 1) / pvc + 1;   // first iteration at which `seen` is full
    const int n_run = p.n_iters < k_none ? p.n_iters : k_none;
    const vl_key_t kSent = vl_sentinel_key();
    const uint32_t sent_ord = (uint32_t)(kSent >> 32);

    const int wpb = blockDim.x >> 5;
    const int64_t warp0 = (int64_t)blockIdx.x * wpb + warp;
    const int64_t nwarps = (int64_t)gridDim.x * wpb;
    for (int64_t row = warp0; row < p.rows; row += nwarps) {
        vl_key_t* sq = reinterpret_cast<vl_key_t*>(base + lay.sq_a);
        vl_key_t* sq_n = reinterpret_cast<vl_key_t*>(base + lay.sq_b);
        vl_key_t* vq = reinterpret_cast<vl_key_t*>(base + lay.vq_a);
        vl_key_t* vq_n = reinterpret_cast<vl_key_t*>(base + lay.vq_b);
        const float* q = p.queries + row * (int64_t)p.dim;
        constexpr int JQ = JU > 0 ? JU : JP;
        float4 qr[JQ];
        if constexpr (JU > 0) vl_load_exact<LPR, JU>(q, lg, qr);
        else vl_load_query<LPR, JP, true>(q, p.dim, lg, qr);

        // ---- prologue: Queue.insert of the seeds into an empty queue (queue.py:37-61) ----
        for (int i = lane; i < sq_len; i += 32) sq[i] = kSent;
        for (int i = lane; i < lay.hash_slots; i += 32) hash[i] = kHashEmpty;
        __syncwarp();
        for (int c0 = 0; c0 < p.seed_cols; c0 += 32) {
            int c = c0 + lane;
            vl_key_t key = kSent;
            if (c < p.seed_cols)
                key = vl_entry_key(__ldg(p.seed_dist + row * p.seed_ld + c), __ldg(p.seed_ids + row * p.seed_ld + c));
            bool want = key < sq[sq_len - 1];
            if (__any_sync(0xffffffffu, want)) merge_chunk(sq, sq_n, sq_len, key, want, lane, mpos);
        }
        // visit_queue.initialize_from_queue (queue.py:30-35)
        {
            const int head = sq_len < vq_len ? sq_len : vq_len;
            for (int i = lane; i < vq_len; i += 32) vq[i] = i < head ? sq[i] : kSent;
        }
        __syncwarp();

        bool always_full = true;
        const int32_t self_id = p.self_base >= 0 ? (int32_t)(p.self_base + row) : VL_MAXINT;
        const int32_t* excl = p.exclude_w > 0 ? p.exclude + row * (int64_t)p.exclude_w : nullptr;
        const int64_t group = p.group_rows > 0 ? row / p.group_rows : 0;
        bool dumped = false;

        for (int k = 1; k <= n_run; ++k) {
            const int first = (k - 1) * pvc;
            const bool seen_live = first < e_cap;    // utils.py:62-69
            // ---- pop_n_ids (queue.py:87-95) ----
            {
                vl_key_t head = lane < pvc ? vq[lane] : kSent;
                if (lane < pvc) pop[lane] = vl_key_id(head);
                for (int i = lane; i < vq_len; i += 32) vq_n[i] = (i + pvc < vq_len) ? vq[i + pvc] : kSent;
                __syncwarp();
                vl_key_t* t = vq; vq = vq_n; vq_n = t;
            }
            // ---- neighbour ids of the popped nodes (kernels.py:244) ----
            for (int v = 0; v < pvc; ++v) {
                int32_t node = pop[v];
                if (node != VL_MAXINT && (node < 0 || (int64_t)node >= p.n)) {
                    if (lane == 0) atomicOr(p.status, VL_STATUS_BAD_ID);
                    node = VL_MAXINT;
                }
                const int32_t* grow = p.graph + (int64_t)(node == VL_MAXINT ? 0 : node) * wb;
                for (int j = lane; j < wb; j += 32) {
                    int32_t id = VL_MAXINT;
                    if (node != VL_MAXINT) {
                        id = __ldg(grow + j);
                        if (id != VL_MAXINT && (id < 0 || (int64_t)id >= p.n)) { atomicOr(p.status, VL_STATUS_BAD_ID); id = VL_MAXINT; }
                    }
                    cand[v * wb + j] = make_uint2((uint32_t)id, sent_ord);
                }
            }
            __syncwarp();
            // ---- gathered distances (kernels.py:248-257), two steps in flight ----
            for (int m0 = 0; m0 < m_total; m0 += 2 * G) {
                const int ma = m0 + g, mb = m0 + G + g;
                int32_t ida = ma < m_total ? (int32_t)cand[ma].x : VL_MAXINT;
                int32_t idb = mb < m_total ? (int32_t)cand[mb].x : VL_MAXINT;
                const bool la = ida != VL_MAXINT, lb = idb != VL_MAXINT;
                const float* ra = p.vectors + (int64_t)(la ? ida : 0) * p.dim;
                const float* rb = p.vectors + (int64_t)(lb ? idb : 0) * p.dim;
                float da, db;
                if constexpr (JU > 0) {
                    float4 xa[JU], xb[JU];
                    vl_load_exact<LPR, JU>(ra, lg, xa);
                    vl_load_exact<LPR, JU>(rb, lg, xb);
                    da = vl_exact_distance<LPR, JP, JU, METRIC>(xa, qr);
                    db = vl_exact_distance<LPR, JP, JU, METRIC>(xb, qr);
                } else {
                    float4 xa[JP], xb[JP];
                    vl_load_row<LPR, JP, true>(ra, p.dim, lg, la, xa);
                    vl_load_row<LPR, JP, true>(rb, p.dim, lg, lb, xb);
                    da = vl_row_distance<LPR, JP, METRIC, true>(xa, qr, ra, q, p.dim, lg, la);
                    db = vl_row_distance<LPR, JP, METRIC, true>(xb, qr, rb, q, p.dim, lg, lb);
                }
                if (lg == 0) {
                    if (la) cand[ma].y = vl_ord(da);
                    if (lb) cand[mb].y = vl_ord(db);
                }
            }
            __syncwarp();
            // ---- search_queue.insert(..., exclude) (ann.py:75-80) ----
            if (p.dump_last && k == p.n_iters) {
                // leave this insert to the caller's full-row sort: head, then the raw candidates
                for (int i = lane; i < sq_len; i += 32) {
                    p.out_ids[row * p.out_ld + i] = vl_key_id(sq[i]);
                    p.out_dist[row * p.out_ld + i] = vl_key_dist(sq[i]);
                }
                for (int i = lane; i < m_total; i += 32) {
                    vl_key_t key = candk[i];
                    int32_t id = vl_key_id(key);
                    bool drop = (id == self_id);
                    if (!drop && excl)
                        for (int t = 0; t < p.exclude_w; ++t) {
                            int32_t x = excl[t];
                            if (x == VL_MAXINT) break;
                            if (x == id) { drop = true; break; }
                        }
                    if (drop) key = kSent;
                    p.out_ids[row * p.out_ld + sq_len + i] = vl_key_id(key);
                    p.out_dist[row * p.out_ld + sq_len + i] = vl_key_dist(key);
                }
                for (int i = sq_len + m_total + lane; i < p.out_cols; i += 32) {
                    p.out_ids[row * p.out_ld + i] = VL_MAXINT;
                    p.out_dist[row * p.out_ld + i] = VL_MAXFLOAT;
                }
                dumped = true;
                break;
            }
            bool changed = false;
            vl_key_t cut = sq[sq_len - 1];
            for (int c0 = 0; c0 < m_total; c0 += 32) {
                const int c = c0 + lane;
                vl_key_t key = c < m_total ? candk[c] : kSent;
                bool want = key < cut;
                if (!__any_sync(0xffffffffu, want)) continue;
                if (want) {
                    int32_t id = vl_key_id(key);
                    if (id == self_id) want = false;
                    else if (excl)
                        for (int t = 0; t < p.exclude_w; ++t) {   // kernels.py:478-488
                            int32_t x = excl[t];
                            if (x == VL_MAXINT) break;
                            if (x == id) { want = false; break; }
                        }
                }
                if (!__any_sync(0xffffffffu, want)) continue;
                changed |= merge_chunk(sq, sq_n, sq_len, key, want, lane, mpos);
                cut = sq[sq_len - 1];
            }
            if (changed && (k % p.readahead) == 0 && lane == 0) {
                int chk = k / p.readahead - 1;
                if (chk < p.n_checks) atomicOr(p.changed_flags + group * p.n_checks + chk, 1u);
            }
            // ---- add_new_to_seen_ (utils.py:61-82) + visit_queue.insert(..., exclude=seen) ----
            if (seen_live) {
                const int ncopy = (e_cap - first) < pvc ? (e_cap - first) : pvc;
                int32_t mine = lane < ncopy ? pop[lane] : 0;
                if (lane < ncopy && mine != VL_MAXINT) hash_insert(hash, lay.hash_slots, lay.hash_shift, mine, p.status);
                if (__any_sync(0xffffffffu, lane < ncopy && mine == VL_MAXINT)) always_full = false;
                __syncwarp();
                vl_key_t vcut = vq[vq_len - 1];
                for (int c0 = 0; c0 < m_total; c0 += 32) {
                    const int c = c0 + lane;
                    vl_key_t key = c < m_total ? candk[c] : kSent;
                    bool want = key < vcut;
                    if (!__any_sync(0xffffffffu, want)) continue;
                    if (want && hash_contains(hash, lay.hash_slots, lay.hash_shift, vl_key_id(key))) want = false;
                    if (!__any_sync(0xffffffffu, want)) continue;
                    merge_chunk(vq, vq_n, vq_len, key, want, lane, mpos);
                    vcut = vq[vq_len - 1];
                }
            }
        }

        if (!dumped) {
            for (int i = lane; i < p.out_cols; i += 32) {
                vl_key_t key = i < sq_len ? sq[i] : kSent;
                p.out_ids[row * p.out_ld + i] = vl_key_id(key);
                p.out_dist[row * p.out_ld + i] = vl_key_dist(key);
            }
        }
        if (always_full && lane == 0) atomicOr(p.group_full + group, 1u);
        __syncwarp();
    }
}

struct BeamPlan { BeamSmem lay; int warps; int blocks; size_t smem; };

template <int LPR, int JP, int JU, int METRIC>
int plan_and_launch(const vl_beam_params& p, BeamPlan& plan, bool launch, cudaStream_t stream)
{
    auto kernel = beam_search_kernel<LPR, JP, JU, METRIC>;
    plan.lay = beam_smem_layout(p.pvc * p.graph_w, p.sq_len, p.vq_len, p.seen_cap);
    int dev = 0, sms = 0, max_smem = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    VL_CHECK_ARG(e == cudaSuccess, "vl_beam_search: %s", cudaGetErrorString(e));
    plan.warps = kBeamWarps;
    while (plan.warps > 1 && (size_t)plan.warps * plan.lay.total > (size_t)max_smem) plan.warps >>= 1;
    plan.smem = (size_t)plan.warps * plan.lay.total;
    VL_CHECK_ARG(plan.smem <= (size_t)max_smem, "vl_beam_search: one row needs %d bytes of shared memory, the device offers %d",
                 plan.lay.total, max_smem);
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);
    VL_CHECK_ARG(e == cudaSuccess, "vl_beam_search: %s", cudaGetErrorString(e));
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, plan.warps * 32, plan.smem);
    VL_CHECK_ARG(e == cudaSuccess && per_sm > 0, "vl_beam_search: occupancy query failed");
    int64_t want = (p.rows + plan.warps - 1) / plan.warps;
    int64_t resident = (int64_t)sms * per_sm;   // one resident wave; rows beyond it are strided
    plan.blocks = (int)(want < resident ? want : resident);
    if (launch && plan.blocks > 0) {
        kernel<<<plan.blocks, plan.warps * 32, plan.smem, stream>>>(p, plan.lay);
        VL_CHECK_LAUNCH("beam_search_kernel");
    }
    return 0;
}

int beam_dispatch(const vl_beam_params* pp, BeamPlan& plan, bool launch, cudaStream_t stream)
{
    VL_CHECK_ARG(pp, "vl_beam_search: null params");
    const vl_beam_params& p = *pp;
    VL_CHECK_ARG(p.vectors && p.graph && p.queries && p.seed_ids && p.seed_dist && p.out_ids && p.out_dist &&
                 p.changed_flags && p.group_full && p.status, "vl_beam_search: null pointer");
    VL_CHECK_ARG(p.n > 0 && p.rows >= 0 && p.dim > 0, "vl_beam_search: bad size");
    VL_CHECK_ARG(p.dim % 4 == 0 && ((uintptr_t)p.vectors | (uintptr_t)p.queries) % 16 == 0,
                 "vl_beam_search: needs dim %% 4 == 0 and 16-byte aligned rows (dim=%d)", p.dim);
    VL_CHECK_ARG(p.metric == VL_METRIC_COSINE || p.metric == VL_METRIC_SQL2, "vl_beam_search: unknown metric %d", p.metric);
    VL_CHECK_ARG(p.pvc >= 1 && p.pvc <= 32, "vl_beam_search: parallel_visit_count %d outside 1..32", p.pvc);
    VL_CHECK_ARG(p.graph_w >= 1 && p.sq_len >= 1 && p.sq_len <= 4096, "vl_beam_search: bad queue shape");
    VL_CHECK_ARG(p.vq_len >= p.pvc, "vl_beam_search: visit queue of %d shorter than parallel_visit_count %d", p.vq_len, p.pvc);
    VL_CHECK_ARG(p.seen_cap >= 0 && p.readahead >= 1 && p.n_iters >= 0, "vl_beam_search: bad loop parameters");
    VL_CHECK_ARG(p.seed_cols >= 0 && p.seed_cols <= p.seed_ld, "vl_beam_search: bad seed shape");
    VL_CHECK_ARG(p.out_cols >= p.sq_len && p.out_cols <= p.out_ld, "vl_beam_search: bad output shape");
    VL_CHECK_ARG(!p.dump_last || p.out_cols >= p.sq_len + p.pvc * p.graph_w, "vl_beam_search: dump_last needs out_cols >= length + candidates");
    VL_CHECK_ARG(!p.dump_last || p.n_iters <= (p.seen_cap + p.pvc - 1) / p.pvc + 1, "vl_beam_search: dump_last past the last productive iteration");
    VL_CHECK_ARG(p.exclude_w == 0 || p.exclude, "vl_beam_search: exclusion width without a list");
    VL_CHECK_ARG(p.n_checks >= 0 && p.group_rows >= 0, "vl_beam_search: bad flag shape");
    if (p.rows == 0) { plan.blocks = 0; plan.warps = kBeamWarps; plan.lay = beam_smem_layout(p.pvc * p.graph_w, p.sq_len, p.vq_len, p.seen_cap); return 0; }
    VlShape shape = vl_pick_shape(p.dim);
    int rc = 0;
    const int chunks = p.dim / 4;
    // exact-fit instantiations for the row sizes that matter (no per-chunk bounds tests)
#define VL_EXACT(L, J, U)                                                                              \
    if (shape.lpr == L && shape.jp == J && chunks == L * U) {                                          \
        if (p.metric == VL_METRIC_COSINE) return plan_and_launch<L, J, U, VL_METRIC_COSINE>(p, plan, launch, stream); \
        return plan_and_launch<L, J, U, VL_METRIC_SQL2>(p, plan, launch, stream);                      \
    }
    VL_EXACT(8, 2, 2)     // dim 64
    VL_EXACT(8, 4, 3)     // dim 96
    VL_EXACT(8, 4, 4)     // dim 128
    VL_EXACT(16, 4, 4)    // dim 256
    VL_EXACT(32, 4, 3)    // dim 384
    VL_EXACT(32, 4, 4)    // dim 512
    VL_EXACT(32, 8, 6)    // dim 768
    VL_EXACT(32, 8, 8)    // dim 1024
#undef VL_EXACT
    VL_DISPATCH_SHAPE(shape, {
        if (p.metric == VL_METRIC_COSINE) rc = plan_and_launch<LPR, JP, 0, VL_METRIC_COSINE>(p, plan, launch, stream);
        else rc = plan_and_launch<LPR, JP, 0, VL_METRIC_SQL2>(p, plan, launch, stream);
    });
    return rc;
}

}  // namespace

extern "C" int vl_beam_search(const vl_beam_params* params, void* stream)
{
    BeamPlan plan;
    return beam_dispatch(params, plan, true, (cudaStream_t)stream);
}

extern "C" int vl_beam_search_plan(const vl_beam_params* params, int* smem_per_warp, int* warps_per_block, int* blocks)
{
    BeamPlan plan;
    int rc = beam_dispatch(params, plan, false, nullptr);
    if (rc) return rc;
    if (smem_per_warp) *smem_per_warp = plan.lay.total;
    if (warps_per_block) *warps_per_block = plan.warps;
    if (blocks) *blocks = plan.blocks;
    return 0;
}
