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

#ifndef VL_MB
#define VL_MB 4     // CTAs per SM the register allocation aims for (4 x 4 warps measured fastest)
#endif
#ifndef VL_PB
#define VL_PB 6     // chunks of 32 candidates per round of id / memo loads
#endif
#ifndef VL_U8
#define VL_U8 2     // gather steps in flight for rows of 8 chunks per lane
#endif
constexpr int kBeamWarps = 4;             // most warps (= rows in flight) per CTA
constexpr int32_t kHashEmpty = -1;

struct BeamSmem {      // per-warp carve-up, in bytes from the warp's base
    int cand, sq_a, sq_b, vq_a, vq_b, hash, pop, mpos, todo, query, total;
    int hash_slots, hash_shift;
};

__host__ __device__ inline BeamSmem beam_smem_layout(int m, int sq_len, int vq_len, int seen_cap, int query_bytes)
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
    s.todo = off; off += 2 * m;
    off = (off + 15) & ~15;
    s.query = off; off += query_bytes;
    s.total = (off + 15) & ~15;
    return s;
}

__device__ __forceinline__ unsigned hash_slot(int32_t id, int shift) { return ((uint32_t)id * 2654435761u) >> shift; }

__device__ __noinline__ void hash_insert(int32_t* table, int slots, int shift, int32_t id, int* status)
{
    unsigned s = hash_slot(id, shift);
#pragma unroll 1
    for (int probe = 0; probe < slots; ++probe) {
        int32_t prev = atomicCAS(&table[s], kHashEmpty, id);
        if (prev == kHashEmpty || prev == id) return;
        s = (s + 1) & (slots - 1);
    }
    atomicOr(status, VL_STATUS_OVERFLOW);
}

__device__ __noinline__ bool hash_contains(const int32_t* table, int slots, int shift, int32_t id)
{
    unsigned s = hash_slot(id, shift);
#pragma unroll 1
    for (int probe = 0; probe < slots; ++probe) {
        int32_t v = table[s];
        if (v == id) return true;
        if (v == kHashEmpty) return false;
        s = (s + 1) & (slots - 1);
    }
    return false;
}

// Distance memo: 2-entry buckets of (ordered distance << 32 | id) keys, newest first.
__device__ __forceinline__ unsigned memo_bucket(uint32_t id, int shift, int buckets)
{
    return buckets > 1 ? (id * 2654435761u) >> shift : 0u;
}
// A new key goes to way `way` of its bucket (the caller alternates the way between
// iterations: first-in-first-out over two ways without reading the bucket).  An entry is one
// aligned 64-bit word, so lanes that collide on a slot can only lose an entry, never pair an
// id with another id's distance.
__device__ __forceinline__ void memo_put(vl_key_t* memo, int buckets, int shift, vl_key_t key, int way)
{
    memo[2 * (size_t)memo_bucket((uint32_t)key, shift, buckets) + way] = key;
}

// ascending sort of one 64-bit key per lane across the warp (bitonic network on shuffles)
__device__ __noinline__ vl_key_t warp_sort32(vl_key_t k, int lane)
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

// (Not inlined, like the other helpers above: the kernel's warps are in different phases at any
// time and an instruction footprint that outgrows the instruction cache stalls all of them -
// the profile of the fully inlined kernel was dominated by instruction-fetch stalls.)
// Merge the keys of the lanes flagged `want` into the sorted list `cur` (length len, sentinels
// last), dropping keys already present and repeats; result in `nxt`, cut at len, and the two
// pointers swapped.  `mpos` is a 32-int scratch of the warp.  Every `want` key is below
// cur[len-1], so the smallest new distinct key always enters: returns true iff one did.
// Most offered keys are already in the list (good candidates come back all the time), so the
// membership test comes first and costs one binary search per offering lane; the common
// single-survivor case is a plain shift, only several survivors need the warp sort.
// All 32 lanes call this.
__device__ __noinline__ bool merge_chunk(vl_key_t*& cur, vl_key_t*& nxt, int len, vl_key_t key, bool want,
                                         int lane, int* mpos)
{
    const vl_key_t kNone = ~0ull;
    int lo = 0;
    if (want) {   // lo = number of list keys below key
        int hi = len;
#pragma unroll 1
        while (lo < hi) {
            int mid = (lo + hi) >> 1;
            if (cur[mid] < key) lo = mid + 1; else hi = mid;
        }
        if (lo < len && cur[lo] == key) want = false;
    }
    const unsigned wmask = __ballot_sync(0xffffffffu, want);
    if (!wmask) return false;
    if (__popc(wmask) == 1) {
        const int src = __ffs(wmask) - 1;
        const vl_key_t k0 = __shfl_sync(0xffffffffu, key, src);
        const int pos = __shfl_sync(0xffffffffu, lo, src);
#pragma unroll 1
        for (int jb = 0; jb < len; jb += 32) {
            const int j = jb + lane;
            if (j < len) {
                const vl_key_t e = cur[j];
                const int dst = j + (j >= pos);
                if (dst < len) nxt[dst] = e;
            }
        }
        if (lane == 0) nxt[pos] = k0;
        __syncwarp();
        vl_key_t* t = cur; cur = nxt; nxt = t;
        return true;
    }
    // several new keys: each needs its rank among them (repeats dropped), then all are spliced in by rank.
    // Up to kRankByCount entrants (the usual case: a handful per iteration) the rank is counted directly -
    // one broadcast per entrant - and the positions found above stay valid; more entrants, or a repeated
    // key among them, go through the 32-key sort.
    constexpr int kRankByCount = 16;
    vl_key_t k = key;
    bool valid = want;
    int rank = 0, nv = __popc(wmask);
    bool counted = false;
    if (nv <= kRankByCount) {
        bool dup = false;
        unsigned m = wmask;
#pragma unroll 1
        while (m) {                                   // warp-uniform: one pass per entrant
            const int src = __ffs(m) - 1;
            m &= m - 1;
            const vl_key_t o = __shfl_sync(0xffffffffu, key, src);
            rank += (want && o < key);
            dup |= (want && o == key && src < lane);
        }
        counted = !__any_sync(0xffffffffu, dup);
    }
    if (!counted) {
        k = warp_sort32(want ? key : kNone, lane);
        valid = (k != kNone);
        const vl_key_t prev = __shfl_up_sync(0xffffffffu, k, 1);
        if (lane > 0 && prev == k) valid = false;
        lo = 0;
        if (valid) {
            int hi = len;
#pragma unroll 1
            while (lo < hi) {
                int mid = (lo + hi) >> 1;
                if (cur[mid] < k) lo = mid + 1; else hi = mid;
            }
        }
        const unsigned vmask = __ballot_sync(0xffffffffu, valid);
        rank = __popc(vmask & ((1u << lane) - 1u));
        nv = __popc(vmask);
    }
    if (valid) mpos[rank] = lo;
    __syncwarp();
    // a list element moves down by the number of entering keys below it (those with pos <= j)
#pragma unroll 1
    for (int jb = 0; jb < len; jb += 32) {
        const int j = jb + lane;
        if (j < len) {
            const vl_key_t e = cur[j];
            int shift = 0;
#pragma unroll 1
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
__global__ void __launch_bounds__(kBeamWarps * 32, VL_MB)
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
    unsigned short* todo = reinterpret_cast<unsigned short*>(base + lay.todo);
    // distance memo of this warp's row: memo_entries 64-bit (ordered distance, id) keys as
    // 2-entry buckets; ~0 = empty.  Only this warp touches its slice.
    const int memo_buckets = p.memo ? (p.memo_entries >> 1) : 0;
    int memo_shift = 32;
#pragma unroll 1
    for (int b = memo_buckets; b > 1; b >>= 1) --memo_shift;
    vl_key_t* const memo_base = p.memo ? p.memo + ((size_t)blockIdx.x * (blockDim.x >> 5) + warp) * (size_t)p.memo_entries : nullptr;

    const int wb = p.graph_w, pvc = p.pvc, m_total = p.pvc * p.graph_w;
    const int sq_len = p.sq_len, vq_len = p.vq_len, e_cap = p.seen_cap;
    const int k_none = (e_cap + pvc - 1) / pvc + 1;   // first iteration at which `seen` is full
    const int n_run = p.n_iters < k_none ? p.n_iters : k_none;
    const vl_key_t kSent = vl_sentinel_key();
    const uint32_t sent_ord = (uint32_t)(kSent >> 32);
    const uint32_t kPoppedOrd = 0xffffffffu;                      // above every real ordered distance
    const vl_key_t kPopped = (vl_key_t)kPoppedOrd << 32;
    const float inv_wb = 1.0f / (float)p.graph_w;
    // With the memo on, a candidate row is read about once per query row: stream it through L2
    // and keep the graph rows and the memo there instead (measured 4 % on 1M x 128).  Without the
    // memo (first build round) the rows themselves are what L2 has to hold.
    const uint64_t pol_stream = p.memo ? vl_policy_evict_first() : vl_policy_evict_normal();
    const uint64_t pol_keep = p.memo ? vl_policy_evict_last() : vl_policy_evict_normal();

    const int wpb = blockDim.x >> 5;
    const int64_t warp0 = (int64_t)blockIdx.x * wpb + warp;
    const int64_t nwarps = (int64_t)gridDim.x * wpb;
    // Row schedule: the first row of a warp is fixed; after that either a fixed stride or, when the
    // caller provides a zeroed counter, the next row nobody has taken yet (rows take unequal time).
    int64_t row = warp0;
#pragma unroll 1
    while (row < p.rows) {
        vl_key_t* sq = reinterpret_cast<vl_key_t*>(base + lay.sq_a);
        vl_key_t* sq_n = reinterpret_cast<vl_key_t*>(base + lay.sq_b);
        vl_key_t* vq = reinterpret_cast<vl_key_t*>(base + lay.vq_a);
        vl_key_t* vq_n = reinterpret_cast<vl_key_t*>(base + lay.vq_b);
        const float* q = p.queries + row * (int64_t)p.dim;
        // Rows of 8 chunks per lane keep the query in shared memory (read back per step: 8
        // conflict-free 16-byte loads) so that the registers hold two steps of candidate rows;
        // shorter rows keep it in registers.
        constexpr bool QSMEM = (JU >= 8);
        constexpr int JQ = QSMEM ? 1 : (JU > 0 ? JU : JP);
        float4 qr[JQ];
        const float4* qs = reinterpret_cast<const float4*>(base + lay.query);
        if constexpr (QSMEM) {
            float4* qw = reinterpret_cast<float4*>(base + lay.query);
#pragma unroll 1
            for (int c = lane; c < p.dim / 4; c += 32) qw[c] = __ldg(reinterpret_cast<const float4*>(q) + c);
            qr[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        } else if constexpr (JU > 0) vl_load_exact<LPR, JU>(q, lg, qr);
        else vl_load_query<LPR, JP, true>(q, p.dim, lg, qr);

        // ---- prologue: Queue.insert of the seeds into an empty queue (queue.py:37-61) ----
#pragma unroll 1
        for (int i = lane; i < sq_len; i += 32) sq[i] = kSent;
#pragma unroll 1
        for (int i = lane; i < lay.hash_slots; i += 32) hash[i] = kHashEmpty;
        vl_key_t* memo = memo_base;
        if (memo) {
            ulonglong2* m2 = reinterpret_cast<ulonglong2*>(memo);
#pragma unroll 1
            for (int i = lane; i < memo_buckets; i += 32) m2[i] = make_ulonglong2(~0ull, ~0ull);
        }
        __syncwarp();
#pragma unroll 1
        for (int c0 = 0; c0 < p.seed_cols; c0 += 32) {
            int c = c0 + lane;
            vl_key_t key = kSent;
            if (c < p.seed_cols)
                key = vl_entry_key(__ldg(p.seed_dist + row * p.seed_ld + c), __ldg(p.seed_ids + row * p.seed_ld + c));
            if (memo && key != kSent) memo_put(memo, memo_buckets, memo_shift, key, 0);   // a seed's distance is known
            bool want = key < sq[sq_len - 1];
            if (__any_sync(0xffffffffu, want)) merge_chunk(sq, sq_n, sq_len, key, want, lane, mpos);
        }
        // visit_queue.initialize_from_queue (queue.py:30-35)
        {
            const int head = sq_len < vq_len ? sq_len : vq_len;
#pragma unroll 1
            for (int i = lane; i < vq_len; i += 32) vq[i] = i < head ? sq[i] : kSent;
        }
        __syncwarp();

        bool always_full = true;
        unsigned long long st_todo = 0, st_sm = 0, st_vm = 0, st_iter = 0, st_a = 0, st_b = 0;
        long long tk[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};     // cycles per phase when p.stats is given
        const bool timing = p.stats != nullptr && (p.flags & 1);
        long long t_prev = timing ? clock64() : 0;
#define VL_PHASE(i) do { if (timing) { long long t_now = clock64(); tk[i] += t_now - t_prev; t_prev = t_now; } } while (0)
        const int32_t self_id = p.self_base >= 0 ? (int32_t)(p.self_base + row) : VL_MAXINT;
        const int32_t* excl = p.exclude_w > 0 ? p.exclude + row * (int64_t)p.exclude_w : nullptr;
        const int64_t group = p.group_rows > 0 ? (p.group_row0 + row) / p.group_rows : 0;
        bool dumped = false;

#pragma unroll 1
        for (int k = 1; k <= n_run; ++k) {
            const int first = (k - 1) * pvc;
            const bool seen_live = first < e_cap;    // utils.py:62-69
            const int ncopy = seen_live ? ((e_cap - first) < pvc ? (e_cap - first) : pvc) : 0;
            // ---- pop_n_ids (queue.py:87-95) ----
            {
                vl_key_t head = lane < pvc ? vq[lane] : kSent;
                int32_t node = vl_key_id(head);
                if (lane < pvc) {
                    if (node != VL_MAXINT && (node < 0 || (int64_t)node >= p.n)) {
                        atomicOr(p.status, VL_STATUS_BAD_ID);
                        node = VL_MAXINT;
                    }
                    pop[lane] = node;
                    // An id that enters `seen` now can never enter the visit queue again, and the
                    // search queue only looks at newly gathered ids: from here on its memo entry
                    // only has to say "popped" (an ordered distance above every real one).
                    // The mark goes into both entries of the id's bucket without reading them first: a load
                    // here would stall the whole iteration for a memory round trip, while losing the
                    // bucket's other entry only costs one gather if that id comes back.
                    if (memo && lane < ncopy && node != VL_MAXINT) {
                        ulonglong2* bk = reinterpret_cast<ulonglong2*>(memo + 2 * (size_t)memo_bucket((uint32_t)node, memo_shift, memo_buckets));
                        const vl_key_t mark = kPopped | (uint32_t)node;
                        *bk = make_ulonglong2(mark, mark);
                    }
                }
#pragma unroll 1
                for (int i = lane; i < vq_len; i += 32) vq_n[i] = (i + pvc < vq_len) ? vq[i + pvc] : kSent;
                __syncwarp();
                vl_key_t* t = vq; vq = vq_n; vq_n = t;
            }
            VL_PHASE(0);   // pop
            // ---- neighbour ids of the popped nodes (kernels.py:244), then which of them need a
            // gather: live ids the memo does not know.  VL_PB chunks of 32 candidates per round so
            // that the graph-row loads, and then the memo loads, of a round are in flight together.
            constexpr int PB = VL_PB;
            int n_todo = 0;
            const bool raw_iteration = p.dump_last && k == p.n_iters;   // needs every real distance
#pragma unroll 1
            for (int cb = 0; cb < m_total; cb += 32 * PB) {
                int32_t idr[PB];
#pragma unroll
                for (int u = 0; u < PB; ++u) {
                    const int c = cb + 32 * u + lane;
                    idr[u] = VL_MAXINT;
                    if (c < m_total) {
                        const int v = __float2int_rz(((float)c + 0.5f) * inv_wb);
                        const int32_t node = pop[v];
                        if (node != VL_MAXINT) idr[u] = vl_ldg_hint(p.graph + (int64_t)node * wb + (c - v * wb), pol_keep);
                    }
                }
                ulonglong2 bk[PB];
#pragma unroll
                for (int u = 0; u < PB; ++u) {
                    if (idr[u] != VL_MAXINT && (idr[u] < 0 || (int64_t)idr[u] >= p.n)) {
                        atomicOr(p.status, VL_STATUS_BAD_ID);
                        idr[u] = VL_MAXINT;
                    }
                    bk[u] = make_ulonglong2(~0ull, ~0ull);
                    if (memo && idr[u] != VL_MAXINT)
                        bk[u] = vl_ld_hint(reinterpret_cast<const ulonglong2*>(memo + 2 * (size_t)memo_bucket((uint32_t)idr[u], memo_shift, memo_buckets)), pol_keep);
                }
#pragma unroll
                for (int u = 0; u < PB; ++u) {
                    const int c = cb + 32 * u + lane;
                    const uint32_t id = (uint32_t)idr[u];
                    bool need = (idr[u] != VL_MAXINT);
                    uint32_t ord = sent_ord;
                    if (need) {
                        if ((uint32_t)bk[u].x == id) { ord = (uint32_t)(bk[u].x >> 32); need = false; }
                        else if ((uint32_t)bk[u].y == id) { ord = (uint32_t)(bk[u].y >> 32); need = false; }
                        if (!need && raw_iteration && ord == kPoppedOrd) need = true;
                    }
                    if (c < m_total) cand[c] = make_uint2(id, ord);
                    const unsigned mask = __ballot_sync(0xffffffffu, need);
                    if (need) todo[n_todo + __popc(mask & ((1u << lane) - 1u))] = (unsigned short)c;
                    n_todo += __popc(mask);
                }
            }

            __syncwarp();
            st_todo += n_todo;
            st_iter += 1;
            VL_PHASE(1);   // neighbour ids + memo probe
            // ---- gathered distances (kernels.py:248-257): G rows per step, U steps in flight ----
            // two steps in flight where the registers allow it (6-chunk rows: measured 3-9 % faster on 16 and 32
            // lanes per row, 5 % slower on 4)
            constexpr int U = QSMEM ? VL_U8 : ((JQ <= 4 || (JQ <= 6 && LPR >= 16)) ? 2 : 1);
#pragma unroll 1
            for (int t0 = 0; t0 < n_todo; t0 += U * G) {
                bool live[U];
                int mi[U];
                const float* rp[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int t = t0 + u * G + g;
                    live[u] = t < n_todo;
                    mi[u] = live[u] ? todo[t] : 0;
                    const int32_t id = live[u] ? (int32_t)cand[mi[u]].x : 0;
                    rp[u] = p.vectors + (int64_t)id * p.dim;
                }
                float dd[U];
#ifndef VL_NO_PREFETCH
                if constexpr (JU > 0) {
                    // pull the next round of candidate rows into L1 while this one is reduced: the
                    // registers can only hold one round of rows, the cache can hold the next
                    constexpr int LINES = (4 * LPR * JU * 4) / 128;          // 128-byte lines per row
                    const int tn = t0 + U * G;
#pragma unroll
                    for (int l0 = 0; l0 < U * G * LINES; l0 += 32) {
                        const int l = l0 + lane;
                        const int t = tn + l / LINES;
                        if (l < U * G * LINES && t < n_todo) {
                            const int32_t nid = (int32_t)cand[todo[t]].x;
                            const float* np_ = p.vectors + (int64_t)nid * p.dim + (l % LINES) * 32;
                            asm volatile("prefetch.global.L1 [%0];" : : "l"(np_));
                        }
                    }
                }
#endif
                if constexpr (JU > 0) {
                    float4 x[U][JU];
#pragma unroll
                    for (int u = 0; u < U; ++u) vl_load_exact_hint<LPR, JU>(rp[u], lg, x[u], pol_stream);
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if constexpr (QSMEM) dd[u] = vl_exact_distance_q<LPR, JP, JU, METRIC>(x[u], qs + lg);
                        else dd[u] = vl_exact_distance<LPR, JP, JU, METRIC>(x[u], qr);
                    }
                } else {
                    float4 x[U][JP];
#pragma unroll
                    for (int u = 0; u < U; ++u) vl_load_row<LPR, JP, true>(rp[u], p.dim, lg, live[u], x[u]);
#pragma unroll
                    for (int u = 0; u < U; ++u) dd[u] = vl_row_distance<LPR, JP, METRIC, true>(x[u], qr, rp[u], q, p.dim, lg, live[u]);
                }
                if (lg == 0) {
#pragma unroll
                    for (int u = 0; u < U; ++u)
                        if (live[u]) cand[mi[u]].y = vl_ord(dd[u]);
                }
            }
            __syncwarp();
            VL_PHASE(2);   // gather
            if (memo) {   // remember what was just computed
#pragma unroll 1
                for (int t = lane; t < n_todo; t += 32) memo_put(memo, memo_buckets, memo_shift, candk[todo[t]], k & 1);
                __syncwarp();
            }
            // ---- search_queue.insert(..., exclude) (ann.py:75-80) ----
            if (p.dump_last && k == p.n_iters) {
                // leave this insert to the caller's full-row sort: head, then the raw candidates
#pragma unroll 1
                for (int i = lane; i < sq_len; i += 32) {
                    p.out_ids[row * p.out_ld + i] = vl_key_id(sq[i]);
                    p.out_dist[row * p.out_ld + i] = vl_key_dist(sq[i]);
                }
#pragma unroll 1
                for (int i = lane; i < m_total; i += 32) {
                    vl_key_t key = candk[i];
                    int32_t id = vl_key_id(key);
                    bool drop = (id == self_id);
                    if (!drop && excl) {
#pragma unroll 1
                        for (int t = 0; t < p.exclude_w; ++t) {
                            int32_t x = excl[t];
                            if (x == VL_MAXINT) break;
                            if (x == id) { drop = true; break; }
                        }
                    }
                    if (drop) key = kSent;
                    p.out_ids[row * p.out_ld + sq_len + i] = vl_key_id(key);
                    p.out_dist[row * p.out_ld + sq_len + i] = vl_key_dist(key);
                }
#pragma unroll 1
                for (int i = sq_len + m_total + lane; i < p.out_cols; i += 32) {
                    p.out_ids[row * p.out_ld + i] = VL_MAXINT;
                    p.out_dist[row * p.out_ld + i] = VL_MAXFLOAT;
                }
                dumped = true;
                break;
            }
            VL_PHASE(3);   // memo put
            // Only candidates gathered in this iteration are offered: an id the memo already knew
            // was offered when it was first gathered, and the search queue's cut-off only falls, so
            // offering it again can neither add nor move anything.
            bool changed = false;
            vl_key_t cut = sq[sq_len - 1];
            // First gather the few candidates that can enter at all (below the queue's current last key,
            // not the row itself, not excluded) to the front of `todo`, then merge them 32 at a time:
            // usually one merge per iteration instead of one per 32-candidate chunk that holds an entrant.
            // "The L best of a union" does not depend on the grouping, so the queue is the same.
            int n_in = 0;
#pragma unroll 1
            for (int t0 = 0; t0 < n_todo; t0 += 32) {
                const int t = t0 + lane;
                const unsigned short ci = t < n_todo ? todo[t] : (unsigned short)0;
                const vl_key_t key = t < n_todo ? candk[ci] : kSent;
                bool want = key < cut;
                if (__any_sync(0xffffffffu, want)) {
                    if (want) {
                        int32_t id = vl_key_id(key);
                        if (id == self_id) want = false;
                        else if (excl) {
#pragma unroll 1
                            for (int x = 0; x < p.exclude_w; ++x) {   // kernels.py:478-488
                                int32_t ex = excl[x];
                                if (ex == VL_MAXINT) break;
                                if (ex == id) { want = false; break; }
                            }
                        }
                    }
                    const unsigned mask = __ballot_sync(0xffffffffu, want);
                    __syncwarp();                                     // every lane has read its todo[t] of this chunk
                    if (want) todo[n_in + __popc(mask & ((1u << lane) - 1u))] = ci;   // n_in <= t0: never ahead of the reads
                    n_in += __popc(mask);
                }
            }
            __syncwarp();
#pragma unroll 1
            for (int t0 = 0; t0 < n_in; t0 += 32) {
                const int t = t0 + lane;
                const vl_key_t key = t < n_in ? candk[todo[t]] : kSent;
                const bool want = key < cut;
                if (!__any_sync(0xffffffffu, want)) continue;
                changed |= merge_chunk(sq, sq_n, sq_len, key, want, lane, mpos);
                st_sm += 1;
                cut = sq[sq_len - 1];
            }
            VL_PHASE(4);   // search-queue merge
            if (changed && (k % p.readahead) == 0 && lane == 0) {
                int chk = k / p.readahead - 1;
                if (chk < p.n_checks) atomicOr(p.changed_flags + group * p.n_checks + chk, 1u);
            }
            // ---- add_new_to_seen_ (utils.py:61-82) + visit_queue.insert(..., exclude=seen) ----
            if (seen_live) {
                int32_t mine = lane < ncopy ? pop[lane] : 0;
                if (lane < ncopy && mine != VL_MAXINT) hash_insert(hash, lay.hash_slots, lay.hash_shift, mine, p.status);
                if (__any_sync(0xffffffffu, lane < ncopy && mine == VL_MAXINT)) always_full = false;
                __syncwarp();
                // The popped entries left `free` slots, so the new queue is: every candidate
                // below the largest kept key T0 that is neither visited nor already queued (class A,
                // merged by rank), then - only if slots remain - the smallest unvisited candidates
                // above T0 (class B, appended one by one in rising order).  Same queue as offering
                // every candidate, without sorting the many that are already in it.
                int n_old = 0;
#pragma unroll 1
                for (int i0 = 0; i0 < vq_len; i0 += 32)
                    n_old += __popc(__ballot_sync(0xffffffffu, i0 + lane < vq_len && vq[i0 + lane] != kSent));
                if (n_old > 0 && vq_len - n_old <= 8) {
                    VL_PHASE(6);
                    const vl_key_t t0key = vq[n_old - 1];
                    int n_a = 0;
#pragma unroll 1
                    for (int c0 = 0; c0 < m_total; c0 += 32) {
                        const int c = c0 + lane;
                        const bool in_a = c < m_total && candk[c] < t0key;
                        const unsigned mask = __ballot_sync(0xffffffffu, in_a);
                        if (in_a) todo[n_a + __popc(mask & ((1u << lane) - 1u))] = (unsigned short)c;
                        n_a += __popc(mask);
                    }
                    __syncwarp();
                    VL_PHASE(7);
                    st_a += n_a;
                    vl_key_t vcut = vq[vq_len - 1];
#pragma unroll 1
                    for (int t0 = 0; t0 < n_a; t0 += 32) {
                        const int t = t0 + lane;
                        vl_key_t key = t < n_a ? candk[todo[t]] : kSent;
                        bool want = key < vcut;
                        if (want && hash_contains(hash, lay.hash_slots, lay.hash_shift, vl_key_id(key))) want = false;
                        if (!__any_sync(0xffffffffu, want)) continue;
                        merge_chunk(vq, vq_n, vq_len, key, want, lane, mpos);
                        st_vm += 1;
                        vcut = vq[vq_len - 1];
                    }
                    VL_PHASE(8);
                    int n_real = 0;
#pragma unroll 1
                    for (int i0 = 0; i0 < vq_len; i0 += 32)
                        n_real += __popc(__ballot_sync(0xffffffffu, i0 + lane < vq_len && vq[i0 + lane] != kSent));
                    vl_key_t last = t0key;
#pragma unroll 1
                    while (n_real < vq_len) {
                        st_b += 1;
                        vl_key_t best = ~0ull;
#pragma unroll 1
                        for (int c = lane; c < m_total; c += 32) {
                            const vl_key_t kk = candk[c];
                            if (kk > last && kk < kSent && kk < best) best = kk;
                        }
#pragma unroll
                        for (int off = 16; off >= 1; off >>= 1) {
                            const vl_key_t o = __shfl_xor_sync(0xffffffffu, best, off);
                            best = o < best ? o : best;
                        }
                        if (best == ~0ull) break;
                        last = best;
                        if (hash_contains(hash, lay.hash_slots, lay.hash_shift, vl_key_id(best))) continue;
                        if (lane == 0) vq[n_real] = best;
                        ++n_real;
                        st_vm += 1;
                    }
                    __syncwarp();
                    VL_PHASE(9);
                } else {
                    // an (almost) empty queue: offer every candidate, 32 at a time
                    vl_key_t vcut = vq[vq_len - 1];
#pragma unroll 1
                    for (int c0 = 0; c0 < m_total; c0 += 32) {
                        const int c = c0 + lane;
                        vl_key_t key = c < m_total ? candk[c] : kSent;
                        bool want = key < vcut;
                        if (!__any_sync(0xffffffffu, want)) continue;
                        if (want && hash_contains(hash, lay.hash_slots, lay.hash_shift, vl_key_id(key))) want = false;
                        if (!__any_sync(0xffffffffu, want)) continue;
                        merge_chunk(vq, vq_n, vq_len, key, want, lane, mpos);
                        st_vm += 1;
                        vcut = vq[vq_len - 1];
                    }
                }
            }
            VL_PHASE(5);   // seen update + visit-queue merge
        }

        VL_PHASE(5);       // visit-queue merge of the last iteration + epilogue
        if (!dumped) {
#pragma unroll 1
            for (int i = lane; i < p.out_cols; i += 32) {
                vl_key_t key = i < sq_len ? sq[i] : kSent;
                p.out_ids[row * p.out_ld + i] = vl_key_id(key);
                p.out_dist[row * p.out_ld + i] = vl_key_dist(key);
            }
        }
        if (always_full && lane == 0) atomicOr(p.group_full + group, 1u);
        if (p.stats && lane == 0) {
            atomicAdd(p.stats + 1, st_todo);
            atomicAdd(p.stats + 2, st_sm);
            atomicAdd(p.stats + 3, st_vm);
            atomicAdd(p.stats + 4, st_a);
            atomicAdd(p.stats + 5, st_b);
            atomicAdd(p.stats + 6, 1ull);
            atomicAdd(p.stats + 7, st_iter);
            if (timing)
#pragma unroll 1
                for (int i = 0; i < 10; ++i) atomicAdd(p.stats + 8 + i, (unsigned long long)tk[i]);
        }
        __syncwarp();
        if (p.row_ticket) {
            unsigned long long t = 0;
            if (lane == 0) t = atomicAdd(p.row_ticket, 1ull);
            row = nwarps + (int64_t)__shfl_sync(0xffffffffu, t, 0);
        } else {
            row += nwarps;
        }
    }
}

struct BeamPlan { BeamSmem lay; int warps; int blocks; size_t smem; };

template <int LPR, int JP, int JU, int METRIC>
int plan_and_launch(const vl_beam_params& p, BeamPlan& plan, bool launch, cudaStream_t stream)
{
    auto kernel = beam_search_kernel<LPR, JP, JU, METRIC>;
    plan.lay = beam_smem_layout(p.pvc * p.graph_w, p.sq_len, p.vq_len, p.seen_cap, (JU >= 8) ? p.dim * 4 : 0);
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
    if (launch && p.memo)
        VL_CHECK_ARG(p.memo_slots >= (int64_t)plan.blocks * plan.warps, "vl_beam_search: memo has %lld slots, the launch keeps %lld rows in flight",
                     (long long)p.memo_slots, (long long)plan.blocks * plan.warps);
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
    VL_CHECK_ARG(p.n_checks >= 0 && p.group_rows >= 0 && p.group_row0 >= 0, "vl_beam_search: bad flag shape");
    VL_CHECK_ARG(p.pvc * (int64_t)p.graph_w <= 65535, "vl_beam_search: %d candidates per iteration exceed 65535", p.pvc * p.graph_w);
    VL_CHECK_ARG(!p.memo || (p.memo_entries >= 2 && (p.memo_entries & (p.memo_entries - 1)) == 0 && (uintptr_t)p.memo % 16 == 0),
                 "vl_beam_search: memo_entries must be a power of two >= 2 and the memo 16-byte aligned");
    if (p.rows == 0) { plan.blocks = 0; plan.warps = kBeamWarps; plan.lay = beam_smem_layout(p.pvc * p.graph_w, p.sq_len, p.vq_len, p.seen_cap, 0); return 0; }
    VlShape shape = vl_pick_shape(p.dim);
    int rc = 0;
    const int chunks = p.dim / 4;
    // exact-fit instantiations for the row sizes that matter (no per-chunk bounds tests)
#define VL_EXACT(L, J, U)                                                                              \
    if (chunks == L * U) {                                                                             \
        if (p.metric == VL_METRIC_COSINE) return plan_and_launch<L, J, U, VL_METRIC_COSINE>(p, plan, launch, stream); \
        return plan_and_launch<L, J, U, VL_METRIC_SQL2>(p, plan, launch, stream);                      \
    }
    VL_EXACT(4, 4, 4)     // dim 64
    VL_EXACT(4, 8, 6)     // dim 96
    VL_EXACT(8, 4, 4)     // dim 128: one 128-byte line per 8-lane load, query in registers (measured 12 % faster than 4 x 8)
    VL_EXACT(8, 8, 8)     // dim 256
    VL_EXACT(16, 8, 6)    // dim 384
    VL_EXACT(16, 8, 8)    // dim 512
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
