// Shared device helpers for the VectorLink B200 kernels (sm_100a).
//
// Conventions used by every kernel in this directory:
//   * ids are int32, distances fp32, the sentinels are MAXINT / MAXFLOAT of the reference
//     (vectorlink_gpu/constants.py:5-6);
//   * a queue entry travels as one 64-bit key: high word = the distance mapped to an
//     order-preserving unsigned integer, low word = the id.  Unsigned comparison of keys is
//     the reference's queue order (distance ascending, then id ascending;
//     vectorlink_gpu/utils.py:44-53), and the sentinel pair is the largest key in use;
//   * a distance is the reference's fixed summation tree (vectorlink_gpu/kernels.py:27-114)
//     evaluated with 128-bit row loads and sub-warp shuffles, bit for bit.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "vlgpu.h"

#define VL_ID_FLAG (1 << 30)  // kernels.py:322: bit 30 marks a duplicate, so ids must stay below 2^30

typedef unsigned long long vl_key_t;

__device__ __forceinline__ uint32_t vl_ord(float f)
{
    f = __fadd_rn(f, 0.0f);  // -0 -> +0: torch.sort treats them as equal
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float vl_unord(uint32_t o)
{
    uint32_t u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
    return __uint_as_float(u);
}
__device__ __forceinline__ vl_key_t vl_make_key(float d, int32_t id)
{
    return ((vl_key_t)vl_ord(d) << 32) | (uint32_t)id;
}
__device__ __forceinline__ vl_key_t vl_sentinel_key() { return vl_make_key(VL_MAXFLOAT, VL_MAXINT); }
__device__ __forceinline__ int32_t vl_key_id(vl_key_t k) { return (int32_t)(uint32_t)(k & 0xffffffffu); }
__device__ __forceinline__ float vl_key_dist(vl_key_t k) { return vl_unord((uint32_t)(k >> 32)); }
// the reference punches every entry whose id has bit 30 set (kernels.py:333-349), MAXINT included
__device__ __forceinline__ vl_key_t vl_entry_key(float d, int32_t id)
{
    return (id & VL_ID_FLAG) ? vl_sentinel_key() : vl_make_key(d, id);
}

// One term of the sum: a*b for the cosine metric, (a-b)^2 for squared L2.  Explicit
// round-to-nearest intrinsics keep the compiler from contracting anything into an FMA: the
// reference stores every product to shared memory before the first add (kernels.py:98).
template <int METRIC>
__device__ __forceinline__ float vl_term(float a, float b)
{
    if (METRIC == VL_METRIC_COSINE) return __fmul_rn(a, b);
    float d = __fsub_rn(a, b);
    return __fmul_rn(d, d);
}
template <int METRIC>
__device__ __forceinline__ float4 vl_term4(float4 a, float4 b)
{
    return make_float4(vl_term<METRIC>(a.x, b.x), vl_term<METRIC>(a.y, b.y), vl_term<METRIC>(a.z, b.z),
                       vl_term<METRIC>(a.w, b.w));
}
__device__ __forceinline__ float4 vl_add4(float4 a, float4 b)
{
    return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}
template <int METRIC>
__device__ __forceinline__ float vl_finish(float s)
{
    if (METRIC == VL_METRIC_COSINE) {
        float r = __fmul_rn(__fsub_rn(1.0f, s), 0.5f);  // (1 - c) / 2, exact either way
        return r < 0.0f ? 0.0f : (r > 1.0f ? 1.0f : r);  // kernels.py:108-112
    }
    return s;
}

// 16-byte chunk `c` of a row (elements 4c .. 4c+3); elements at or past `dim` read as zero.
// ALIGNED rows (dim % 4 == 0, 16-byte aligned base) take one 128-bit load.
template <bool ALIGNED>
__device__ __forceinline__ float4 vl_load_chunk(const float* __restrict__ row, int c, int dim)
{
    if (ALIGNED) return __ldg(reinterpret_cast<const float4*>(row) + c);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    int e = 4 * c;
    if (e + 0 < dim) v.x = __ldg(row + e + 0);
    if (e + 1 < dim) v.y = __ldg(row + e + 1);
    if (e + 2 < dim) v.z = __ldg(row + e + 2);
    if (e + 3 < dim) v.w = __ldg(row + e + 3);
    return v;
}

// The reference's sum (kernels.py:38-72 + 27-35) is a halving tree over a 1024-slot buffer:
// slot t += slot t+h for h = 512 ... 1, after slots 1024k+t were folded onto t in rising k.
// A row is spread over LPR lanes (4, 8, 16 or 32) as 16-byte chunks, lane l holding chunks
// l + LPR*j, j < JP (LPR*JP*4 >= min(dim,1024)).  Then tree levels h >= 4*LPR are adds between a lane's own
// registers (largest stride first), levels 4*LPR > h >= 4 are shuffles between lanes, and the
// last two levels combine the four components of the remaining float4 - the same additions in
// the same order, so the result is bit-identical.
// JU > 0 says only registers j < JU hold data (the rest are zero by construction): adds of
// a known zero are skipped, which changes nothing (x + 0 == x; the sign of an all-zero sum
// does not survive vl_finish).
template <int LPR, int JP, int JU = 0>
__device__ __forceinline__ float vl_tree_reduce(float4 (&acc)[JP])
{
    constexpr int USED = JU > 0 ? JU : JP;
#pragma unroll
    for (int h = JP / 2; h >= 1; h >>= 1) {
#pragma unroll
        for (int j = 0; j < h; ++j)
            if (j + h < USED) acc[j] = vl_add4(acc[j], acc[j + h]);
    }
    float4 a = acc[0];
#pragma unroll
    for (int off = LPR / 2; off >= 1; off >>= 1) {
        a.x = __fadd_rn(a.x, __shfl_down_sync(0xffffffffu, a.x, off, LPR));
        a.y = __fadd_rn(a.y, __shfl_down_sync(0xffffffffu, a.y, off, LPR));
        a.z = __fadd_rn(a.z, __shfl_down_sync(0xffffffffu, a.z, off, LPR));
        a.w = __fadd_rn(a.w, __shfl_down_sync(0xffffffffu, a.w, off, LPR));
    }
    return __fadd_rn(__fadd_rn(a.x, a.z), __fadd_rn(a.y, a.w));
}

// L2 eviction-priority hints (createpolicy + ld/st ...L2::cache_hint): candidate rows are streamed
// (evict first), while a row's memo and the graph rows are what the next iterations come back to
// (evict last).
__device__ __forceinline__ uint64_t vl_policy_evict_first()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t vl_policy_evict_normal()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t vl_policy_evict_last()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ float4 vl_ldg_hint(const float4* ptr, uint64_t pol)
{
    float4 v;
    asm volatile("ld.global.nc.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(ptr), "l"(pol));
    return v;
}
__device__ __forceinline__ int32_t vl_ldg_hint(const int32_t* ptr, uint64_t pol)
{
    int32_t v;
    asm volatile("ld.global.nc.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(ptr), "l"(pol));
    return v;
}
__device__ __forceinline__ ulonglong2 vl_ld_hint(const ulonglong2* ptr, uint64_t pol)
{
    ulonglong2 v;
    asm volatile("ld.global.L2::cache_hint.v2.u64 {%0,%1}, [%2], %3;" : "=l"(v.x), "=l"(v.y) : "l"(ptr), "l"(pol) : "memory");
    return v;
}
template <int LPR, int JU>
__device__ __forceinline__ void vl_load_exact_hint(const float* __restrict__ row, int lg, float4 (&xr)[JU], uint64_t pol)
{
    const float4* r4 = reinterpret_cast<const float4*>(row) + lg;
#pragma unroll
    for (int j = 0; j < JU; ++j) xr[j] = vl_ldg_hint(r4 + LPR * j, pol);
}

// Exact-fit fast path: the row is exactly LPR*JU 16-byte chunks (dim == 4*LPR*JU <= 1024,
// aligned), so every lane loads JU chunks with no bounds test; `row` must be a readable row
// even for a dead candidate (its result is discarded).
template <int LPR, int JU>
__device__ __forceinline__ void vl_load_exact(const float* __restrict__ row, int lg, float4 (&xr)[JU])
{
    const float4* r4 = reinterpret_cast<const float4*>(row) + lg;
#pragma unroll
    for (int j = 0; j < JU; ++j) xr[j] = __ldg(r4 + LPR * j);
}
// Packed fp32x2 arithmetic of sm_100 (add/sub/mul.rn.f32x2): two IEEE round-to-nearest
// operations per instruction, the same bits as the scalar intrinsics, half the issue slots.
typedef unsigned long long vl_f2;
__device__ __forceinline__ vl_f2 vl_f2_pack(float lo, float hi)
{
    vl_f2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void vl_f2_unpack(vl_f2 v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ vl_f2 vl_f2_add(vl_f2 a, vl_f2 b)
{
    vl_f2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ vl_f2 vl_f2_sub(vl_f2 a, vl_f2 b)
{
    vl_f2 d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// Packed product.  ptxas 12.9 contracts a packed multiply (and a packed FMA with a -0 addend,
// which it may simplify to a multiply) with the packed add that consumes it into one packed
// FMA - one rounding instead of two, which breaks bit parity - even when both carry .rn.
// fma(a, b, +0) cannot be simplified (it differs from a*b when the product is -0) and an FMA
// cannot absorb a following add, so this form keeps both roundings.  Its value is round(a*b)
// except that a -0 product becomes +0, which no sum downstream can tell apart.
__device__ __forceinline__ vl_f2 vl_f2_mul(vl_f2 a, vl_f2 b)
{
    vl_f2 d;
    const vl_f2 zero = 0ull;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(zero));
    return d;
}
template <int METRIC>
__device__ __forceinline__ vl_f2 vl_f2_term(float ax, float ay, float bx, float by)
{
#ifndef VL_PACKED_PRODUCTS   // default: scalar products (measured equally fast, and independent of how ptxas treats packed FMAs)
    if (METRIC == VL_METRIC_COSINE) return vl_f2_pack(__fmul_rn(ax, bx), __fmul_rn(ay, by));
    float dx, dy;
    vl_f2_unpack(vl_f2_sub(vl_f2_pack(ax, ay), vl_f2_pack(bx, by)), dx, dy);
    return vl_f2_pack(__fmul_rn(dx, dx), __fmul_rn(dy, dy));
#else
    if (METRIC == VL_METRIC_COSINE) return vl_f2_mul(vl_f2_pack(ax, ay), vl_f2_pack(bx, by));
    const vl_f2 d = vl_f2_sub(vl_f2_pack(ax, ay), vl_f2_pack(bx, by));
    return vl_f2_mul(d, d);
#endif
}

// Exact-fit distance on packed pairs: (x,y) and (z,w) of every chunk travel as fp32x2 through
// the differences, the register fold and the lane shuffles; the order of additions is that of
// vl_tree_reduce.
template <int LPR, int JP, int JU, int METRIC>
__device__ __forceinline__ float vl_exact_distance(const float4 (&xr)[JU], const float4 (&qr)[JU])
{
    vl_f2 axy[JU], azw[JU];
#pragma unroll
    for (int j = 0; j < JU; ++j) {
        axy[j] = vl_f2_term<METRIC>(xr[j].x, xr[j].y, qr[j].x, qr[j].y);
        azw[j] = vl_f2_term<METRIC>(xr[j].z, xr[j].w, qr[j].z, qr[j].w);
    }
#pragma unroll
    for (int h = JP / 2; h >= 1; h >>= 1) {
#pragma unroll
        for (int j = 0; j < h; ++j)
            if (j + h < JU) {
                axy[j] = vl_f2_add(axy[j], axy[j + h]);
                azw[j] = vl_f2_add(azw[j], azw[j + h]);
            }
    }
    vl_f2 xy = axy[0], zw = azw[0];
#pragma unroll
    for (int off = LPR / 2; off >= 1; off >>= 1) {
        xy = vl_f2_add(xy, __shfl_down_sync(0xffffffffu, xy, off, LPR));
        zw = vl_f2_add(zw, __shfl_down_sync(0xffffffffu, zw, off, LPR));
    }
    float lo, hi;
    vl_f2_unpack(vl_f2_add(xy, zw), lo, hi);       // (x+z, y+w)
    return vl_finish<METRIC>(__fadd_rn(lo, hi));
}

// The same with the query read from memory (shared): q4[LPR*j] is the lane's j-th query chunk.
template <int LPR, int JP, int JU, int METRIC>
__device__ __forceinline__ float vl_exact_distance_q(const float4 (&xr)[JU], const float4* q4)
{
    vl_f2 axy[JU], azw[JU];
#pragma unroll
    for (int j = 0; j < JU; ++j) {
        const float4 qv = q4[LPR * j];
        axy[j] = vl_f2_term<METRIC>(xr[j].x, xr[j].y, qv.x, qv.y);
        azw[j] = vl_f2_term<METRIC>(xr[j].z, xr[j].w, qv.z, qv.w);
    }
#pragma unroll
    for (int h = JP / 2; h >= 1; h >>= 1) {
#pragma unroll
        for (int j = 0; j < h; ++j)
            if (j + h < JU) {
                axy[j] = vl_f2_add(axy[j], axy[j + h]);
                azw[j] = vl_f2_add(azw[j], azw[j + h]);
            }
    }
    vl_f2 xy = axy[0], zw = azw[0];
#pragma unroll
    for (int off = LPR / 2; off >= 1; off >>= 1) {
        xy = vl_f2_add(xy, __shfl_down_sync(0xffffffffu, xy, off, LPR));
        zw = vl_f2_add(zw, __shfl_down_sync(0xffffffffu, zw, off, LPR));
    }
    float lo, hi;
    vl_f2_unpack(vl_f2_add(xy, zw), lo, hi);
    return vl_finish<METRIC>(__fadd_rn(lo, hi));
}

// The query-side registers of one lane: chunks lg + LPR*j of the first 1024 elements.
template <int LPR, int JP, bool ALIGNED>
__device__ __forceinline__ void vl_load_query(const float* __restrict__ q, int dim, int lg, float4 (&qr)[JP])
{
    const int nchunks = (dim + 3) >> 2;
#pragma unroll
    for (int j = 0; j < JP; ++j) {
        int c = lg + LPR * j;
        qr[j] = (c < nchunks && c < 256) ? vl_load_chunk<ALIGNED>(q, c, dim) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// Issue the loads of one candidate row (first 1024 elements) into registers.
template <int LPR, int JP, bool ALIGNED>
__device__ __forceinline__ void vl_load_row(const float* __restrict__ row, int dim, int lg, bool live, float4 (&xr)[JP])
{
    const int nchunks = (dim + 3) >> 2;
#pragma unroll
    for (int j = 0; j < JP; ++j) {
        int c = lg + LPR * j;
        xr[j] = (live && c < nchunks && c < 256) ? vl_load_chunk<ALIGNED>(row, c, dim) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// Distance of the loaded row against the query registers; valid in the group's lane 0.
// `qfull` is the whole query row, read again only for elements past 1024.
template <int LPR, int JP, int METRIC, bool ALIGNED>
__device__ __forceinline__ float vl_row_distance(const float4 (&xr)[JP], const float4 (&qr)[JP],
                                                 const float* __restrict__ row, const float* __restrict__ qfull,
                                                 int dim, int lg, bool live)
{
    float4 acc[JP];
#pragma unroll
    for (int j = 0; j < JP; ++j) acc[j] = vl_term4<METRIC>(xr[j], qr[j]);
    if (dim > 1024) {  // kernels.py:43-47: fold element 1024k+t onto t, k rising
        const int nchunks = (dim + 3) >> 2;
        for (int k = 1; 256 * k < nchunks; ++k) {
#pragma unroll
            for (int j = 0; j < JP; ++j) {
                int c = 256 * k + lg + LPR * j;
                if (live && c < nchunks && lg + LPR * j < 256) {
                    float4 x = vl_load_chunk<ALIGNED>(row, c, dim);
                    float4 y = vl_load_chunk<ALIGNED>(qfull, c, dim);
                    float4 t = vl_term4<METRIC>(x, y);
                    // a chunk that straddles `dim` must add nothing for its missing elements
                    // (the reference never touches those slots); zero terms do exactly that,
                    // except that (0-0)^2 and 0*0 are +0 and x + 0 == x
                    acc[j] = vl_add4(acc[j], t);
                }
            }
        }
    }
    return vl_finish<METRIC>(vl_tree_reduce<LPR, JP>(acc));
}

// Shape of the lane layout for a dimension: the smallest (LPR, JP) with LPR*JP >= chunks.
struct VlShape { int lpr, jp; };
static inline VlShape vl_pick_shape(int dim)
{
    int chunks = (dim + 3) / 4;
    if (chunks > 256) chunks = 256;
    if (chunks <= 4) return {4, 1};
    if (chunks <= 8) return {4, 2};
    if (chunks <= 16) return {4, 4};
    if (chunks <= 32) return {4, 8};
    if (chunks <= 64) return {8, 8};
    if (chunks <= 128) return {16, 8};
    return {32, 8};
}

#define VL_DISPATCH_SHAPE(shape, ...)                                                   \
    do {                                                                                \
        if ((shape).lpr == 4 && (shape).jp == 1) { constexpr int LPR = 4, JP = 1; __VA_ARGS__ }        \
        else if ((shape).lpr == 4 && (shape).jp == 2) { constexpr int LPR = 4, JP = 2; __VA_ARGS__ }   \
        else if ((shape).lpr == 4 && (shape).jp == 4) { constexpr int LPR = 4, JP = 4; __VA_ARGS__ }   \
        else if ((shape).lpr == 4 && (shape).jp == 8) { constexpr int LPR = 4, JP = 8; __VA_ARGS__ }   \
        else if ((shape).lpr == 8 && (shape).jp == 8) { constexpr int LPR = 8, JP = 8; __VA_ARGS__ }   \
        else if ((shape).lpr == 16 && (shape).jp == 8) { constexpr int LPR = 16, JP = 8; __VA_ARGS__ } \
        else { constexpr int LPR = 32, JP = 8; __VA_ARGS__ }                            \
    } while (0)

// host-side error plumbing shared by the extern "C" entry points
void vl_set_error(const char* fmt, ...);
int vl_sm_count();   // SMs of the current device
#define VL_CHECK_ARG(cond, ...)          \
    do {                                 \
        if (!(cond)) {                   \
            vl_set_error(__VA_ARGS__);   \
            return -1;                   \
        }                                \
    } while (0)
#define VL_CHECK_LAUNCH(name)                                                        \
    do {                                                                             \
        cudaError_t e__ = cudaGetLastError();                                        \
        if (e__ != cudaSuccess) {                                                    \
            vl_set_error("%s: launch failed: %s", name, cudaGetErrorString(e__));    \
            return -2;                                                               \
        }                                                                            \
    } while (0)
