// Hand-written sm_100a SpMV kernels, one family per reduce operator ("template") of the
// reference. Every family is parameterised at run time: value dtype and column-index width
// are template parameters, every metadata array is a `Meta` (device array of width 1/2/4/8 or
// a closed form), launch shape comes from the tuner.
//
// Array semantics follow the reference's emitted kernels (code_of_template_kernal in
// direct_atom_op*.cc, shared_memory_*.cc, unaligned_warp_reduce_same_TLB_size_op*.cc); the
// device code itself is new: vectorised streaming loads of values/indices, read-only-path
// gathers of x, shuffle reductions, segmented warp scan without prefix-sum cancellation,
// red.global atomics only where a row is shared.
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernel_args.h"
#include "kernels.h"

namespace asp
{

typedef unsigned long long u64;
typedef unsigned int u32;

// ---------------------------------------------------------------------------------------------
// metadata access
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ u64 mload(const void *p, int width, u64 i)
{
    switch (width)
    {
    case 1: return __ldg((const unsigned char *)p + i);
    case 2: return __ldg((const unsigned short *)p + i);
    case 4: return __ldg((const unsigned int *)p + i);
    default: return __ldg((const u64 *)p + i);
    }
}

__device__ __forceinline__ u64 mget(const Meta &m, u64 i)
{
    switch (m.kind)
    {
    case MK_ARRAY: return mload(m.p, m.width, i);
    case MK_LINEAR: return i * m.coef + m.icpt;
    case MK_CONSTANT: return m.icpt;
    case MK_CYCLE_LINEAR: return (i % m.cycle) * m.coef + m.icpt;
    case MK_CYCLE_INCREASE: return i / m.cycle + m.icpt;
    default:
    {
        u64 v = m.bval[0];
#pragma unroll
        for (int b = 1; b < 5; b++)
            if (b < m.nb && i > m.bhi[b - 1]) v = m.bval[b];
        return v;
    }
    }
}

// ---------------------------------------------------------------------------------------------
// streaming vector loads: values and column indices are touched once per SpMV, so they are
// loaded with the evict-first policy and leave L1/L2 to the x gathers.
// ---------------------------------------------------------------------------------------------
template <class T, int V>
struct alignas(sizeof(T) * V) Vec
{
    T v[V];
};

template <int BYTES>
struct RawLoad;
template <>
struct RawLoad<1>
{
    typedef unsigned char type;
};
template <>
struct RawLoad<2>
{
    typedef unsigned short type;
};
template <>
struct RawLoad<4>
{
    typedef unsigned int type;
};
template <>
struct RawLoad<8>
{
    typedef uint2 type;
};
template <>
struct RawLoad<16>
{
    typedef uint4 type;
};

template <class T, int V>
__device__ __forceinline__ Vec<T, V> ld_stream(const T *p)
{
    typedef typename RawLoad<sizeof(T) * V>::type R;
    union
    {
        R r;
        Vec<T, V> v;
    } u;
    u.r = __ldcs(reinterpret_cast<const R *>(p));
    return u.v;
}
// The same loads as volatile PTX: the compiler keeps volatile asm statements in program order, so a
// batch of loads written before its uses is issued as a batch (it otherwise interleaves loads and
// uses to save registers, which serialises the memory latency).
template <int BYTES>
__device__ __forceinline__ void ld_cs_raw(const void *p, unsigned int (&r)[(BYTES + 3) / 4])
{
    if constexpr (BYTES == 16)
        asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "l"(p));
    else if constexpr (BYTES == 8)
        asm volatile("ld.global.cs.v2.u32 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "l"(p));
    else if constexpr (BYTES == 4)
        asm volatile("ld.global.cs.u32 %0, [%1];" : "=r"(r[0]) : "l"(p));
    else if constexpr (BYTES == 2)
    {
        unsigned short t;
        asm volatile("ld.global.cs.u16 %0, [%1];" : "=h"(t) : "l"(p));
        r[0] = t;
    }
    else
    {
        unsigned int t;
        asm volatile("ld.global.cs.u8 %0, [%1];" : "=r"(t) : "l"(p));
        r[0] = t;
    }
}

template <class T, int V>
__device__ __forceinline__ void ld_stream_pinned(const T *p, T (&out)[V])
{
    constexpr int BYTES = sizeof(T) * V;
    if constexpr (BYTES <= 16)
    {
        unsigned int r[(BYTES + 3) / 4];
        ld_cs_raw<BYTES>(p, r);
        if constexpr (sizeof(T) == 8)
        {
#pragma unroll
            for (int j = 0; j < V; j++)
            {
                const unsigned long long w = ((unsigned long long)r[2 * j + 1] << 32) | r[2 * j];
                out[j] = *reinterpret_cast<const T *>(&w);
            }
        }
        else if constexpr (sizeof(T) == 4)
        {
#pragma unroll
            for (int j = 0; j < V; j++) out[j] = *reinterpret_cast<const T *>(&r[j]);
        }
        else if constexpr (sizeof(T) == 2)
        {
#pragma unroll
            for (int j = 0; j < V; j++) out[j] = (T)((r[j / 2] >> (16 * (j & 1))) & 0xffffu);
        }
        else
        {
#pragma unroll
            for (int j = 0; j < V; j++) out[j] = (T)((r[j / 4] >> (8 * (j & 3))) & 0xffu);
        }
    }
    else
    {
        constexpr int H = 16 / sizeof(T);
#pragma unroll
        for (int h = 0; h < V / H; h++)
        {
            T half[H];
            ld_stream_pinned<T, H>(p + h * H, half);
#pragma unroll
            for (int j = 0; j < H; j++) out[h * H + j] = half[j];
        }
    }
}

__device__ __forceinline__ float ld_x_pinned(const float *p)
{
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ double ld_x_pinned(const double *p)
{
    double v;
    asm volatile("ld.global.nc.f64 %0, [%1];" : "=d"(v) : "l"(p));
    return v;
}

// 32-byte groups (8 x f32 / 4 x f64) are fetched as two 16-byte halves
template <class T, int V>
__device__ __forceinline__ void ld_stream_n(const T *p, T (&out)[V])
{
    if constexpr (sizeof(T) * V <= 16)
    {
        Vec<T, V> t = ld_stream<T, V>(p);
#pragma unroll
        for (int j = 0; j < V; j++) out[j] = t.v[j];
    }
    else
    {
        constexpr int H = 16 / sizeof(T);
#pragma unroll
        for (int h = 0; h < V / H; h++)
        {
            Vec<T, H> t = ld_stream<T, H>(p + h * H);
#pragma unroll
            for (int j = 0; j < H; j++) out[h * H + j] = t.v[j];
        }
    }
}

template <class VT>
__device__ __forceinline__ void out_add(VT *y, u64 row, VT v, bool atomic)
{
    if (atomic)
        atomicAdd(y + row, v); // result unused: compiles to red.global.add
    else
        y[row] = v;
}

// rows whose permutation is applied on the device (shared-memory and CSR5-like families)
__device__ __forceinline__ u64 row_on_device(const KArgs &a, u64 r)
{
    if (a.sort_kind == 1) return mget(a.perm, r + a.first_row);
    if (a.sort_kind == 2) return mget(a.perm, r) + a.first_row;
    return r + a.first_row;
}

template <class VT>
__device__ __forceinline__ VT warp_sum(VT v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------------------------
// DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS (ELL-like): thread t owns row map[t]; element k of
// TLB t sits at t + k*P, P = padded TLB count. V adjacent TLBs per thread give 16-byte loads.
// ---------------------------------------------------------------------------------------------
// KS > 0: the TLB size is a compile-time constant, so every value / index load of a thread is in
// flight before the first gather of x is issued. KS == 0: any size, in predicated chunks of 4.
template <class VT, int V>
__device__ __forceinline__ void store_rows(VT *__restrict__ y, u64 row0, const VT (&acc)[V])
{
    if constexpr (sizeof(VT) * V >= 16)
    {
        constexpr int H = 16 / sizeof(VT);
        typedef Vec<VT, H> P16;
#pragma unroll
        for (int h = 0; h < V / H; h++)
        {
            P16 t;
#pragma unroll
            for (int j = 0; j < H; j++) t.v[j] = acc[h * H + j];
            *reinterpret_cast<P16 *>(y + row0 + h * H) = t;
        }
    }
    else
    {
#pragma unroll
        for (int j = 0; j < V; j++) y[row0 + j] = acc[j];
    }
}

template <class VT, class CT, int V, int KS>
__global__ void __launch_bounds__(512) k_ell(const KArgs a)
{
    const VT *__restrict__ val = (const VT *)a.val;
    const CT *__restrict__ col = (const CT *)a.col;
    const VT *__restrict__ x = (const VT *)a.x + a.first_col;
    VT *__restrict__ y = (VT *)a.y;
    const u64 P = a.n_tlb;
    const u32 S = KS > 0 ? (u32)KS : a.tlb_size;
    const u64 ngroup = P / V;
    const u64 stride = (u64)gridDim.x * blockDim.x;
    const u64 radd = a.row_add ? a.first_row : 0;
    // consecutive TLBs map to consecutive rows: whole groups can be stored as vectors
    const bool unit_rows = a.m[MS_ROW_OF_TLB].kind == MK_LINEAR && a.m[MS_ROW_OF_TLB].coef == 1 && !a.atomic &&
                           ((a.m[MS_ROW_OF_TLB].icpt + radd) % V) == 0;
    for (u64 g = (u64)blockIdx.x * blockDim.x + threadIdx.x; g < ngroup; g += stride)
    {
        const u64 t0 = g * V;
        if (t0 >= a.effective) break;
        VT acc[V];
#pragma unroll
        for (int j = 0; j < V; j++) acc[j] = 0;
        const VT *vp = val + t0;
        const CT *cp = col + t0;
        if constexpr (KS > 0)
        {
            VT v[KS][V];
            CT c[KS][V];
#pragma unroll
            for (int k = 0; k < KS; k++)
            {
                ld_stream_n<VT, V>(vp + (u64)k * P, v[k]);
                ld_stream_n<CT, V>(cp + (u64)k * P, c[k]);
            }
#pragma unroll
            for (int k = 0; k < KS; k++)
#pragma unroll
                for (int j = 0; j < V; j++) acc[j] += v[k][j] * __ldg(x + c[k][j]);
        }
        else
        {
            constexpr int U = 4;
            u32 k = 0;
            for (; k + U <= S; k += U)
            {
                VT v[U][V];
                CT c[U][V];
#pragma unroll
                for (int u = 0; u < U; u++) ld_stream_pinned<CT, V>(cp + (u64)(k + u) * P, c[u]);
#pragma unroll
                for (int u = 0; u < U; u++) ld_stream_pinned<VT, V>(vp + (u64)(k + u) * P, v[u]);
                VT xv[U][V];
#pragma unroll
                for (int u = 0; u < U; u++)
#pragma unroll
                    for (int j = 0; j < V; j++) xv[u][j] = ld_x_pinned(x + c[u][j]);
#pragma unroll
                for (int u = 0; u < U; u++)
#pragma unroll
                    for (int j = 0; j < V; j++) acc[j] += v[u][j] * xv[u][j];
            }
            if (k < S)
            {
                VT v[U - 1][V];
                CT c[U - 1][V];
#pragma unroll
                for (int u = 0; u < U - 1; u++)
                    if (k + u < S)
                    {
                        ld_stream_n<VT, V>(vp + (u64)(k + u) * P, v[u]);
                        ld_stream_n<CT, V>(cp + (u64)(k + u) * P, c[u]);
                    }
#pragma unroll
                for (int u = 0; u < U - 1; u++)
                    if (k + u < S)
                    {
#pragma unroll
                        for (int j = 0; j < V; j++) acc[j] += v[u][j] * __ldg(x + c[u][j]);
                    }
            }
        }
        if (unit_rows && t0 + V <= a.effective)
            store_rows<VT, V>(y, t0 + a.m[MS_ROW_OF_TLB].icpt + radd, acc);
        else
        {
#pragma unroll
            for (int j = 0; j < V; j++)
            {
                const u64 t = t0 + j;
                if (t < a.effective) out_add(y, mget(a.m[MS_ROW_OF_TLB], t) + radd, acc[j], a.atomic != 0);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// DIRECT_ATOM_TEMPLATE_WARP_COMPRESS (SELL-like): inside BLB b (a row strip of n TLBs) element k
// of local TLB i sits at nz0 + i + k*n.
//
// Strips of equal size (block_begin_thread_index_offset is linear, as ROW_PADDING + even row
// division gives) are cut into warp tasks of 32*V TLBs that a persistent grid of warps walks, so
// thousands of tiny strips cost no CTA launches; otherwise one CTA takes one strip at a time.
// ---------------------------------------------------------------------------------------------
template <class VT, int V>
__device__ __forceinline__ void sell_store(const KArgs &a, VT *__restrict__ y, const VT (&acc)[V], u64 t0, u64 radd)
{
    const Meta &rm = a.m[MS_ROW_OF_TLB];
    if (V > 1 && rm.kind == MK_LINEAR && rm.coef == 1 && !a.atomic && t0 + V <= a.effective && ((t0 + rm.icpt + radd) % V) == 0)
    {
        store_rows<VT, V>(y, t0 + rm.icpt + radd, acc);
        return;
    }
    if (V == 4 && rm.kind == MK_ARRAY && rm.width == 4 && (t0 & 3) == 0 && t0 + V <= a.effective)
    {
        const uint4 r = __ldg(reinterpret_cast<const uint4 *>((const unsigned int *)rm.p + t0));
        out_add(y, (u64)r.x + radd, acc[0], a.atomic != 0);
        out_add(y, (u64)r.y + radd, acc[1 % V], a.atomic != 0);
        out_add(y, (u64)r.z + radd, acc[2 % V], a.atomic != 0);
        out_add(y, (u64)r.w + radd, acc[3 % V], a.atomic != 0);
        return;
    }
#pragma unroll
    for (int j = 0; j < V; j++)
    {
        const u64 t = t0 + j;
        if (t < a.effective) out_add(y, mget(rm, t) + radd, acc[j], a.atomic != 0);
    }
}

template <class VT, class CT, int V>
__device__ __forceinline__ void sell_group(const KArgs &a, const VT *__restrict__ val, const CT *__restrict__ col, const VT *__restrict__ x,
                                           VT *__restrict__ y, u64 nz, u64 n, u32 S, u64 t0, u64 radd)
{
    VT acc[V];
#pragma unroll
    for (int j = 0; j < V; j++) acc[j] = 0;
    const VT *vp = val + nz;
    const CT *cp = col + nz;
    constexpr int U = 4;
    u32 k = 0;
    // full batches: U value and U index vectors in flight, then U*V gathers, then the FMAs
    for (; k + U <= S; k += U)
    {
        VT v[U][V];
        CT c[U][V];
#pragma unroll
        for (int u = 0; u < U; u++) ld_stream_pinned<CT, V>(cp + (u64)u * n, c[u]);
#pragma unroll
        for (int u = 0; u < U; u++) ld_stream_pinned<VT, V>(vp + (u64)u * n, v[u]);
        VT xv[U][V];
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int j = 0; j < V; j++) xv[u][j] = ld_x_pinned(x + c[u][j]);
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int j = 0; j < V; j++) acc[j] += v[u][j] * xv[u][j];
        vp += (u64)U * n;
        cp += (u64)U * n;
    }
    if (k < S)
    {
        // the last S % U steps (all of a short TLB) as one predicated batch
        VT v[U - 1][V];
        CT c[U - 1][V];
#pragma unroll
        for (int u = 0; u < U - 1; u++)
            if (k + u < S)
            {
                ld_stream_n<VT, V>(vp + (u64)u * n, v[u]);
                ld_stream_n<CT, V>(cp + (u64)u * n, c[u]);
            }
#pragma unroll
        for (int u = 0; u < U - 1; u++)
            if (k + u < S)
            {
#pragma unroll
                for (int j = 0; j < V; j++) acc[j] += v[u][j] * __ldg(x + c[u][j]);
            }
    }
    sell_store<VT, V>(a, y, acc, t0, radd);
}

template <class VT, class CT, int V>
__global__ void __launch_bounds__(256) k_sell(const KArgs a)
{
    const VT *__restrict__ val = (const VT *)a.val;
    const CT *__restrict__ col = (const CT *)a.col;
    const VT *__restrict__ x = (const VT *)a.x + a.first_col;
    VT *__restrict__ y = (VT *)a.y;
    const u64 radd = a.row_add ? a.first_row : 0;
    const Meta &bt = a.m[MS_BLK_THR];
    if ((a.path & 1) == 0 && V > 1 && bt.kind == MK_LINEAR && bt.coef > 0 && (bt.coef % (32 * V)) == 0)
    {
        const u64 n = bt.coef;
        const u64 tasks_per_blb = n / (32 * V);
        const u64 total = a.n_units * tasks_per_blb;
        const u32 lane = threadIdx.x & 31;
        const u64 wstride = ((u64)gridDim.x * blockDim.x) >> 5;
        for (u64 task = ((u64)blockIdx.x * blockDim.x + threadIdx.x) >> 5; task < total; task += wstride)
        {
            const u64 b = task / tasks_per_blb;
            const u64 i = (task - b * tasks_per_blb) * (32 * V) + (u64)lane * V;
            const u64 t0 = bt.icpt + b * n + i;
            if (t0 >= a.effective) continue;
            const u64 nz0 = mget(a.m[MS_BLK_NZ], b);
            const u32 S = (u32)mget(a.m[MS_TLB_SIZE], b);
            if ((nz0 % V) == 0)
                sell_group<VT, CT, V>(a, val, col, x, y, nz0 + i, n, S, t0, radd);
            else
            {
#pragma unroll
                for (int j = 0; j < V; j++) sell_group<VT, CT, 1>(a, val, col, x, y, nz0 + i + j, n, S, t0 + j, radd);
            }
        }
        return;
    }
    for (u64 b = blockIdx.x; b < a.n_units; b += gridDim.x)
    {
        const u64 nz0 = mget(a.m[MS_BLK_NZ], b);
        const u64 t0 = mget(bt, b);
        const u64 t1 = mget(bt, b + 1);
        const u32 S = (u32)mget(a.m[MS_TLB_SIZE], b);
        const u64 n = t1 - t0;
        if (t0 >= a.effective) continue;
        if (V > 1 && (n % V == 0) && (nz0 % V == 0))
        {
            for (u64 i = (u64)threadIdx.x * V; i < n; i += (u64)blockDim.x * V)
            {
                if (t0 + i >= a.effective) break;
                sell_group<VT, CT, V>(a, val, col, x, y, nz0 + i, n, S, t0 + i, radd);
            }
        }
        else
        {
            for (u64 i = threadIdx.x; i < n; i += blockDim.x)
            {
                if (t0 + i >= a.effective) break;
                sell_group<VT, CT, 1>(a, val, col, x, y, nz0 + i, n, S, t0 + i, radd);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// DIRECT_ATOM_TEMPLATE: BLB -> WLB -> groups of 32 TLBs, values warp-staggered (element k of
// lane l in group g at base + g*32*S + k*32 + l). The reference accumulates this template in
// double and always adds atomically when rows are shared.
// ---------------------------------------------------------------------------------------------
template <class VT, class CT>
__global__ void __launch_bounds__(1024) k_direct3(const KArgs a)
{
    const VT *__restrict__ val = (const VT *)a.val;
    const CT *__restrict__ col = (const CT *)a.col;
    const VT *__restrict__ x = (const VT *)a.x + a.first_col;
    VT *__restrict__ y = (VT *)a.y;
    const u32 lane = threadIdx.x & 31, wid = threadIdx.x >> 5, wnum = blockDim.x >> 5;
    const u64 radd = a.row_add ? a.first_row : 0;
    for (u64 b = blockIdx.x; b < a.n_units; b += gridDim.x)
    {
        const u64 bnz = mget(a.m[MS_BLK_NZ], b);
        const u64 w0 = mget(a.m[MS_BLK_WARP], b), w1 = mget(a.m[MS_BLK_WARP], b + 1);
        for (u64 w = w0 + wid; w < w1; w += wnum)
        {
            const u64 wnz = bnz + mget(a.m[MS_WARP_NZ], w);
            const u32 S = (u32)mget(a.m[MS_TLB_SIZE], w);
            const u64 t0 = mget(a.m[MS_WARP_THR], w), t1 = mget(a.m[MS_WARP_THR], w + 1);
            const u64 groups = (t1 - t0) >> 5;
            if ((wnz & 3) == 0)
            {
                // a lane takes 4 adjacent TLBs of a group (one 16-byte load of values and of indices per step), so a
                // warp walks 4 groups per trip: lane l -> group g0 + l / 8, TLBs 4 (l % 8) .. + 3
                for (u64 g = lane >> 3; g < groups; g += 4)
                {
                    double acc[4] = {0, 0, 0, 0};
                    u64 nz = wnz + g * 32 * S + 4 * (lane & 7);
                    for (u32 k = 0; k < S; k++, nz += 32)
                    {
                        VT v[4];
                        CT c[4];
                        ld_stream_n<VT, 4>(val + nz, v);
                        ld_stream_n<CT, 4>(col + nz, c);
#pragma unroll
                        for (int j = 0; j < 4; j++) acc[j] += (double)(v[j] * __ldg(x + c[j]));
                    }
                    const u64 t = t0 + g * 32 + 4 * (lane & 7);
#pragma unroll
                    for (int j = 0; j < 4; j++) out_add(y, mget(a.m[MS_ROW_OF_TLB], t + j) + radd, (VT)acc[j], a.atomic != 0);
                }
            }
            else
                for (u64 g = 0; g < groups; g++)
                {
                    double acc = 0;
                    u64 nz = wnz + g * 32 * S + lane;
                    for (u32 k = 0; k < S; k++, nz += 32) acc += (double)(__ldcs(val + nz) * __ldg(x + __ldcs(col + nz)));
                    const u64 t = t0 + g * 32 + lane;
                    out_add(y, mget(a.m[MS_ROW_OF_TLB], t) + radd, (VT)acc, a.atomic != 0);
                }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE (CSR-vector-like): warp <-> WLB = a chunk of one row.
// ---------------------------------------------------------------------------------------------
template <class VT, class CT>
__device__ __forceinline__ VT warp_chunk_dot(const VT *__restrict__ val, const CT *__restrict__ col, const VT *__restrict__ x, u64 beg, u64 end, u32 lane)
{
    VT acc = 0;
    constexpr int V = 16 / sizeof(VT) >= 4 ? 4 : 2; // 4 x f32 or 2 x f64 per lane and step
    if (((beg | end) & (V - 1)) == 0 && end - beg >= 32 * V)
    {
        u64 i = beg + (u64)lane * V;
        for (; i + V <= end; i += 32 * V)
        {
            VT v[V];
            CT c[V];
            ld_stream_n<VT, V>(val + i, v);
            ld_stream_n<CT, V>(col + i, c);
#pragma unroll
            for (int j = 0; j < V; j++) acc += v[j] * __ldg(x + c[j]);
        }
    }
    else
    {
        for (u64 i = beg + lane; i < end; i += 32) acc += __ldcs(val + i) * __ldg(x + __ldcs(col + i));
    }
    return acc;
}

template <class VT, class CT>
__global__ void __launch_bounds__(1024) k_warp_row(const KArgs a)
{
    const VT *__restrict__ val = (const VT *)a.val;
    const CT *__restrict__ col = (const CT *)a.col;
    const VT *__restrict__ x = (const VT *)a.x + a.first_col;
    VT *__restrict__ y = (VT *)a.y;
    const u32 lane = threadIdx.x & 31;
    const u64 wstride = ((u64)gridDim.x * blockDim.x) >> 5;
    const u64 radd = a.row_add ? a.first_row : 0;
    for (u64 w = ((u64)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < a.effective; w += wstride)
    {
        const u64 beg = mget(a.m[MS_WARP_NZ], w), end = mget(a.m[MS_WARP_NZ], w + 1);
        VT acc = warp_sum(warp_chunk_dot<VT, CT>(val, col, x, beg, end, lane));
        if (lane == 0) out_add(y, mget(a.m[MS_ROW_OF_UNIT], w) + radd, acc, a.atomic != 0);
    }
}

// ---------------------------------------------------------------------------------------------
// SHARED_MEMORY_LONG_ROW_TEMPLATE: CTA <-> BLB = a chunk of one long row.
// ---------------------------------------------------------------------------------------------
template <class VT, class CT>
__global__ void __launch_bounds__(1024) k_long_row(const KArgs a)
{
    __shared__ VT part[32];
    const VT *__restrict__ val = (const VT *)a.val;
    const CT *__restrict__ col = (const CT *)a.col;
    const VT *__restrict__ x = (const VT *)a.x + a.first_col;
    VT *__restrict__ y = (VT *)a.y;
    const u32 lane = threadIdx.x & 31, wid = threadIdx.x >> 5, wnum = blockDim.x >> 5;
    const u64 radd = a.row_add ? a.first_row : 0;
    constexpr int V = 16 / sizeof(VT) >= 4 ? 4 : 2;
    for (u64 b = blockIdx.x; b < a.n_units; b += gridDim.x)
    {
        const u64 beg = mget(a.m[MS_BLK_NZ], b), end = mget(a.m[MS_BLK_NZ], b + 1);
        VT acc = 0;
        if (((beg | end) & (V - 1)) == 0)
        {
            const u64 step = (u64)blockDim.x * V;
            u64 i = beg + (u64)threadIdx.x * V;
            // two CTA-strides per trip: both index vectors, both value vectors, then 2V gathers
            for (; i + step < end; i += 2 * step)
            {
                VT v[2][V];
                CT c[2][V];
                ld_stream_pinned<CT, V>(col + i, c[0]);
                ld_stream_pinned<CT, V>(col + i + step, c[1]);
                ld_stream_pinned<VT, V>(val + i, v[0]);
                ld_stream_pinned<VT, V>(val + i + step, v[1]);
                VT xv[2][V];
#pragma unroll
                for (int u = 0; u < 2; u++)
#pragma unroll
                    for (int j = 0; j < V; j++) xv[u][j] = ld_x_pinned(x + c[u][j]);
#pragma unroll
                for (int u = 0; u < 2; u++)
#pragma unroll
                    for (int j = 0; j < V; j++) acc += v[u][j] * xv[u][j];
            }
            for (; i < end; i += step)
            {
                VT v[V];
                CT c[V];
                ld_stream_n<VT, V>(val + i, v);
                ld_stream_n<CT, V>(col + i, c);
#pragma unroll
                for (int j = 0; j < V; j++) acc += v[j] * __ldg(x + c[j]);
            }
        }
        else
        {
            for (u64 i = beg + threadIdx.x; i < end; i += blockDim.x) acc += __ldcs(val + i) * __ldg(x + __ldcs(col + i));
        }
        acc = warp_sum(acc);
        __syncthreads(); // previous iteration's readers are done with part[]
        if (lane == 0) part[wid] = acc;
        __syncthreads();
        if (wid == 0)
        {
            VT s = lane < wnum ? part[lane] : (VT)0;
            s = warp_sum(s);
            if (lane == 0) out_add(y, mget(a.m[MS_ROW_OF_UNIT], b) + radd, s, a.atomic != 0);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// phase 2 of the shared-memory family: `w` lanes per row sum the row's slice of the CTA's
// partial results (CSR over partials), combine by shuffle, lane 0 of the group writes y.
// Every warp runs the same trip count so full-mask shuffles are legal.
// ---------------------------------------------------------------------------------------------
template <class VT>
__device__ __forceinline__ void smem_row_reduce(const KArgs &a, const VT *part, VT *__restrict__ y, u64 r0, u64 r1, u64 g0)
{
    const u32 w = (u32)a.row_reduce;
    const u32 lane = threadIdx.x & 31;
    const u32 sub = lane & (w - 1);
    const u32 rows_per_warp = 32 / w;
    const u64 rows_per_cta = (u64)(blockDim.x >> 5) * rows_per_warp;
    for (u64 rb = r0 + (u64)(threadIdx.x >> 5) * rows_per_warp; rb < r1; rb += rows_per_cta)
    {
        const u64 r = rb + lane / w;
        const bool valid = r < r1;
        VT s = 0;
        if (valid)
        {
            const u64 lo = mget(a.m[MS_ROW_OFF], r) - g0, hi = mget(a.m[MS_ROW_OFF], r + 1) - g0;
            for (u64 j = lo + sub; j < hi; j += w) s += part[j];
        }
        for (u32 o = w >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (valid && sub == 0 && r < a.effective) out_add(y, row_on_device(a, r), s, a.atomic != 0);
    }
}

// SHARED_MEMORY_TEMPLATE_WARP_COMPRESS (row-grouped CSR): CTA <-> BLB; TLB partials in smem.
template <class VT, class CT>
__global__ void __launch_bounds__(1024) k_smem_tlb(const KArgs a)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    VT *part = reinterpret_cast<VT *>(smem_raw);
    const VT *__restrict__ val = (const VT *)a.val;
    const CT *__restrict__ col = (const CT *)a.col;
    const VT *__restrict__ x = (const VT *)a.x + a.first_col;
    VT *__restrict__ y = (VT *)a.y;
    for (u64 b = blockIdx.x; b < a.n_units; b += gridDim.x)
    {
        const u64 nz0 = mget(a.m[MS_BLK_NZ], b);
        const u64 t0 = mget(a.m[MS_BLK_THR], b), t1 = mget(a.m[MS_BLK_THR], b + 1);
        const u64 r0 = mget(a.m[MS_BLK_ROW], b), r1 = mget(a.m[MS_BLK_ROW], b + 1);
        const u32 S = (u32)mget(a.m[MS_TLB_SIZE], b);
        const u64 n = t1 - t0;
        const u64 g0 = mget(a.m[MS_ROW_OFF], r0);
        __syncthreads(); // the previous strip's phase 2 has finished reading part[]
        constexpr int V = 4;
        if ((n % V) == 0 && (nz0 % V) == 0)
        {
            // the strip's TLB count is padded to a multiple of 32 by the TLB operator: a thread takes V adjacent TLBs,
            // so every value / index load is one 16-byte (fp32) or two 16-byte (fp64) vectors, batches of 4 steps in flight
            for (u64 i = (u64)threadIdx.x * V; i < n; i += (u64)blockDim.x * V)
            {
                VT acc[V];
#pragma unroll
                for (int j = 0; j < V; j++) acc[j] = 0;
                const VT *vp = val + nz0 + i;
                const CT *cp = col + nz0 + i;
                constexpr int U = 4;
                u32 k = 0;
                for (; k + U <= S; k += U)
                {
                    VT v[U][V], xv[U][V];
                    CT c[U][V];
#pragma unroll
                    for (int u = 0; u < U; u++) ld_stream_pinned<CT, V>(cp + (u64)u * n, c[u]);
#pragma unroll
                    for (int u = 0; u < U; u++) ld_stream_pinned<VT, V>(vp + (u64)u * n, v[u]);
#pragma unroll
                    for (int u = 0; u < U; u++)
#pragma unroll
                        for (int j = 0; j < V; j++) xv[u][j] = ld_x_pinned(x + c[u][j]);
#pragma unroll
                    for (int u = 0; u < U; u++)
#pragma unroll
                        for (int j = 0; j < V; j++) acc[j] += v[u][j] * xv[u][j];
                    vp += (u64)U * n;
                    cp += (u64)U * n;
                }
                for (; k < S; k++)
                {
                    VT v[V];
                    CT c[V];
                    ld_stream_n<VT, V>(vp, v);
                    ld_stream_n<CT, V>(cp, c);
#pragma unroll
                    for (int j = 0; j < V; j++) acc[j] += v[j] * __ldg(x + c[j]);
                    vp += n;
                    cp += n;
                }
#pragma unroll
                for (int j = 0; j < V; j++) part[i + j] = acc[j];
            }
        }
        else
        {
            for (u64 i = threadIdx.x; i < n; i += blockDim.x)
            {
                VT acc = 0;
                const VT *vp = val + nz0 + i;
                const CT *cp = col + nz0 + i;
#pragma unroll 4
                for (u32 k = 0; k < S; k++)
                {
                    acc += __ldcs(vp) * __ldg(x + __ldcs(cp));
                    vp += n;
                    cp += n;
                }
                part[i] = acc;
            }
        }
        __syncthreads();
        smem_row_reduce<VT>(a, part, y, r0, r1, g0);
    }
}

// SHARED_MEMORY_TEMPLATE: BLB -> WLB -> TLB with WLB-level interleave (element k of local TLB i
// of a WLB at bnz + wnz + i + k*n_w), partials of the whole BLB in smem, then the row reduce.
template <class VT, class CT>
__global__ void __launch_bounds__(1024) k_smem3(const KArgs a)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    VT *part = reinterpret_cast<VT *>(smem_raw);
    const VT *__restrict__ val = (const VT *)a.val;
    const CT *__restrict__ col = (const CT *)a.col;
    const VT *__restrict__ x = (const VT *)a.x + a.first_col;
    VT *__restrict__ y = (VT *)a.y;
    const u32 lane = threadIdx.x & 31, wid = threadIdx.x >> 5, wnum = blockDim.x >> 5;
    for (u64 b = blockIdx.x; b < a.n_units; b += gridDim.x)
    {
        const u64 bnz = mget(a.m[MS_BLK_NZ], b);
        const u64 w0 = mget(a.m[MS_BLK_WARP], b), w1 = mget(a.m[MS_BLK_WARP], b + 1);
        const u64 r0 = mget(a.m[MS_BLK_ROW], b), r1 = mget(a.m[MS_BLK_ROW], b + 1);
        const u64 tb0 = mget(a.m[MS_WARP_THR], w0);
        const u64 g0 = mget(a.m[MS_ROW_OFF], r0);
        __syncthreads();
        for (u64 w = w0 + wid; w < w1; w += wnum)
        {
            const u64 wnz = bnz + mget(a.m[MS_WARP_NZ], w);
            const u32 S = (u32)mget(a.m[MS_TLB_SIZE], w);
            const u64 t0 = mget(a.m[MS_WARP_THR], w), t1 = mget(a.m[MS_WARP_THR], w + 1);
            const u64 n = t1 - t0;
            if ((n & 3) == 0 && (wnz & 3) == 0)
            {
                // the WLB's TLB count is padded to a multiple of 32: a lane takes 4 adjacent TLBs, 16-byte loads per step
                for (u64 i = (u64)lane * 4; i < n; i += 128)
                {
                    VT acc[4] = {0, 0, 0, 0};
                    u64 nz = wnz + i;
                    for (u32 k = 0; k < S; k++, nz += n)
                    {
                        VT v[4];
                        CT c[4];
                        ld_stream_n<VT, 4>(val + nz, v);
                        ld_stream_n<CT, 4>(col + nz, c);
#pragma unroll
                        for (int j = 0; j < 4; j++) acc[j] += v[j] * __ldg(x + c[j]);
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) part[t0 + i + j - tb0] = acc[j];
                }
            }
            else
                for (u64 i = lane; i < n; i += 32)
                {
                    VT acc = 0;
                    u64 nz = wnz + i;
                    for (u32 k = 0; k < S; k++, nz += n) acc += __ldcs(val + nz) * __ldg(x + __ldcs(col + nz));
                    part[t0 + i - tb0] = acc;
                }
        }
        __syncthreads();
        smem_row_reduce<VT>(a, part, y, r0, r1, g0);
    }
}

// SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE: CTA <-> BLB (a few rows); warp <-> WLB (chunk of
// one row) reduced by shuffle into smem; then the row reduce over WLB partials.
template <class VT, class CT>
__global__ void __launch_bounds__(1024) k_smem_wlb(const KArgs a)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    VT *part = reinterpret_cast<VT *>(smem_raw);
    const VT *__restrict__ val = (const VT *)a.val;
    const CT *__restrict__ col = (const CT *)a.col;
    const VT *__restrict__ x = (const VT *)a.x + a.first_col;
    VT *__restrict__ y = (VT *)a.y;
    const u32 lane = threadIdx.x & 31, wid = threadIdx.x >> 5, wnum = blockDim.x >> 5;
    for (u64 b = blockIdx.x; b < a.n_units; b += gridDim.x)
    {
        const u64 w0 = mget(a.m[MS_BLK_WARP], b), w1 = mget(a.m[MS_BLK_WARP], b + 1);
        const u64 r0 = mget(a.m[MS_BLK_ROW], b), r1 = mget(a.m[MS_BLK_ROW], b + 1);
        const u64 g0 = mget(a.m[MS_ROW_OFF], r0);
        __syncthreads();
        for (u64 w = w0 + wid; w < w1; w += wnum)
        {
            const u64 beg = mget(a.m[MS_WARP_NZ], w), end = mget(a.m[MS_WARP_NZ], w + 1);
            VT acc = warp_sum(warp_chunk_dot<VT, CT>(val, col, x, beg, end, lane));
            if (lane == 0) part[w - w0] = acc;
        }
        __syncthreads();
        smem_row_reduce<VT>(a, part, y, r0, r1, g0);
    }
}

// ---------------------------------------------------------------------------------------------
// UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE[_WITH_WARP_REDUCE] (CSR5-like): every thread
// owns S consecutive non-zeros regardless of row boundaries; the packed per-thread word holds
// S row-start flags (MSB first), the count of following threads that continue this thread's
// last row, and the first row (relative to the warp's first row) that starts in this thread.
//
// Cross-thread tails are combined with a flag-segmented suffix scan (no subtraction of prefix
// sums), and the thread that holds a row's start writes the row's total. The reference's
// emitted code writes the per-thread partial instead of the total for rows that span threads.
// ---------------------------------------------------------------------------------------------
// products val[nz + 32u] * x[col[nz + 32u]], u < cnt <= U. A full batch issues its U index loads,
// U value loads and U gathers in that order (volatile PTX keeps the order), so U gathers are in flight.
template <class VT, class CT, int U>
__device__ __forceinline__ void strided_products(const VT *__restrict__ val, const CT *__restrict__ col, const VT *__restrict__ x, u64 nz, u32 cnt, VT (&p)[U])
{
    if (cnt >= (u32)U)
    {
        CT c[U][1];
        VT v[U][1];
#pragma unroll
        for (int u = 0; u < U; u++) ld_stream_pinned<CT, 1>(col + nz + 32 * u, c[u]);
#pragma unroll
        for (int u = 0; u < U; u++) ld_stream_pinned<VT, 1>(val + nz + 32 * u, v[u]);
        VT xv[U];
#pragma unroll
        for (int u = 0; u < U; u++) xv[u] = ld_x_pinned(x + c[u][0]);
#pragma unroll
        for (int u = 0; u < U; u++) p[u] = v[u][0] * xv[u];
    }
    else
    {
#pragma unroll
        for (int u = 0; u < U; u++) p[u] = (u32)u < cnt ? __ldcs(val + nz + 32 * u) * __ldg(x + __ldcs(col + nz + 32 * u)) : VT(0);
    }
}

template <class VT, class CT, bool WARP_FAST>
__global__ void __launch_bounds__(256) k_csr5(const KArgs a)
{
    const VT *__restrict__ val = (const VT *)a.val;
    const CT *__restrict__ col = (const CT *)a.col;
    const VT *__restrict__ x = (const VT *)a.x + a.first_col;
    VT *__restrict__ y = (VT *)a.y;
    const u32 lane = threadIdx.x & 31;
    const u32 S = a.tlb_size;
    const u64 wstride = ((u64)gridDim.x * blockDim.x) >> 5;
    for (u64 w = ((u64)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < a.n_units; w += wstride)
    {
        const u64 R0 = mget(a.m[MS_ROW_OF_UNIT], w);
        u64 nz = w * 32 * S + lane;
        if (WARP_FAST)
        {
            // the first-row array of this template carries one sentinel entry past the last warp
            const u64 R1 = (w + 1 < (u64)a.warps_first_row_len) ? mget(a.m[MS_ROW_OF_UNIT], w + 1) : R0 + 1;
            if (R0 == R1)
            {
                VT s = 0;
                constexpr int UF = 8;
                for (u32 k0 = 0; k0 < S; k0 += UF, nz += 32 * UF)
                {
                    VT pr[UF];
                    strided_products<VT, CT, UF>(val, col, x, nz, S - k0, pr);
#pragma unroll
                    for (int u = 0; u < UF; u++) s += pr[u];
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0) atomicAdd(y + row_on_device(a, R0), s);
                continue;
            }
        }
        const u64 meta = mload(a.m[MS_COMBINE].p, a.m[MS_COMBINE].width, w * 32 + lane);
        const u32 frow = (u32)(meta & ((1ull << a.bits_row) - 1));
        const u32 roff = (u32)((meta >> a.bits_row) & ((1ull << a.bits_off) - 1));
        u32 yo = frow;
        bool seen = false;
        VT sum = 0, tail = 0;
        // products of U elements are fetched together (independent gathers in flight) before the
        // sequential walk over the row-start flags
        constexpr u32 U = 8;
        for (u32 k0 = 0; k0 < S; k0 += U, nz += 32 * U)
        {
            VT v[U];
            strided_products<VT, CT, (int)U>(val, col, x, nz, S - k0, v);
#pragma unroll
            for (u32 u = 0; u < U; u++)
                if (k0 + u < S)
                {
                    const bool flag = (meta >> (a.bits_word - 1 - (k0 + u))) & 1ull;
                    if (flag)
                    {
                        if (seen)
                        {
                            // a row that starts and ends inside this thread; only the warp's very
                            // first row can also receive contributions from the previous warp
                            const bool at = a.atomic || (lane == 0 && yo == frow);
                            out_add(y, row_on_device(a, R0 + yo), sum, at);
                            yo++;
                        }
                        else
                            tail = sum;
                        seen = true;
                        sum = 0;
                    }
                    sum += v[u];
                }
        }
        if (!seen) tail = sum;
        // suffix scan of the tails, segmented at threads that start a row: after the scan
        // lane j holds the sum of tail[j..] up to and including the next row-starting lane.
        const u32 heads = __ballot_sync(0xffffffffu, seen);
        VT sc = tail;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1)
        {
            const VT o = __shfl_down_sync(0xffffffffu, sc, d);
            // lanes [lane, lane+d) must contain no row start for lane+d to belong to my segment
            const bool same = (lane + d < 32) && (((heads >> lane) & ((1u << d) - 1u)) == 0u);
            if (same) sc += o;
        }
        VT extra = __shfl_down_sync(0xffffffffu, sc, 1);
        if (lane == 31) extra = 0;
        if (seen)
        {
            const bool at = a.atomic || (lane == 0 && yo == frow) || (lane + roff == 31);
            out_add(y, row_on_device(a, R0 + yo), sum + extra, at);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// launch dispatch
// ---------------------------------------------------------------------------------------------
template <class VT, class CT, int V>
static void launch_ell_v(const KArgs &a, dim3 grid, dim3 block, cudaStream_t st)
{
    if constexpr (V == 2 || V == 4)
    {
        switch (a.tlb_size)
        {
        case 1: k_ell<VT, CT, V, 1><<<grid, block, 0, st>>>(a); return;
        case 2: k_ell<VT, CT, V, 2><<<grid, block, 0, st>>>(a); return;
        case 3: k_ell<VT, CT, V, 3><<<grid, block, 0, st>>>(a); return;
        case 4: k_ell<VT, CT, V, 4><<<grid, block, 0, st>>>(a); return;
        case 5: k_ell<VT, CT, V, 5><<<grid, block, 0, st>>>(a); return;
        case 6: k_ell<VT, CT, V, 6><<<grid, block, 0, st>>>(a); return;
        case 7: k_ell<VT, CT, V, 7><<<grid, block, 0, st>>>(a); return;
        case 8: k_ell<VT, CT, V, 8><<<grid, block, 0, st>>>(a); return;
        default: break;
        }
    }
    k_ell<VT, CT, V, 0><<<grid, block, 0, st>>>(a);
}

template <class VT, class CT>
static void launch_ell(const KArgs &a, dim3 grid, dim3 block, cudaStream_t st, int vec)
{
    if (vec >= 8) launch_ell_v<VT, CT, 8>(a, grid, block, st);
    else if (vec >= 4) launch_ell_v<VT, CT, 4>(a, grid, block, st);
    else if (vec == 2) launch_ell_v<VT, CT, 2>(a, grid, block, st);
    else launch_ell_v<VT, CT, 1>(a, grid, block, st);
}

template <class VT, class CT>
static cudaError_t launch_vc(int templ, const KArgs &a, dim3 grid, dim3 block, size_t smem, cudaStream_t st, int vec)
{
    switch (templ)
    {
    case 2: // ELL-like
        launch_ell<VT, CT>(a, grid, block, st, vec);
        break;
    case 1: // SELL-like
        if (vec >= 4) k_sell<VT, CT, 4><<<grid, block, 0, st>>>(a);
        else if (vec == 2) k_sell<VT, CT, 2><<<grid, block, 0, st>>>(a);
        else k_sell<VT, CT, 1><<<grid, block, 0, st>>>(a);
        break;
    case 0: k_direct3<VT, CT><<<grid, block, 0, st>>>(a); break;
    case 7: k_warp_row<VT, CT><<<grid, block, 0, st>>>(a); break;
    case 5: k_long_row<VT, CT><<<grid, block, 0, st>>>(a); break;
    case 4: k_smem_tlb<VT, CT><<<grid, block, smem, st>>>(a); break;
    case 3: k_smem3<VT, CT><<<grid, block, smem, st>>>(a); break;
    case 6: k_smem_wlb<VT, CT><<<grid, block, smem, st>>>(a); break;
    case 8:
    case 9:
        // TLB sizes 4 / 8 / 16 / 32 with 32-bit columns run the specialised kernels; everything else the generic one
        if (csr5_specialised((int)a.tlb_size, (int)sizeof(CT), a.bits_word) && ((a.path & 2) == 0 || (a.path & 1) || a.y_mc))
            return launch_csr5(sizeof(VT) == 8, (int)sizeof(CT), (templ == 9 ? 1 : 0) | ((a.path & 1) ? 2 : 0) | (a.y_mc ? 6 : 0), a, grid.x, block.x, st);
        if (a.y_mc) return cudaErrorInvalidValue;
        if (templ == 8) k_csr5<VT, CT, false><<<grid, block, 0, st>>>(a);
        else k_csr5<VT, CT, true><<<grid, block, 0, st>>>(a);
        break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

template <class VT>
static cudaError_t launch_v(int templ, int col_width, const KArgs &a, dim3 grid, dim3 block, size_t smem, cudaStream_t st, int vec)
{
    switch (col_width)
    {
    case 1: return launch_vc<VT, unsigned char>(templ, a, grid, block, smem, st, vec);
    case 2: return launch_vc<VT, unsigned short>(templ, a, grid, block, smem, st, vec);
    case 4: return launch_vc<VT, unsigned int>(templ, a, grid, block, smem, st, vec);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_template(int templ, int val_is_f64, int col_width, const KArgs &a, unsigned grid, unsigned block, size_t smem, cudaStream_t st, int vec)
{
    if (templ == 12) return col_width == 8 ? launch_diag(val_is_f64, a, grid, block, st) : cudaErrorInvalidValue; // diagonal-value template
    if (templ == 11) // block-value template: r and c travel in the two bit-count fields the CSR5-like templates use
        return col_width == 4 ? launch_block_ell(val_is_f64, a.bits_row, a.bits_off, a, grid, block, st) : cudaErrorInvalidValue;
    if (val_is_f64) return launch_v<double>(templ, col_width, a, dim3(grid), dim3(block), smem, st, vec);
    return launch_v<float>(templ, col_width, a, dim3(grid), dim3(block), smem, st, vec);
}

template <class VT, class CT>
static cudaError_t smem_attr_vc(int templ, size_t smem)
{
    const void *f = NULL;
    switch (templ)
    {
    case 4: f = (const void *)k_smem_tlb<VT, CT>; break;
    case 3: f = (const void *)k_smem3<VT, CT>; break;
    case 6: f = (const void *)k_smem_wlb<VT, CT>; break;
    default: return cudaSuccess;
    }
    return cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

// opt in to more than 48 KB of dynamic shared memory for the shared-memory family
cudaError_t allow_dynamic_smem(int templ, int val_is_f64, int col_width, size_t smem)
{
    if (smem <= 48 * 1024) return cudaSuccess;
#define ASP_SMEM_CASE(VT)                                                      \
    switch (col_width)                                                         \
    {                                                                          \
    case 1: return smem_attr_vc<VT, unsigned char>(templ, smem);               \
    case 2: return smem_attr_vc<VT, unsigned short>(templ, smem);              \
    case 4: return smem_attr_vc<VT, unsigned int>(templ, smem);                \
    default: return cudaErrorInvalidValue;                                     \
    }
    if (val_is_f64)
    {
        ASP_SMEM_CASE(double)
    }
    ASP_SMEM_CASE(float)
#undef ASP_SMEM_CASE
}

} // namespace asp
