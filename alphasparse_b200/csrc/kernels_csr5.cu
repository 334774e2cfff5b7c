// CSR5-like family (UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE and ..._WITH_WARP_REDUCE of the
// reference, unaligned_warp_reduce_same_TLB_size_op.cc:793-1258) specialised on the TLB size.
//
// The format: every thread owns S consecutive non-zeros regardless of row boundaries, stored
// warp-interleaved (element k of lane l of warp w at w*32*S + k*32 + l); a packed word per thread
// holds S row-start flags (MSB first), the number of following threads that continue this
// thread's last row, and the first row (relative to the warp's first row) that starts in the
// thread. The first non-zero of every warp carries a flag, so a warp's rows are the contiguous
// range R0 .. R0 + (#flags in the warp) - 1; only the first and the last of them can also receive
// sums from the neighbouring warps.
//
// What bounds this family on matrices with scattered columns is the rate at which an SM can look
// up cache lines for the x gathers (one line per clock), not DRAM. Everything else is therefore
// kept off that path: S is a compile-time constant (all index and value loads of a thread are in
// flight before the first gather, the walk over the flags is straight-line predicated code, no
// branch per element), and with STAGE the row sums of a warp are collected in shared memory and
// written as one contiguous run (two `red` per warp for the shared end rows, coalesced stores for
// the rest) instead of one scattered 4-byte store per row.
//
// PUBLISH (sharded repeated SpMV): the contiguous run goes out through an NVLink multicast
// address with multimem.st, so a rank's rows of the next x reach every GPU from inside the SpMV
// kernel, warp by warp, while the other warps still compute. The two end rows of each warp are
// accumulated locally with `red` and published afterwards by k_publish_rows.
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernel_args.h"
#include "kernels.h"

namespace asp
{
typedef unsigned long long u64;
typedef unsigned int u32;

namespace
{
__device__ __forceinline__ u64 mload5(const void *p, int width, u64 i)
{
    switch (width)
    {
    case 1: return __ldg((const unsigned char *)p + i);
    case 2: return __ldg((const unsigned short *)p + i);
    case 4: return __ldg((const unsigned int *)p + i);
    default: return __ldg((const u64 *)p + i);
    }
}
__device__ __forceinline__ u64 mget5(const Meta &m, u64 i)
{
    switch (m.kind)
    {
    case MK_ARRAY: return mload5(m.p, m.width, i);
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
// row of y for relative row r of the sub-matrix
__device__ __forceinline__ u64 row_of(const KArgs &a, u64 r)
{
    if (a.sort_kind == 1) return mget5(a.perm, r + a.first_row);
    if (a.sort_kind == 2) return mget5(a.perm, r) + a.first_row;
    return r + a.first_row;
}

template <class CT>
__device__ __forceinline__ u32 ld_col(const CT *p)
{
    if constexpr (sizeof(CT) == 4)
    {
        u32 v;
        asm volatile("ld.global.cs.u32 %0, [%1];" : "=r"(v) : "l"(p));
        return v;
    }
    else
    {
        unsigned short v;
        asm volatile("ld.global.cs.u16 %0, [%1];" : "=h"(v) : "l"(p));
        return v;
    }
}
__device__ __forceinline__ float ld_val(const float *p)
{
    float v;
    asm volatile("ld.global.cs.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ double ld_val(const double *p)
{
    double v;
    asm volatile("ld.global.cs.f64 %0, [%1];" : "=d"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_x(const float *p)
{
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ double ld_x(const double *p)
{
    double v;
    asm volatile("ld.global.nc.f64 %0, [%1];" : "=d"(v) : "l"(p));
    return v;
}

// one value to every GPU bound to the multicast object that `mc` addresses
__device__ __forceinline__ void mc_store(float *mc, float v)
{
    asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc), "f"(v) : "memory");
}
__device__ __forceinline__ void mc_store(double *mc, double v)
{
    asm volatile("multimem.st.relaxed.sys.global.f64 [%0], %1;" ::"l"(mc), "d"(v) : "memory");
}
__device__ __forceinline__ void mc_store4(float *mc, float a, float b, float c, float d)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <class VT>
__device__ __forceinline__ void put(VT *y, u64 row, VT v, bool atomic)
{
    if (atomic)
        atomicAdd(y + row, v); // result unused: red.global.add
    else
        y[row] = v;
}

// MODE bit 0: WARP_FAST (second CSR5-like template: a warp that lies inside one row takes a butterfly
// reduction), bit 1: STAGE (row sums through shared memory, contiguous write-out), bit 2: PUBLISH
// (write-out through the multicast address; implies STAGE). B: elements per load batch. BRANCHY: the walk
// over the row-start flags branches per flagged element instead of running predicated straight-line code.
template <class VT, class CT, int S, int MODE, int B, bool BRANCHY>
__global__ void __launch_bounds__(256) k_csr5s(const KArgs a)
{
    constexpr bool WARP_FAST = (MODE & 1) != 0, STAGE = (MODE & 2) != 0, PUBLISH = (MODE & 4) != 0;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const VT *__restrict__ val = (const VT *)a.val;
    const CT *__restrict__ col = (const CT *)a.col;
    const VT *__restrict__ x = (const VT *)a.x + a.first_col;
    VT *__restrict__ y = (VT *)a.y;
    VT *__restrict__ ymc = (VT *)a.y_mc;
    const u32 lane = threadIdx.x & 31;
    const int fshift = a.bits_word - S; // the S flags are the top bits of the word
    const u64 rmask = (1ull << a.bits_row) - 1, omask = (1ull << a.bits_off) - 1;
    const bool all_atomic = a.atomic != 0;
    // staging area of this warp: the first `cap` rows a warp produces go through it, later ones straight out
    const u32 cap = STAGE ? (u32)a.stage_cap : 0u;
    VT *stage = STAGE ? reinterpret_cast<VT *>(smem_raw) + (size_t)(threadIdx.x >> 5) * cap : nullptr;
    const u64 wstride = ((u64)gridDim.x * blockDim.x) >> 5;

    // a finished row sum that does not go through the staging area
    auto out = [&](u64 rel_row, VT v, bool atomic) {
        const u64 r = row_of(a, rel_row);
        if (atomic) atomicAdd(y + r, v); // result unused: red.global.add
        else if (PUBLISH) mc_store(ymc + r, v);
        else y[r] = v;
    };

    for (u64 w = ((u64)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < a.n_units; w += wstride)
    {
        const u64 R0 = mget5(a.m[MS_ROW_OF_UNIT], w);
        const u64 nz0 = w * (32 * S) + lane;
        if (WARP_FAST)
        {
            const u64 R1 = (w + 1 < (u64)a.warps_first_row_len) ? mget5(a.m[MS_ROW_OF_UNIT], w + 1) : R0 + 1;
            if (R0 == R1)
            {
                VT s = 0;
#pragma unroll
                for (int k0 = 0; k0 < S; k0 += B)
                {
                    u32 c[B];
                    VT v[B], xv[B];
#pragma unroll
                    for (int u = 0; u < B; u++) c[u] = ld_col(col + nz0 + 32 * (k0 + u));
#pragma unroll
                    for (int u = 0; u < B; u++) v[u] = ld_val(val + nz0 + 32 * (k0 + u));
#pragma unroll
                    for (int u = 0; u < B; u++) xv[u] = ld_x(x + c[u]);
#pragma unroll
                    for (int u = 0; u < B; u++) s += v[u] * xv[u];
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0) atomicAdd(y + row_of(a, R0), s);
                continue;
            }
        }
        const u64 meta = mload5(a.m[MS_COMBINE].p, a.m[MS_COMBINE].width, w * 32 + lane);
        const u32 frow = (u32)(meta & rmask);
        const u32 roff = (u32)((meta >> a.bits_row) & omask);
        // bit k of F: element k of this thread starts a row
        const u32 F = __brev((u32)(meta >> fshift)) >> (32 - S);
        u32 yo = frow;
        bool seen = false;
        VT sum = 0, tail = 0;
        // (the batch loop stays rolled: unrolling it for S = 32 quadruples the code without gaining anything)
#pragma unroll 1
        for (int k0 = 0; k0 < S; k0 += B)
        {
            u32 c[B];
            VT p[B], xv[B];
#pragma unroll
            for (int u = 0; u < B; u++) c[u] = ld_col(col + nz0 + 32 * (k0 + u));
#pragma unroll
            for (int u = 0; u < B; u++) p[u] = ld_val(val + nz0 + 32 * (k0 + u));
#pragma unroll
            for (int u = 0; u < B; u++) xv[u] = ld_x(x + c[u]);
#pragma unroll
            for (int u = 0; u < B; u++) p[u] *= xv[u];
#pragma unroll
            for (int u = 0; u < B; u++)
            {
                const bool f = (F >> (k0 + u)) & 1u;
                if (BRANCHY)
                {
                    if (f)
                    {
                        if (seen)
                        {
                            // a row that starts and ends inside this thread; only the warp's very first row can
                            // also receive sums from the previous warp
                            if (STAGE && yo < cap) stage[yo] = sum;
                            else out(R0 + yo, sum, all_atomic || (lane == 0 && yo == frow));
                            yo++;
                        }
                        else
                            tail = sum;
                        seen = true;
                        sum = 0;
                    }
                    sum += p[u];
                }
                else
                {
                    // straight-line walk: a row that ends inside the thread is emitted under a predicate
                    const bool e = f && seen;
                    if (e)
                    {
                        if (STAGE && yo < cap) stage[yo] = sum;
                        else out(R0 + yo, sum, all_atomic || (lane == 0 && yo == frow));
                    }
                    yo += e ? 1u : 0u;
                    tail = (f && !seen) ? sum : tail;
                    seen = seen || f;
                    sum = f ? p[u] : sum + p[u];
                }
            }
        }
        if (!seen) tail = sum;
        // suffix scan of the tails, segmented at threads that start a row: afterwards lane j holds the
        // sum of tail[j..] up to the lane before the next row-starting lane
        const u32 heads = __ballot_sync(0xffffffffu, seen);
        VT sc = tail;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1)
        {
            const VT o = __shfl_down_sync(0xffffffffu, sc, d);
            const bool same = (lane + d < 32) && (((heads >> lane) & ((1u << d) - 1u)) == 0u);
            if (same) sc += o;
        }
        VT extra = __shfl_down_sync(0xffffffffu, sc, 1);
        if (lane == 31) extra = 0;
        if (seen)
        {
            // the last row this thread starts; it is the warp's last row when no later lane starts one
            if (STAGE && yo < cap) stage[yo] = sum + extra;
            else out(R0 + yo, sum + extra, all_atomic || (lane == 0 && yo == frow) || (lane + roff == 31));
        }
        if (!STAGE) continue;
        // ---- staged write-out: rows R0 .. R0 + min(nrows, cap) - 1 are in stage[]
        const u32 last_head = 31 - __clz(heads); // heads has bit 0 set: every warp starts with a flag
        const u32 nrows = __shfl_sync(0xffffffffu, yo, last_head) + 1;
        const u32 nst = nrows < cap ? nrows : cap;
        __syncwarp();
        if (all_atomic)
        {
            for (u32 j = lane; j < nst; j += 32) atomicAdd(y + row_of(a, R0 + j), stage[j]);
        }
        else
        {
            // the warp's first and last row may continue in the neighbouring warps
            if (lane == 0) atomicAdd(y + row_of(a, R0), stage[0]);
            if (lane == 1 && nrows > 1 && nrows <= cap) atomicAdd(y + row_of(a, R0 + nrows - 1), stage[nrows - 1]);
            const u32 jend = nrows <= cap ? nrows - 1 : cap; // one past the last staged row that is not an end row
            if (PUBLISH && a.sort_kind != 0)
            {
                // permuted rows: one multicast store per row (a stable partition keeps them ascending)
                for (u32 j = 1 + lane; j < jend; j += 32) mc_store(ymc + row_of(a, R0 + j), stage[j]);
            }
            else if (PUBLISH)
            {
                // unpermuted rows: y[first_row + R0 + j], and the same offset behind the multicast address
                VT *mc = ymc + a.first_row + R0;
                if constexpr (sizeof(VT) == 4)
                {
                    // 16-byte multicast stores where the run allows it
                    const u32 g0 = (u32)(((uintptr_t)(mc + 1) >> 2) & 3); // position of the first interior row inside its 16 bytes
                    const u32 n_in = jend > 1 ? jend - 1 : 0;
                    const u32 head = ((4 - g0) & 3) < n_in ? ((4 - g0) & 3) : n_in;
                    const u32 body = (n_in - head) >> 2;
                    if (lane < head) mc_store(mc + 1 + lane, stage[1 + lane]);
                    for (u32 q = lane; q < body; q += 32)
                    {
                        const u32 j = 1 + head + 4 * q;
                        mc_store4(mc + j, stage[j], stage[j + 1], stage[j + 2], stage[j + 3]);
                    }
                    const u32 t0 = 1 + head + 4 * body;
                    if (t0 + lane < jend) mc_store(mc + t0 + lane, stage[t0 + lane]);
                }
                else
                {
                    for (u32 j = 1 + lane; j < jend; j += 32) mc_store(mc + j, stage[j]);
                }
            }
            else
            {
                for (u32 j = 1 + lane; j < jend; j += 32) y[row_of(a, R0 + j)] = stage[j];
            }
        }
        __syncwarp(); // the next warp task of this warp reuses the staging area
    }
    if (PUBLISH) __threadfence_system();
}

template <class VT, class CT, int S, int B, bool BRANCHY>
cudaError_t launch_sb(int mode, const KArgs &a, unsigned grid, unsigned block, cudaStream_t st)
{
    const size_t smem = (mode & 2) ? (size_t)(block / 32) * a.stage_cap * sizeof(VT) : 0;
#define ASP_CSR5_MODE(M)                                                       \
    case M: k_csr5s<VT, CT, S, M, B, BRANCHY><<<grid, block, smem, st>>>(a); break;
    switch (mode)
    {
        ASP_CSR5_MODE(0)
        ASP_CSR5_MODE(1)
        ASP_CSR5_MODE(2)
        ASP_CSR5_MODE(3)
        ASP_CSR5_MODE(6)
        ASP_CSR5_MODE(7)
    default: return cudaErrorInvalidValue;
    }
#undef ASP_CSR5_MODE
    return cudaGetLastError();
}

template <class VT, class CT, int S>
cudaError_t launch_s(int mode, const KArgs &a, unsigned grid, unsigned block, cudaStream_t st)
{
    // Load batches, measured on a power-law matrix with random columns and on R-MAT: 8 elements in flight per
    // thread are best when rows go straight out (more CTAs fit), 16 with the staged write-out; a branch per
    // flagged element never beat the predicated walk by more than 1 %.
    if (mode & 2) return launch_sb<VT, CT, S, (S < 16 ? S : 16), false>(mode, a, grid, block, st);
    return launch_sb<VT, CT, S, (S < 8 ? S : 8), false>(mode, a, grid, block, st);
}

template <class VT, class CT>
cudaError_t launch_vc5(int S, int mode, const KArgs &a, unsigned grid, unsigned block, cudaStream_t st)
{
    switch (S)
    {
    case 4: return launch_s<VT, CT, 4>(mode, a, grid, block, st);
    case 8: return launch_s<VT, CT, 8>(mode, a, grid, block, st);
    case 16: return launch_s<VT, CT, 16>(mode, a, grid, block, st);
    case 32: return launch_s<VT, CT, 32>(mode, a, grid, block, st);
    default: return cudaErrorInvalidValue;
    }
}

// ---- the end rows of every warp (sharded repeated SpMV) ----------------------------------------
// rows[i]: global row of y that some warp accumulates with `red`. Before the SpMV kernel they are cleared
// (locally); after it they hold their totals and are sent to every GPU.
template <class VT>
__global__ void __launch_bounds__(256) k_zero_rows(VT *__restrict__ y, const u32 *__restrict__ rows, u64 n)
{
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (u64)gridDim.x * blockDim.x) y[rows[i]] = 0;
}
template <class VT>
__global__ void __launch_bounds__(256) k_publish_rows(const VT *__restrict__ y, VT *y_mc, const u32 *__restrict__ rows, u64 n)
{
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (u64)gridDim.x * blockDim.x)
    {
        const u32 r = rows[i];
        mc_store(y_mc + r, y[r]);
    }
    __threadfence_system();
}
} // namespace

bool csr5_specialised(int tlb_size, int col_width, int bits_word)
{
    return (tlb_size == 4 || tlb_size == 8 || tlb_size == 16 || tlb_size == 32) && col_width == 4 && bits_word - tlb_size >= 0;
}

cudaError_t launch_csr5(int val_is_f64, int col_width, int mode, const KArgs &a, unsigned grid, unsigned block, cudaStream_t st)
{
    const int S = (int)a.tlb_size;
    if (a.stage_cap <= 0) mode &= ~2; // no staging area configured: rows go straight out
    if ((mode & 4) && !(mode & 2)) return cudaErrorInvalidValue;
    if (col_width != 4) return cudaErrorInvalidValue;
    if (val_is_f64) return launch_vc5<double, unsigned int>(S, mode, a, grid, block, st);
    return launch_vc5<float, unsigned int>(S, mode, a, grid, block, st);
}

cudaError_t launch_zero_rows(int val_is_f64, void *y, const unsigned *rows, unsigned long long n, cudaStream_t st)
{
    if (n == 0) return cudaSuccess;
    const unsigned grid = (unsigned)((n + 255) / 256 < 1024 ? (n + 255) / 256 : 1024);
    if (val_is_f64) k_zero_rows<double><<<grid, 256, 0, st>>>((double *)y, rows, n);
    else k_zero_rows<float><<<grid, 256, 0, st>>>((float *)y, rows, n);
    return cudaGetLastError();
}

cudaError_t launch_publish_rows(int val_is_f64, const void *y, void *y_mc, const unsigned *rows, unsigned long long n, cudaStream_t st)
{
    if (n == 0) return cudaSuccess;
    const unsigned grid = (unsigned)((n + 255) / 256 < 256 ? (n + 255) / 256 : 256);
    if (val_is_f64) k_publish_rows<double><<<grid, 256, 0, st>>>((const double *)y, (double *)y_mc, rows, n);
    else k_publish_rows<float><<<grid, 256, 0, st>>>((const float *)y, (float *)y_mc, rows, n);
    return cudaGetLastError();
}

} // namespace asp
