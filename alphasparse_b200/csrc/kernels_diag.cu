// Diagonal-value template (no counterpart among the reference's ten reduce templates): DIA storage for matrices
// whose non-zeros lie on a few diagonals, produced by the `diag_value` operator.
//
// The reference's formats store a column index per non-zero even where the index is a closed form of the row:
// the 5-point Laplacian keeps 84 MB of indices that are row - n, row - 1, row, row + 1, row + n. Here a diagonal
// carries ONE offset; values are stored diagonal-major, val[d * NR + r] = A[r, r + off[d]] (zero where the
// diagonal leaves the matrix or the entry is absent), so that
//   bytes per stored non-zero  12 -> 8 (fp64), 8 -> 4 (fp32)
//   x is read as D contiguous, shifted runs instead of gathers.
// A thread owns V consecutive rows (16 bytes of values per diagonal); all loads of a diagonal batch are issued
// before the first use.
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernel_args.h"
#include "kernels.h"

namespace asp
{
typedef unsigned long long u64;
typedef long long i64;

namespace
{
template <class VT, int V>
__device__ __forceinline__ void ld_vals(const VT *p, VT (&v)[V])
{
    static_assert(sizeof(VT) * V == 16, "one 16-byte load");
    unsigned r[4];
    asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "l"(p));
    if constexpr (sizeof(VT) == 8)
    {
#pragma unroll
        for (int j = 0; j < V; j++)
        {
            const u64 w = ((u64)r[2 * j + 1] << 32) | r[2 * j];
            v[j] = *reinterpret_cast<const VT *>(&w);
        }
    }
    else
    {
#pragma unroll
        for (int j = 0; j < V; j++) v[j] = *reinterpret_cast<const VT *>(&r[j]);
    }
}

// offsets are stored biased by the column count (so that they are unsigned): off = stored - n_cols
template <class VT, int U>
__global__ void __launch_bounds__(256) k_diag(const KArgs a)
{
    constexpr int V = 16 / sizeof(VT);
    const VT *__restrict__ val = (const VT *)a.val;
    const u64 *__restrict__ offs = (const u64 *)a.col;
    const VT *__restrict__ x = (const VT *)a.x + a.first_col;
    VT *__restrict__ y = (VT *)a.y + a.first_row;
    const u64 NR = a.n_tlb;       // padded rows (multiple of V)
    const unsigned D = a.tlb_size; // diagonals
    const i64 rows = (i64)a.effective, ncols = (i64)a.n_units; // rows and columns of the sub-matrix
    const u64 stride = (u64)gridDim.x * blockDim.x;
    for (u64 g = (u64)blockIdx.x * blockDim.x + threadIdx.x; g * V < NR; g += stride)
    {
        const i64 r0 = (i64)(g * V);
        VT acc[V];
#pragma unroll
        for (int j = 0; j < V; j++) acc[j] = 0;
        unsigned d = 0;
        for (; d + U <= D; d += U)
        {
            VT v[U][V], xv[U][V];
            i64 off[U];
#pragma unroll
            for (int u = 0; u < U; u++) off[u] = (i64)__ldg(offs + d + u) - ncols;
#pragma unroll
            for (int u = 0; u < U; u++) ld_vals<VT, V>(val + (u64)(d + u) * NR + (u64)r0, v[u]);
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int j = 0; j < V; j++)
                {
                    const i64 c = r0 + j + off[u];
                    xv[u][j] = (c >= 0 && c < ncols) ? __ldg(x + c) : VT(0);
                }
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int j = 0; j < V; j++) acc[j] += v[u][j] * xv[u][j];
        }
        for (; d < D; d++)
        {
            VT v[V];
            const i64 off = (i64)__ldg(offs + d) - ncols;
            ld_vals<VT, V>(val + (u64)d * NR + (u64)r0, v);
#pragma unroll
            for (int j = 0; j < V; j++)
            {
                const i64 c = r0 + j + off;
                if (c >= 0 && c < ncols) acc[j] += v[j] * __ldg(x + c);
            }
        }
        if (r0 + V <= rows && (((uintptr_t)(y + r0)) & 15) == 0)
        {
            if constexpr (sizeof(VT) == 8) *reinterpret_cast<double2 *>(y + r0) = make_double2(acc[0], acc[1]);
            else *reinterpret_cast<float4 *>(y + r0) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        }
        else
        {
#pragma unroll
            for (int j = 0; j < V; j++)
                if (r0 + j < rows) y[r0 + j] = acc[j];
        }
    }
}
} // namespace

cudaError_t launch_diag(int val_is_f64, const KArgs &a, unsigned grid, unsigned block, cudaStream_t st)
{
    if (block > 256) return cudaErrorInvalidValue;
    if (val_is_f64) k_diag<double, 5><<<grid, block, 0, st>>>(a);
    else k_diag<float, 5><<<grid, block, 0, st>>>(a);
    return cudaGetLastError();
}

} // namespace asp
