// Block-value template (no counterpart among the reference's ten reduce templates): blocked ELL over
// dense R x C blocks, produced by the `block_value R C` operator.
//
// The reference's formats store one column index per non-zero. A matrix assembled from small dense blocks
// (finite elements with several unknowns per node: 3 x 3 blocks for 3-D elasticity) repeats that index R*C
// times per block and gathers every x value R times. Here a block carries ONE block-column index, its R*C
// values, and each thread gathers the C values of x once per block:
//   bytes per stored non-zero  12 -> 8 + 4 / (R*C)   (fp64, 3 x 3: 8.44)
//   gathers per stored non-zero 1 -> 1 / R
//
// Layout (NB = block rows padded to a multiple of 2, W = blocks per block row, padded with zero blocks):
//   block column of slot k of block row b     idx[k * NB + b]
//   element (i, j) of that block              val[((k * R + i) * C + j) * NB + b]
// so that the 2 block rows of a thread are adjacent: 16-byte loads of values, 8-byte loads of indices, all
// coalesced across the warp. A thread owns two block rows (2 R rows of y, stored as 16-byte vectors).
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
template <class VT>
struct Pair;
template <>
struct Pair<double>
{
    typedef double2 type;
};
template <>
struct Pair<float>
{
    typedef float2 type;
};

// two adjacent values, streamed (touched once per SpMV)
__device__ __forceinline__ void ld_pair(const double *p, double &a, double &b)
{
    asm volatile("ld.global.cs.v2.f64 {%0, %1}, [%2];" : "=d"(a), "=d"(b) : "l"(p));
}
__device__ __forceinline__ void ld_pair(const float *p, float &a, float &b)
{
    asm volatile("ld.global.cs.v2.f32 {%0, %1}, [%2];" : "=f"(a), "=f"(b) : "l"(p));
}
__device__ __forceinline__ void ld_idx2(const u32 *p, u32 &a, u32 &b)
{
    asm volatile("ld.global.cs.v2.u32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "l"(p));
}
__device__ __forceinline__ double ld_xv(const double *p)
{
    double v;
    asm volatile("ld.global.nc.f64 %0, [%1];" : "=d"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_xv(const float *p)
{
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// U block slots per trip: their index pairs, then their value pairs, then their x values are issued as one batch
template <class VT, int R, int C, int U>
__global__ void __launch_bounds__(128) k_block_ell(const KArgs a)
{
    const VT *__restrict__ val = (const VT *)a.val;
    const u32 *__restrict__ idx = (const u32 *)a.col;
    const VT *__restrict__ x = (const VT *)a.x + a.first_col;
    VT *__restrict__ y = (VT *)a.y + a.first_row;
    const u64 NB = a.n_tlb;      // padded block rows (even)
    const u32 W = a.tlb_size;    // block slots per block row
    const u64 rows = a.effective; // rows of the sub-matrix (the last block row may be partial)
    const u64 stride = (u64)gridDim.x * blockDim.x;
    for (u64 g = (u64)blockIdx.x * blockDim.x + threadIdx.x; 2 * g < NB; g += stride)
    {
        const u64 b0 = 2 * g;
        VT acc[2][R];
#pragma unroll
        for (int v = 0; v < 2; v++)
#pragma unroll
            for (int i = 0; i < R; i++) acc[v][i] = 0;
        const u32 *ip = idx + b0;
        const VT *vp = val + b0;
        u32 k = 0;
        for (; k + U <= W; k += U)
        {
            u32 bc[U][2];
            VT v[U][R * C][2], xv[U][2][C];
#pragma unroll
            for (int u = 0; u < U; u++) ld_idx2(ip + (u64)(k + u) * NB, bc[u][0], bc[u][1]);
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int e = 0; e < R * C; e++) ld_pair(vp + ((u64)(k + u) * (R * C) + e) * NB, v[u][e][0], v[u][e][1]);
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int s = 0; s < 2; s++)
#pragma unroll
                    for (int j = 0; j < C; j++) xv[u][s][j] = ld_xv(x + (u64)bc[u][s] * C + j);
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int s = 0; s < 2; s++)
#pragma unroll
                    for (int i = 0; i < R; i++)
#pragma unroll
                        for (int j = 0; j < C; j++) acc[s][i] += v[u][i * C + j][s] * xv[u][s][j];
        }
        for (; k < W; k++)
        {
            u32 bc[2];
            ld_idx2(ip + (u64)k * NB, bc[0], bc[1]);
#pragma unroll
            for (int i = 0; i < R; i++)
#pragma unroll
                for (int j = 0; j < C; j++)
                {
                    VT v0, v1;
                    ld_pair(vp + ((u64)k * (R * C) + i * C + j) * NB, v0, v1);
                    acc[0][i] += v0 * ld_xv(x + (u64)bc[0] * C + j);
                    acc[1][i] += v1 * ld_xv(x + (u64)bc[1] * C + j);
                }
        }
        // rows b0*R .. b0*R + 2R - 1 are contiguous in y
        const u64 r0 = b0 * R;
        if (r0 + 2 * R <= rows && ((2 * R * sizeof(VT)) % 16 == 0) && (((uintptr_t)(y + r0)) & 15) == 0)
        {
            typedef typename Pair<VT>::type P2;
            constexpr int PER = 16 / sizeof(VT); // values per 16-byte store
            VT flat[2 * R];
#pragma unroll
            for (int s = 0; s < 2; s++)
#pragma unroll
                for (int i = 0; i < R; i++) flat[s * R + i] = acc[s][i];
            if constexpr (PER == 2)
            {
#pragma unroll
                for (int q = 0; q < R; q++)
                {
                    P2 t;
                    t.x = flat[2 * q];
                    t.y = flat[2 * q + 1];
                    *reinterpret_cast<P2 *>(y + r0 + 2 * q) = t;
                }
            }
            else
            {
#pragma unroll
                for (int q = 0; q + 4 <= 2 * R; q += 4) *reinterpret_cast<float4 *>(y + r0 + q) = make_float4(flat[q], flat[q + 1], flat[q + 2], flat[q + 3]);
#pragma unroll
                for (int q = (2 * R) / 4 * 4; q < 2 * R; q++) y[r0 + q] = flat[q];
            }
        }
        else
        {
#pragma unroll
            for (int s = 0; s < 2; s++)
#pragma unroll
                for (int i = 0; i < R; i++)
                    if (r0 + s * R + i < rows) y[r0 + s * R + i] = acc[s][i];
        }
    }
}

template <class VT>
cudaError_t launch_rc(int r, int c, const KArgs &a, unsigned grid, unsigned block, cudaStream_t st)
{
    if (r == 3 && c == 3) k_block_ell<VT, 3, 3, 2><<<grid, block, 0, st>>>(a);
    else if (r == 2 && c == 2) k_block_ell<VT, 2, 2, 4><<<grid, block, 0, st>>>(a);
    else if (r == 4 && c == 4) k_block_ell<VT, 4, 4, 1><<<grid, block, 0, st>>>(a);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}
} // namespace

bool block_ell_supported(int r, int c) { return (r == 2 && c == 2) || (r == 3 && c == 3) || (r == 4 && c == 4); }

cudaError_t launch_block_ell(int val_is_f64, int r, int c, const KArgs &a, unsigned grid, unsigned block, cudaStream_t st)
{
    if (block > 128) return cudaErrorInvalidValue;
    return val_is_f64 ? launch_rc<double>(r, c, a, grid, block, st) : launch_rc<float>(r, c, a, grid, block, st);
}

} // namespace asp
