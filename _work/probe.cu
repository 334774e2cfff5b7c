// Ceiling probe for the x gathers of SpMV: a kernel that does nothing but read an index vector
// (coalesced, streaming) and gather 4-byte values of a vector that fits L2 at those indices, eight
// independent gathers per thread in flight. Its rate bounds every SpMV kernel on a matrix whose
// columns are uniformly random, whatever the format: each non-zero costs one such gather.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/asp_b200.h"

namespace
{
template <int U>
__global__ void __launch_bounds__(512) k_probe_gather(const unsigned *__restrict__ idx, const float *__restrict__ x, float *__restrict__ out, size_t n)
{
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    float acc = 0.f;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + (U - 1) * stride < n; i += U * stride)
    {
        unsigned c[U];
#pragma unroll
        for (int u = 0; u < U; ++u) c[u] = __ldcs(idx + i + u * stride);
#pragma unroll
        for (int u = 0; u < U; ++u) acc += __ldg(x + c[u]);
    }
    for (; i < n; i += stride) acc += __ldg(x + __ldcs(idx + i));
    if (acc == 123.456f) out[0] = acc; // keeps the loads alive without a store per thread
}
} // namespace

extern "C" asp_status asp_probe_gather(const void *d_idx_u32, const void *d_x_f32, void *d_out_f32, size_t n_gathers, int threads, int ctas, int reps, void *stream,
                                       float *ms_per_pass)
{
    if (!d_idx_u32 || !d_x_f32 || !d_out_f32 || !ms_per_pass || threads <= 0 || threads > 512 || ctas <= 0 || reps <= 0) return ASP_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return ASP_ERR_CUDA;
    for (int w = 0; w < 3; ++w) k_probe_gather<8><<<ctas, threads, 0, st>>>((const unsigned *)d_idx_u32, (const float *)d_x_f32, (float *)d_out_f32, n_gathers);
    cudaEventRecord(e0, st);
    for (int r = 0; r < reps; ++r) k_probe_gather<8><<<ctas, threads, 0, st>>>((const unsigned *)d_idx_u32, (const float *)d_x_f32, (float *)d_out_f32, n_gathers);
    cudaEventRecord(e1, st);
    cudaError_t e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess || cudaGetLastError() != cudaSuccess) return ASP_ERR_CUDA;
    *ms_per_pass = ms / (float)reps;
    return ASP_OK;
}
