// One-to-all store of a finished slice of y through an NVLink multicast address (NVSwitch replicates
// the stores to every GPU bound to the multicast object, the issuing GPU included): the slice leaves
// its owner once, however many peers there are. Used by the sharded repeated SpMV, where the owner of
// a row block publishes its part of the next x to all ranks.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/asp_b200.h"

namespace
{
__device__ __forceinline__ void mc_store4(void *mc, uint4 v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)),
                 "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}
__device__ __forceinline__ void mc_store1(void *mc, unsigned v)
{
    asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc), "f"(__uint_as_float(v)) : "memory");
}

// words: 32-bit units. src (local memory) and mc (multicast address of the same offset in the
// symmetric buffer) have the same alignment modulo 16 bytes; the ragged head and tail go as scalars.
__global__ void __launch_bounds__(512) k_mc_store(const unsigned *__restrict__ src, unsigned *mc, size_t words)
{
    const size_t head = ((16 - ((uintptr_t)src & 15)) & 15) / 4 < words ? ((16 - ((uintptr_t)src & 15)) & 15) / 4 : words;
    const size_t body = (words - head) / 4; // 16-byte units
    const size_t tail0 = head + body * 4;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthr = (size_t)gridDim.x * blockDim.x;
    if (tid < head) mc_store1(mc + tid, src[tid]);
    const uint4 *s4 = reinterpret_cast<const uint4 *>(src + head);
    unsigned *m4 = mc + head;
    for (size_t i = tid; i < body; i += nthr) mc_store4(m4 + i * 4, __ldcs(s4 + i));
    if (tid < words - tail0) mc_store1(mc + tail0 + tid, src[tail0 + tid]);
    __threadfence_system();
}
} // namespace

extern "C" asp_status asp_multicast_store(const void *src, void *multicast_dst, size_t bytes, void *stream, int ctas)
{
    if (bytes == 0) return ASP_OK;
    if (!src || !multicast_dst || (bytes & 3) != 0 || (((uintptr_t)src ^ (uintptr_t)multicast_dst) & 15) != 0 || ((uintptr_t)src & 3) != 0) return ASP_ERR_INVALID_ARG;
    if (ctas <= 0) ctas = 32;
    k_mc_store<<<ctas, 512, 0, (cudaStream_t)stream>>>((const unsigned *)src, (unsigned *)multicast_dst, bytes / 4);
    return cudaGetLastError() == cudaSuccess ? ASP_OK : ASP_ERR_CUDA;
}
