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
// Barrier of the ranks of one NVLink multicast group, as a kernel on the stream that carries the SpMV:
// every rank announces `epoch` in its own slot of a small symmetric flag array (one multicast store reaches
// all replicas) and then waits until every slot of its LOCAL replica has reached `epoch`. The announcing
// thread first issues a system-scope fence, so everything this GPU stored before the barrier (the rows it
// published from the kernels launched earlier on the stream) is visible to a peer that sees the flag.
//
// The wait is bounded: after `max_polls` polls of a slot the thread records 1 + the slot it gave up on in
// *status and returns, so a rank that never arrives costs a second or two, not a hung GPU. Ranks live on
// different GPUs; two ranks of one group must never share a GPU (nothing guarantees that kernels that wait
// on one another run at the same time).
__global__ void __launch_bounds__(32) k_rank_barrier(const unsigned *flags_local, unsigned *flags_mc, int rank, int world, unsigned epoch,
                                                     unsigned *status, unsigned max_polls)
{
    if (threadIdx.x == 0)
    {
        __threadfence_system();
        asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(flags_mc + rank), "r"(epoch) : "memory");
    }
    if ((int)threadIdx.x < world)
    {
        unsigned seen = 0, polls = 0;
        for (;;)
        {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags_local + threadIdx.x) : "memory");
            if ((int)(seen - epoch) >= 0) break; // (wrap-safe comparison of epochs)
            if (++polls >= max_polls)
            {
                atomicExch(status, 1u + threadIdx.x);
                break;
            }
            __nanosleep(200);
        }
    }
    __syncwarp();
    __threadfence_system();
}
} // namespace

extern "C" asp_status asp_rank_barrier(const void *flags_local, void *flags_multicast, int rank, int world, unsigned epoch, void *status_u32, unsigned max_polls,
                                       void *stream)
{
    if (!flags_local || !flags_multicast || !status_u32 || world < 1 || world > 32 || rank < 0 || rank >= world) return ASP_ERR_INVALID_ARG;
    if (max_polls == 0) max_polls = 4000000u; // about a second or two
    k_rank_barrier<<<1, 32, 0, (cudaStream_t)stream>>>((const unsigned *)flags_local, (unsigned *)flags_multicast, rank, world, epoch, (unsigned *)status_u32, max_polls);
    return cudaGetLastError() == cudaSuccess ? ASP_OK : ASP_ERR_CUDA;
}

extern "C" asp_status asp_multicast_store(const void *src, void *multicast_dst, size_t bytes, void *stream, int ctas)
{
    if (bytes == 0) return ASP_OK;
    if (!src || !multicast_dst || (bytes & 3) != 0 || (((uintptr_t)src ^ (uintptr_t)multicast_dst) & 15) != 0 || ((uintptr_t)src & 3) != 0) return ASP_ERR_INVALID_ARG;
    if (ctas <= 0) ctas = 32;
    k_mc_store<<<ctas, 512, 0, (cudaStream_t)stream>>>((const unsigned *)src, (unsigned *)multicast_dst, bytes / 4);
    return cudaGetLastError() == cudaSuccess ? ASP_OK : ASP_ERR_CUDA;
}
