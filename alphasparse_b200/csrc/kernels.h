// Launch entry of the kernel families (kernels.cu); used by the C ABI only.
#ifndef ASP_KERNELS_H
#define ASP_KERNELS_H
#include <cuda_runtime.h>
#include "kernel_args.h"
namespace asp
{
// templ: asp_template_type; vec: TLBs handled per thread by the ELL-like / SELL-like families
cudaError_t launch_template(int templ, int val_is_f64, int col_width, const KArgs &a, unsigned grid, unsigned block, size_t smem, cudaStream_t st, int vec);
cudaError_t allow_dynamic_smem(int templ, int val_is_f64, int col_width, size_t smem);
} // namespace asp
#endif
