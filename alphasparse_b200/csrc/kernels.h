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
// CSR5-like family specialised on the TLB size (kernels_csr5.cu). mode: bit 0 = the second template's whole-warp
// fast path, bit 1 = staged contiguous write-out, bit 2 = write-out through KArgs::y_mc (needs bit 1).
bool csr5_specialised(int tlb_size, int col_width, int bits_word);
cudaError_t launch_csr5(int val_is_f64, int col_width, int mode, const KArgs &a, unsigned grid, unsigned block, cudaStream_t st);
// block-value template (kernels_block.cu): blocked ELL over dense r x c blocks; KArgs::n_tlb = padded block rows,
// tlb_size = block slots per block row, effective = rows of the sub-matrix
bool block_ell_supported(int r, int c);
cudaError_t launch_block_ell(int val_is_f64, int r, int c, const KArgs &a, unsigned grid, unsigned block, cudaStream_t st);
// diagonal-value template (kernels_diag.cu): KArgs::col = u64 offsets biased by the column count, n_tlb = padded rows,
// tlb_size = diagonals, effective = rows, n_units = columns of the sub-matrix
cudaError_t launch_diag(int val_is_f64, const KArgs &a, unsigned grid, unsigned block, cudaStream_t st);
// end rows of the warps (the rows the CSR5-like kernel accumulates with `red`): cleared before, published after
cudaError_t launch_zero_rows(int val_is_f64, void *y, const unsigned *rows, unsigned long long n, cudaStream_t st);
cudaError_t launch_publish_rows(int val_is_f64, const void *y, void *y_mc, const unsigned *rows, unsigned long long n, cudaStream_t st);
} // namespace asp
#endif
