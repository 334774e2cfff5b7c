// Kernel-side view of one uploaded template ("plan"): device pointers, metadata references
// (array or closed form) and the scalars the reference baked into emitted source as literals.
#ifndef ASP_KERNEL_ARGS_H
#define ASP_KERNEL_ARGS_H

#include <stdint.h>

namespace asp
{

enum MetaKind : int
{
    MK_ARRAY = 0,
    MK_LINEAR = 1,
    MK_CONSTANT = 2,
    MK_BRANCH = 3,
    MK_CYCLE_LINEAR = 4,
    MK_CYCLE_INCREASE = 5
};

// One metadata array of a template, or the closed form that replaces it
// (arr_optimization.cc of the reference: linear / constant / branch / cycle-linear / cycle-increase).
// Closed forms are always evaluated in 64 bits: the reference evaluates them in the array's
// narrowed type, which can wrap for masked-off ids.
struct Meta
{
    const void *p;
    unsigned long long coef, icpt, cycle;
    unsigned long long bval[5];
    unsigned long long bhi[5];
    int kind;
    int width; // bytes per element when kind == MK_ARRAY
    int nb;
    int pad_;
};

// slots of KArgs::m, by template
enum MetaSlot : int
{
    // ELL-like / SELL-like / 3-level direct (K1, K2, K3)
    MS_ROW_OF_TLB = 0,
    MS_BLK_THR = 1,     // block_begin_thread_index_offset
    MS_BLK_NZ = 2,      // block_nz_begin_offset
    MS_TLB_SIZE = 3,    // thread_block_size_in_block | thread_block_size_in_warp
    MS_BLK_WARP = 4,    // block_begin_warp_index_offset
    MS_WARP_THR = 5,    // warp_begin_thread_index_offset
    MS_WARP_NZ = 6,     // warp_nz_begin_offset | global_warp_nz_begin_offset | global_warp_block_first_nz
    // shared-memory family (K5, K6, K8)
    MS_ROW_OFF = 7,     // row_offset_in_thread_tmp_result | row_offset_in_warp_tmp_result
    MS_BLK_ROW = 8,     // block_first_row_index
    // warp / block per row chunk (K4, K7), CSR5-like (K9, K10)
    MS_ROW_OF_UNIT = 9, // global_row_index_of_warp_level_block | row_index_of_block_level_block | global_first_row_index_of_warp_level_block
    MS_COMBINE = 10,    // combine_meta_of_thread_level_block
    MS_COUNT = 11
};

struct KArgs
{
    const void *val;
    const void *col;
    const void *x;
    void *y;
    void *y_mc; // CSR5-like family in publish mode: NVLink multicast address of y (same offsets), else NULL
    Meta m[MS_COUNT];
    Meta perm; // row_index_before_sort
    unsigned long long first_row, first_col;
    unsigned long long n_units;   // #BLB | #WLB | #TLB depending on the template
    unsigned long long n_tlb;     // padded TLB count (k-stride of the ELL-like layout)
    unsigned long long effective; // effective_TLB_num | effective_WLB_num | effective_row_num
    unsigned int tlb_size;
    int atomic;
    int sort_kind;  // 0 none, 1 global (perm[row + first_row]), 2 local (perm[row] + first_row)
    int row_add;    // 1: add first_row to a host-permuted row map (not for global sort)
    int row_reduce; // thread_num_of_row_reduce
    int bits_word, bits_flag, bits_row, bits_off;
    int warps_first_row_len; // length of the WLB first-row array (K10 has a +1 sentinel)
    int stage_cap;           // CSR5-like, staged write-out: rows per warp that go through shared memory (the rest go straight out)
    int path;                // kernel-specific walk: SELL-like 0 = warp tasks when strips are equal, 1 = one CTA per strip;
                             // CSR5-like 1 = the row sums of a warp go through shared memory and out as one contiguous run
};

} // namespace asp
#endif
