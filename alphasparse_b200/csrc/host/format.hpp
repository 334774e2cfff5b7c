// Host-side data model and format operators: the Operator Graph's nodes (dense-view sort /
// row division / compress, compressed-view row padding and BLB / WLB / TLB tiling) and the
// lowering of a tiled sub-matrix into the flat arrays of each reduce template.
//
// Outputs are bit-identical to the reference's host code (op_manager.cc, the init_* functions of
// the ten template files, arr_optimization.cc) -- same values, same narrowed element types, same
// closed forms -- but the implementation is CSR-based and O(nnz): the reference keeps COO row
// indices per non-zero, copies vectors by value and scans linearly for bins and blocks.
#ifndef ASP_HOST_FORMAT_HPP
#define ASP_HOST_FORMAT_HPP

#include <stdint.h>

#include <memory>
#include <string>
#include <vector>

#include "../../../include/asp_b200.h"

namespace asp
{
namespace host
{

typedef uint64_t u64;
typedef uint32_t u32;

// smallest unsigned type that holds `max_value` (find_most_suitable_data_type, op_manager.cc:1103)
int suitable_dtype(u64 max_value);
int dtype_bytes(int dt);

// a metadata array kept wide on the host, with the narrowed element type it will be stored in
struct IndexArr
{
    std::vector<u64> v;
    int dt = ASP_U8;
};

struct ClosedForm
{
    int kind = ASP_COMPRESS_NONE;
    u64 coef = 0, icpt = 0, cycle = 0;
    std::vector<u64> lo, hi, val;
};

// closed-form detectors (arr_optimization.cc:6-57, 81-105, 113-170, 206-260, 277-337)
bool detect_linear(const std::vector<u64> &a, ClosedForm &out);
bool detect_constant(const std::vector<u64> &a, ClosedForm &out);
bool detect_branch(const std::vector<u64> &a, ClosedForm &out);
bool detect_cycle_linear(const std::vector<u64> &a, u64 cycle, ClosedForm &out);
bool detect_cycle_increase(const std::vector<u64> &a, ClosedForm &out);

// one (ptr, dtype, size) triple of a template, in its final narrowed bytes
struct TemplateArray
{
    int role = 0; // asp_array_role
    int dt = ASP_U8;
    u64 len = 0;
    std::vector<uint8_t> bytes;           // owned storage ...
    std::shared_ptr<std::vector<uint8_t>> shared; // ... or storage shared between sub-matrices (global row permutation)
    ClosedForm comp;
    const uint8_t *data() const { return shared ? shared->data() : bytes.data(); }
};

// everything one template struct of the reference carries (see include/asp_b200.h: asp_plan_desc)
struct TemplateData
{
    int template_type = ASP_EMPTY_TEMPLATE;
    int val_dt = ASP_F32;
    u64 first_row = 0, first_col = 0, true_nnz = 0;
    u64 effective_num = 0, tlb_size = 0;
    int bits_word = 0, bits_flag = 0, bits_row = 0, bits_off = 0;
    bool is_atom_add = false;
    int sort_kind = ASP_SORT_NONE;
    u64 n_blb = 0, n_wlb = 0, n_tlb = 0;
    long tblock_num = 120, thread_num_in_block = 512, thread_num_of_row_reduce = 1; // DEFAULT_THREAD_* of global_config.json
    std::vector<TemplateArray> arrays;
    const TemplateArray *find(int role) const;
};

// values are only ever moved or zero-filled, never computed with: raw bytes + element size
struct ValBuf
{
    int es = 4; // 4: f32, 8: f64
    std::vector<uint8_t> b;
    u64 size() const { return b.size() / es; }
    void resize(u64 n) { b.assign(n * es, 0); }
};

// One level of the BLB -> WLB -> TLB tiling (index_of_compress_block_t of the reference,
// struct.hpp:60-125), restricted to the arrays later stages read.
struct Level
{
    u64 block_num = 0;
    IndexArr index;     // CSR over the next level (first child id), block_num + 1 entries
    IndexArr first_row; // relative to the parent block
    IndexArr row_num;
    IndexArr coo_begin; // BLB: absolute, block_num + 1 entries; WLB: relative to its BLB, block_num entries
    IndexArr coo_size;  // WLB: nnz of the block; TLB level: TLB size of each WLB
    bool built = false;
};

// compressed_block_t: one sub-matrix after COMPRESS, rows / columns relative to the block
struct CompressedBlock
{
    // dense-view bounds of the block (dense_block_table_item_t)
    u64 min_row = 0, max_row = 0, min_col = 0, max_col = 0;
    u64 begin_coo = 0, end_coo = 0;
    // compressed view; n_rows grows with COMPRESSED_ROW_PADDING
    u64 n_rows = 0;
    std::vector<u64> rowptr;
    std::vector<u32> col;
    ValBuf val;
    int row_dt = ASP_U8, col_dt = ASP_U8; // element types of read_index[0] / read_index[1]
    Level blb, wlb, tlb;
    bool tlb_is_nnz_div = false;  // read_index[4] built by sep_thread_level_acc_to_nnz
    IndexArr tlb_row_span;        // rows spanned per TLB (nnz-div only)
    bool share_row_with_other_block = false, share_row_with_other_warp = false, share_row_with_other_thread = false;
    // read_index[5] / padding_val_arr: padded arrays, row-major inside each WLB
    std::vector<u32> pad_col;
    ValBuf pad_val;
    bool padded = false;
    // block_value operator (not one of the reference's): the sub-matrix is to be stored as dense block_r x block_c blocks
    u64 block_r = 0, block_c = 0;
    // diag_value operator (not one of the reference's): DIA storage; the most diagonals it may take
    u64 diag_max = 0;

    int n_index() const { return 2 + (blb.built ? 1 : 0) + (wlb.built ? 1 : 0) + (tlb.built ? 3 : 0); }
    u64 nnz() const { return col.size(); }
};

// sparse_struct_t
struct Matrix
{
    u64 n_rows = 0, n_cols = 0, nnz = 0;
    int val_dt = ASP_F32;
    // dense view, CSR (rows are in sorted order after DENSE_ROW_COARSE_SORT)
    std::vector<u64> rowptr;
    std::vector<u32> col;
    ValBuf val;
    bool is_sorted = false;
    std::shared_ptr<std::vector<uint8_t>> sorted_row_index; // new -> old, narrowed to perm_dt
    int perm_dt = ASP_U8;
    std::vector<u64> perm; // wide copy of sorted_row_index
    bool is_blocked = false, is_compressed = false;
    std::vector<CompressedBlock> blocks; // block_coor_table
    struct BlockRange
    {
        u64 min_row, max_row, begin_coo, end_coo;
    };
    std::vector<BlockRange> ranges;
};

// ---- BEGIN_* nodes ---------------------------------------------------------------------------
// BEGIN_MEMORY_CACHE_INPUT_FILE: from CSR arrays (row offsets int64, column indices u32, values)
std::unique_ptr<Matrix> matrix_from_csr(u64 n_rows, u64 n_cols, const int64_t *indptr, const u32 *indices, const void *values, int val_dt);
std::unique_ptr<Matrix> relabel_by_column_count(const Matrix &m, bool empty_rows_last, std::vector<u32> &labels, u64 &n_active);
// BEGIN_INPUT_FILE: parse the `.mtx.coo` text grammar (struct.cc:92-174)
std::unique_ptr<Matrix> matrix_from_coo_file(const std::string &path, int val_dt, std::string &err);

// ---- dense-view operators --------------------------------------------------------------------
// DENSE_ROW_COARSE_SORT (total_dense_block_coarse_sort, op_manager.cc:5492): stable bucket sort by
// row-nnz bins, largest bin first. `step` = row_nnz_low_bound_step_size of the fixed strategy.
void dense_row_coarse_sort(Matrix &m, u64 step);
// DENSE_ROW_DIV with the exponential strategy (parameter_set_strategy.cc:542, graph_enumerate.cc:183)
std::vector<u64> row_div_position_exponential(const Matrix &m, u64 lowest, u64 highest, u64 rate);
// var_len_row_div (op_manager.cc:370)
void dense_row_div(Matrix &m, const std::vector<u64> &positions);
// COMPRESS (compress_dense_view, op_manager.cc:968)
void compress_dense_view(Matrix &m);

// ---- compressed-view operators ---------------------------------------------------------------
// COMPRESSED_ROW_PADDING (compress_block_end_block_multiple_padding, op_manager.cc:5735)
void row_padding(CompressedBlock &b, u64 multiple, u64 padding_row_length);
// COMPRESSED_TBLOCK_LEVEL_ROW_DIV (sep_tblock_level_row_csr, op_manager.cc:1270)
void sep_tblock_level_row_csr(CompressedBlock &b, const std::vector<u64> &rows_of_each_blb);
std::vector<u64> blb_rows_evenly(const CompressedBlock &b, u64 block_row_num);      // graph_enumerate.cc: row_block_size_of_a_sub_matrix_by_fixed_div
std::vector<u64> blb_rows_by_nnz_low_bound(const CompressedBlock &b, u64 nnz_low_bound); // graph_enumerate.cc: row_block_size_of_a_sub_matrix_by_nnz_low_bound
// COMPRESSED_TBLOCK_LEVEL_COL_DIV with the fixed strategy (one_row_sep_tblock_level_row_csr +
// sep_tblock_level_col_csr, op_manager.cc:1540,1797; col_block_size_of_each_row, graph_enumerate.cc:337)
void sep_tblock_level_col_fixed(CompressedBlock &b, u64 col_block_nnz);
// COMPRESSED_WARP_LEVEL_ROW_DIV (sep_warp_level_row_csr, op_manager.cc:1970); empty vectors = one WLB per BLB
void sep_warp_level_row_csr(CompressedBlock &b, const std::vector<std::vector<u64>> &rows_of_each_wlb_in_blb);
std::vector<std::vector<u64>> wlb_rows_evenly(const CompressedBlock &b, u64 rows);
// COMPRESSED_WARP_LEVEL_COL_DIV with the fixed strategy (one_row_sep_warp_level_row_csr +
// sep_warp_level_col_csr, op_manager.cc:2376,2416; col_block_size_of_each_row_without_block_merge)
void sep_warp_level_col_fixed(CompressedBlock &b, u64 col_block_nnz);
// COMPRESSED_THREAD_LEVEL_ROW_DIV / _COL_DIV (sep_thread_level_col_ell_with_padding, op_manager.cc:3105):
// tlb_size == 0 means "one TLB per row" (TLB size = the WLB's longest row)
void sep_thread_level_col_ell_with_padding(CompressedBlock &b, u64 tlb_size);
// COMPRESSED_THREAD_LEVEL_NNZ_DIV (sep_thread_level_acc_to_nnz, op_manager.cc:3807)
void sep_thread_level_acc_to_nnz(CompressedBlock &b, u64 tlb_nnz);
// execute_default_div_to_complete_each_level_blocking (default_auto_tuner.cc:384)
void complete_each_level_blocking(CompressedBlock &b);

// ---- templates: init_<template> + try_all_compress -------------------------------------------
// returns false and sets err when the tiling does not fit the template
bool init_template(const Matrix &m, size_t sub, int template_type, TemplateData &out, std::string &err);

} // namespace host
} // namespace asp
#endif
