// Test infrastructure (format oracle). NOT part of the product: only tests, the smoke check
// and the fixture generator run the binary built from this file.
//
// Links against the UNMODIFIED reference host sources (compiled where they lie) and drives
// them exactly the way the reference's own tuner does:
//   dense view   : add_a_exe_node_and_param_strategy_to_exe_dense_sub_graph +
//                  execute_dense_matrix_exe_graph_with_param_strategy   (default_auto_tuner.cc:2073)
//   compressed   : add_a_exe_node_and_param_strategy_to_exe_compressed_sub_graph +
//                  execute_sub_matrix_exe_graph_with_param_strategy     (default_auto_tuner.cc:2034)
//   completion   : execute_default_div_to_complete_each_level_blocking  (default_auto_tuner.cc:384)
//   template     : init_<template>(builder, sub) + try_all_compress     (e.g. direct_atom_op_warp_compress.cc:6,1719)
// and then writes every array of every template (name, dtype, length, raw bytes, closed-form
// compression kind and coefficients, scalars, flags) into <out>/manifest.json + <out>/arrays.bin.
//
// Usage: ref_dump <matrix.mtx.coo> <spec-file> <out-dir>
// Spec file, one directive per line ('#' comments):
//   dtype float|double
//   dense sort <step>
//   dense rowdiv_exp <lowest> <highest> <rate>
//   dense compress
//   sub <id|all> row_padding <multiple> <row_len>
//   sub <id|all> blb_row_evenly <rows> | blb_row_nnz <nnz_low_bound> | blb_col_fixed <nnz>
//   sub <id|all> wlb_row_evenly <rows> | wlb_col_fixed <nnz>
//   sub <id|all> tlb_row | tlb_col_fixed <nnz> | tlb_nnz <nnz>
//   sub <id|all> template K1..K10 [tblock threads [row_reduce]]
//   fix_values 0|1     (default 1: repair two value-array defects of the reference so that the
//                       dumped arrays describe A: sub-matrices > 0 are filled from offset 0 of the
//                       COO values, op_manager.cc:1077-1087; the row-grouped template never
//                       re-interleaves its last BLB, shared_memory_op_warp_compress.cc:472.
//                       Index arrays and permutations are never touched.)
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "default_auto_tuner.hpp"

namespace
{
struct sub_spec
{
    std::vector<std::vector<std::string>> nodes;
    std::string templ;
    long tblock = -1, threads = -1, reduce = -1;
};

FILE *g_bin = NULL;
unsigned long g_off = 0;
std::ostringstream g_js;

const char *dt_name(data_type t)
{
    switch (t)
    {
    case UNSIGNED_CHAR: return "u8";
    case UNSIGNED_SHORT: return "u16";
    case UNSIGNED_INT: return "u32";
    case UNSIGNED_LONG: return "u64";
    case FLOAT: return "f32";
    case DOUBLE: return "f64";
    case BOOL: return "bool";
    default: return "other";
    }
}
size_t dt_size(data_type t)
{
    switch (t)
    {
    case UNSIGNED_CHAR: case BOOL: case CHAR: return 1;
    case UNSIGNED_SHORT: case SHORT: return 2;
    case UNSIGNED_INT: case INT: case FLOAT: return 4;
    default: return 8;
    }
}

std::string compress_json(arr_compress_type type, void *meta)
{
    std::ostringstream o;
    switch (type)
    {
    case NONE_COMPRESS: o << "{\"kind\":\"none\"}"; break;
    case LINEAR_COMPRESS:
    {
        linear_compress_t *m = (linear_compress_t *)meta;
        o << "{\"kind\":\"linear\",\"coef\":" << m->coefficient << ",\"icpt\":" << m->intercept << "}";
        break;
    }
    case CONSTANT_COMPRESS:
    {
        constant_compress_t *m = (constant_compress_t *)meta;
        o << "{\"kind\":\"constant\",\"icpt\":" << m->constant << "}";
        break;
    }
    case BRANCH_COMPRESS:
    {
        branch_compress_t *m = (branch_compress_t *)meta;
        o << "{\"kind\":\"branch\",\"lo\":[";
        for (size_t i = 0; i < m->index_low_bound.size(); i++) o << (i ? "," : "") << m->index_low_bound[i];
        o << "],\"hi\":[";
        for (size_t i = 0; i < m->index_up_bound.size(); i++) o << (i ? "," : "") << m->index_up_bound[i];
        o << "],\"val\":[";
        for (size_t i = 0; i < m->constant.size(); i++) o << (i ? "," : "") << m->constant[i];
        o << "]}";
        break;
    }
    case CYCLE_LINEAR_COMPRESS:
    {
        cycle_linear_compress_t *m = (cycle_linear_compress_t *)meta;
        o << "{\"kind\":\"cycle_linear\",\"cycle\":" << m->cycle << ",\"coef\":" << m->coefficient << ",\"icpt\":" << m->intercept << "}";
        break;
    }
    case CYCLE_INCREASE_COMPRESS:
    {
        cycle_increase_compress_t *m = (cycle_increase_compress_t *)meta;
        o << "{\"kind\":\"cycle_increase\",\"cycle\":" << m->cycle << ",\"icpt\":" << m->intercept << "}";
        break;
    }
    }
    return o.str();
}

bool g_first_arr = true;
bool g_fix_values = true;
void *g_tp = NULL;
template_type g_tt = NONE_TEMPLATE;
void dump_arr(const char *name, void *ptr, data_type t, unsigned long n, arr_compress_type ct = NONE_COMPRESS, void *meta = NULL)
{
    if (ptr == NULL) return;
    size_t bytes = dt_size(t) * n;
    fwrite(ptr, 1, bytes, g_bin);
    g_js << (g_first_arr ? "" : ",") << "\n    {\"name\":\"" << name << "\",\"dtype\":\"" << dt_name(t) << "\",\"len\":" << n
         << ",\"offset\":" << g_off << ",\"compress\":" << compress_json(ct, meta) << "}";
    g_first_arr = false;
    g_off += bytes;
    size_t pad = (8 - (g_off & 7)) & 7;
    const char z[8] = {0};
    fwrite(z, 1, pad, g_bin);
    g_off += pad;
}

#define ARR(t, f) dump_arr(#f, t->f, t->data_type_of_##f, t->size_of_##f)
#define ARRC(t, f, c) dump_arr(#f, t->f, t->data_type_of_##f, t->size_of_##f, t->c, t->c##_meta)

template <class T>
void common_head(T *t, const char *kname)
{
    g_js << "\"template\":\"" << kname << "\",\"first_row\":" << t->kernal_first_row_index << ",\"first_col\":" << t->kernal_first_col_index
         << ",\"global_sort\":" << (t->global_sort_index ? 1 : 0) << ",\"local_sort\":" << (t->local_sort_index ? 1 : 0)
         << ",\"threads\":" << t->thread_num_in_block;
}
template <class T>
void common_tail(T *t)
{
    ARRC(t, row_index_before_sort, row_index_before_sort_compress);
    ARR(t, val_arr);
    ARR(t, col_index_arr);
}

void set_launch(unsigned long &tb, unsigned long &th, const sub_spec &s)
{
    if (s.tblock > 0) tb = s.tblock;
    if (s.threads > 0) th = s.threads;
}

void dump_template(code_builder_t *builder, unsigned long sub, const sub_spec &s)
{
    const std::string &k = s.templ;
    g_first_arr = true;
    if (k == "K1")
    {
        direct_atom_template_t *t = init_direct_atom_template(builder, sub);
        try_all_compress(t);
        set_launch(t->tblock_num, t->thread_num_in_block, s);
        common_head(t, "K1");
        g_tp = t; g_tt = DIRECT_ATOM_TEMPLATE;
        g_js << ",\"tblock\":" << t->tblock_num << ",\"is_atom_add\":" << (t->is_atom_add ? 1 : 0) << ",\n   \"arrays\":[";
        ARRC(t, global_row_index_of_thread_level_block, global_row_index_compress);
        ARRC(t, block_begin_warp_index_offset, block_begin_warp_index_compress);
        ARRC(t, warp_begin_thread_index_offset, warp_begin_thread_index_compress);
        ARRC(t, thread_block_size_in_warp, thread_block_size_compress);
        ARRC(t, block_nz_begin_offset, block_nz_begin_offset_compress);
        ARRC(t, warp_nz_begin_offset, warp_nz_begin_offset_compress);
        common_tail(t);
    }
    else if (k == "K2")
    {
        direct_atom_template_warp_compress_t *t = init_direct_atom_template_warp_compress(builder, sub);
        try_all_compress(t);
        set_launch(t->tblock_num, t->thread_num_in_block, s);
        common_head(t, "K2");
        g_tp = t; g_tt = DIRECT_ATOM_TEMPLATE_WARP_COMPRESS;
        g_js << ",\"tblock\":" << t->tblock_num << ",\"is_atom_add\":" << (t->is_atom_add ? 1 : 0)
             << ",\"effective_TLB_num\":" << t->effective_TLB_num << ",\n   \"arrays\":[";
        ARRC(t, global_row_index_of_thread_level_block, global_row_index_compress);
        ARRC(t, block_begin_thread_index_offset, block_begin_thread_index_offset_compress);
        ARRC(t, block_nz_begin_offset, block_nz_begin_offset_compress);
        ARRC(t, thread_block_size_in_block, thread_block_size_in_block_compress);
        common_tail(t);
    }
    else if (k == "K3")
    {
        direct_atom_template_warp_block_compress_t *t = init_direct_atom_template_warp_block_compress(builder, sub);
        try_all_compress(t);
        set_launch(t->tblock_num, t->thread_num_in_block, s);
        common_head(t, "K3");
        g_tp = t; g_tt = DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS;
        g_js << ",\"tblock\":" << t->tblock_num << ",\"is_atom_add\":" << (t->is_atom_add ? 1 : 0)
             << ",\"effective_TLB_num\":" << t->effective_TLB_num << ",\"thread_block_size_in_block\":" << t->thread_block_size_in_block
             << ",\n   \"arrays\":[";
        ARRC(t, global_row_index_of_thread_level_block, global_row_index_compress);
        common_tail(t);
    }
    else if (k == "K4")
    {
        direct_atom_total_warp_reduce_template_t *t = init_direct_atom_total_warp_reduce_template(builder, sub);
        try_all_compress(t);
        set_launch(t->tblock_num, t->thread_num_in_block, s);
        common_head(t, "K4");
        g_tp = t; g_tt = DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE;
        g_js << ",\"tblock\":" << t->tblock_num << ",\"is_atom_add\":" << (t->is_atom_add ? 1 : 0)
             << ",\"effective_WLB_num\":" << t->effective_WLB_num << ",\n   \"arrays\":[";
        ARRC(t, global_row_index_of_warp_level_block, global_row_index_of_warp_level_block_compress);
        ARRC(t, global_warp_nz_begin_offset, global_warp_nz_begin_offset_compress);
        common_tail(t);
    }
    else if (k == "K5")
    {
        shared_memory_template_t *t = init_shared_memory_template(builder, sub);
        try_all_compress(t);
        set_launch(t->tblock_num, t->thread_num_in_block, s);
        if (s.reduce > 0) t->thread_num_of_row_reduce = s.reduce;
        common_head(t, "K5");
        g_tp = t; g_tt = SHARED_MEMORY_TEMPLATE;
        g_js << ",\"tblock\":" << t->tblock_num << ",\"is_atom_add\":" << (t->is_atom_add ? 1 : 0)
             << ",\"row_reduce\":" << t->thread_num_of_row_reduce << ",\n   \"arrays\":[";
        ARRC(t, row_offset_in_thread_tmp_result, row_offset_in_thread_tmp_result_compress);
        ARRC(t, block_first_row_index, block_first_row_index_compress);
        ARRC(t, block_begin_warp_index_offset, block_begin_warp_index_offset_compress);
        ARRC(t, warp_begin_thread_index_offset, warp_begin_thread_index_offset_compress);
        ARRC(t, thread_block_size_in_warp, thread_block_size_in_warp_compress);
        ARRC(t, block_nz_begin_offset, block_nz_begin_offset_compress);
        ARRC(t, warp_nz_begin_offset, warp_nz_begin_offset_compress);
        common_tail(t);
    }
    else if (k == "K6")
    {
        shared_memory_template_warp_compress_t *t = init_shared_memory_template_warp_compress(builder, sub);
        if (g_fix_values)
        {
            // the reference's re-interleave loop stops one BLB early (shared_memory_op_warp_compress.cc:472,
            // "block_index < block_num - 1"), leaving the last BLB's slice of val_arr / col_index_arr as
            // uninitialised heap memory; complete it from the padded row-major arrays with the same rule.
            compressed_block_t *cb = builder->op_manager->matrix->block_coor_table.item_arr[sub]->compressed_block_ptr;
            unsigned long b = t->size_of_block_nz_begin_offset - 1;
            unsigned long nz0 = read_from_array_with_data_type(t->block_nz_begin_offset, t->data_type_of_block_nz_begin_offset, b);
            unsigned long t0 = read_from_array_with_data_type(t->block_begin_thread_index_offset, t->data_type_of_block_begin_thread_index_offset, b);
            unsigned long t1 = read_from_array_with_data_type(t->block_begin_thread_index_offset, t->data_type_of_block_begin_thread_index_offset, b + 1);
            unsigned long S = read_from_array_with_data_type(t->thread_block_size_in_block, t->data_type_of_thread_block_size_in_block, b);
            unsigned long n = t1 - t0;
            for (unsigned long i = 0; i < n; i++)
                for (unsigned long k = 0; k < S; k++)
                {
                    unsigned long src = nz0 + i * S + k, dst = nz0 + i + k * n;
                    write_double_to_array_with_data_type(t->val_arr, t->data_type_of_val_arr, dst, read_double_from_array_with_data_type(cb->padding_val_arr, cb->val_data_type, src));
                    write_to_array_with_data_type(t->col_index_arr, t->data_type_of_col_index_arr, dst, read_from_array_with_data_type(cb->read_index[5]->index_arr, cb->read_index[5]->index_data_type, src));
                }
        }
        try_all_compress(t);
        set_launch(t->tblock_num, t->thread_num_in_block, s);
        if (s.reduce > 0) t->thread_num_of_row_reduce = s.reduce;
        common_head(t, "K6");
        g_tp = t; g_tt = SHARED_MEMORY_TEMPLATE_WARP_COMPRESS;
        g_js << ",\"tblock\":" << t->tblock_num << ",\"is_atom_add\":" << (t->is_atom_add ? 1 : 0)
             << ",\"row_reduce\":" << t->thread_num_of_row_reduce << ",\"effective_row_num\":" << t->effective_row_num << ",\n   \"arrays\":[";
        ARRC(t, row_offset_in_thread_tmp_result, row_offset_in_thread_tmp_result_compress);
        ARRC(t, block_first_row_index, block_first_row_index_compress);
        ARRC(t, block_begin_thread_index_offset, block_begin_thread_index_offset_compress);
        ARRC(t, thread_block_size_in_block, thread_block_size_in_block_compress);
        ARRC(t, block_nz_begin_offset, block_nz_begin_offset_compress);
        common_tail(t);
    }
    else if (k == "K7")
    {
        shared_memory_long_row_template_t *t = init_shared_memory_long_row_template(builder, sub);
        try_all_compress(t);
        set_launch(t->tblock_num, t->thread_num_in_block, s);
        common_head(t, "K7");
        g_tp = t; g_tt = SHARED_MEMORY_LONG_ROW_TEMPLATE;
        g_js << ",\"tblock\":" << t->tblock_num << ",\"is_atom_add\":" << (t->is_atom_add ? 1 : 0) << ",\n   \"arrays\":[";
        ARRC(t, row_index_of_block_level_block, row_index_of_block_level_block_compress);
        ARRC(t, block_nz_begin_offset, block_nz_begin_offset_compress);
        common_tail(t);
    }
    else if (k == "K8")
    {
        shared_memory_total_warp_reduce_template_t *t = init_shared_memory_total_warp_reduce_template(builder, sub);
        try_all_compress(t);
        set_launch(t->tblock_num, t->thread_num_in_block, s);
        if (s.reduce > 0) t->thread_num_of_row_reduce = s.reduce;
        common_head(t, "K8");
        g_tp = t; g_tt = SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE;
        g_js << ",\"tblock\":" << t->tblock_num << ",\"is_atom_add\":" << (t->is_atom_add ? 1 : 0)
             << ",\"row_reduce\":" << t->thread_num_of_row_reduce << ",\"effective_row_num\":" << t->effective_row_num << ",\n   \"arrays\":[";
        ARRC(t, row_offset_in_warp_tmp_result, row_offset_in_warp_tmp_result_compress);
        ARRC(t, block_first_row_index, block_first_row_index_compress);
        ARRC(t, block_begin_warp_index_offset, block_begin_warp_index_offset_compress);
        ARRC(t, global_warp_block_first_nz, global_warp_block_first_nz_compress);
        common_tail(t);
    }
    else if (k == "K9")
    {
        unaligned_warp_reduce_same_TLB_size_template_t *t = init_unaligned_warp_reduce_same_TLB_size_template(builder, sub);
        try_all_compress(t);
        set_launch(t->tblock_num, t->thread_num_in_block, s);
        common_head(t, "K9");
        g_tp = t; g_tt = UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE;
        g_js << ",\"tblock\":" << t->tblock_num << ",\"is_all_force_atom_add\":" << (t->is_all_force_atom_add ? 1 : 0)
             << ",\"tlb_size\":" << t->global_thread_level_block_size << ",\"bits_word\":" << t->bit_num_of_thread_level_combine_meta
             << ",\"bits_flag\":" << t->bit_num_of_sum_begin_bit_flag << ",\"bits_row\":" << t->bit_num_of_first_relative_reduce_row_of_thread_level_block
             << ",\"bits_off\":" << t->bit_num_of_tmp_result_reduce_offset_of_thread_level_block << ",\n   \"arrays\":[";
        ARRC(t, global_first_row_index_of_warp_level_block, global_first_row_index_of_warp_level_block_compress);
        ARR(t, first_relative_reduce_row_of_thread_level_block);
        ARR(t, tmp_result_reduce_offset_of_thread_level_block);
        ARR(t, combine_meta_of_thread_level_block);
        common_tail(t);
    }
    else if (k == "K10")
    {
        unaligned_warp_reduce_same_TLB_size_template_with_warp_reduce_t *t = init_unaligned_warp_reduce_same_TLB_size_template_with_warp_reduce(builder, sub);
        try_all_compress(t);
        if (s.threads > 0) t->thread_num_in_block = s.threads;
        common_head(t, "K10");
        g_tp = t; g_tt = UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE;
        g_js << ",\"is_all_force_atom_add\":" << (t->is_all_force_atom_add ? 1 : 0)
             << ",\"tlb_size\":" << t->global_thread_level_block_size << ",\"bits_word\":" << t->bit_num_of_thread_level_combine_meta
             << ",\"bits_flag\":" << t->bit_num_of_sum_begin_bit_flag << ",\"bits_row\":" << t->bit_num_of_first_relative_reduce_row_of_thread_level_block
             << ",\"bits_off\":" << t->bit_num_of_tmp_result_reduce_offset_of_thread_level_block << ",\n   \"arrays\":[";
        ARRC(t, global_first_row_index_of_warp_level_block, global_first_row_index_of_warp_level_block_compress);
        ARR(t, first_relative_reduce_row_of_thread_level_block);
        ARR(t, tmp_result_reduce_offset_of_thread_level_block);
        ARR(t, combine_meta_of_thread_level_block);
        common_tail(t);
    }
    else
    {
        fprintf(stderr, "unknown template %s\n", k.c_str());
        exit(3);
    }
    g_js << "\n   ]";
}

void add_sub_node(exe_compressed_sub_graph_t *g, param_strategy_of_sub_graph_t *p, const std::vector<std::string> &tok)
{
    const std::string &op = tok[0];
    auto L = [&](int i) { return atol(tok.at(i).c_str()); };
    if (op == "row_padding")
    {
        compressed_row_padding_direct_param_strategy_t s;
        s.multiply = L(1);
        s.padding_row_length = L(2);
        add_a_exe_node_and_param_strategy_to_exe_compressed_sub_graph(g, p, COMPRESSED_ROW_PADDING, COMPRESSED_ROW_PADDING_DIRECT_PARAM_STRATEGY, &s);
    }
    else if (op == "blb_row_evenly")
    {
        compressed_tblock_level_row_div_evenly_param_strategy_t s;
        s.block_row_num = L(1);
        add_a_exe_node_and_param_strategy_to_exe_compressed_sub_graph(g, p, COMPRESSED_TBLOCK_LEVEL_ROW_DIV, COMPRESSED_TBLOCK_LEVEL_ROW_DIV_EVENLY_PARAM_STRATEGY, &s);
    }
    else if (op == "blb_row_nnz")
    {
        compressed_tblock_level_row_div_acc_to_least_nnz_param_strategy_t s;
        s.nnz_low_bound = L(1);
        add_a_exe_node_and_param_strategy_to_exe_compressed_sub_graph(g, p, COMPRESSED_TBLOCK_LEVEL_ROW_DIV, COMPRESSED_TBLOCK_LEVEL_ROW_DIV_ACC_TO_LEAST_NNZ_PARAM_STRATEGY, &s);
    }
    else if (op == "blb_col_fixed")
    {
        compressed_tblock_level_col_div_fixed_param_strategy_t s;
        s.col_block_nnz_num = L(1);
        add_a_exe_node_and_param_strategy_to_exe_compressed_sub_graph(g, p, COMPRESSED_TBLOCK_LEVEL_COL_DIV, COMPRESSED_TBLOCK_LEVEL_COL_DIV_FIXED_PARAM_STRATEGY, &s);
    }
    else if (op == "wlb_row_evenly")
    {
        compressed_warp_level_row_div_evenly_param_strategy_t s;
        s.warp_row_num_of_each_BLB = L(1);
        add_a_exe_node_and_param_strategy_to_exe_compressed_sub_graph(g, p, COMPRESSED_WARP_LEVEL_ROW_DIV, COMPRESSED_WARP_LEVEL_ROW_DIV_EVENLY_PARAM_STRATEGY, &s);
    }
    else if (op == "wlb_col_fixed")
    {
        compressed_warp_level_col_div_fixed_param_strategy_t s;
        s.col_block_nnz_num = L(1);
        add_a_exe_node_and_param_strategy_to_exe_compressed_sub_graph(g, p, COMPRESSED_WARP_LEVEL_COL_DIV, COMPRESSED_WARP_LEVEL_COL_DIV_FIXED_PARAM_STRATEGY, &s);
    }
    else if (op == "tlb_row")
    {
        compressed_thread_level_row_div_none_param_strategy_t s;
        add_a_exe_node_and_param_strategy_to_exe_compressed_sub_graph(g, p, COMPRESSED_THREAD_LEVEL_ROW_DIV, COMPRESSED_THREAD_LEVEL_ROW_DIV_NONE_PARAM_STRATEGY, &s);
    }
    else if (op == "tlb_col_fixed")
    {
        compressed_thread_level_col_div_fixed_param_strategy_t s;
        s.col_block_nnz_num = L(1);
        add_a_exe_node_and_param_strategy_to_exe_compressed_sub_graph(g, p, COMPRESSED_THREAD_LEVEL_COL_DIV, COMPRESSED_THREAD_LEVEL_COL_DIV_FIXED_PARAM_STRATEGY, &s);
    }
    else if (op == "tlb_nnz")
    {
        compressed_thread_level_nnz_div_direct_param_strategy_t s;
        s.block_nnz_num = L(1);
        add_a_exe_node_and_param_strategy_to_exe_compressed_sub_graph(g, p, COMPRESSED_THREAD_LEVEL_NNZ_DIV, COMPRESSED_THREAD_LEVEL_NNZ_DIV_DIRECT_PARAM_STRATEGY, &s);
    }
    else
    {
        fprintf(stderr, "unknown sub op %s\n", op.c_str());
        exit(3);
    }
}
} // namespace

int main(int argc, char **argv)
{
    if (argc < 4)
    {
        fprintf(stderr, "usage: %s <matrix.mtx.coo> <spec> <outdir>\n", argv[0]);
        return 2;
    }
    std::string mtx = argv[1], spec_path = argv[2], out = argv[3];
    data_type vt = FLOAT;
    std::vector<std::vector<std::string>> dense_ops;
    std::map<long, sub_spec> subs; // -1 == all
    {
        std::ifstream f(spec_path);
        if (!f) { fprintf(stderr, "cannot open spec\n"); return 2; }
        std::string line;
        while (std::getline(f, line))
        {
            size_t h = line.find('#');
            if (h != std::string::npos) line = line.substr(0, h);
            std::istringstream is(line);
            std::vector<std::string> tok;
            std::string w;
            while (is >> w) tok.push_back(w);
            if (tok.empty()) continue;
            if (tok[0] == "dtype") vt = (tok.at(1) == "double") ? DOUBLE : FLOAT;
            else if (tok[0] == "fix_values") g_fix_values = atoi(tok.at(1).c_str()) != 0;
            else if (tok[0] == "dense") dense_ops.push_back(std::vector<std::string>(tok.begin() + 1, tok.end()));
            else if (tok[0] == "sub")
            {
                long id = (tok.at(1) == "all") ? -1 : atol(tok[1].c_str());
                sub_spec &s = subs[id];
                if (tok.at(2) == "template")
                {
                    s.templ = tok.at(3);
                    if (tok.size() > 4) s.tblock = atol(tok[4].c_str());
                    if (tok.size() > 5) s.threads = atol(tok[5].c_str());
                    if (tok.size() > 6) s.reduce = atol(tok[6].c_str());
                }
                else s.nodes.push_back(std::vector<std::string>(tok.begin() + 2, tok.end()));
            }
            else { fprintf(stderr, "bad directive %s\n", tok[0].c_str()); return 2; }
        }
    }

    // ---- dense view -------------------------------------------------------------------
    dense_begin_memory_cache_input_file_direct_param_strategy_t in = get_begin_memory_cache_input_file_direct_param_strategy_from_coo_file(mtx, vt);
    std::vector<double> orig_val;
    if (vt == DOUBLE) orig_val.assign(in.double_val_cache.begin(), in.double_val_cache.end());
    else orig_val.assign(in.float_val_cache.begin(), in.float_val_cache.end());

    exe_dense_sub_graph_t dg;
    param_strategy_of_sub_graph_t dp;
    add_a_exe_node_and_param_strategy_to_exe_dense_sub_graph(&dg, &dp, BEGIN_MEMORY_CACHE_INPUT_FILE, DENSE_BEGIN_MEMORY_CACHE_INPUT_FILE_DIRECT_PARAM_STRATEGY, &in);
    bool has_compress = false;
    for (auto &tok : dense_ops)
    {
        if (tok[0] == "sort")
        {
            dense_row_coarse_sort_fixed_param_strategy_t s;
            s.row_nnz_low_bound_step_size = atol(tok.at(1).c_str());
            add_a_exe_node_and_param_strategy_to_exe_dense_sub_graph(&dg, &dp, DENSE_ROW_COARSE_SORT, DENSE_ROW_COARSE_SORT_FIXED_PARAM_STRATEGY, &s);
        }
        else if (tok[0] == "rowdiv_exp")
        {
            dense_row_div_acc_to_exponential_increase_row_nnz_param_strategy_t s;
            s.lowest_nnz_bound_of_row = atol(tok.at(1).c_str());
            s.highest_nnz_bound_of_row = atol(tok.at(2).c_str());
            s.expansion_rate = atol(tok.at(3).c_str());
            s.sub_dense_block_id = 0;
            add_a_exe_node_and_param_strategy_to_exe_dense_sub_graph(&dg, &dp, DENSE_ROW_DIV, DENSE_ROW_DIV_ACC_TO_EXPONENTIAL_INCREASE_ROW_NNZ_PARAM_STRATEGY, &s);
        }
        else if (tok[0] == "compress")
        {
            compress_none_param_strategy_t s;
            add_a_exe_node_and_param_strategy_to_exe_dense_sub_graph(&dg, &dp, COMPRESS, COMPRESS_NONE_PARAM_STRATEGY, &s);
            has_compress = true;
        }
        else { fprintf(stderr, "bad dense op %s\n", tok[0].c_str()); return 2; }
    }
    if (!has_compress)
    {
        compress_none_param_strategy_t s;
        add_a_exe_node_and_param_strategy_to_exe_dense_sub_graph(&dg, &dp, COMPRESS, COMPRESS_NONE_PARAM_STRATEGY, &s);
    }
    sparse_struct_t *matrix = execute_dense_matrix_exe_graph_with_param_strategy(&dg, &dp);
    unsigned long nsub = matrix->block_coor_table.item_arr.size();

    if (g_fix_values)
    {
        // the dense-view value cache is in (possibly sorted) COO order; each compressed block
        // must hold the slice [begin_coo_index, end_coo_index] of it.
        for (unsigned long b = 0; b < nsub; b++)
        {
            dense_block_table_item_t *it = matrix->block_coor_table.item_arr[b];
            compressed_block_t *cb = it->compressed_block_ptr;
            unsigned long n = it->end_coo_index - it->begin_coo_index + 1;
            for (unsigned long i = 0; i < n; i++)
            {
                double v = read_double_from_array_with_data_type(matrix->coo_value_cache, matrix->val_data_type, it->begin_coo_index + i);
                write_double_to_array_with_data_type(cb->val_arr, cb->val_data_type, i, v);
            }
        }
    }

    // ---- compressed view per sub-matrix --------------------------------------------------
    std::vector<sub_spec> per(nsub);
    for (unsigned long b = 0; b < nsub; b++)
    {
        if (subs.count((long)b)) per[b] = subs[(long)b];
        else if (subs.count(-1)) per[b] = subs[-1];
        else { fprintf(stderr, "no spec for sub %lu\n", b); return 2; }
        if (!per[b].nodes.empty())
        {
            exe_compressed_sub_graph_t g;
            param_strategy_of_sub_graph_t p;
            for (auto &tok : per[b].nodes) add_sub_node(&g, &p, tok);
            execute_sub_matrix_exe_graph_with_param_strategy(matrix, b, &g, &p);
        }
        execute_default_div_to_complete_each_level_blocking(matrix, b);
    }

    operator_manager_t *op_manager = init_op_manager(matrix);
    code_builder_t *builder = init_code_builder(op_manager);

    std::string bin_path = out + "/arrays.bin";
    g_bin = fopen(bin_path.c_str(), "wb");
    if (!g_bin) { fprintf(stderr, "cannot write %s\n", bin_path.c_str()); return 2; }

    g_js << "{\"rows\":" << matrix->dense_row_number << ",\"cols\":" << matrix->dense_col_number << ",\"nnz\":" << matrix->nnz
         << ",\"origin_nnz\":" << matrix->origin_nnz << ",\"val_dtype\":\"" << dt_name(matrix->val_data_type) << "\""
         << ",\"is_sorted\":" << (matrix->is_sorted ? 1 : 0) << ",\n \"global\":[";
    g_first_arr = true;
    if (matrix->is_sorted && matrix->sorted_row_index != NULL)
        dump_arr("sorted_row_index", matrix->sorted_row_index, matrix->data_type_of_sorted_row_index, matrix->dense_row_number);
    g_js << "],\n \"subs\":[";
    for (unsigned long b = 0; b < nsub; b++)
    {
        dense_block_table_item_t *it = matrix->block_coor_table.item_arr[b];
        compressed_block_t *cb = it->compressed_block_ptr;
        g_js << (b ? "," : "") << "\n  {\"min_row\":" << it->min_dense_row_index << ",\"max_row\":" << it->max_dense_row_index
             << ",\"min_col\":" << it->min_dense_col_index << ",\"max_col\":" << it->max_dense_col_index
             << ",\"begin_coo\":" << it->begin_coo_index << ",\"end_coo\":" << it->end_coo_index
             << ",\"n_blb\":" << cb->read_index[2]->block_num << ",\"n_wlb\":" << cb->read_index[3]->block_num
             << ",\"n_tlb\":" << cb->read_index[4]->block_num << ",\n   ";
        dump_template(builder, b, per[b]);
        g_js << "}";
    }
    g_js << "\n ]}\n";
    fclose(g_bin);
    std::ofstream mf(out + "/manifest.json");
    mf << g_js.str();
    mf.close();
    return 0;
}
