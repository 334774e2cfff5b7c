// Test infrastructure (oracle side, reference -> product, never the other way): a replacement for the
// reference's executor.cc that lowers its code_builder_t to the C ABI of include/asp_b200.h.
//
// The reference's tuner reaches the GPU through two functions only (executor.hpp:12-22):
// part_execute_code_builder (every launch-parameter trial, default_auto_tuner.cc:513) and
// execute_code_builder (the whole matrix, whilte_list_path_impl.cc:5372). Their original bodies write text
// files, print template.cu, shell out to nvcc and run ./a.out (executor.cc:6-260). Linked in place of
// executor.cc, this file makes the UNMODIFIED tuner time the hand-written sm_100a kernels instead: every
// template struct of builder->template_vec becomes an asp_plan_desc (all ten templates below), the group
// is uploaded with asp_plan_group_create and timed with asp_time. INTEGRATION.md shows the same text as
// what a maintainer of the reference adds.
//
// Two extras exist only for the tests that drive it (environment variables, read once):
//   ASP_SHIM_RECORD=<file>  every call appends one line "template;n_blb;n_wlb;n_tlb;padded_nnz;tblock;threads;
//                           reduce;ms;gflops" (the fingerprint of the trial point);
//   ASP_SHIM_NO_GPU=1       nothing is uploaded or timed: every trial "runs" in 1 ms (a recording stub, so that
//                           the enumeration of the reference's tuner can be compared with asp_search on a CPU box);
//   ASP_SHIM_X=<raw file of n_cols values>, ASP_SHIM_Y=<file>: after timing, one SpMV with this x is run through
//                           asp_spmv_host and the y of the fastest whole-sub-matrix trial so far is written.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "default_auto_tuner.hpp" // the ten template structs (one header per reduce operator) and executor.hpp
#include "executor.hpp"

#include "../include/asp_b200.h"

namespace
{
asp_ctx *ctx()
{
    static asp_ctx *c = NULL;
    if (!c && asp_ctx_create((int)get_config()["DEFAULT_DEVICE_ID"].as_integer(), &c) != ASP_OK)
    {
        fprintf(stderr, "shim: asp_ctx_create failed: %s\n", asp_last_error());
        c = NULL;
    }
    return c;
}

int dt(data_type t) // struct.hpp:32-48 -> asp_dtype
{
    switch (t)
    {
    case UNSIGNED_CHAR: return ASP_U8;
    case UNSIGNED_SHORT: return ASP_U16;
    case UNSIGNED_INT: return ASP_U32;
    case UNSIGNED_LONG: return ASP_U64;
    case FLOAT: return ASP_F32;
    default: return ASP_F64;
    }
}

asp_array_desc arr(int role, void *p, data_type t, unsigned long n, arr_compress_type c = NONE_COMPRESS, void *meta = NULL)
{
    asp_array_desc d;
    memset(&d, 0, sizeof(d));
    d.role = role;
    d.dtype = dt(t);
    d.host_ptr = p;
    d.len = n;
    d.compress = (int)c; // arr_compress_type and asp_compress_kind share their order (arr_optimization.hpp:12-20)
    if (meta == NULL) d.compress = ASP_COMPRESS_NONE;
    else if (c == LINEAR_COMPRESS)
    {
        d.coef = ((linear_compress_t *)meta)->coefficient;
        d.icpt = ((linear_compress_t *)meta)->intercept;
    }
    else if (c == CONSTANT_COMPRESS) d.icpt = ((constant_compress_t *)meta)->constant;
    else if (c == CYCLE_LINEAR_COMPRESS)
    {
        cycle_linear_compress_t *m = (cycle_linear_compress_t *)meta;
        d.cycle = m->cycle, d.coef = m->coefficient, d.icpt = m->intercept;
    }
    else if (c == CYCLE_INCREASE_COMPRESS)
    {
        cycle_increase_compress_t *m = (cycle_increase_compress_t *)meta;
        d.cycle = m->cycle, d.icpt = m->intercept;
    }
    else if (c == BRANCH_COMPRESS)
    {
        branch_compress_t *m = (branch_compress_t *)meta;
        d.n_branch = (int)m->constant.size();
        for (int i = 0; i < d.n_branch && i < ASP_MAX_BRANCH; i++)
        {
            d.branch_lo[i] = m->index_low_bound[i];
            d.branch_hi[i] = m->index_up_bound[i];
            d.branch_val[i] = m->constant[i];
        }
    }
    return d;
}

// (ptr, data_type_of_<f>, size_of_<f>) triple of a template struct, with or without its closed form
#define A(role, t, f) a.push_back(arr(role, t->f, t->data_type_of_##f, t->size_of_##f))
#define AC(role, t, f, c) a.push_back(arr(role, t->f, t->data_type_of_##f, t->size_of_##f, t->c, t->c##_meta))

// what every template struct carries
template <class T>
void common(T *t, std::vector<asp_array_desc> &a, asp_plan_desc &d, int type)
{
    if (t->row_index_before_sort != NULL) AC(ASP_ARR_ROW_INDEX_BEFORE_SORT, t, row_index_before_sort, row_index_before_sort_compress);
    A(ASP_ARR_VAL, t, val_arr);
    A(ASP_ARR_COL_INDEX, t, col_index_arr);
    d.template_type = type; // asp_template_type has the values of the reference's template_type (code_builder.hpp:15-29)
    d.first_row = t->kernal_first_row_index;
    d.first_col = t->kernal_first_col_index;
    d.sort_kind = t->global_sort_index ? ASP_SORT_GLOBAL : (t->local_sort_index ? ASP_SORT_LOCAL : ASP_SORT_NONE);
    d.thread_num_in_block = t->thread_num_in_block;
    d.thread_num_of_row_reduce = 1;
}

void lower(direct_atom_template_t *t, std::vector<asp_array_desc> &a, asp_plan_desc &d)
{
    AC(ASP_ARR_GLOBAL_ROW_INDEX_OF_THREAD_LEVEL_BLOCK, t, global_row_index_of_thread_level_block, global_row_index_compress);
    AC(ASP_ARR_BLOCK_BEGIN_WARP_INDEX_OFFSET, t, block_begin_warp_index_offset, block_begin_warp_index_compress);
    AC(ASP_ARR_WARP_BEGIN_THREAD_INDEX_OFFSET, t, warp_begin_thread_index_offset, warp_begin_thread_index_compress);
    AC(ASP_ARR_THREAD_BLOCK_SIZE_IN_WARP, t, thread_block_size_in_warp, thread_block_size_compress);
    AC(ASP_ARR_BLOCK_NZ_BEGIN_OFFSET, t, block_nz_begin_offset, block_nz_begin_offset_compress);
    AC(ASP_ARR_WARP_NZ_BEGIN_OFFSET, t, warp_nz_begin_offset, warp_nz_begin_offset_compress);
    common(t, a, d, ASP_DIRECT_ATOM_TEMPLATE);
    d.is_atom_add = t->is_atom_add;
    d.tblock_num = t->tblock_num;
}
void lower(direct_atom_template_warp_compress_t *t, std::vector<asp_array_desc> &a, asp_plan_desc &d)
{
    AC(ASP_ARR_GLOBAL_ROW_INDEX_OF_THREAD_LEVEL_BLOCK, t, global_row_index_of_thread_level_block, global_row_index_compress);
    AC(ASP_ARR_BLOCK_BEGIN_THREAD_INDEX_OFFSET, t, block_begin_thread_index_offset, block_begin_thread_index_offset_compress);
    AC(ASP_ARR_BLOCK_NZ_BEGIN_OFFSET, t, block_nz_begin_offset, block_nz_begin_offset_compress);
    AC(ASP_ARR_THREAD_BLOCK_SIZE_IN_BLOCK, t, thread_block_size_in_block, thread_block_size_in_block_compress);
    common(t, a, d, ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS);
    d.is_atom_add = t->is_atom_add;
    d.effective_num = t->effective_TLB_num;
    d.tblock_num = t->tblock_num;
}
void lower(direct_atom_template_warp_block_compress_t *t, std::vector<asp_array_desc> &a, asp_plan_desc &d)
{
    AC(ASP_ARR_GLOBAL_ROW_INDEX_OF_THREAD_LEVEL_BLOCK, t, global_row_index_of_thread_level_block, global_row_index_compress);
    common(t, a, d, ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS);
    d.is_atom_add = t->is_atom_add;
    d.effective_num = t->effective_TLB_num;
    d.tlb_size = t->thread_block_size_in_block;
    d.tblock_num = t->tblock_num;
}
void lower(direct_atom_total_warp_reduce_template_t *t, std::vector<asp_array_desc> &a, asp_plan_desc &d)
{
    AC(ASP_ARR_GLOBAL_ROW_INDEX_OF_WARP_LEVEL_BLOCK, t, global_row_index_of_warp_level_block, global_row_index_of_warp_level_block_compress);
    AC(ASP_ARR_GLOBAL_WARP_NZ_BEGIN_OFFSET, t, global_warp_nz_begin_offset, global_warp_nz_begin_offset_compress);
    common(t, a, d, ASP_DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE);
    d.is_atom_add = t->is_atom_add;
    d.effective_num = t->effective_WLB_num;
    d.tblock_num = t->tblock_num;
}
void lower(shared_memory_template_t *t, std::vector<asp_array_desc> &a, asp_plan_desc &d)
{
    AC(ASP_ARR_ROW_OFFSET_IN_THREAD_TMP_RESULT, t, row_offset_in_thread_tmp_result, row_offset_in_thread_tmp_result_compress);
    AC(ASP_ARR_BLOCK_FIRST_ROW_INDEX, t, block_first_row_index, block_first_row_index_compress);
    AC(ASP_ARR_BLOCK_BEGIN_WARP_INDEX_OFFSET, t, block_begin_warp_index_offset, block_begin_warp_index_offset_compress);
    AC(ASP_ARR_WARP_BEGIN_THREAD_INDEX_OFFSET, t, warp_begin_thread_index_offset, warp_begin_thread_index_offset_compress);
    AC(ASP_ARR_THREAD_BLOCK_SIZE_IN_WARP, t, thread_block_size_in_warp, thread_block_size_in_warp_compress);
    AC(ASP_ARR_BLOCK_NZ_BEGIN_OFFSET, t, block_nz_begin_offset, block_nz_begin_offset_compress);
    AC(ASP_ARR_WARP_NZ_BEGIN_OFFSET, t, warp_nz_begin_offset, warp_nz_begin_offset_compress);
    common(t, a, d, ASP_SHARED_MEMORY_TEMPLATE);
    d.is_atom_add = t->is_atom_add;
    d.tblock_num = t->tblock_num;
    d.thread_num_of_row_reduce = t->thread_num_of_row_reduce;
}
void lower(shared_memory_template_warp_compress_t *t, std::vector<asp_array_desc> &a, asp_plan_desc &d)
{
    AC(ASP_ARR_ROW_OFFSET_IN_THREAD_TMP_RESULT, t, row_offset_in_thread_tmp_result, row_offset_in_thread_tmp_result_compress);
    AC(ASP_ARR_BLOCK_FIRST_ROW_INDEX, t, block_first_row_index, block_first_row_index_compress);
    AC(ASP_ARR_BLOCK_BEGIN_THREAD_INDEX_OFFSET, t, block_begin_thread_index_offset, block_begin_thread_index_offset_compress);
    AC(ASP_ARR_THREAD_BLOCK_SIZE_IN_BLOCK, t, thread_block_size_in_block, thread_block_size_in_block_compress);
    AC(ASP_ARR_BLOCK_NZ_BEGIN_OFFSET, t, block_nz_begin_offset, block_nz_begin_offset_compress);
    common(t, a, d, ASP_SHARED_MEMORY_TEMPLATE_WARP_COMPRESS);
    d.is_atom_add = t->is_atom_add;
    d.effective_num = t->effective_row_num;
    d.tblock_num = t->tblock_num;
    d.thread_num_of_row_reduce = t->thread_num_of_row_reduce;
}
void lower(shared_memory_long_row_template_t *t, std::vector<asp_array_desc> &a, asp_plan_desc &d)
{
    AC(ASP_ARR_ROW_INDEX_OF_BLOCK_LEVEL_BLOCK, t, row_index_of_block_level_block, row_index_of_block_level_block_compress);
    AC(ASP_ARR_BLOCK_NZ_BEGIN_OFFSET, t, block_nz_begin_offset, block_nz_begin_offset_compress);
    common(t, a, d, ASP_SHARED_MEMORY_LONG_ROW_TEMPLATE);
    d.is_atom_add = t->is_atom_add;
    d.tblock_num = t->tblock_num;
}
void lower(shared_memory_total_warp_reduce_template_t *t, std::vector<asp_array_desc> &a, asp_plan_desc &d)
{
    AC(ASP_ARR_ROW_OFFSET_IN_WARP_TMP_RESULT, t, row_offset_in_warp_tmp_result, row_offset_in_warp_tmp_result_compress);
    AC(ASP_ARR_BLOCK_FIRST_ROW_INDEX, t, block_first_row_index, block_first_row_index_compress);
    AC(ASP_ARR_BLOCK_BEGIN_WARP_INDEX_OFFSET, t, block_begin_warp_index_offset, block_begin_warp_index_offset_compress);
    AC(ASP_ARR_GLOBAL_WARP_BLOCK_FIRST_NZ, t, global_warp_block_first_nz, global_warp_block_first_nz_compress);
    common(t, a, d, ASP_SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE);
    d.is_atom_add = t->is_atom_add;
    d.effective_num = t->effective_row_num;
    d.tblock_num = t->tblock_num;
    d.thread_num_of_row_reduce = t->thread_num_of_row_reduce;
}
template <class T>
void lower_csr5(T *t, std::vector<asp_array_desc> &a, asp_plan_desc &d, int type)
{
    AC(ASP_ARR_GLOBAL_FIRST_ROW_INDEX_OF_WARP_LEVEL_BLOCK, t, global_first_row_index_of_warp_level_block, global_first_row_index_of_warp_level_block_compress);
    A(ASP_ARR_COMBINE_META_OF_THREAD_LEVEL_BLOCK, t, combine_meta_of_thread_level_block);
    common(t, a, d, type);
    d.is_atom_add = t->is_all_force_atom_add;
    d.tlb_size = t->global_thread_level_block_size;
    d.bits_word = (int)t->bit_num_of_thread_level_combine_meta;
    d.bits_flag = (int)t->bit_num_of_sum_begin_bit_flag;
    d.bits_row = (int)t->bit_num_of_first_relative_reduce_row_of_thread_level_block;
    d.bits_off = (int)t->bit_num_of_tmp_result_reduce_offset_of_thread_level_block;
}
void lower(unaligned_warp_reduce_same_TLB_size_template_t *t, std::vector<asp_array_desc> &a, asp_plan_desc &d)
{
    lower_csr5(t, a, d, ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE);
    d.tblock_num = t->tblock_num;
}
void lower(unaligned_warp_reduce_same_TLB_size_template_with_warp_reduce_t *t, std::vector<asp_array_desc> &a, asp_plan_desc &d)
{
    lower_csr5(t, a, d, ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE);
    // this template has no tblock_num: its grid covers one thread per TLB (code_of_kernal_function_call of the template)
    d.tblock_num = (long)((t->size_of_combine_meta_of_thread_level_block + t->thread_num_in_block - 1) / t->thread_num_in_block);
}
#undef A
#undef AC

bool lower_sub(code_builder_t *b, int id, std::vector<asp_array_desc> &a, asp_plan_desc &d)
{
    sparse_struct_t *m = b->op_manager->matrix;
    memset(&d, 0, sizeof(d));
    d.val_dtype = dt(m->val_data_type);
    d.n_rows = m->dense_row_number;
    d.n_cols = m->dense_col_number;
    dense_block_table_item_t *it = m->block_coor_table.item_arr[id];
    d.true_nnz = it->end_coo_index - it->begin_coo_index + 1; // code_builder.cc:1676-1686
    void *t = b->template_vec[id];
    switch (b->template_type_vec[id])
    {
    case DIRECT_ATOM_TEMPLATE: lower((direct_atom_template_t *)t, a, d); break;
    case DIRECT_ATOM_TEMPLATE_WARP_COMPRESS: lower((direct_atom_template_warp_compress_t *)t, a, d); break;
    case DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS: lower((direct_atom_template_warp_block_compress_t *)t, a, d); break;
    case DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE: lower((direct_atom_total_warp_reduce_template_t *)t, a, d); break;
    case SHARED_MEMORY_TEMPLATE: lower((shared_memory_template_t *)t, a, d); break;
    case SHARED_MEMORY_TEMPLATE_WARP_COMPRESS: lower((shared_memory_template_warp_compress_t *)t, a, d); break;
    case SHARED_MEMORY_LONG_ROW_TEMPLATE: lower((shared_memory_long_row_template_t *)t, a, d); break;
    case SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE: lower((shared_memory_total_warp_reduce_template_t *)t, a, d); break;
    case UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE: lower((unaligned_warp_reduce_same_TLB_size_template_t *)t, a, d); break;
    case UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE: lower((unaligned_warp_reduce_same_TLB_size_template_with_warp_reduce_t *)t, a, d); break;
    case EMPTY_TEMPLATE: d.template_type = ASP_EMPTY_TEMPLATE; break;
    default: return false;
    }
    d.n_arrays = (int)a.size();
    d.arrays = a.data();
    return true;
}

double g_best_gflops_with_y = 0;

bool run(code_builder_t *b, const std::vector<int> &ids, float &ms, float &gflops)
{
    ms = 0;
    gflops = 0;
    if (b == NULL || ids.empty()) return false;
    std::vector<std::vector<asp_array_desc>> arrays(ids.size());
    std::vector<asp_plan_desc> descs(ids.size());
    for (size_t k = 0; k < ids.size(); k++)
        if (!lower_sub(b, ids[k], arrays[k], descs[k])) return false;
    const bool no_gpu = getenv("ASP_SHIM_NO_GPU") != NULL;
    bool ok = true;
    if (no_gpu)
    {
        ok = asp_plan_descs_validate(descs.data(), (int)descs.size()) == ASP_OK;
        ms = 1.0f;
        double nnz = 0;
        for (const asp_plan_desc &d : descs) nnz += (double)d.true_nnz;
        gflops = (float)(2.0 * nnz * 1e-6);
    }
    else
    {
        if (!ctx()) return false;
        std::vector<asp_plan *> plans(ids.size(), (asp_plan *)NULL);
        if (asp_plan_group_create(ctx(), descs.data(), (int)descs.size(), plans.data()) != ASP_OK)
        {
            fprintf(stderr, "shim: plan rejected: %s\n", asp_last_error());
            return false; // the tuner scores 0 and moves on, as after a failed compile (whilte_list_path_impl.cc:5374-5378)
        }
        // the reference's GFLOPS_UP_BOUND (500, executor.cc:51-56) is below every B200 roofline: no bound here
        ok = asp_time(ctx(), plans.data(), (int)plans.size(), 3, 20, 2, 0.0, &ms, &gflops) == ASP_OK;
        const char *xf = getenv("ASP_SHIM_X"), *yf = getenv("ASP_SHIM_Y");
        if (ok && xf && yf && gflops > g_best_gflops_with_y)
        {
            const size_t es = descs[0].val_dtype == ASP_F64 ? 8 : 4;
            std::vector<char> x(descs[0].n_cols * es), y(descs[0].n_rows * es);
            FILE *f = fopen(xf, "rb");
            if (f && fread(x.data(), 1, x.size(), f) == x.size() && asp_spmv_host(ctx(), plans.data(), (int)plans.size(), x.data(), y.data()) == ASP_OK)
            {
                FILE *o = fopen(yf, "wb");
                if (o)
                {
                    fwrite(y.data(), 1, y.size(), o);
                    fclose(o);
                    g_best_gflops_with_y = gflops;
                }
            }
            if (f) fclose(f);
        }
        for (asp_plan *p : plans) asp_plan_destroy(p);
    }
    if (const char *rec = getenv("ASP_SHIM_RECORD"))
    {
        FILE *f = fopen(rec, "a");
        if (f)
        {
            for (size_t k = 0; k < ids.size(); k++)
            {
                compressed_block_t *cb = b->op_manager->matrix->block_coor_table.item_arr[ids[k]]->compressed_block_ptr;
                unsigned long padded = 0;
                for (int j = 0; j < descs[k].n_arrays; j++)
                    if (descs[k].arrays[j].role == ASP_ARR_VAL) padded = descs[k].arrays[j].len;
                fprintf(f, "%d;%lu;%lu;%lu;%lu;%ld;%ld;%ld;%g;%g\n", descs[k].template_type, cb->read_index[2]->block_num, cb->read_index[3]->block_num,
                        cb->read_index[4]->block_num, padded, (long)descs[k].tblock_num, (long)descs[k].thread_num_in_block, (long)descs[k].thread_num_of_row_reduce,
                        (double)ms, (double)gflops);
            }
            fclose(f);
        }
    }
    return ok;
}
} // namespace

bool part_execute_code_builder(code_builder_t *b, vector<int> ids, float &time_ms, float &gflops, string, string, bool) { return run(b, ids, time_ms, gflops); }
bool part_execute_code_builder(code_builder_t *b, vector<int> ids, float &time_ms, float &gflops, string, string, bool, bool) { return run(b, ids, time_ms, gflops); }
bool execute_code_builder(code_builder_t *b, float &time_ms, float &gflops, string, string, bool)
{
    std::vector<int> ids;
    for (size_t i = 0; i < b->template_vec.size(); i++) ids.push_back((int)i);
    return run(b, ids, time_ms, gflops);
}
// nothing is compiled or executed as a separate program any more
bool compile_spmv_code(string) { return true; }
bool execute_binary(string, float &t, float &g)
{
    t = 0;
    g = 0;
    return false;
}
