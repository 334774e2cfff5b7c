/*
 * asp_b200_host.h -- C ABI of the host side: the Operator Graph (dense-view and compressed-view
 * format operators) and the lowering of every sub-matrix into the flat arrays of a reduce
 * template. It mirrors what a caller of the reference does with exe_graph / op_manager /
 * code_builder (exe_graph.hpp, op_manager.hpp, code_builder.hpp): build a matrix, run graph
 * nodes on it, init a template per sub-matrix, try_all_compress -- and then hands the result to
 * the device side (asp_b200.h) instead of to the nvcc-driven executor.
 */
#ifndef ASP_B200_HOST_H
#define ASP_B200_HOST_H

#include "asp_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct asp_matrix asp_matrix; /* sparse_struct_t of the reference */
typedef struct asp_format asp_format; /* code_builder_t: one template per sub-matrix */

/* BEGIN_MEMORY_CACHE_INPUT_FILE node (exe_graph.hpp:162-175): a matrix from CSR arrays that are
 * sorted by row then column. indptr has n_rows + 1 entries; values are f32 or f64. */
asp_status asp_matrix_from_csr(uint64_t n_rows, uint64_t n_cols, const int64_t *indptr, const uint32_t *indices,
                               const void *values, int val_dtype, asp_matrix **out);
/* BEGIN_INPUT_FILE node: the `.mtx.coo` text format (struct.cc:92-174) */
asp_status asp_matrix_from_coo_file(const char *path, int val_dtype, asp_matrix **out);
void asp_matrix_destroy(asp_matrix *m);
uint64_t asp_matrix_rows(const asp_matrix *m);
uint64_t asp_matrix_cols(const asp_matrix *m);
uint64_t asp_matrix_nnz(const asp_matrix *m);

/*
 * Run an Operator Graph on (a copy of) the matrix and lower every sub-matrix to a template.
 * `spec` is a line-oriented description of the graph, one node per line:
 *   dense sort <step>                       DENSE_ROW_COARSE_SORT (fixed-step strategy)
 *   dense rowdiv_exp <low> <high> <rate>    DENSE_ROW_DIV (exponential row-nnz ranges)
 *   dense compress                          COMPRESS (implied when absent)
 *   sub <id|all> row_padding <mult> <len>   COMPRESSED_ROW_PADDING
 *   sub <id|all> blb_row_evenly <rows> | blb_row_nnz <nnz> | blb_col_fixed <nnz>
 *   sub <id|all> wlb_row_evenly <rows> | wlb_col_fixed <nnz>
 *   sub <id|all> tlb_row | tlb_col_fixed <nnz> | tlb_nnz <nnz>
 *   sub <id|all> template K1..K10 [tblock threads [row_reduce]]
 * (node names: exe_graph.hpp:36-57; strategies: parameter_set_strategy.hpp:10-25; K1..K10 are
 * the templates of code_builder.hpp:15-29 in the order DIRECT_ATOM, _WARP_COMPRESS,
 * _WARP_BLOCK_COMPRESS, DIRECT_ATOM_TOTAL_WARP_REDUCE, SHARED_MEMORY, _WARP_COMPRESS, _LONG_ROW,
 * _TOTAL_WARP_REDUCE, UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE, _WITH_WARP_REDUCE).
 * Levels a graph leaves untiled are completed the way the reference's tuner does
 * (execute_default_div_to_complete_each_level_blocking, default_auto_tuner.cc:384).
 */
asp_status asp_graph_execute(const asp_matrix *m, const char *spec, asp_format **out);

/* Dense-view part of a graph on its own (`dense ...` lines only; compress is implied): returns a
 * compressed matrix whose sub-matrices can then be lowered again and again with
 * asp_graph_execute(`sub ...` lines only). This is how the reference's tuner works: the dense
 * view is executed once per dense strategy (execute_dense_matrix_exe_graph_with_param_strategy,
 * default_auto_tuner.cc:2073) and value-copied for every compressed-view trial
 * (val_copy_from_old_matrix_struct, struct.cc:392). Sub-matrices whose spec names the template
 * EMPTY are neither copied nor lowered (EMPTY_TEMPLATE of the reference, empty_op.cc). */
asp_status asp_dense_execute(const asp_matrix *m, const char *dense_spec, asp_matrix **out);
/* number of sub-matrices of a compressed matrix (0 before compress) */
int asp_matrix_num_subs(const asp_matrix *m);
/* row statistics of one sub-matrix: what the tuner's rule gates look at (matrix_info.cc:122-190) */
asp_status asp_matrix_sub_rows(const asp_matrix *m, int sub, uint64_t *n_rows, uint64_t *nnz, uint64_t *min_row_nnz, uint64_t *max_row_nnz);
void asp_format_destroy(asp_format *f);

int asp_format_num_subs(const asp_format *f);
/* the global row permutation (sorted_row_index, new -> old); *ptr == NULL when unsorted */
asp_status asp_format_global_perm(const asp_format *f, const void **ptr, int *dtype, uint64_t *len);

typedef struct asp_sub_info
{
    uint64_t min_row, max_row, min_col, max_col, begin_coo, end_coo; /* dense_block_table_item_t */
    uint64_t n_blb, n_wlb, n_tlb;
    int32_t template_type, n_arrays;
} asp_sub_info;
asp_status asp_format_sub_info(const asp_format *f, int sub, asp_sub_info *out);

/* plan descriptors for asp_plan_group_create(); the pointers stay valid until
 * asp_format_destroy(). `descs` must have room for asp_format_num_subs() entries. */
asp_status asp_format_plan_descs(const asp_format *f, asp_plan_desc *descs);

/* per-point padding rate the tuner gates on (PADDING_RATE_UP_BOUND): padded nnz / true nnz */
double asp_format_padding_rate(const asp_format *f, int sub);

/* No counterpart in the reference (it is single-GPU, code_builder.cc:1483-1489): contiguous row
 * blocks with about nnz / parts non-zeros each, for sharding a matrix over `parts` GPUs with x
 * replicated. bounds gets parts + 1 entries, bounds[p] .. bounds[p + 1] is the row range of
 * part p; a row is never split. */
asp_status asp_partition_rows_by_nnz(uint64_t n_rows, const int64_t *indptr, int parts, uint64_t *bounds);

/* text of the last error a host-side entry point reported on this thread */
const char *asp_host_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* ASP_B200_HOST_H */
