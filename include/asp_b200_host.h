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
 *   dense rowdiv <p1> <p2> ...               DENSE_ROW_DIV at explicit rows: strips [0,p1), [p1,p2), ..., [pk,rows)
 *   dense compress                          COMPRESS (implied when absent)
 *   sub <id|all> row_padding <mult> <len>   COMPRESSED_ROW_PADDING
 *   sub <id|all> blb_row_evenly <rows> | blb_row_nnz <nnz> | blb_col_fixed <nnz>
 *   sub <id|all> wlb_row_evenly <rows> | wlb_col_fixed <nnz>
 *   sub <id|all> tlb_row | tlb_col_fixed <nnz> | tlb_nnz <nnz>
 *   sub <id|all> block_value <r> <c>        (no node of the reference) store the sub-matrix as dense r x c blocks:
 *                                            2 x 2, 3 x 3 or 4 x 4; alone in its sub-graph, followed by `template B1`
 *   sub <id|all> diag_value [<max diagonals>] (no node of the reference) DIA storage for matrices whose non-zeros lie on at
 *                                            most <max> (default 64) diagonals; alone in its sub-graph, followed by `template D1`
 *   sub <id|all> template K1..K10 | B1 | D1 [tblock threads [row_reduce]]
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
/* process-unique, never reused: lets a cache of uploaded plans tell formats apart after their addresses are recycled */
uint64_t asp_format_id(const asp_format *f);
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

/* Binary file of a lowered format (all template arrays, closed forms, scalars, launch parameters and the row
 * permutation): tune once, then asp_format_load() + asp_format_plan_descs() + asp_plan_group_create() without
 * executing the Operator Graph again. Counterpart of the reference's directory of data files next to its
 * generated program (store_code_builder_data, code_builder.cc:2429-2517). A loaded format answers every
 * asp_format_* query like the one that was saved. */
asp_status asp_format_save(const asp_format *f, const char *path);
asp_status asp_format_load(const char *path, asp_format **out);

/* per-point padding rate the tuner gates on (PADDING_RATE_UP_BOUND): padded nnz / true nnz */
double asp_format_padding_rate(const asp_format *f, int sub);

/* No counterpart in the reference. For square matrices that are iterated (x <- A x on a graph), where the
 * numbering of the vertices is free: renumbers them by how often their column occurs, most frequent first
 * (ties keep their order), with the vertices whose row is empty last when empty_rows_last != 0, and returns
 * P A P^T as a new matrix. labels (n entries, may be NULL): labels[v] = new number of vertex v, so the caller
 * feeds x'[labels[v]] = x[v] and reads y[v] = y'[labels[v]]; *n_active (may be NULL) = rows with non-zeros
 * (with empty_rows_last the rows from n_active on are empty). The often-read entries of x become contiguous:
 * whole cache lines of x are hot, and what an L2 smaller than x keeps is what is read (measured on R-MAT
 * scale 26: 15 % less SpMV time). Call it before any dense-view node. */
asp_status asp_matrix_relabel_by_column_count(const asp_matrix *m, int empty_rows_last, asp_matrix **out, uint32_t *labels, uint64_t *n_active);

/* No counterpart in the reference (it is single-GPU, code_builder.cc:1483-1489): contiguous row
 * blocks with about nnz / parts non-zeros each, for sharding a matrix over `parts` GPUs with x
 * replicated. bounds gets parts + 1 entries, bounds[p] .. bounds[p + 1] is the row range of
 * part p; a row is never split. */
asp_status asp_partition_rows_by_nnz(uint64_t n_rows, const int64_t *indptr, int parts, uint64_t *bounds);

/* ---- the search loop (search_strategy.cc, whilte_list_path_impl.cc:3411-4579, default_auto_tuner.cc:449-2030) ----
 *
 * Enumerate-and-time over Operator Graphs: the dense-view strategies G1 (compress only), G2 (exponential
 * row division) and G3 (coarse sort + exponential row division); per sub-matrix the whitelist strategies
 * that its row statistics admit, each with a small node-parameter grid, one template and a sweep of launch
 * parameters; points whose padded / true non-zeros exceed `padding_rate_up_bound` are skipped; then the
 * whole matrix with the per-strip winners, and the fastest dense strategy wins. A trial costs one lowering
 * and one call of `time_fn` instead of an nvcc compile and a run of a generated program. */
typedef struct asp_search_options
{
    int32_t quick;              /* 1: one or two node-parameter points per strategy and a short launch sweep; 0: the reference's
                                 * node-parameter grids (whilte_list_path_impl.cc:228, 613-643, 1072-1110, 1483-1520, 2093-2127,
                                 * 2481-2530, 2838-2867, 3119-3176) and its launch sweeps derived from the lowered format
                                 * (default_auto_tuner.cc:465-498, 587-700, 849-883, 970-1110, 1215-1360, 1495-1625, 1749-1798,
                                 * 1911-1933), plus this build's extensions (TLB sizes 8 / 16 / 32 for the CSR5-like templates on
                                 * long rows, their staged write-out, no 65535-CTA grid cap); 2: the reference's space exactly */
    int32_t warmup, reps;       /* handed to time_fn */
    int32_t max_subs;           /* row divisions that give more strips are abandoned (reference: 5) */
    int32_t struggle_step_num;  /* < 0: time every candidate; else the stop rule of search_strategy.cc per strip */
    double time_limit_s;        /* <= 0: none; wall-clock limit of one strip's sweep under the stop rule */
    double padding_rate_up_bound; /* <= 0: the reference's 4.0 (global_config.json) */
    double prune_gbs;           /* > 0: a point whose format bytes / prune_gbs (an upper bound of the memory bandwidth, GB/s)
                                 * already exceed the best time of its strip is not timed: it cannot win. Only applied to
                                 * formats of at least prune_min_bytes (cache-resident ones can beat the memory bound). */
    uint64_t prune_min_bytes;   /* 0: 256 MiB */
    void (*log_fn)(void *user, const char *line); /* may be NULL */
    void *log_user;
    uint32_t strategy_mask;     /* 0: every whitelist strategy the row statistics admit; else bit k set = enumerate strategy k
                                 * (1..9, find_best_path_of_white_list_strategy<k> of the reference) */
    const char *checkpoint_path; /* NULL: none. Else a text file that receives every timed point as soon as it is timed (one
                                 * trial line each, flushed); a search started with the same file, matrix and options takes the
                                 * recorded times of those points instead of timing them again, so an interrupted search picks
                                 * up where it stopped. The reference keeps only the best graph of a finished strategy
                                 * (whilte_list_path_impl.cc:5395-5412). */
} asp_search_options;

/* Times one SpMV over `fmt` (sub-matrices with the EMPTY template are skipped) with the given launch
 * parameters per sub-matrix (arrays of asp_format_num_subs(fmt) entries; entries of EMPTY sub-matrices are
 * ignored). Returns 0 and the milliseconds per SpMV, or non-zero when this point cannot run (the search
 * moves on, as the reference does when a generated program fails). */
typedef int (*asp_time_fn)(void *user, const asp_format *fmt, const int64_t *tblock_num, const int64_t *thread_num_in_block,
                           const int64_t *thread_num_of_row_reduce, int warmup, int reps, float *ms_per_spmv);

typedef struct asp_search_result asp_search_result;
asp_status asp_search(const asp_matrix *m, const asp_search_options *opt, asp_time_fn time_fn, void *time_user, asp_search_result **out);
void asp_search_result_destroy(asp_search_result *r);
/* the winner: dense-view spec (lines as asp_dense_execute takes them), per sub-matrix the compressed-view
 * lines ("sub <i> ..." incl. the template line, as asp_graph_execute takes them), its strategy name and launch */
const char *asp_search_result_dense(const asp_search_result *r);
int asp_search_result_num_subs(const asp_search_result *r);
const char *asp_search_result_sub_spec(const asp_search_result *r, int sub);
const char *asp_search_result_sub_name(const asp_search_result *r, int sub);
asp_status asp_search_result_sub_launch(const asp_search_result *r, int sub, int64_t *thread_num_in_block, int64_t *thread_num_of_row_reduce);
float asp_search_result_ms(const asp_search_result *r);
/* every timed point, one text line each: "<dense> ; sub <i> ; <strategy> ; threads ; reduce ; ms ; padding" */
int asp_search_result_num_trials(const asp_search_result *r);
const char *asp_search_result_trial(const asp_search_result *r, int i);

/* The strategies that apply to a sub-matrix with row non-zeros in [min, max] (mean avg), as text: one line
 * per candidate, "<name> ; <template> ; <node>|<node>... ; <threads>:<reduce>,..." (what asp_search sweeps).
 * quick = 1: the short table; 0: the long table with fixed launch lists; 2: the reference's node grids exactly,
 * without launch lists (asp_search derives them from the lowered format, as the reference does). */
const char *asp_search_candidates(uint64_t min_row_nnz, uint64_t max_row_nnz, double avg_row_nnz, int is_sorted, int quick);
/* launch shapes the reference derives instead of searching (default_auto_tuner.cc:465-498, 688-693) */
int64_t asp_search_derive_tblock(int template_type, uint64_t n_tlb, uint64_t n_wlb, uint64_t n_blb, int64_t thread_num_in_block);

/* text of the last error a host-side entry point reported on this thread */
const char *asp_host_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* ASP_B200_HOST_H */
