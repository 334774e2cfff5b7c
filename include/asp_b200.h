/*
 * asp_b200.h -- C ABI of the B200-native SpMV path for AlphaSparse's machine-designed formats.
 *
 * This boundary replaces the reference's executor seam: where the reference wrote text files,
 * emitted template.cu / template.h, shelled out to nvcc and ran ./a.out to time y = A*x
 * (executor.hpp:12-22, executor.cc:6-260, code_builder.cc:1471-1575), a caller now hands the
 * per-sub-matrix template arrays to asp_plan_group_create() once and launches / times
 * precompiled sm_100a kernels.
 *
 * All entry points use C linkage, plain pointers and sizes, return an asp_status and never
 * throw or abort. Handles are opaque. One asp_ctx per GPU and per host thread.
 */
#ifndef ASP_B200_H
#define ASP_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum asp_status
{
    ASP_OK = 0,
    ASP_ERR_INVALID_ARG = 1, /* NULL pointer, bad length, inconsistent descriptor          */
    ASP_ERR_UNSUPPORTED = 2, /* a dtype / template / width the kernels do not implement     */
    ASP_ERR_CUDA = 3,        /* a CUDA runtime call failed; asp_last_error() has the text   */
    ASP_ERR_ALLOC = 4,       /* host or device allocation failed                            */
    ASP_ERR_BOUNDS = 5,      /* a format array refers outside val/col/x/y                   */
    ASP_ERR_IMPLAUSIBLE = 6, /* measured throughput above the configured sanity bound       */
    ASP_ERR_TIMEOUT = 7      /* a bounded wait on the device expired (asp_dist_status)      */
} asp_status;

/* element types of format arrays; the reference narrows every index array to the smallest
 * unsigned type that holds its maximum (op_manager.cc:1103-1134). */
typedef enum asp_dtype
{
    ASP_U8 = 0,
    ASP_U16 = 1,
    ASP_U32 = 2,
    ASP_U64 = 3,
    ASP_F32 = 4,
    ASP_F64 = 5
} asp_dtype;

/* closed forms that stand in for a metadata array (arr_optimization.hpp:12-81). The
 * reference bakes them into the emitted source; here they are kernel parameters. */
typedef enum asp_compress_kind
{
    ASP_COMPRESS_NONE = 0,           /* a[i] is loaded                       */
    ASP_COMPRESS_LINEAR = 1,         /* a[i] = i*coef + icpt                 */
    ASP_COMPRESS_CONSTANT = 2,       /* a[i] = icpt                          */
    ASP_COMPRESS_BRANCH = 3,         /* a[i] = val[b] for lo[b] <= i <= hi[b]*/
    ASP_COMPRESS_CYCLE_LINEAR = 4,   /* a[i] = (i % cycle)*coef + icpt       */
    ASP_COMPRESS_CYCLE_INCREASE = 5  /* a[i] = i / cycle + icpt              */
} asp_compress_kind;

/* same order as the reference's template_type (code_builder.hpp:15-29) */
typedef enum asp_template_type
{
    ASP_DIRECT_ATOM_TEMPLATE = 0,
    ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS = 1,
    ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS = 2,
    ASP_SHARED_MEMORY_TEMPLATE = 3,
    ASP_SHARED_MEMORY_TEMPLATE_WARP_COMPRESS = 4,
    ASP_SHARED_MEMORY_LONG_ROW_TEMPLATE = 5,
    ASP_SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE = 6,
    ASP_DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE = 7,
    ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE = 8,
    ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE = 9,
    ASP_EMPTY_TEMPLATE = 10,
    /* Not one of the reference's templates: blocked ELL over dense r x c blocks, built by the `block_value r c`
     * operator of asp_b200_host.h (2 x 2, 3 x 3, 4 x 4). One block-column index per block instead of one column
     * index per non-zero, and the c values of x are gathered once per block. Arrays: ASP_ARR_COL_INDEX = block
     * column of slot k of block row b at [k * NB + b] (u32), ASP_ARR_VAL = element (i, j) of that block at
     * [((k * r + i) * c + j) * NB + b]. Scalars of asp_plan_desc: tlb_size = block slots per block row,
     * effective_num = rows of the sub-matrix, bits_row = r, bits_off = c; NB = len(col) / tlb_size (even). */
    ASP_BLOCK_ELL_TEMPLATE = 11,
    /* Not one of the reference's templates either: DIA storage, built by the `diag_value` operator, for matrices
     * whose non-zeros lie on a few diagonals (banded stencils). One offset per diagonal instead of one column index
     * per non-zero; x is read as shifted contiguous runs. Arrays: ASP_ARR_COL_INDEX = the D offsets as u64, biased by
     * (n_cols - first_col) so that they are unsigned; ASP_ARR_VAL = A[r, r + off[d]] at [d * NR + r] (zero where the
     * diagonal leaves the matrix). Scalars: tlb_size = D, effective_num = rows of the sub-matrix; NR = len(val) / D,
     * a multiple of 16 / sizeof(value). */
    ASP_DIAG_TEMPLATE = 12
} asp_template_type;

/* role of an array inside a template; names are the reference's struct field names
 * (direct_atom_op.hpp, shared_memory_op_warp_compress.hpp, ... one struct per template). */
typedef enum asp_array_role
{
    ASP_ARR_VAL = 0,
    ASP_ARR_COL_INDEX = 1,
    ASP_ARR_ROW_INDEX_BEFORE_SORT = 2,
    ASP_ARR_GLOBAL_ROW_INDEX_OF_THREAD_LEVEL_BLOCK = 3,
    ASP_ARR_BLOCK_BEGIN_WARP_INDEX_OFFSET = 4,
    ASP_ARR_WARP_BEGIN_THREAD_INDEX_OFFSET = 5,
    ASP_ARR_THREAD_BLOCK_SIZE_IN_WARP = 6,
    ASP_ARR_BLOCK_NZ_BEGIN_OFFSET = 7,
    ASP_ARR_WARP_NZ_BEGIN_OFFSET = 8,
    ASP_ARR_BLOCK_BEGIN_THREAD_INDEX_OFFSET = 9,
    ASP_ARR_THREAD_BLOCK_SIZE_IN_BLOCK = 10,
    ASP_ARR_GLOBAL_ROW_INDEX_OF_WARP_LEVEL_BLOCK = 11,
    ASP_ARR_GLOBAL_WARP_NZ_BEGIN_OFFSET = 12,
    ASP_ARR_ROW_OFFSET_IN_THREAD_TMP_RESULT = 13,
    ASP_ARR_BLOCK_FIRST_ROW_INDEX = 14,
    ASP_ARR_ROW_INDEX_OF_BLOCK_LEVEL_BLOCK = 15,
    ASP_ARR_ROW_OFFSET_IN_WARP_TMP_RESULT = 16,
    ASP_ARR_GLOBAL_WARP_BLOCK_FIRST_NZ = 17,
    ASP_ARR_GLOBAL_FIRST_ROW_INDEX_OF_WARP_LEVEL_BLOCK = 18,
    ASP_ARR_COMBINE_META_OF_THREAD_LEVEL_BLOCK = 19,
    ASP_ARR_ROLE_COUNT = 20
} asp_array_role;

#define ASP_MAX_BRANCH 5 /* BRANCH_COMPRESS_MAX_SIZE of the reference's global_config.json */

/* one (ptr, dtype, size) triple of a template struct plus its arr_compress_type + meta */
typedef struct asp_array_desc
{
    int32_t role;           /* asp_array_role */
    int32_t dtype;          /* asp_dtype */
    const void *host_ptr;   /* may be NULL when compress != NONE */
    uint64_t len;           /* elements */
    int32_t compress;       /* asp_compress_kind */
    int32_t n_branch;
    uint64_t coef, icpt, cycle;
    uint64_t branch_lo[ASP_MAX_BRANCH], branch_hi[ASP_MAX_BRANCH], branch_val[ASP_MAX_BRANCH];
} asp_array_desc;

typedef enum asp_sort_kind
{
    ASP_SORT_NONE = 0,
    ASP_SORT_GLOBAL = 1, /* matrix->sorted_row_index, indexed by row + first_row */
    ASP_SORT_LOCAL = 2   /* per sub-matrix y_write_index, indexed by row         */
} asp_sort_kind;

/* everything one template struct of the reference carries for one sub-matrix */
typedef struct asp_plan_desc
{
    int32_t template_type;   /* asp_template_type */
    int32_t val_dtype;       /* ASP_F32 | ASP_F64 */
    uint64_t n_rows, n_cols; /* of the WHOLE matrix: lengths of y and x */
    uint64_t first_row;      /* kernal_first_row_index */
    uint64_t first_col;      /* kernal_first_col_index */
    uint64_t true_nnz;       /* nnz of this sub-matrix before padding (for GFLOP/s) */
    int32_t n_arrays;
    const asp_array_desc *arrays;
    /* scalars */
    uint64_t effective_num;  /* effective_TLB_num | effective_WLB_num | effective_row_num; 0 = all */
    uint64_t tlb_size;       /* thread_block_size_in_block (ELL-like) | global_thread_level_block_size (CSR5-like) */
    int32_t bits_word, bits_flag, bits_row, bits_off; /* combine-meta layout, CSR5-like templates */
    int32_t is_atom_add;     /* is_atom_add | is_all_force_atom_add */
    int32_t sort_kind;       /* asp_sort_kind */
    /* launch parameters, as the tuner sets them */
    int64_t tblock_num, thread_num_in_block, thread_num_of_row_reduce;
} asp_plan_desc;

typedef struct asp_ctx asp_ctx;
typedef struct asp_plan asp_plan;

/* replaces cudaSetDevice(DEFAULT_DEVICE_ID) + stream creation of the generated main()
 * (code_builder.cc:1483-1518). */
asp_status asp_ctx_create(int device, asp_ctx **out);
void asp_ctx_destroy(asp_ctx *ctx);
/* raw cudaStream_t the context launches on (for callers that enqueue their own work) */
void *asp_ctx_stream(asp_ctx *ctx);

/* replaces store_code_builder_data + read_dense_block_k_from_file + the cudaMalloc/cudaMemcpy
 * block (code_builder.cc:2429-2517, 2119-2129; e.g. direct_atom_op.cc:289-370,1524-1692):
 * validates and uploads all sub-matrix templates of one matrix. Arrays that share a host
 * pointer (the global row permutation) are uploaded once. Validation covers the contents too:
 * every column index must lie inside x, every row a kernel can write inside y, every offset
 * inside the array it indexes (ASP_ERR_BOUNDS otherwise; one parallel pass over each index array).
 * Every entry point makes the context's device current for its own duration and restores the
 * caller's device before it returns. */
asp_status asp_plan_group_create(asp_ctx *ctx, const asp_plan_desc *descs, int n, asp_plan **out_plans);
void asp_plan_destroy(asp_plan *plan);
/* The validation of asp_plan_group_create on its own: same checks, same status and message, no device
 * needed, nothing allocated or uploaded. For a caller that wants to vet template arrays (a loaded
 * format file, the output of its own operators) before it touches a GPU. The reference has no
 * counterpart: its init_<template> functions assert (e.g. direct_atom_op_warp_compress.cc:88-92). */
asp_status asp_plan_descs_validate(const asp_plan_desc *descs, int n);

/* replaces re-emitting + recompiling the program for every launch-parameter trial
 * (default_auto_tuner.cc:449-2030): tblock_num / thread_num_in_block / thread_num_of_row_reduce.
 * The two CSR5-like templates have no row-reduce phase; for them the third parameter selects the
 * write-out: 1 = every finished row is stored on its own (what the reference's kernel does), 2 = the rows
 * of a warp are collected in shared memory and leave as one contiguous run (an extension of the launch
 * space for sm_100a; which one is faster depends on the matrix, so the search times both). */
asp_status asp_plan_set_launch(asp_plan *plan, int64_t tblock_num, int64_t thread_num_in_block, int64_t thread_num_of_row_reduce);
/* The launch asp_spmv will actually use. The kernels are compiled for a bounded CTA width per family
 * (ELL-like 512, SELL-like and CSR5-like 256 threads) and never launch CTAs without work, so a request
 * outside those bounds is folded into an equivalent launch (wider requests become more CTAs); a tuner
 * that sweeps thread_num_in_block reads back here which points of its sweep coincide. The reference has
 * no such query: its launch is the literal it printed into the program (code_of_kernal_function_call,
 * e.g. direct_atom_op_warp_block_compress.cc:1012-1040). Any pointer may be NULL. */
asp_status asp_plan_get_launch(const asp_plan *plan, int64_t *tblock_num, int64_t *thread_num_in_block, int64_t *thread_num_of_row_reduce);
/* Work decomposition knobs, for launch-space experiments (the defaults are what the measurements in this
 * repository use): `vec` = TLBs per thread (1, 2, 4, 8 for ELL-like; 1, 2, 4 for SELL-like; 0 keeps the
 * current value), `path` (-1 keeps): SELL-like 0 = warp tasks over equal strips, 1 = one CTA per strip;
 * CSR5-like bit 0 = staged write-out (the same switch as thread_num_of_row_reduce = 2), bits 4..7 = log2
 * of the rows per warp that go through shared memory (0 keeps the size chosen at plan creation).
 * Re-applies the last requested launch. No counterpart in the reference (its generated kernels handle
 * one TLB per thread). */
asp_status asp_plan_set_tuning(asp_plan *plan, int vec, int path);
/* bytes of device memory the plan's format arrays occupy (B_fmt without x and y) */
uint64_t asp_plan_format_bytes(const asp_plan *plan);
/* number of kernel launches one asp_spmv over this plan issues (excluding the y clear) */
int asp_plan_launches(const asp_plan *plan);

/* replaces the spmv_<k><<<...>>> calls of the generated main() (code_builder.cc:1534-1550):
 * y (+)= A*x over all sub-matrix plans of one matrix; d_x and d_y are device pointers of
 * the value dtype, lengths n_cols and n_rows. zero_y: 0 = leave y as it is (the reference
 * never clears y between repeats), 1 = clear y first, 2 = clear y only when one of the plans
 * accumulates with atomics (plans that store every row of a matrix without empty rows
 * overwrite y completely). Asynchronous on the context's stream. */
asp_status asp_spmv(asp_ctx *ctx, asp_plan *const *plans, int n_plans, const void *d_x, void *d_y, int zero_y);

/* same with HOST x and y: copies x in, runs, copies y out, waits. This is the shape of the
 * reference's a.out run (host arrays in, host y out) without the text files. */
asp_status asp_spmv_host(asp_ctx *ctx, asp_plan *const *plans, int n_plans, const void *h_x, void *h_y);

/* asp_spmv_host for matrices whose rows read a bounded band of columns (stencils, finite elements in a
 * band-reducing numbering): the rows are cut into chunks, each with its own plan group built over ALL columns
 * (global column indices, n_rows = the chunk's rows), and chunk k declares col_hi, an exclusive upper bound of
 * the columns its rows read. x is uploaded as a growing prefix: chunk k's kernel starts as soon as x[0, col_hi)
 * is on the device, and its rows of y leave for the host while the next chunk's part of x is still arriving, on
 * three streams (copy in, kernels, copy out). With h_x and h_y in pinned memory a host-to-host SpMV then costs
 * about one PCIe direction instead of two in series. A wrong col_hi makes a kernel read entries of x that are not
 * there yet (stale values of an earlier call): declare the maximum column + 1, or n_cols when in doubt. The
 * chunks must tile [0, n_rows) in ascending order. Returns when y is complete. No counterpart in the reference
 * (its generated program copies x in, runs, copies y out: code_builder.cc:2119-2129, 1534-1557). */
typedef struct
{
    asp_plan *const *plans;
    int n_plans;
    uint64_t row_lo, row_hi; /* rows [row_lo, row_hi) of the matrix */
    uint64_t col_hi;         /* every column these rows read is < col_hi */
} asp_host_chunk;
asp_status asp_spmv_host_pipelined(asp_ctx *ctx, const asp_host_chunk *chunks, int n_chunks, const void *h_x, void *h_y);

/* No counterpart in the reference. asp_spmv_host for callers that must not trigger a device
 * allocation (a solver whose own pool owns all device memory; a loop that cannot afford the
 * device-wide synchronisation of cudaMalloc / cudaFree): x and y are staged in a fixed device
 * array of asp_static_stage_bytes() bytes (half for x, half for y) that every GPU loading the
 * library holds until exit. Fails with ASP_ERR_INVALID_ARG when n_cols or n_rows times the
 * value size exceeds half of it. The first call for a device looks up the array's address and
 * should be made before any stream capture; calls that overlap on one GPU race on the array. */
asp_status asp_spmv_host_static(asp_ctx *ctx, asp_plan *const *plans, int n_plans, const void *h_x, void *h_y);
uint64_t asp_static_stage_bytes(void);

/* Publishes `bytes` of finished results at `src` (this GPU's memory) to every GPU of an NVLink
 * multicast group: `multicast_dst` is the multicast address of the same offset of a buffer that all
 * the GPUs mapped symmetrically (e.g. torch.distributed._symmetric_memory). The stores are issued by a
 * small kernel (`ctas` CTAs, 0 = default) on `stream` (a cudaStream_t) and replicated by NVSwitch, so
 * the data leaves this GPU once. `bytes` must be a multiple of 4 and src / multicast_dst congruent
 * modulo 16. Completion on the peers is ordered by whatever the caller enqueues next on `stream`
 * across the ranks (a collective). No counterpart in the reference, which is single-GPU
 * (code_builder.cc:1483-1489). */
asp_status asp_multicast_store(const void *src, void *multicast_dst, size_t bytes, void *stream, int ctas);

/* The sharded repeated SpMV (x <- A x over the GPUs of one NVLink domain, every rank owning a row block) as
 * ONE kernel per plan that computes and publishes: like asp_spmv, but the rows a warp finishes leave the
 * kernel through `d_y_multicast`, the NVLink multicast address of the buffer that `d_y` is this GPU's
 * replica of (same offsets), so they land in every rank's copy of the next x while the other warps are
 * still computing. Only the first and last row of each warp, which neighbouring warps may share, are
 * accumulated locally (cleared before the kernel, sent by a small kernel after it). Every plan must be a
 * CSR5-like template (TLB size 4, 8, 16 or 32; 16- or 32-bit columns; not forced to atomics), else
 * ASP_ERR_UNSUPPORTED. Rows the plans never write (rows without non-zeros that the format dropped) are not
 * touched in any replica: the caller clears the buffer once, when it creates it. Follow the call with
 * asp_rank_barrier (or a collective) before any rank reads the result. No counterpart in the reference,
 * which is single-GPU (code_builder.cc:1483-1489). */
asp_status asp_spmv_publish(asp_ctx *ctx, asp_plan *const *plans, int n_plans, const void *d_x, void *d_y, void *d_y_multicast);
/* number of rows asp_spmv_publish sends after the kernel (at most two per warp) */
uint64_t asp_plan_end_rows(const asp_plan *plan);

/* Barrier of the `world` ranks of a multicast group as a one-warp kernel on `stream` (see asp_spmv_publish):
 * `flags_local` / `flags_multicast` are this GPU's replica and the multicast address of a symmetric array of
 * `world` 32-bit words, zero at first; `epoch` must grow by one per barrier, the same on every rank. Stores
 * issued earlier on the stream are visible to a peer that passes the barrier. The wait is bounded
 * (`max_polls` polls per slot, 0 = about a second): on expiry the kernel writes 1 + the slot it gave up on
 * to *status_u32 (device memory, cleared by the caller) and returns. One rank per GPU only. No counterpart
 * in the reference. */
asp_status asp_rank_barrier(const void *flags_local, void *flags_multicast, int rank, int world, unsigned epoch, void *status_u32, unsigned max_polls,
                            void *stream);

/* The sharded repeated SpMV (x <- A x, square matrix, x replicated on the GPUs of one NVLink domain, every rank
 * owning a contiguous row block) as one native loop per rank; no counterpart in the reference, which is
 * single-GPU (code_builder.cc:1483-1489). A rank's block is cut into row chunks, each with its own plan group
 * built over ALL columns; the chunks are computed in the order given, and as soon as one is finished its rows
 * are stored once through the NVLink multicast address of the result vector (asp_multicast_store) on a second
 * stream, under the next chunk's kernels, so only the LAST chunk's exchange is exposed: put the chunk with
 * the fewest rows last. One asp_rank_barrier per SpMV orders the ranks. The ranks may cut their blocks into
 * different numbers of chunks. Vectors and the flag array are symmetric memory that the caller allocated,
 * bound to multicast objects and zeroed (e.g. torch.distributed._symmetric_memory); the library sees plain
 * pointers only. One rank per GPU. The plans, the flag array and the context must outlive the asp_dist, which
 * only refers to them. The ranks must enter a loop together (a host barrier after anything that takes a
 * different time on every rank): the barrier kernel waits for a late rank only as long as max_polls allows. */
typedef struct asp_dist asp_dist;
typedef struct
{
    asp_plan *const *plans; /* the chunk's plan group; n_rows = row_hi - row_lo, n_cols = the vector length */
    int n_plans;            /* 0: the chunk has no non-zeros, its rows are cleared */
    uint64_t row_lo, row_hi; /* global rows [row_lo, row_hi) the group produces */
} asp_dist_chunk;
typedef struct
{
    int rank, world;       /* at most 32 ranks */
    int value_is_f64;
    uint64_t n;            /* length of the replicated vector */
    const asp_dist_chunk *chunks; /* tile one contiguous row block, in the order they are computed */
    int n_chunks;
    const void *flags_local; /* world > 1: this GPU's replica and the multicast address of a symmetric array of */
    void *flags_multicast;   /* at least `world` 32-bit words, zero at first, used by nothing else              */
    unsigned max_polls;      /* bound of the barrier's wait, 0 = about a second */
} asp_dist_desc;
asp_status asp_dist_create(asp_ctx *ctx, const asp_dist_desc *desc, asp_dist **out);
void asp_dist_destroy(asp_dist *d);
/* y <- A x on every rank: d_y is this GPU's replica of the result vector, d_y_multicast the multicast address
 * of the same vector (ignored when world == 1). Asynchronous on the context's stream, on which the result is
 * complete in every replica. x and y must be different vectors. */
asp_status asp_dist_spmv(asp_dist *d, const void *d_x, void *d_y, void *d_y_multicast);
/* x <- A x, `iters` times, starting from d_x0 (only read); the results alternate between the two buffers
 * (iteration i writes d_buf[i & 1]); *final_buf = index of the buffer that holds the last result (-1 when
 * iters == 0). */
asp_status asp_dist_spmv_iter(asp_dist *d, const void *d_x0, void *const d_buf[2], void *const d_buf_multicast[2], int iters, int *final_buf);
/* Waits for the context's stream, then ASP_OK, or ASP_ERR_TIMEOUT with *waiting_for_rank = the rank a barrier
 * gave up on (its wait is bounded by design: a rank that never arrives costs seconds, not a hung GPU). */
asp_status asp_dist_status(asp_dist *d, int *waiting_for_rank);

/* replaces execute_binary + perf_result parsing (executor.cc:6-59): CUDA-event timing of
 * `reps` SpMVs after `warmup`, x and y internal (x = 100 everywhere, as the generated main()
 * does). gflops = 2*sum(true_nnz)*1e-6/ms. Returns ASP_ERR_IMPLAUSIBLE when gflops exceeds
 * gflops_up_bound > 0 (the reference's GFLOPS_UP_BOUND check, executor.cc:51-56). */
asp_status asp_time(asp_ctx *ctx, asp_plan *const *plans, int n_plans, int warmup, int reps, int zero_y,
                    double gflops_up_bound, float *ms_per_spmv, float *gflops);

/* asp_search (asp_b200_host.h) with the GPU as the timer: every trial is uploaded once
 * (asp_plan_group_create), its launch parameters are swept with asp_plan_set_launch, and asp_time
 * measures it on the context's stream. `matrix`, `options` and `result` are the asp_matrix,
 * asp_search_options and asp_search_result of asp_b200_host.h (void here so that this header stays
 * independent of the host one). Replaces the reference's compile-and-run trial
 * (part_execute_code_builder + execute_binary, executor.cc:6-260). */
asp_status asp_search_gpu(asp_ctx *ctx, const void *matrix, const void *options, void **result);

asp_status asp_synchronize(asp_ctx *ctx);
const char *asp_status_str(asp_status s);
/* text of the last CUDA error seen by this thread ("" if none) */
const char *asp_last_error(void);
/* 1 when the library was built with device code for sm_100a */
int asp_built_for_sm100a(void);

#ifdef __cplusplus
}
#endif
#endif /* ASP_B200_H */
