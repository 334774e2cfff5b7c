// C ABI over the kernel families: context, plan upload / validation, launch, timing.
// Replaces the reference's "emit source -> nvcc -> a.out -> parse perf_result" executor
// (executor.cc:6-260) and the generated main() (code_builder.cc:1471-1575).
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <memory>
#include <new>
#include <string>
#include <vector>

#include "../../include/asp_b200.h"
#include "kernel_args.h"
#include "kernels.h"

namespace
{
thread_local std::string g_last_error;

asp_status cuda_fail(cudaError_t e, const char *what)
{
    g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
    return ASP_ERR_CUDA;
}
asp_status fail(asp_status s, const std::string &msg)
{
    g_last_error = msg;
    return s;
}
#define ASP_CUDA(call)                                      \
    do                                                      \
    {                                                       \
        cudaError_t e__ = (call);                           \
        if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
    } while (0)

// Makes `device` current for the lifetime of the object and restores the caller's device afterwards:
// every entry point that launches or allocates runs under one, so a process that holds contexts on
// several GPUs never launches into a stream of a device that is not current.
struct DeviceGuard
{
    int prev = -1;
    cudaError_t err = cudaSuccess;
    explicit DeviceGuard(int device)
    {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) err = cudaSetDevice(device);
        else if (err == cudaSuccess) prev = -1; // nothing to restore
    }
    ~DeviceGuard()
    {
        if (prev >= 0) cudaSetDevice(prev);
    }
};
#define ASP_ON_DEVICE(ctx)                \
    DeviceGuard guard__((ctx)->device); \
    if (guard__.err != cudaSuccess) return cuda_fail(guard__.err, "cudaSetDevice")

int dtype_size(int dt)
{
    switch (dt)
    {
    case ASP_U8: return 1;
    case ASP_U16: return 2;
    case ASP_U32: case ASP_F32: return 4;
    case ASP_U64: case ASP_F64: return 8;
    default: return 0;
    }
}

// device memory shared by the plans of one group (one cudaMalloc per matrix)
struct Arena
{
    void *base = nullptr;
    size_t bytes = 0;
    int device = 0;
    ~Arena()
    {
        if (base) cudaFree(base);
    }
};

// host copy of a metadata reference, for validation and shared-memory sizing
struct HostMeta
{
    const void *p = nullptr;
    int dtype = ASP_U32;
    uint64_t len = 0;
    int kind = ASP_COMPRESS_NONE;
    uint64_t coef = 0, icpt = 0, cycle = 1;
    int nb = 0;
    uint64_t bhi[5] = {0, 0, 0, 0, 0}, bval[5] = {0, 0, 0, 0, 0};
    bool present = false;
    uint64_t get(uint64_t i) const
    {
        switch (kind)
        {
        case ASP_COMPRESS_NONE:
            switch (dtype)
            {
            case ASP_U8: return ((const uint8_t *)p)[i];
            case ASP_U16: return ((const uint16_t *)p)[i];
            case ASP_U32: return ((const uint32_t *)p)[i];
            default: return ((const uint64_t *)p)[i];
            }
        case ASP_COMPRESS_LINEAR: return i * coef + icpt;
        case ASP_COMPRESS_CONSTANT: return icpt;
        case ASP_COMPRESS_CYCLE_LINEAR: return (i % cycle) * coef + icpt;
        case ASP_COMPRESS_CYCLE_INCREASE: return i / cycle + icpt;
        default:
        {
            uint64_t v = bval[0];
            for (int b = 1; b < nb; b++)
                if (i > bhi[b - 1]) v = bval[b];
            return v;
        }
        }
    }
};
} // namespace

struct asp_ctx
{
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    // side streams: the sub-matrix kernels of one SpMV run concurrently (the reference gives every
    // sub-matrix kernel its own stream, code_builder.cc:1515-1518)
    static const int kAux = 3;
    cudaStream_t aux[kAux] = {nullptr, nullptr, nullptr};
    cudaEvent_t ev_fork = nullptr, ev_join[kAux] = {nullptr, nullptr, nullptr};
    int sm_count = 0;
    int max_smem_optin = 0;
    // scratch x / y used by asp_time and asp_spmv_host; grown on demand
    void *x = nullptr, *y = nullptr;
    size_t x_bytes = 0, y_bytes = 0;
    // copy streams and events of the pipelined host SpMV, created on first use
    cudaStream_t h2d = nullptr, d2h = nullptr;
    std::vector<cudaEvent_t> pipe_events;
};

struct asp_plan
{
    std::shared_ptr<Arena> arena;
    asp::KArgs args;
    int templ = 0;
    int val_is_f64 = 0;
    int col_width = 4;
    uint64_t n_rows = 0, n_cols = 0, true_nnz = 0;
    unsigned grid = 1, block = 32;
    size_t smem = 0;
    int vec = 1;
    uint64_t fmt_bytes = 0;
    uint64_t smem_elems = 0; // partial results per CTA (shared-memory family)
    uint64_t units_for_grid = 0;
    uint64_t warp_tasks = 0; // SELL-like with equal strips: warp-sized work items
    uint64_t sell_strip = 0; // SELL-like: TLBs per strip when all strips are equal, else 0
    bool needs_zero = false;
    // CSR5-like family: the rows of y that warps accumulate with `red` (first and last row of every warp), as
    // indices into y; kept on the device for the publishing SpMV (asp_spmv_publish)
    std::shared_ptr<Arena> end_rows;
    uint64_t n_end_rows = 0;
    int64_t asked_tblock = 0, asked_threads = 0, asked_reduce = 0; // the launch last requested (re-applied when vec / path change)
};

namespace
{
int slot_of_role(int templ, int role)
{
    using namespace asp;
    switch (role)
    {
    case ASP_ARR_GLOBAL_ROW_INDEX_OF_THREAD_LEVEL_BLOCK: return MS_ROW_OF_TLB;
    case ASP_ARR_BLOCK_BEGIN_THREAD_INDEX_OFFSET: return MS_BLK_THR;
    case ASP_ARR_BLOCK_NZ_BEGIN_OFFSET: return MS_BLK_NZ;
    case ASP_ARR_THREAD_BLOCK_SIZE_IN_BLOCK:
    case ASP_ARR_THREAD_BLOCK_SIZE_IN_WARP: return MS_TLB_SIZE;
    case ASP_ARR_BLOCK_BEGIN_WARP_INDEX_OFFSET: return MS_BLK_WARP;
    case ASP_ARR_WARP_BEGIN_THREAD_INDEX_OFFSET: return MS_WARP_THR;
    case ASP_ARR_WARP_NZ_BEGIN_OFFSET:
    case ASP_ARR_GLOBAL_WARP_NZ_BEGIN_OFFSET:
    case ASP_ARR_GLOBAL_WARP_BLOCK_FIRST_NZ: return MS_WARP_NZ;
    case ASP_ARR_ROW_OFFSET_IN_THREAD_TMP_RESULT:
    case ASP_ARR_ROW_OFFSET_IN_WARP_TMP_RESULT: return MS_ROW_OFF;
    case ASP_ARR_BLOCK_FIRST_ROW_INDEX: return MS_BLK_ROW;
    case ASP_ARR_GLOBAL_ROW_INDEX_OF_WARP_LEVEL_BLOCK:
    case ASP_ARR_ROW_INDEX_OF_BLOCK_LEVEL_BLOCK:
    case ASP_ARR_GLOBAL_FIRST_ROW_INDEX_OF_WARP_LEVEL_BLOCK: return MS_ROW_OF_UNIT;
    case ASP_ARR_COMBINE_META_OF_THREAD_LEVEL_BLOCK: return MS_COMBINE;
    default: return -1;
    }
}

// which metadata slots each template must provide
std::vector<int> required_slots(int templ)
{
    using namespace asp;
    switch (templ)
    {
    case ASP_DIRECT_ATOM_TEMPLATE: return {MS_ROW_OF_TLB, MS_BLK_WARP, MS_WARP_THR, MS_TLB_SIZE, MS_BLK_NZ, MS_WARP_NZ};
    case ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS: return {MS_ROW_OF_TLB, MS_BLK_THR, MS_BLK_NZ, MS_TLB_SIZE};
    case ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS: return {MS_ROW_OF_TLB};
    case ASP_SHARED_MEMORY_TEMPLATE: return {MS_ROW_OFF, MS_BLK_ROW, MS_BLK_WARP, MS_WARP_THR, MS_TLB_SIZE, MS_BLK_NZ, MS_WARP_NZ};
    case ASP_SHARED_MEMORY_TEMPLATE_WARP_COMPRESS: return {MS_ROW_OFF, MS_BLK_ROW, MS_BLK_THR, MS_TLB_SIZE, MS_BLK_NZ};
    case ASP_SHARED_MEMORY_LONG_ROW_TEMPLATE: return {MS_ROW_OF_UNIT, MS_BLK_NZ};
    case ASP_SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE: return {MS_ROW_OFF, MS_BLK_ROW, MS_BLK_WARP, MS_WARP_NZ};
    case ASP_DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE: return {MS_ROW_OF_UNIT, MS_WARP_NZ};
    case ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE:
    case ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE: return {MS_ROW_OF_UNIT, MS_COMBINE};
    default: return {};
    }
}

bool is_smem_family(int t)
{
    return t == ASP_SHARED_MEMORY_TEMPLATE || t == ASP_SHARED_MEMORY_TEMPLATE_WARP_COMPRESS || t == ASP_SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE;
}
bool perm_on_device(int t)
{
    return is_smem_family(t) || t == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE || t == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE;
}

asp_status apply_launch(asp_ctx *ctx, asp_plan *p, int64_t tblock, int64_t threads, int64_t reduce)
{
    if (threads <= 0 || threads > 1024) return fail(ASP_ERR_INVALID_ARG, "thread_num_in_block must be in 1..1024");
    p->asked_tblock = tblock;
    p->asked_threads = threads;
    p->asked_reduce = reduce;
    const int t = p->templ;
    const bool warp_based = t != ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS && t != ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS && t != ASP_BLOCK_ELL_TEMPLATE && t != ASP_DIAG_TEMPLATE;
    if (warp_based && (threads % 32) != 0) return fail(ASP_ERR_INVALID_ARG, "thread_num_in_block must be a multiple of 32 for this template");
    if (is_smem_family(t))
    {
        if (reduce <= 0) reduce = 1;
        if (reduce > 32 || (reduce & (reduce - 1)) != 0) return fail(ASP_ERR_INVALID_ARG, "thread_num_of_row_reduce must be a power of two <= 32");
        if ((threads % 32) != 0) return fail(ASP_ERR_INVALID_ARG, "thread_num_in_block must be a multiple of 32 for this template");
        p->args.row_reduce = (int)reduce;
    }
    if (tblock <= 0) tblock = 1;
    if (tblock > 2147483647LL) tblock = 2147483647LL;
    if (t == ASP_DIAG_TEMPLATE)
    {
        threads = std::min<int64_t>(256, (threads + 31) / 32 * 32);
        tblock = (int64_t)std::max<uint64_t>(1, (p->units_for_grid + (uint64_t)threads - 1) / (uint64_t)threads);
    }
    if (t == ASP_BLOCK_ELL_TEMPLATE)
    {
        // one thread per pair of block rows, CTAs of at most 128 threads, never more CTAs than work
        threads = std::min<int64_t>(128, (threads + 31) / 32 * 32);
        tblock = (int64_t)std::max<uint64_t>(1, (p->units_for_grid + (uint64_t)threads - 1) / (uint64_t)threads);
    }
    if (t == ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS)
    {
        // the ELL-like kernel handles `vec` TLBs per thread and is compiled for at most 512 threads
        // per CTA: fold wider requests into more CTAs and never launch CTAs without work
        if (threads > 512)
        {
            tblock *= (threads + 511) / 512;
            threads = 512;
        }
        const int64_t needed = (int64_t)((p->units_for_grid + (uint64_t)threads - 1) / (uint64_t)threads);
        if (tblock > needed) tblock = needed > 0 ? needed : 1;
    }
    if (t == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE || t == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE)
    {
        // these templates have no row-reduce phase; the third launch parameter selects their write-out instead:
        // 1 = every finished row is stored on its own, 2 = the rows of a warp leave through shared memory as one run
        if (reduce > 2) return fail(ASP_ERR_INVALID_ARG, "CSR5-like templates: thread_num_of_row_reduce is 1 (rows stored one by one) or 2 (staged write-out)");
        p->args.path = (p->args.path & ~1) | (reduce == 2 ? 1 : 0);
        p->args.row_reduce = reduce == 2 ? 2 : 1;
    }
    if ((t == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE || t == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE) && threads > 256)
    {
        // compiled for at most 256 threads per CTA; the warp loop is grid-stride, so more CTAs
        // of 256 threads walk the same warps
        tblock = std::min<int64_t>(tblock * ((threads + 255) / 256), 2147483647LL);
        threads = 256;
    }
    if (t == ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS && threads > 256)
    {
        // the SELL-like kernel is compiled for at most 256 threads per CTA (register budget); its
        // strip loop is CTA-stride, so a narrower CTA only changes how a strip is walked
        threads = 256;
    }
    if (t == ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS && p->warp_tasks > 0)
    {
        threads = (threads + 31) / 32 * 32;
        const int64_t needed = (int64_t)((p->warp_tasks + (uint64_t)(threads / 32) - 1) / (uint64_t)(threads / 32));
        if (tblock > needed) tblock = needed > 0 ? needed : 1;
    }
    p->grid = (unsigned)tblock;
    p->block = (unsigned)threads;
    return ASP_OK;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- content validation --------------------------------------------------------------------------
// The structural checks of asp_plan_group_create look at lengths and offsets; these look at what the
// arrays SAY: every column a kernel will gather and every row it will write must lie inside x and y.
// A caller that hands over one bad index would otherwise make a kernel read or write outside its
// buffers on a GPU it shares with other jobs. Cost: one OpenMP pass over each index array.
uint64_t max_of(const HostMeta &h, uint64_t count)
{
    if (count == 0) return 0;
    switch (h.kind)
    {
    case ASP_COMPRESS_NONE:
    {
        uint64_t mx = 0;
        const int64_t n = (int64_t)count;
        switch (h.dtype)
        {
#define ASP_MAX_CASE(DT, T)                                                            \
    case DT:                                                                           \
    {                                                                                  \
        const T *q = (const T *)h.p;                                                   \
        _Pragma("omp parallel for reduction(max : mx) schedule(static)") for (int64_t i = 0; i < n; i++) mx = q[i] > mx ? (uint64_t)q[i] : mx; \
        break;                                                                         \
    }
            ASP_MAX_CASE(ASP_U8, uint8_t)
            ASP_MAX_CASE(ASP_U16, uint16_t)
            ASP_MAX_CASE(ASP_U32, uint32_t)
        default:
            ASP_MAX_CASE(ASP_U64, uint64_t)
#undef ASP_MAX_CASE
        }
        return mx;
    }
    case ASP_COMPRESS_LINEAR: return (count - 1) * h.coef + h.icpt;
    case ASP_COMPRESS_CONSTANT: return h.icpt;
    case ASP_COMPRESS_CYCLE_LINEAR: return (std::min<uint64_t>(count, h.cycle) - 1) * h.coef + h.icpt;
    case ASP_COMPRESS_CYCLE_INCREASE: return (count - 1) / h.cycle + h.icpt;
    default:
    {
        uint64_t mx = 0;
        for (int b = 0; b < h.nb && b < 5; b++) mx = std::max(mx, h.bval[b]);
        return mx;
    }
    }
}

// the largest y index a device-permuted template (shared-memory and CSR5-like families) can write for
// relative rows [0, rows); false when the permutation itself is too short
bool device_rows_in_bounds(const asp_plan_desc &d, const HostMeta &perm, uint64_t rows, std::string &why)
{
    if (rows == 0) return true;
    if (d.sort_kind == ASP_SORT_GLOBAL)
    {
        if (rows + d.first_row > perm.len) return why = "row_index_before_sort is shorter than first_row + the rows of this sub-matrix", false;
        if (max_of(perm, perm.len) >= d.n_rows) return why = "row_index_before_sort names a row outside y", false;
    }
    else if (d.sort_kind == ASP_SORT_LOCAL)
    {
        if (rows > perm.len) return why = "row_index_before_sort is shorter than the rows of this sub-matrix", false;
        if (max_of(perm, perm.len) + d.first_row >= d.n_rows) return why = "row_index_before_sort + first_row names a row outside y", false;
    }
    else if (rows + d.first_row > d.n_rows)
        return why = "the sub-matrix has more rows than y below first_row", false;
    return true;
}

bool validate_contents(const asp_plan_desc &d, const std::vector<HostMeta> &hm, const HostMeta &perm, const asp_array_desc *col, const asp::KArgs &a,
                       std::string &why)
{
    using namespace asp;
    {
        HostMeta c;
        c.p = col->host_ptr;
        c.dtype = col->dtype;
        c.kind = ASP_COMPRESS_NONE;
        if (d.template_type == ASP_DIAG_TEMPLATE)
        {
            // offsets are biased by the column count; |offset| beyond the matrix is harmless (the kernel masks every x index)
            // but a bias that does not match makes no sense
            c.dtype = ASP_U64;
            if (max_of(c, col->len) >= 2 * (d.n_cols - d.first_col) + d.n_rows) return why = "a diagonal offset lies outside the matrix", false;
            return true;
        }
        if (d.template_type == ASP_BLOCK_ELL_TEMPLATE)
        {
            // a block column covers bits_off columns of x
            if ((max_of(c, col->len) + 1) * (uint64_t)d.bits_off + d.first_col > d.n_cols) return why = "col_index_arr names a column outside x", false;
            return true;
        }
        if (max_of(c, col->len) + d.first_col >= d.n_cols) return why = "col_index_arr names a column outside x", false;
    }
    const uint64_t radd = (d.sort_kind == ASP_SORT_GLOBAL) ? 0 : d.first_row;
    switch (d.template_type)
    {
    case ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS:
    case ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS:
        if (max_of(hm[MS_ROW_OF_TLB], a.effective) + radd >= d.n_rows) return why = "global_row_index_of_thread_level_block names a row outside y", false;
        return true;
    case ASP_DIRECT_ATOM_TEMPLATE:
        if (hm[MS_ROW_OF_TLB].kind == ASP_COMPRESS_NONE && hm[MS_ROW_OF_TLB].len < a.n_tlb) return why = "3-level: row map shorter than the TLB count", false;
        if (max_of(hm[MS_ROW_OF_TLB], a.n_tlb) + radd >= d.n_rows) return why = "global_row_index_of_thread_level_block names a row outside y", false;
        return true;
    case ASP_DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE:
        if (max_of(hm[MS_ROW_OF_UNIT], a.effective) + radd >= d.n_rows) return why = "global_row_index_of_warp_level_block names a row outside y", false;
        return true;
    case ASP_SHARED_MEMORY_LONG_ROW_TEMPLATE:
        if (max_of(hm[MS_ROW_OF_UNIT], a.n_units) + radd >= d.n_rows) return why = "row_index_of_block_level_block names a row outside y", false;
        return true;
    case ASP_SHARED_MEMORY_TEMPLATE:
    case ASP_SHARED_MEMORY_TEMPLATE_WARP_COMPRESS:
    case ASP_SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE:
    {
        // rows: block_first_row_index is a CSR over BLBs; the partial-result offsets of every BLB must stay
        // inside the BLB's own partials (they index shared memory)
        const uint64_t B = a.n_units;
        const HostMeta &br = hm[MS_BLK_ROW], &ro = hm[MS_ROW_OFF];
        const uint64_t rows_all = br.get(B);
        if (ro.kind == ASP_COMPRESS_NONE && ro.len < rows_all + 1) return why = "row offsets shorter than the row count", false;
        bool ok = true;
#pragma omp parallel for schedule(static) reduction(&& : ok)
        for (int64_t b = 0; b < (int64_t)B; b++)
        {
            const uint64_t r0 = br.get(b), r1 = br.get(b + 1);
            if (r1 < r0 || r1 > rows_all) { ok = false; continue; }
            uint64_t partials;
            if (d.template_type == ASP_SHARED_MEMORY_TEMPLATE_WARP_COMPRESS) partials = hm[MS_BLK_THR].get(b + 1) - hm[MS_BLK_THR].get(b);
            else if (d.template_type == ASP_SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE) partials = hm[MS_BLK_WARP].get(b + 1) - hm[MS_BLK_WARP].get(b);
            else partials = hm[MS_WARP_THR].get(hm[MS_BLK_WARP].get(b + 1)) - hm[MS_WARP_THR].get(hm[MS_BLK_WARP].get(b));
            const uint64_t g0 = ro.get(r0);
            uint64_t prev = g0;
            for (uint64_t r = r0; r < r1; r++)
            {
                const uint64_t nx = ro.get(r + 1);
                if (nx < prev || nx - g0 > partials) { ok = false; break; }
                prev = nx;
            }
        }
        if (!ok) return why = "a row's partial-result range leaves its BLB (row offsets / block_first_row_index inconsistent)", false;
        return device_rows_in_bounds(d, perm, std::min<uint64_t>(rows_all, a.effective), why);
    }
    case ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE:
    case ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE:
    {
        // thread t of warp w writes rows R0[w] + frow .. + (#row starts in t) - 1
        const HostMeta &cm = hm[MS_COMBINE], &fr = hm[MS_ROW_OF_UNIT];
        const uint64_t W = a.n_units;
        const int S = (int)d.tlb_size, bw = d.bits_word;
        const uint64_t rmask = (1ull << d.bits_row) - 1;
        uint64_t top = 0; // one past the largest relative row written
#pragma omp parallel for schedule(static) reduction(max : top)
        for (int64_t w = 0; w < (int64_t)W; w++)
        {
            const uint64_t R0 = fr.get(w);
            for (int l = 0; l < 32; l++)
            {
                const uint64_t m = cm.get((uint64_t)w * 32 + l);
                const uint64_t flags = S >= 64 ? m : (m >> (bw - S)) & ((S >= 64) ? ~0ull : ((1ull << S) - 1));
                const int starts = __builtin_popcountll(flags);
                if (starts) top = std::max<uint64_t>(top, R0 + (m & rmask) + starts);
            }
        }
        return device_rows_in_bounds(d, perm, top, why);
    }
    default: return true;
    }
}

asp_status ensure_xy(asp_ctx *ctx, size_t xb, size_t yb)
{
    if (ctx->x_bytes < xb)
    {
        if (ctx->x) cudaFree(ctx->x);
        ctx->x = nullptr;
        ctx->x_bytes = 0;
        ASP_CUDA(cudaMalloc(&ctx->x, xb));
        ctx->x_bytes = xb;
    }
    if (ctx->y_bytes < yb)
    {
        if (ctx->y) cudaFree(ctx->y);
        ctx->y = nullptr;
        ctx->y_bytes = 0;
        ASP_CUDA(cudaMalloc(&ctx->y, yb));
        ctx->y_bytes = yb;
    }
    return ASP_OK;
}
} // namespace

extern "C" {

const char *asp_status_str(asp_status s)
{
    switch (s)
    {
    case ASP_OK: return "ok";
    case ASP_ERR_INVALID_ARG: return "invalid argument";
    case ASP_ERR_UNSUPPORTED: return "unsupported";
    case ASP_ERR_CUDA: return "CUDA error";
    case ASP_ERR_ALLOC: return "allocation failed";
    case ASP_ERR_BOUNDS: return "format array out of bounds";
    case ASP_ERR_IMPLAUSIBLE: return "implausible throughput";
    case ASP_ERR_TIMEOUT: return "bounded device-side wait expired";
    default: return "unknown";
    }
}

const char *asp_last_error(void) { return g_last_error.c_str(); }

int asp_built_for_sm100a(void)
{
#ifdef ASP_SM100A
    return 1;
#else
    return 0;
#endif
}

asp_status asp_ctx_create(int device, asp_ctx **out)
{
    if (!out) return fail(ASP_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    int n = 0;
    ASP_CUDA(cudaGetDeviceCount(&n));
    if (device < 0 || device >= n) return fail(ASP_ERR_INVALID_ARG, "no such CUDA device");
    DeviceGuard guard(device); // the caller's current device is left as it was
    if (guard.err != cudaSuccess) return cuda_fail(guard.err, "cudaSetDevice");
    asp_ctx *c = new (std::nothrow) asp_ctx();
    if (!c) return fail(ASP_ERR_ALLOC, "host allocation failed");
    c->device = device;
    cudaError_t e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&c->ev0);
    if (e == cudaSuccess) e = cudaEventCreate(&c->ev1);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming);
    for (int i = 0; i < asp_ctx::kAux && e == cudaSuccess; i++)
    {
        e = cudaStreamCreateWithFlags(&c->aux[i], cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_join[i], cudaEventDisableTiming);
    }
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&c->max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    if (e != cudaSuccess)
    {
        asp_ctx_destroy(c);
        return cuda_fail(e, "context setup");
    }
    *out = c;
    return ASP_OK;
}

void asp_ctx_destroy(asp_ctx *c)
{
    if (!c) return;
    DeviceGuard guard(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->x) cudaFree(c->x);
    if (c->y) cudaFree(c->y);
    if (c->ev0) cudaEventDestroy(c->ev0);
    if (c->ev1) cudaEventDestroy(c->ev1);
    if (c->ev_fork) cudaEventDestroy(c->ev_fork);
    for (int i = 0; i < asp_ctx::kAux; i++)
    {
        if (c->ev_join[i]) cudaEventDestroy(c->ev_join[i]);
        if (c->aux[i]) cudaStreamDestroy(c->aux[i]);
    }
    if (c->h2d) cudaStreamSynchronize(c->h2d);
    if (c->d2h) cudaStreamSynchronize(c->d2h);
    for (cudaEvent_t e : c->pipe_events) cudaEventDestroy(e);
    if (c->h2d) cudaStreamDestroy(c->h2d);
    if (c->d2h) cudaStreamDestroy(c->d2h);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

void *asp_ctx_stream(asp_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

asp_status asp_synchronize(asp_ctx *ctx)
{
    if (!ctx) return fail(ASP_ERR_INVALID_ARG, "ctx is NULL");
    ASP_ON_DEVICE(ctx);
    ASP_CUDA(cudaStreamSynchronize(ctx->stream));
    return ASP_OK;
}

} // extern "C"

namespace
{
// dry == true: everything asp_plan_group_create checks, without a device (no allocation, no upload, no
// plan objects returned); ctx may then be NULL.
asp_status plan_group_build(asp_ctx *ctx, const asp_plan_desc *descs, int n, asp_plan **out_plans, bool dry)
{

    // ---- pass 1: validate descriptors, lay out the arena (arrays sharing a host pointer once)
    struct Slot
    {
        size_t off, bytes;
    };
    std::map<const void *, Slot> placed;
    size_t total = 0;
    std::vector<std::vector<HostMeta>> metas(n, std::vector<HostMeta>(asp::MS_COUNT));
    std::vector<HostMeta> perms(n);
    std::vector<const asp_array_desc *> vals(n, nullptr), cols(n, nullptr);
    for (int i = 0; i < n; i++)
    {
        const asp_plan_desc &d = descs[i];
        if (d.template_type < 0 || d.template_type > ASP_DIAG_TEMPLATE) return fail(ASP_ERR_INVALID_ARG, "unknown template_type");
        // (also for EMPTY plans: the host-buffer entry points size x and y from the value type)
        if (d.val_dtype != ASP_F32 && d.val_dtype != ASP_F64) return fail(ASP_ERR_UNSUPPORTED, "val_dtype must be f32 or f64");
        if (d.n_rows == 0 || d.n_cols == 0) return fail(ASP_ERR_INVALID_ARG, "matrix without rows or columns");
        if (d.template_type == ASP_EMPTY_TEMPLATE) continue;
        if (!d.arrays || d.n_arrays <= 0) return fail(ASP_ERR_INVALID_ARG, "plan without arrays");
        if (d.first_row >= d.n_rows || d.first_col >= d.n_cols) return fail(ASP_ERR_BOUNDS, "first_row/first_col outside the matrix");
        for (int k = 0; k < d.n_arrays; k++)
        {
            const asp_array_desc &ad = d.arrays[k];
            if (ad.role < 0 || ad.role >= ASP_ARR_ROLE_COUNT) return fail(ASP_ERR_INVALID_ARG, "unknown array role");
            const int es = dtype_size(ad.dtype);
            if (es == 0) return fail(ASP_ERR_UNSUPPORTED, "unknown array dtype");
            if (ad.compress < ASP_COMPRESS_NONE || ad.compress > ASP_COMPRESS_CYCLE_INCREASE) return fail(ASP_ERR_INVALID_ARG, "unknown compress kind");
            if (ad.compress == ASP_COMPRESS_NONE && (!ad.host_ptr || ad.len == 0)) return fail(ASP_ERR_INVALID_ARG, "array without data");
            if (ad.compress == ASP_COMPRESS_BRANCH && (ad.n_branch < 1 || ad.n_branch > ASP_MAX_BRANCH)) return fail(ASP_ERR_INVALID_ARG, "bad branch count");
            if ((ad.compress == ASP_COMPRESS_CYCLE_LINEAR || ad.compress == ASP_COMPRESS_CYCLE_INCREASE) && ad.cycle == 0) return fail(ASP_ERR_INVALID_ARG, "cycle == 0");
            if (ad.role == ASP_ARR_VAL)
            {
                if (ad.dtype != d.val_dtype) return fail(ASP_ERR_INVALID_ARG, "val_arr dtype differs from val_dtype");
                vals[i] = &ad;
            }
            else if (ad.role == ASP_ARR_COL_INDEX)
            {
                if (d.template_type == ASP_DIAG_TEMPLATE ? ad.dtype != ASP_U64 : (ad.dtype != ASP_U8 && ad.dtype != ASP_U16 && ad.dtype != ASP_U32))
                    return fail(ASP_ERR_UNSUPPORTED, "col_index_arr must be u8/u16/u32 (u64 diagonal offsets for the diagonal-value template)");
                cols[i] = &ad;
            }
            else
            {
                if (ad.dtype == ASP_F32 || ad.dtype == ASP_F64) return fail(ASP_ERR_INVALID_ARG, "metadata array with float dtype");
                HostMeta hm;
                hm.p = ad.host_ptr;
                hm.dtype = ad.dtype;
                hm.len = ad.len;
                hm.kind = ad.compress;
                hm.coef = ad.coef;
                hm.icpt = ad.icpt;
                hm.cycle = ad.cycle ? ad.cycle : 1;
                hm.nb = ad.n_branch;
                for (int b = 0; b < ASP_MAX_BRANCH; b++)
                {
                    hm.bhi[b] = ad.branch_hi[b];
                    hm.bval[b] = ad.branch_val[b];
                }
                hm.present = true;
                if (ad.role == ASP_ARR_ROW_INDEX_BEFORE_SORT) perms[i] = hm;
                else
                {
                    const int s = slot_of_role(d.template_type, ad.role);
                    if (s < 0) return fail(ASP_ERR_INVALID_ARG, "array role not used by any template");
                    metas[i][s] = hm;
                }
            }
            if (ad.compress == ASP_COMPRESS_NONE && !placed.count(ad.host_ptr))
            {
                Slot s{total, (size_t)ad.len * es};
                placed[ad.host_ptr] = s;
                total = align_up(total + s.bytes + 32, 256); // 32 B of slack: vector loads may over-read masked tails
            }
        }
        if (!vals[i] || !cols[i]) return fail(ASP_ERR_INVALID_ARG, "val_arr or col_index_arr missing");
        if (d.template_type != ASP_BLOCK_ELL_TEMPLATE && d.template_type != ASP_DIAG_TEMPLATE && vals[i]->len != cols[i]->len) return fail(ASP_ERR_INVALID_ARG, "val_arr and col_index_arr differ in length");
        for (int s : required_slots(d.template_type))
            if (!metas[i][s].present) return fail(ASP_ERR_INVALID_ARG, "a metadata array this template needs is missing");
        if (perm_on_device(d.template_type) && d.sort_kind != ASP_SORT_NONE && !perms[i].present)
            return fail(ASP_ERR_INVALID_ARG, "sorted plan without row_index_before_sort");
    }

    std::shared_ptr<Arena> arena(new (std::nothrow) Arena());
    if (!arena) return fail(ASP_ERR_ALLOC, "host allocation failed");
    arena->device = dry ? 0 : ctx->device;
    arena->bytes = std::max<size_t>(total, 256);
    if (!dry)
    {
        cudaError_t e = cudaMalloc(&arena->base, arena->bytes);
        if (e != cudaSuccess)
        {
            arena->base = nullptr;
            cudaGetLastError();
            return fail(ASP_ERR_ALLOC, std::string("cudaMalloc of the plan arena failed: ") + cudaGetErrorString(e));
        }
    }
    if (!dry)
        for (auto &kv : placed)
            ASP_CUDA(cudaMemcpyAsync((char *)arena->base + kv.second.off, kv.first, kv.second.bytes, cudaMemcpyHostToDevice, ctx->stream));

    // ---- pass 2: build the kernel arguments
    auto dev_meta = [&](const HostMeta &h) {
        asp::Meta m;
        memset(&m, 0, sizeof(m));
        m.kind = h.kind;
        m.width = dtype_size(h.dtype);
        m.coef = h.coef;
        m.icpt = h.icpt;
        m.cycle = h.cycle;
        m.nb = h.nb;
        for (int b = 0; b < 5; b++)
        {
            m.bhi[b] = h.bhi[b];
            m.bval[b] = h.bval[b];
        }
        m.p = (h.kind == ASP_COMPRESS_NONE && h.p) ? (const void *)((char *)arena->base + placed[h.p].off) : nullptr;
        return m;
    };

    std::vector<asp_plan *> made;
    auto cleanup = [&]() {
        for (asp_plan *p : made) delete p;
        for (int i = 0; i < n; i++) out_plans[i] = nullptr;
    };
    for (int i = 0; i < n; i++)
    {
        const asp_plan_desc &d = descs[i];
        asp_plan *p = new (std::nothrow) asp_plan();
        if (!p)
        {
            cleanup();
            return fail(ASP_ERR_ALLOC, "host allocation failed");
        }
        made.push_back(p);
        out_plans[i] = p;
        p->arena = arena;
        p->templ = d.template_type;
        p->n_rows = d.n_rows;
        p->n_cols = d.n_cols;
        p->true_nnz = d.true_nnz;
        memset(&p->args, 0, sizeof(p->args));
        p->val_is_f64 = d.val_dtype == ASP_F64;
        if (d.template_type == ASP_EMPTY_TEMPLATE) continue;
        p->col_width = dtype_size(cols[i]->dtype);
        asp::KArgs &a = p->args;
        a.val = (char *)arena->base + placed[vals[i]->host_ptr].off;
        a.col = (char *)arena->base + placed[cols[i]->host_ptr].off;
        for (int s = 0; s < asp::MS_COUNT; s++)
            if (metas[i][s].present) a.m[s] = dev_meta(metas[i][s]);
        if (perms[i].present) a.perm = dev_meta(perms[i]);
        a.first_row = d.first_row;
        a.first_col = d.first_col;
        a.tlb_size = (unsigned)d.tlb_size;
        a.atomic = d.is_atom_add ? 1 : 0;
        a.sort_kind = perm_on_device(d.template_type) ? d.sort_kind : 0;
        a.row_add = (d.sort_kind == ASP_SORT_GLOBAL) ? 0 : 1;
        a.row_reduce = 1;
        a.bits_word = d.bits_word;
        a.bits_flag = d.bits_flag;
        a.bits_row = d.bits_row;
        a.bits_off = d.bits_off;
        const uint64_t nnz_pad = vals[i]->len;
        const std::vector<HostMeta> &hm = metas[i];
        uint64_t fmt = 0;
        for (int k = 0; k < d.n_arrays; k++)
            if (d.arrays[k].compress == ASP_COMPRESS_NONE) fmt += d.arrays[k].len * (uint64_t)dtype_size(d.arrays[k].dtype);
        p->fmt_bytes = fmt;

        std::string why;
        asp_status st = ASP_OK;
        switch (d.template_type)
        {
        case ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS:
        {
            const uint64_t P = hm[asp::MS_ROW_OF_TLB].len;
            a.n_tlb = P;
            a.n_units = P;
            a.effective = d.effective_num ? std::min<uint64_t>(d.effective_num, P) : P;
            if (d.tlb_size == 0 || P == 0 || P * d.tlb_size != nnz_pad) st = ASP_ERR_BOUNDS, why = "ELL-like: #TLB * TLB size != padded nnz";
            // TLBs per thread: the widest group that keeps 16-byte alignment of every k-slice
            int v = 4;
            while (v > 1 && (P % v) != 0) v >>= 1;
            p->vec = v;
            p->units_for_grid = (P + v - 1) / v;
            break;
        }
        case ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS:
        {
            const uint64_t B = hm[asp::MS_BLK_NZ].len;
            a.n_units = B;
            const uint64_t T = hm[asp::MS_ROW_OF_TLB].len;
            a.n_tlb = T;
            a.effective = d.effective_num ? std::min<uint64_t>(d.effective_num, T) : T;
            if (B == 0 || hm[asp::MS_BLK_THR].len != B + 1) st = ASP_ERR_BOUNDS, why = "SELL-like: block_begin_thread_index_offset must have #BLB + 1 entries";
            else
            {
                for (uint64_t b = 0; b < B && st == ASP_OK; b++)
                {
                    const uint64_t t0 = hm[asp::MS_BLK_THR].get(b), t1 = hm[asp::MS_BLK_THR].get(b + 1);
                    if (t1 < t0 || t1 > T || hm[asp::MS_BLK_NZ].get(b) + (t1 - t0) * hm[asp::MS_TLB_SIZE].get(b) > nnz_pad) st = ASP_ERR_BOUNDS, why = "SELL-like: a BLB reaches outside val_arr";
                }
            }
            {
                // 32 bytes of values per lane and k-step keep enough bytes in flight per warp; fp64
                // strips that are not a multiple of 128 TLBs fall back to 16-byte lanes
                const HostMeta &bt = hm[asp::MS_BLK_THR];
                const bool eq128 = bt.kind == ASP_COMPRESS_LINEAR && bt.coef > 0 && bt.coef % 128 == 0;
                p->vec = (p->val_is_f64 && !eq128) ? 2 : 4;
                p->sell_strip = (bt.kind == ASP_COMPRESS_LINEAR && bt.coef > 0) ? bt.coef : 0;
            }
            p->units_for_grid = B;
            // equal strips: the kernel walks warp tasks of 32 * vec TLBs (see k_sell)
            if (p->sell_strip && p->sell_strip % (32ull * p->vec) == 0) p->warp_tasks = B * (p->sell_strip / (32ull * p->vec));
            break;
        }
        case ASP_DIRECT_ATOM_TEMPLATE:
        case ASP_SHARED_MEMORY_TEMPLATE:
        {
            const uint64_t B = hm[asp::MS_BLK_NZ].len;
            a.n_units = B;
            a.n_tlb = hm[asp::MS_WARP_THR].len ? hm[asp::MS_WARP_THR].get(hm[asp::MS_WARP_THR].len - 1) : 0;
            a.effective = d.effective_num ? d.effective_num : ~0ull;
            if (B == 0 || hm[asp::MS_BLK_WARP].len != B + 1) st = ASP_ERR_BOUNDS, why = "3-level: block_begin_warp_index_offset must have #BLB + 1 entries";
            else
            {
                const uint64_t W = hm[asp::MS_WARP_NZ].len;
                uint64_t mx = 0;
                for (uint64_t b = 0; b < B && st == ASP_OK; b++)
                {
                    const uint64_t w0 = hm[asp::MS_BLK_WARP].get(b), w1 = hm[asp::MS_BLK_WARP].get(b + 1);
                    if (w1 < w0 || w1 > W || w1 + 1 > hm[asp::MS_WARP_THR].len) { st = ASP_ERR_BOUNDS; why = "3-level: WLB range outside the WLB arrays"; break; }
                    mx = std::max(mx, hm[asp::MS_WARP_THR].get(w1) - hm[asp::MS_WARP_THR].get(w0));
                }
                p->smem_elems = mx;
            }
            p->units_for_grid = B;
            break;
        }
        case ASP_SHARED_MEMORY_TEMPLATE_WARP_COMPRESS:
        {
            const uint64_t B = hm[asp::MS_BLK_NZ].len;
            a.n_units = B;
            a.effective = d.effective_num ? d.effective_num : ~0ull;
            if (B == 0 || hm[asp::MS_BLK_THR].len != B + 1 || hm[asp::MS_BLK_ROW].len != B + 1) st = ASP_ERR_BOUNDS, why = "row-grouped: offset arrays must have #BLB + 1 entries";
            else
            {
                uint64_t mx = 0;
                for (uint64_t b = 0; b < B && st == ASP_OK; b++)
                {
                    const uint64_t t0 = hm[asp::MS_BLK_THR].get(b), t1 = hm[asp::MS_BLK_THR].get(b + 1);
                    if (t1 < t0 || hm[asp::MS_BLK_NZ].get(b) + (t1 - t0) * hm[asp::MS_TLB_SIZE].get(b) > nnz_pad) { st = ASP_ERR_BOUNDS; why = "row-grouped: a BLB reaches outside val_arr"; break; }
                    mx = std::max(mx, t1 - t0);
                }
                p->smem_elems = mx;
                if (hm[asp::MS_BLK_ROW].get(B) + 1 > hm[asp::MS_ROW_OFF].len) st = ASP_ERR_BOUNDS, why = "row-grouped: row offsets shorter than the row count";
            }
            p->units_for_grid = B;
            break;
        }
        case ASP_SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE:
        {
            const uint64_t B = hm[asp::MS_BLK_ROW].len ? hm[asp::MS_BLK_ROW].len - 1 : 0;
            a.n_units = B;
            a.effective = d.effective_num ? d.effective_num : ~0ull;
            if (B == 0 || hm[asp::MS_BLK_WARP].len != B + 1) st = ASP_ERR_BOUNDS, why = "warp-reduce smem: offset arrays must have #BLB + 1 entries";
            else
            {
                uint64_t mx = 0;
                const uint64_t W1 = hm[asp::MS_WARP_NZ].len;
                for (uint64_t b = 0; b < B; b++)
                {
                    const uint64_t w0 = hm[asp::MS_BLK_WARP].get(b), w1 = hm[asp::MS_BLK_WARP].get(b + 1);
                    if (w1 < w0 || w1 + 1 > W1) { st = ASP_ERR_BOUNDS; why = "warp-reduce smem: WLB range outside global_warp_block_first_nz"; break; }
                    mx = std::max(mx, w1 - w0);
                }
                p->smem_elems = mx;
                if (st == ASP_OK && hm[asp::MS_WARP_NZ].get(W1 - 1) > nnz_pad) st = ASP_ERR_BOUNDS, why = "warp-reduce smem: last nz offset outside val_arr";
            }
            p->units_for_grid = B;
            break;
        }
        case ASP_SHARED_MEMORY_LONG_ROW_TEMPLATE:
        {
            const uint64_t B = hm[asp::MS_ROW_OF_UNIT].len;
            a.n_units = B;
            if (B == 0 || hm[asp::MS_BLK_NZ].len != B + 1) st = ASP_ERR_BOUNDS, why = "long-row: block_nz_begin_offset must have #BLB + 1 entries";
            else if (hm[asp::MS_BLK_NZ].get(B) > nnz_pad) st = ASP_ERR_BOUNDS, why = "long-row: last nz offset outside val_arr";
            p->units_for_grid = B;
            break;
        }
        case ASP_DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE:
        {
            const uint64_t W = hm[asp::MS_ROW_OF_UNIT].len;
            a.n_units = W;
            a.effective = d.effective_num ? std::min<uint64_t>(d.effective_num, W) : W;
            if (W == 0 || hm[asp::MS_WARP_NZ].len != W + 1) st = ASP_ERR_BOUNDS, why = "warp-per-row: global_warp_nz_begin_offset must have #WLB + 1 entries";
            else if (hm[asp::MS_WARP_NZ].get(W) > nnz_pad) st = ASP_ERR_BOUNDS, why = "warp-per-row: last nz offset outside val_arr";
            p->units_for_grid = W;
            break;
        }
        case ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE:
        case ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE:
        {
            const uint64_t T = hm[asp::MS_COMBINE].len;
            const uint64_t W = T / 32;
            a.n_units = W;
            a.n_tlb = T;
            a.warps_first_row_len = (int)std::min<uint64_t>(hm[asp::MS_ROW_OF_UNIT].len, 0x7fffffff);
            if (hm[asp::MS_COMBINE].kind != ASP_COMPRESS_NONE) st = ASP_ERR_INVALID_ARG, why = "CSR5-like: combine meta must be an array";
            else if (T == 0 || (T % 32) != 0 || d.tlb_size == 0 || T * d.tlb_size != nnz_pad) st = ASP_ERR_BOUNDS, why = "CSR5-like: #TLB * TLB size != padded nnz";
            else if (hm[asp::MS_ROW_OF_UNIT].len < W) st = ASP_ERR_BOUNDS, why = "CSR5-like: first-row array shorter than #WLB";
            else if (d.bits_word != 8 * dtype_size(hm[asp::MS_COMBINE].dtype) || d.bits_row <= 0 || d.bits_off <= 0 || (int)d.tlb_size + d.bits_row + d.bits_off > d.bits_word)
                st = ASP_ERR_INVALID_ARG, why = "CSR5-like: inconsistent combine-meta bit layout";
            p->units_for_grid = W;
            if (st == ASP_OK && !dry && d.n_rows <= 0xffffffffull && d.bits_word - (int)d.tlb_size >= 0 && d.tlb_size <= 64)
            {
                // first and last row of every warp, mapped to y (duplicates of neighbouring warps dropped)
                const HostMeta &cm = hm[asp::MS_COMBINE], &fr = hm[asp::MS_ROW_OF_UNIT], &pm = perms[i];
                const int S = (int)d.tlb_size, bw = d.bits_word;
                auto row_of = [&](uint64_t r) -> uint64_t {
                    if (d.sort_kind == ASP_SORT_GLOBAL) return pm.get(r + d.first_row);
                    if (d.sort_kind == ASP_SORT_LOCAL) return pm.get(r) + d.first_row;
                    return r + d.first_row;
                };
                std::vector<uint32_t> rows(2 * W);
                uint64_t all_starts = 0;
#pragma omp parallel for schedule(static) reduction(+ : all_starts)
                for (int64_t w = 0; w < (int64_t)W; w++)
                {
                    uint64_t starts = 0;
                    for (int l = 0; l < 32; l++)
                    {
                        const uint64_t m = cm.get((uint64_t)w * 32 + l);
                        const uint64_t flags = S >= 64 ? m : ((m >> (bw - S)) & ((1ull << S) - 1));
                        starts += (uint64_t)__builtin_popcountll(flags);
                    }
                    const uint64_t R0 = fr.get(w);
                    rows[2 * w] = (uint32_t)row_of(R0);
                    rows[2 * w + 1] = (uint32_t)row_of(R0 + (starts ? starts - 1 : 0));
                    all_starts += starts;
                }
                // staging area of the staged write-out: room for twice the average number of rows a warp produces
                // (a power of two between 32 and 256; warps with more rows send the rest straight out)
                {
                    const uint64_t avg = W ? all_starts / W : 1;
                    uint64_t cap = 32;
                    while (cap < 2 * avg && cap < 256) cap <<= 1;
                    a.stage_cap = (int)std::min<uint64_t>(cap, 32ull * S);
                }
                rows.erase(std::unique(rows.begin(), rows.end()), rows.end());
                std::shared_ptr<Arena> er(new (std::nothrow) Arena());
                if (!er || cudaMalloc(&er->base, std::max<size_t>(rows.size() * 4, 4)) != cudaSuccess)
                {
                    cudaGetLastError();
                    cleanup();
                    return fail(ASP_ERR_ALLOC, "allocation of the end-row list failed");
                }
                er->device = ctx->device;
                cudaError_t ce = cudaMemcpy(er->base, rows.data(), rows.size() * 4, cudaMemcpyHostToDevice);
                if (ce != cudaSuccess)
                {
                    cleanup();
                    return cuda_fail(ce, "upload of the end-row list");
                }
                p->end_rows = er;
                p->n_end_rows = rows.size();
            }
            break;
        }
        case ASP_BLOCK_ELL_TEMPLATE:
        {
            const uint64_t W = d.tlb_size, r = (uint64_t)d.bits_row, c = (uint64_t)d.bits_off;
            const uint64_t NB = W ? cols[i]->len / W : 0;
            a.n_tlb = NB;
            a.n_units = NB;
            a.effective = d.effective_num;
            if (!asp::block_ell_supported((int)r, (int)c)) st = ASP_ERR_UNSUPPORTED, why = "block-value template: blocks must be 2 x 2, 3 x 3 or 4 x 4";
            else if (cols[i]->dtype != ASP_U32) st = ASP_ERR_UNSUPPORTED, why = "block-value template: block-column indices must be u32";
            else if (W == 0 || NB == 0 || NB * W != cols[i]->len || (NB & 1) || nnz_pad != cols[i]->len * r * c)
                st = ASP_ERR_BOUNDS, why = "block-value template: arrays do not match slots x padded block rows x r x c";
            else if (d.effective_num == 0 || d.effective_num > NB * r || d.first_row + d.effective_num > d.n_rows)
                st = ASP_ERR_BOUNDS, why = "block-value template: rows of the sub-matrix outside y or the block rows";
            else if (d.sort_kind != ASP_SORT_NONE || d.is_atom_add) st = ASP_ERR_UNSUPPORTED, why = "block-value template: neither sorted nor column-sliced matrices";
            p->units_for_grid = NB / 2;
            break;
        }
        case ASP_DIAG_TEMPLATE:
        {
            const uint64_t D = d.tlb_size, V = p->val_is_f64 ? 2 : 4;
            const uint64_t NR = D ? nnz_pad / D : 0;
            a.n_tlb = NR;
            a.n_units = d.n_cols - d.first_col; // the offsets are biased by this
            a.effective = d.effective_num;
            if (D == 0 || D != cols[i]->len || NR * D != nnz_pad || NR == 0 || (NR % V) != 0) st = ASP_ERR_BOUNDS, why = "diagonal-value template: values do not match diagonals x padded rows";
            else if (d.effective_num == 0 || d.effective_num > NR || d.first_row + d.effective_num > d.n_rows) st = ASP_ERR_BOUNDS, why = "diagonal-value template: rows of the sub-matrix outside y or the padded rows";
            else if (d.sort_kind != ASP_SORT_NONE || d.is_atom_add) st = ASP_ERR_UNSUPPORTED, why = "diagonal-value template: neither sorted nor column-sliced matrices";
            p->units_for_grid = NR / V;
            break;
        }
        default: st = ASP_ERR_UNSUPPORTED; why = "template not implemented"; break;
        }
        if (st == ASP_OK && !validate_contents(d, hm, perms[i], cols[i], a, why)) st = ASP_ERR_BOUNDS;
        if (st != ASP_OK)
        {
            cleanup();
            return fail(st, why);
        }
        if (is_smem_family(d.template_type))
        {
            p->smem = align_up((size_t)p->smem_elems * (p->val_is_f64 ? 8 : 4), 16);
            if (p->smem > (size_t)(dry ? 227 * 1024 : ctx->max_smem_optin))
            {
                cleanup();
                return fail(ASP_ERR_UNSUPPORTED, "partial results of one BLB do not fit in shared memory");
            }
            cudaError_t e = dry ? cudaSuccess : asp::allow_dynamic_smem(d.template_type, p->val_is_f64, p->col_width, p->smem);
            if (e != cudaSuccess)
            {
                cleanup();
                return cuda_fail(e, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
            }
        }
        p->needs_zero = a.atomic != 0 || d.template_type == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE ||
                        d.template_type == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE;
        st = apply_launch(ctx, p, d.tblock_num, d.thread_num_in_block > 0 ? d.thread_num_in_block : 256, d.thread_num_of_row_reduce);
        if (st != ASP_OK)
        {
            cleanup();
            return st;
        }
    }
    if (dry)
    {
        cleanup();
        return ASP_OK;
    }
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess)
    {
        cleanup();
        return cuda_fail(e, "plan upload");
    }
    return ASP_OK;
}
} // namespace

extern "C" {

asp_status asp_plan_group_create(asp_ctx *ctx, const asp_plan_desc *descs, int n, asp_plan **out_plans)
{
    if (!ctx || !descs || !out_plans || n <= 0) return fail(ASP_ERR_INVALID_ARG, "NULL argument or n <= 0");
    for (int i = 0; i < n; i++) out_plans[i] = nullptr;
    ASP_ON_DEVICE(ctx);
    return plan_group_build(ctx, descs, n, out_plans, false);
}

asp_status asp_plan_descs_validate(const asp_plan_desc *descs, int n)
{
    if (!descs || n <= 0) return fail(ASP_ERR_INVALID_ARG, "NULL argument or n <= 0");
    std::vector<asp_plan *> scratch((size_t)n, nullptr);
    return plan_group_build(nullptr, descs, n, scratch.data(), true);
}

void asp_plan_destroy(asp_plan *plan) { delete plan; }

asp_status asp_plan_set_launch(asp_plan *plan, int64_t tblock_num, int64_t thread_num_in_block, int64_t thread_num_of_row_reduce)
{
    if (!plan) return fail(ASP_ERR_INVALID_ARG, "plan is NULL");
    if (plan->templ == ASP_EMPTY_TEMPLATE) return ASP_OK;
    return apply_launch(nullptr, plan, tblock_num, thread_num_in_block, thread_num_of_row_reduce);
}

asp_status asp_plan_get_launch(const asp_plan *plan, int64_t *tblock_num, int64_t *thread_num_in_block, int64_t *thread_num_of_row_reduce)
{
    if (!plan) return fail(ASP_ERR_INVALID_ARG, "plan is NULL");
    const bool empty = plan->templ == ASP_EMPTY_TEMPLATE;
    if (tblock_num) *tblock_num = empty ? 0 : (int64_t)plan->grid;
    if (thread_num_in_block) *thread_num_in_block = empty ? 0 : (int64_t)plan->block;
    if (thread_num_of_row_reduce) *thread_num_of_row_reduce = empty ? 0 : (int64_t)plan->args.row_reduce;
    return ASP_OK;
}

asp_status asp_plan_set_tuning(asp_plan *plan, int vec, int path)
{
    if (!plan) return fail(ASP_ERR_INVALID_ARG, "plan is NULL");
    const int t = plan->templ;
    if (t == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE || t == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE)
    {
        if (vec != 0) return fail(ASP_ERR_INVALID_ARG, "the CSR5-like family has no vec knob");
        if (path >= 0)
        {
            // bit 0: staged write-out; bits 4..7 (optional): log2 of the rows per warp that are staged
            // bit 1: rows stored one by one by the kernel that takes any TLB size at run time (for comparisons)
            plan->args.path = path & 3;
            plan->args.row_reduce = (path & 1) ? 2 : 1;
            const int lg = (path >> 4) & 0xf;
            if (lg) plan->args.stage_cap = (int)std::min<uint64_t>(1ull << lg, 32ull * plan->args.tlb_size);
        }
        return ASP_OK;
    }
    if (t != ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS && t != ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS)
        return fail(ASP_ERR_UNSUPPORTED, "only the ELL-like, SELL-like and CSR5-like families have tuning knobs");
    if (vec != 0 && vec != 1 && vec != 2 && vec != 4 && vec != 8) return fail(ASP_ERR_INVALID_ARG, "vec must be 0 (keep), 1, 2, 4 or 8");
    if (t == ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS)
    {
        if (vec)
        {
            if (plan->args.n_tlb % (uint64_t)vec) return fail(ASP_ERR_INVALID_ARG, "vec must divide the padded TLB count");
            plan->vec = vec;
            plan->units_for_grid = (plan->args.n_tlb + vec - 1) / vec;
        }
    }
    else
    {
        if (vec == 8) return fail(ASP_ERR_INVALID_ARG, "the SELL-like family takes vec 1, 2 or 4");
        if (vec) plan->vec = vec;
        if (path >= 0) plan->args.path = path;
        plan->warp_tasks = 0;
        if ((plan->args.path & 1) == 0 && plan->sell_strip && plan->sell_strip % (32ull * plan->vec) == 0)
            plan->warp_tasks = plan->args.n_units * (plan->sell_strip / (32ull * plan->vec));
    }
    if (plan->asked_threads > 0) return apply_launch(nullptr, plan, plan->asked_tblock, plan->asked_threads, plan->asked_reduce);
    return ASP_OK;
}

uint64_t asp_plan_format_bytes(const asp_plan *plan) { return plan ? plan->fmt_bytes : 0; }
int asp_plan_launches(const asp_plan *plan) { return (plan && plan->templ != ASP_EMPTY_TEMPLATE) ? 1 : 0; }
uint64_t asp_plan_end_rows(const asp_plan *plan) { return plan ? plan->n_end_rows : 0; }

} // extern "C"

namespace
{
// x / y lengths and the value size of a plan group: from the first plan that has a kernel, else from
// plans[0] (a group of EMPTY plans still describes a matrix: y = 0)
struct GroupShape
{
    const asp_plan *first = nullptr; // first non-EMPTY plan, may stay NULL
    uint64_t n_rows = 0, n_cols = 0;
    size_t es = 4;
};
asp_status group_shape(asp_plan *const *plans, int n_plans, GroupShape *g)
{
    for (int i = 0; i < n_plans; i++)
    {
        if (!plans[i]) return fail(ASP_ERR_INVALID_ARG, "NULL plan");
        if (plans[i]->templ != ASP_EMPTY_TEMPLATE && !g->first) g->first = plans[i];
    }
    const asp_plan *ref = g->first ? g->first : plans[0];
    g->n_rows = ref->n_rows;
    g->n_cols = ref->n_cols;
    g->es = ref->val_is_f64 ? 8 : 4;
    for (int i = 0; i < n_plans; i++)
        if (plans[i]->val_is_f64 != ref->val_is_f64 || plans[i]->n_rows != ref->n_rows || plans[i]->n_cols != ref->n_cols)
            return fail(ASP_ERR_INVALID_ARG, "plans of different matrices in one call");
    return ASP_OK;
}
} // namespace

extern "C" {

asp_status asp_spmv(asp_ctx *ctx, asp_plan *const *plans, int n_plans, const void *d_x, void *d_y, int zero_y)
{
    if (!ctx || !plans || n_plans <= 0 || !d_x || !d_y) return fail(ASP_ERR_INVALID_ARG, "NULL argument");
    GroupShape g;
    asp_status gs = group_shape(plans, n_plans, &g);
    if (gs != ASP_OK) return gs;
    ASP_ON_DEVICE(ctx);
    bool clear = zero_y == 1;
    if (zero_y == 2)
    {
        // a group without any kernel is the zero matrix: "clear when needed" means clear
        clear = g.first == nullptr;
        for (int i = 0; i < n_plans; i++) clear = clear || (plans[i]->templ != ASP_EMPTY_TEMPLATE && plans[i]->needs_zero);
    }
    if (clear) ASP_CUDA(cudaMemsetAsync(d_y, 0, g.n_rows * g.es, ctx->stream));
    if (!g.first) return ASP_OK;
    int active = 0;
    for (int i = 0; i < n_plans; i++) active += plans[i]->templ != ASP_EMPTY_TEMPLATE;
    const bool fork = active > 1;
    if (fork) ASP_CUDA(cudaEventRecord(ctx->ev_fork, ctx->stream));
    bool used[asp_ctx::kAux] = {false, false, false};
    int k = 0;
    asp_status result = ASP_OK;
    for (int i = 0; i < n_plans && result == ASP_OK; i++)
    {
        const asp_plan *p = plans[i];
        if (p->templ == ASP_EMPTY_TEMPLATE) continue;
        cudaStream_t st = ctx->stream;
        if (fork && k > 0)
        {
            const int j = (k - 1) % asp_ctx::kAux;
            st = ctx->aux[j];
            if (!used[j])
            {
                cudaError_t e = cudaStreamWaitEvent(st, ctx->ev_fork, 0);
                if (e != cudaSuccess)
                {
                    result = cuda_fail(e, "cudaStreamWaitEvent");
                    break;
                }
                used[j] = true;
            }
        }
        k++;
        asp::KArgs args = p->args; // plans are shared, read-only objects: x / y travel in a copy
        args.x = d_x;
        args.y = d_y;
        cudaError_t e = asp::launch_template(p->templ, p->val_is_f64, p->col_width, args, p->grid, p->block, p->smem, st, p->vec);
        if (e != cudaSuccess) result = cuda_fail(e, "kernel launch");
    }
    // always join the side streams that were forked, also after a failed launch
    for (int j = 0; j < asp_ctx::kAux; j++)
        if (used[j])
        {
            cudaError_t e = cudaEventRecord(ctx->ev_join[j], ctx->aux[j]);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->stream, ctx->ev_join[j], 0);
            if (e != cudaSuccess && result == ASP_OK) result = cuda_fail(e, "joining a side stream");
        }
    return result;
}

asp_status asp_spmv_host(asp_ctx *ctx, asp_plan *const *plans, int n_plans, const void *h_x, void *h_y)
{
    if (!ctx || !plans || n_plans <= 0 || !h_x || !h_y) return fail(ASP_ERR_INVALID_ARG, "NULL argument");
    GroupShape g;
    asp_status st = group_shape(plans, n_plans, &g);
    if (st != ASP_OK) return st;
    ASP_ON_DEVICE(ctx);
    const size_t xb = g.n_cols * g.es, yb = g.n_rows * g.es;
    st = ensure_xy(ctx, xb, yb);
    if (st != ASP_OK) return st;
    ASP_CUDA(cudaMemcpyAsync(ctx->x, h_x, xb, cudaMemcpyHostToDevice, ctx->stream));
    st = asp_spmv(ctx, plans, n_plans, ctx->x, ctx->y, 1);
    if (st != ASP_OK) return st;
    ASP_CUDA(cudaMemcpyAsync(h_y, ctx->y, yb, cudaMemcpyDeviceToHost, ctx->stream));
    ASP_CUDA(cudaStreamSynchronize(ctx->stream));
    return ASP_OK;
}

asp_status asp_spmv_host_pipelined(asp_ctx *ctx, const asp_host_chunk *chunks, int n_chunks, const void *h_x, void *h_y)
{
    if (!ctx || !chunks || n_chunks <= 0 || !h_x || !h_y) return fail(ASP_ERR_INVALID_ARG, "NULL argument or no chunks");
    // the chunks tile the rows in ascending order; every group spans all columns of the same matrix
    uint64_t n_rows = 0, n_cols = 0;
    size_t es = 0;
    for (int c = 0; c < n_chunks; c++)
    {
        const asp_host_chunk &ch = chunks[c];
        if (!ch.plans || ch.n_plans <= 0) return fail(ASP_ERR_INVALID_ARG, "chunk without plans");
        if (ch.row_lo != n_rows || ch.row_hi <= ch.row_lo) return fail(ASP_ERR_INVALID_ARG, "the chunks must tile the rows in ascending order");
        GroupShape g;
        asp_status gs = group_shape(ch.plans, ch.n_plans, &g);
        if (gs != ASP_OK) return gs;
        if (g.n_rows != ch.row_hi - ch.row_lo) return fail(ASP_ERR_INVALID_ARG, "a chunk's plan group has another number of rows than the chunk");
        if (c == 0)
        {
            n_cols = g.n_cols;
            es = g.es;
        }
        else if (g.n_cols != n_cols || g.es != es) return fail(ASP_ERR_INVALID_ARG, "the chunks belong to different matrices");
        if (ch.col_hi == 0 || ch.col_hi > n_cols) return fail(ASP_ERR_INVALID_ARG, "col_hi outside the matrix");
        n_rows = ch.row_hi;
    }
    ASP_ON_DEVICE(ctx);
    asp_status st = ensure_xy(ctx, n_cols * es, n_rows * es);
    if (st != ASP_OK) return st;
    if (!ctx->h2d) ASP_CUDA(cudaStreamCreateWithFlags(&ctx->h2d, cudaStreamNonBlocking));
    if (!ctx->d2h) ASP_CUDA(cudaStreamCreateWithFlags(&ctx->d2h, cudaStreamNonBlocking));
    while (ctx->pipe_events.size() < 2 * (size_t)n_chunks + 1)
    {
        cudaEvent_t e = nullptr;
        ASP_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        ctx->pipe_events.push_back(e);
    }
    // whatever ran on the context's stream before (an earlier SpMV reading x, writing y) is finished first
    cudaEvent_t start = ctx->pipe_events[2 * (size_t)n_chunks];
    ASP_CUDA(cudaEventRecord(start, ctx->stream));
    ASP_CUDA(cudaStreamWaitEvent(ctx->h2d, start, 0));
    uint64_t uploaded = 0; // x[0, uploaded) is on its way to the device
    for (int c = 0; c < n_chunks; c++)
    {
        const asp_host_chunk &ch = chunks[c];
        cudaEvent_t x_in = ctx->pipe_events[2 * (size_t)c], y_done = ctx->pipe_events[2 * (size_t)c + 1];
        if (ch.col_hi > uploaded)
        {
            ASP_CUDA(cudaMemcpyAsync((unsigned char *)ctx->x + uploaded * es, (const unsigned char *)h_x + uploaded * es, (ch.col_hi - uploaded) * es,
                                     cudaMemcpyHostToDevice, ctx->h2d));
            uploaded = ch.col_hi;
            ASP_CUDA(cudaEventRecord(x_in, ctx->h2d));
            ASP_CUDA(cudaStreamWaitEvent(ctx->stream, x_in, 0));
        }
        unsigned char *y = (unsigned char *)ctx->y + ch.row_lo * es;
        st = asp_spmv(ctx, ch.plans, ch.n_plans, ctx->x, y, 1);
        if (st != ASP_OK) break;
        ASP_CUDA(cudaEventRecord(y_done, ctx->stream));
        ASP_CUDA(cudaStreamWaitEvent(ctx->d2h, y_done, 0));
        ASP_CUDA(cudaMemcpyAsync((unsigned char *)h_y + ch.row_lo * es, y, (ch.row_hi - ch.row_lo) * es, cudaMemcpyDeviceToHost, ctx->d2h));
    }
    // nothing is left in flight when the call returns, also after an error
    cudaError_t e1 = cudaStreamSynchronize(ctx->h2d), e2 = cudaStreamSynchronize(ctx->stream), e3 = cudaStreamSynchronize(ctx->d2h);
    if (st != ASP_OK) return st;
    if (e1 != cudaSuccess) return cuda_fail(e1, "host-to-device copies");
    if (e2 != cudaSuccess) return cuda_fail(e2, "kernels");
    if (e3 != cudaSuccess) return cuda_fail(e3, "device-to-host copies");
    return ASP_OK;
}

asp_status asp_spmv_publish(asp_ctx *ctx, asp_plan *const *plans, int n_plans, const void *d_x, void *d_y, void *d_y_multicast)
{
    if (!ctx || !plans || n_plans <= 0 || !d_x || !d_y || !d_y_multicast) return fail(ASP_ERR_INVALID_ARG, "NULL argument");
    GroupShape g;
    asp_status gs = group_shape(plans, n_plans, &g);
    if (gs != ASP_OK) return gs;
    for (int i = 0; i < n_plans; i++)
    {
        const asp_plan *p = plans[i];
        if (p->templ == ASP_EMPTY_TEMPLATE) continue;
        const bool csr5 = p->templ == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE || p->templ == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE;
        if (!csr5 || !p->end_rows || p->args.atomic || !asp::csr5_specialised((int)p->args.tlb_size, p->col_width, p->args.bits_word))
            return fail(ASP_ERR_UNSUPPORTED, "publishing SpMV: every plan must be a CSR5-like template with TLB size 4, 8, 16 or 32 and 32-bit columns");
    }
    ASP_ON_DEVICE(ctx);
    // the three steps of every plan run back to back on the context's stream
    for (int i = 0; i < n_plans; i++)
    {
        const asp_plan *p = plans[i];
        if (p->templ == ASP_EMPTY_TEMPLATE) continue;
        ASP_CUDA(asp::launch_zero_rows(p->val_is_f64, d_y, (const unsigned *)p->end_rows->base, p->n_end_rows, ctx->stream));
    }
    for (int i = 0; i < n_plans; i++)
    {
        const asp_plan *p = plans[i];
        if (p->templ == ASP_EMPTY_TEMPLATE) continue;
        asp::KArgs args = p->args;
        args.x = d_x;
        args.y = d_y;
        args.y_mc = d_y_multicast;
        ASP_CUDA(asp::launch_template(p->templ, p->val_is_f64, p->col_width, args, p->grid, p->block, p->smem, ctx->stream, p->vec));
    }
    for (int i = 0; i < n_plans; i++)
    {
        const asp_plan *p = plans[i];
        if (p->templ == ASP_EMPTY_TEMPLATE) continue;
        ASP_CUDA(asp::launch_publish_rows(p->val_is_f64, d_y, d_y_multicast, (const unsigned *)p->end_rows->base, p->n_end_rows, ctx->stream));
    }
    return ASP_OK;
}

// ---------------------------------------------------------------------------------------------
// asp_spmv_host_static: the host-buffer SpMV without any allocation.
//
// Who needs it: a solver that has handed the whole device to its own memory pool (a cudaMalloc
// from this library would fail, or break the pool's accounting), and a control loop that cannot
// tolerate the device-wide synchronisation cudaMalloc / cudaFree imply. asp_spmv_host stages x
// and y in buffers it allocates on first use and grows on demand; this variant stages them in the
// fixed array below instead. Every GPU that loads the library holds the array until the process
// exits, which is why it is kept modest: x lives in the first half, y in the second, so
// n_cols * sizeof(value) and n_rows * sizeof(value) must each fit in ASP_STATIC_STAGE_BYTES / 2.
//
// In host code `g_static_stage` is only a handle for the device symbol, not a device address; the
// address is looked up with cudaGetSymbolAddress once per device (with that device current) on
// the first call made for that device, and cached. That first call should therefore be made
// during set-up, before any stream capture is started.
//
// All calls share the array and it keeps whatever the previous call left in it: the y half is
// cleared at the start of every call, the x half is overwritten. Two calls that overlap in time
// on one GPU (different contexts or host threads) race on it; serialise them.
// ---------------------------------------------------------------------------------------------
#define ASP_STATIC_STAGE_BYTES (16u << 20)
static __device__ __align__(256) unsigned char g_static_stage[ASP_STATIC_STAGE_BYTES];

namespace
{
const int kMaxDevices = 64;
unsigned char *g_static_stage_addr[kMaxDevices]; // per device, filled on first use

asp_status static_stage_address(asp_ctx *ctx, unsigned char **out)
{
    // (called with ctx->device current; the table is written with the same value by whichever
    // thread gets there first)
    if (ctx->device < 0 || ctx->device >= kMaxDevices) return fail(ASP_ERR_UNSUPPORTED, "device ordinal too large for the static staging table");
    if (!g_static_stage_addr[ctx->device])
    {
        void *p = nullptr;
        ASP_CUDA(cudaGetSymbolAddress(&p, g_static_stage));
        g_static_stage_addr[ctx->device] = (unsigned char *)p;
    }
    *out = g_static_stage_addr[ctx->device];
    return ASP_OK;
}
} // namespace

asp_status asp_spmv_host_static(asp_ctx *ctx, asp_plan *const *plans, int n_plans, const void *h_x, void *h_y)
{
    if (!ctx || !plans || n_plans <= 0 || !h_x || !h_y) return fail(ASP_ERR_INVALID_ARG, "NULL argument");
    GroupShape g;
    asp_status st = group_shape(plans, n_plans, &g);
    if (st != ASP_OK) return st;
    const size_t xb = g.n_cols * g.es, yb = g.n_rows * g.es;
    const size_t half = ASP_STATIC_STAGE_BYTES / 2;
    if (xb > half || yb > half)
        return fail(ASP_ERR_INVALID_ARG, "matrix too large for the static staging area: x and y must each fit in " + std::to_string(half) + " bytes");
    ASP_ON_DEVICE(ctx);
    unsigned char *stage = nullptr;
    st = static_stage_address(ctx, &stage);
    if (st != ASP_OK) return st;
    unsigned char *sx = stage, *sy = stage + half;
    ASP_CUDA(cudaMemcpyAsync(sx, h_x, xb, cudaMemcpyHostToDevice, ctx->stream));
    st = asp_spmv(ctx, plans, n_plans, sx, sy, 1); // zero_y = 1: the y half still holds the previous call's result
    if (st != ASP_OK) return st;
    ASP_CUDA(cudaMemcpyAsync(h_y, sy, yb, cudaMemcpyDeviceToHost, ctx->stream));
    ASP_CUDA(cudaStreamSynchronize(ctx->stream));
    return ASP_OK;
}

uint64_t asp_static_stage_bytes(void) { return ASP_STATIC_STAGE_BYTES; }

asp_status asp_time(asp_ctx *ctx, asp_plan *const *plans, int n_plans, int warmup, int reps, int zero_y,
                    double gflops_up_bound, float *ms_per_spmv, float *gflops)
{
    if (!ctx || !plans || n_plans <= 0 || reps <= 0 || !ms_per_spmv) return fail(ASP_ERR_INVALID_ARG, "NULL argument or reps <= 0");
    GroupShape g;
    asp_status st = group_shape(plans, n_plans, &g);
    if (st != ASP_OK) return st;
    ASP_ON_DEVICE(ctx);
    const size_t es = g.es;
    const size_t xn = g.n_cols, yn = g.n_rows;
    st = ensure_xy(ctx, xn * es, yn * es);
    if (st != ASP_OK) return st;
    {
        // x = 100 everywhere, as the reference's generated main() sets it (code_builder.cc:1508-1509)
        std::vector<char> hx(xn * es);
        if (es == 8) std::fill((double *)hx.data(), (double *)hx.data() + xn, 100.0);
        else std::fill((float *)hx.data(), (float *)hx.data() + xn, 100.0f);
        ASP_CUDA(cudaMemcpyAsync(ctx->x, hx.data(), xn * es, cudaMemcpyHostToDevice, ctx->stream));
        ASP_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    for (int i = 0; i < warmup; i++)
    {
        st = asp_spmv(ctx, plans, n_plans, ctx->x, ctx->y, zero_y);
        if (st != ASP_OK) return st;
    }
    ASP_CUDA(cudaStreamSynchronize(ctx->stream));
    ASP_CUDA(cudaEventRecord(ctx->ev0, ctx->stream));
    for (int i = 0; i < reps; i++)
    {
        st = asp_spmv(ctx, plans, n_plans, ctx->x, ctx->y, zero_y);
        if (st != ASP_OK) return st;
    }
    ASP_CUDA(cudaEventRecord(ctx->ev1, ctx->stream));
    ASP_CUDA(cudaEventSynchronize(ctx->ev1));
    float ms = 0;
    ASP_CUDA(cudaEventElapsedTime(&ms, ctx->ev0, ctx->ev1));
    ms /= (float)reps;
    *ms_per_spmv = ms;
    uint64_t nnz = 0;
    for (int i = 0; i < n_plans; i++) nnz += plans[i]->true_nnz;
    const double gf = ms > 0 ? 2.0 * (double)nnz * 1e-6 / ms : 0.0;
    if (gflops) *gflops = (float)gf;
    if (gflops_up_bound > 0 && gf > gflops_up_bound) return fail(ASP_ERR_IMPLAUSIBLE, "throughput above the configured GFLOPS_UP_BOUND");
    return ASP_OK;
}

// ---- the sharded repeated SpMV as a native loop -------------------------------------------------
struct asp_dist
{
    asp_ctx *ctx = nullptr;
    int rank = 0, world = 1;
    size_t es = 4;
    uint64_t n = 0;
    struct Chunk
    {
        std::vector<asp_plan *> plans;
        uint64_t lo = 0, hi = 0;
        cudaEvent_t done = nullptr; // the chunk's kernels have finished (recorded on the context's stream)
    };
    std::vector<Chunk> chunks;
    cudaStream_t comm = nullptr;   // carries the store passes and the barrier, under the next chunk's kernels
    cudaEvent_t exchanged = nullptr;
    const void *flags_local = nullptr;
    void *flags_mc = nullptr;
    unsigned *status = nullptr;    // device word the barrier kernel reports to
    unsigned epoch = 0, max_polls = 0;
};

asp_status asp_dist_create(asp_ctx *ctx, const asp_dist_desc *desc, asp_dist **out)
{
    if (!out) return fail(ASP_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    if (!ctx || !desc || !desc->chunks || desc->n_chunks <= 0) return fail(ASP_ERR_INVALID_ARG, "NULL argument or no chunks");
    if (desc->world < 1 || desc->world > 32 || desc->rank < 0 || desc->rank >= desc->world) return fail(ASP_ERR_INVALID_ARG, "rank / world out of range (at most 32 ranks)");
    if (desc->world > 1 && (!desc->flags_local || !desc->flags_multicast)) return fail(ASP_ERR_INVALID_ARG, "more than one rank needs the symmetric flag array");
    std::unique_ptr<asp_dist, void (*)(asp_dist *)> d(new (std::nothrow) asp_dist(), asp_dist_destroy);
    if (!d) return fail(ASP_ERR_ALLOC, "host allocation failed");
    d->ctx = ctx;
    d->rank = desc->rank;
    d->world = desc->world;
    d->es = desc->value_is_f64 ? 8 : 4;
    d->n = desc->n;
    d->flags_local = desc->flags_local;
    d->flags_mc = desc->flags_multicast;
    d->max_polls = desc->max_polls;
    // the chunks must tile one contiguous row block and agree with their plan groups
    std::vector<std::pair<uint64_t, uint64_t>> spans;
    for (int c = 0; c < desc->n_chunks; c++)
    {
        const asp_dist_chunk &in = desc->chunks[c];
        if (in.row_hi < in.row_lo || in.row_hi > desc->n) return fail(ASP_ERR_INVALID_ARG, "chunk rows outside the vector");
        if (in.n_plans < 0 || (in.n_plans > 0 && !in.plans)) return fail(ASP_ERR_INVALID_ARG, "chunk without plans");
        asp_dist::Chunk ch;
        ch.lo = in.row_lo;
        ch.hi = in.row_hi;
        if (in.n_plans > 0)
        {
            GroupShape g;
            asp_status gs = group_shape(in.plans, in.n_plans, &g);
            if (gs != ASP_OK) return gs;
            if (g.n_rows != in.row_hi - in.row_lo) return fail(ASP_ERR_INVALID_ARG, "a chunk's plan group has another number of rows than the chunk");
            if (g.n_cols != desc->n) return fail(ASP_ERR_INVALID_ARG, "a chunk's plan group has another number of columns than the vector");
            if (g.es != d->es) return fail(ASP_ERR_INVALID_ARG, "a chunk's plan group has another value type");
            ch.plans.assign(in.plans, in.plans + in.n_plans);
        }
        if (ch.hi > ch.lo) spans.push_back({ch.lo, ch.hi});
        d->chunks.push_back(std::move(ch));
    }
    std::sort(spans.begin(), spans.end());
    for (size_t i = 1; i < spans.size(); i++)
        if (spans[i].first != spans[i - 1].second) return fail(ASP_ERR_INVALID_ARG, "the chunks do not tile one contiguous row block");
    ASP_ON_DEVICE(ctx);
    for (auto &ch : d->chunks) ASP_CUDA(cudaEventCreateWithFlags(&ch.done, cudaEventDisableTiming));
    if (d->world > 1)
    {
        ASP_CUDA(cudaStreamCreateWithFlags(&d->comm, cudaStreamNonBlocking));
        ASP_CUDA(cudaEventCreateWithFlags(&d->exchanged, cudaEventDisableTiming));
        ASP_CUDA(cudaMalloc((void **)&d->status, 256));
        ASP_CUDA(cudaMemsetAsync(d->status, 0, 256, ctx->stream));
    }
    *out = d.release();
    return ASP_OK;
}

void asp_dist_destroy(asp_dist *d)
{
    if (!d) return;
    if (d->ctx)
    {
        DeviceGuard guard(d->ctx->device);
        if (d->comm) cudaStreamSynchronize(d->comm);
        for (auto &ch : d->chunks)
            if (ch.done) cudaEventDestroy(ch.done);
        if (d->exchanged) cudaEventDestroy(d->exchanged);
        if (d->comm) cudaStreamDestroy(d->comm);
        if (d->status) cudaFree(d->status);
    }
    delete d;
}

asp_status asp_dist_spmv(asp_dist *d, const void *d_x, void *d_y, void *d_y_multicast)
{
    if (!d || !d_x || !d_y) return fail(ASP_ERR_INVALID_ARG, "NULL argument");
    if (d->world > 1 && !d_y_multicast) return fail(ASP_ERR_INVALID_ARG, "more than one rank needs the multicast address of y");
    if (d_x == d_y) return fail(ASP_ERR_INVALID_ARG, "x and y must be different buffers");
    asp_ctx *ctx = d->ctx;
    ASP_ON_DEVICE(ctx);
    for (auto &ch : d->chunks)
    {
        const size_t off = (size_t)ch.lo * d->es, bytes = (size_t)(ch.hi - ch.lo) * d->es;
        if (bytes == 0) continue;
        unsigned char *dst = (unsigned char *)d_y + off;
        if (ch.plans.empty()) ASP_CUDA(cudaMemsetAsync(dst, 0, bytes, ctx->stream));
        else
        {
            // rows without non-zeros are never stored by a kernel: clear the slice first
            asp_status st = asp_spmv(ctx, ch.plans.data(), (int)ch.plans.size(), d_x, dst, 1);
            if (st != ASP_OK) return st;
        }
        if (d->world == 1) continue;
        ASP_CUDA(cudaEventRecord(ch.done, ctx->stream));
        ASP_CUDA(cudaStreamWaitEvent(d->comm, ch.done, 0));
        asp_status st = asp_multicast_store(dst, (unsigned char *)d_y_multicast + off, bytes, d->comm, 0);
        if (st != ASP_OK) return fail(st, "multicast store pass refused (buffers must be congruent modulo 16)");
    }
    if (d->world == 1) return ASP_OK;
    // every rank's stores are in every replica past the barrier; the next SpMV waits for it
    asp_status st = asp_rank_barrier(d->flags_local, d->flags_mc, d->rank, d->world, ++d->epoch, d->status, d->max_polls, d->comm);
    if (st != ASP_OK) return fail(st, "barrier kernel launch failed");
    ASP_CUDA(cudaEventRecord(d->exchanged, d->comm));
    ASP_CUDA(cudaStreamWaitEvent(ctx->stream, d->exchanged, 0));
    return ASP_OK;
}

asp_status asp_dist_spmv_iter(asp_dist *d, const void *d_x0, void *const d_buf[2], void *const d_buf_multicast[2], int iters, int *final_buf)
{
    if (!d || !d_x0 || !d_buf || !d_buf[0] || !d_buf[1] || iters < 0) return fail(ASP_ERR_INVALID_ARG, "NULL argument or negative iteration count");
    if (d->world > 1 && (!d_buf_multicast || !d_buf_multicast[0] || !d_buf_multicast[1])) return fail(ASP_ERR_INVALID_ARG, "more than one rank needs the multicast addresses of both buffers");
    if (d_x0 == d_buf[0] || d_x0 == d_buf[1] || d_buf[0] == d_buf[1]) return fail(ASP_ERR_INVALID_ARG, "x0 and the two buffers must be three different vectors");
    const void *x = d_x0;
    int last = -1;
    for (int i = 0; i < iters; i++)
    {
        const int b = i & 1;
        asp_status st = asp_dist_spmv(d, x, d_buf[b], d->world > 1 ? d_buf_multicast[b] : nullptr);
        if (st != ASP_OK) return st;
        x = d_buf[b];
        last = b;
    }
    if (final_buf) *final_buf = last;
    return ASP_OK;
}

asp_status asp_dist_status(asp_dist *d, int *waiting_for_rank)
{
    if (!d) return fail(ASP_ERR_INVALID_ARG, "NULL argument");
    if (waiting_for_rank) *waiting_for_rank = -1;
    ASP_ON_DEVICE(d->ctx);
    ASP_CUDA(cudaStreamSynchronize(d->ctx->stream));
    if (!d->status) return ASP_OK;
    unsigned v = 0;
    ASP_CUDA(cudaMemcpy(&v, d->status, sizeof(v), cudaMemcpyDeviceToHost));
    if (v == 0) return ASP_OK;
    if (waiting_for_rank) *waiting_for_rank = (int)v - 1;
    return fail(ASP_ERR_TIMEOUT, "a barrier of the sharded SpMV gave up waiting for rank " + std::to_string((int)v - 1));
}

} // extern "C"
