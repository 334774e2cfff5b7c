// init_<template> + try_all_compress for the ten reduce templates: flatten a tiled sub-matrix into
// the arrays a kernel family reads, apply the row permutation where the reference applies it on
// the host, re-interleave values / column indices, detect closed forms. Array contents, element
// types and closed forms equal the reference's (the ten *_op*.cc files and arr_optimization.cc).
#include <string.h>

#include <algorithm>

#include "format.hpp"

#include <set>

namespace asp
{
namespace host
{

// ---------------------------------------------------------------------------------------------
// closed forms (arr_optimization.cc)
// ---------------------------------------------------------------------------------------------
bool detect_linear(const std::vector<u64> &a, ClosedForm &out)
{
    if (a.size() <= 1) return false;
    if (a[1] < a[0]) return false;
    const u64 coef = a[1] - a[0];
    for (size_t i = 0; i + 1 < a.size(); i++)
        if (a[i + 1] < a[i] || a[i + 1] - a[i] != coef) return false;
    out = ClosedForm();
    out.kind = ASP_COMPRESS_LINEAR;
    out.coef = coef;
    out.icpt = a[0];
    return true;
}

bool detect_constant(const std::vector<u64> &a, ClosedForm &out)
{
    if (a.empty()) return false;
    for (u64 v : a)
        if (v != a[0]) return false;
    out = ClosedForm();
    out.kind = ASP_COMPRESS_CONSTANT;
    out.icpt = a[0];
    return true;
}

bool detect_branch(const std::vector<u64> &a, ClosedForm &out)
{
    // the reference asserts arr_size > 2 here (arr_optimization.cc:117) and aborts on shorter arrays;
    // shorter arrays simply stay uncompressed
    if (a.size() <= 2) return false;
    ClosedForm f;
    f.kind = ASP_COMPRESS_BRANCH;
    f.lo.push_back(0);
    f.val.push_back(a[0]);
    for (size_t i = 0; i < a.size(); i++)
    {
        if (a[i] != f.val.back())
        {
            f.hi.push_back(i - 1);
            f.lo.push_back(i);
            f.val.push_back(a[i]);
            if (f.hi.size() >= ASP_MAX_BRANCH) return false;
        }
    }
    f.hi.push_back(a.size() - 1);
    out = f;
    return true;
}

bool detect_cycle_linear(const std::vector<u64> &a, u64 cycle, ClosedForm &out)
{
    if (!(cycle < a.size()) || a.size() % cycle != 0 || cycle <= 1) return false;
    const u64 icpt = a[0], coef = a[1] - a[0];
    for (size_t i = 0; i < a.size(); i++)
    {
        const u64 k = i % cycle;
        if (k == 0) continue;
        // the reference asserts divisibility inside this check (arr_optimization.cc:271); a
        // mismatch is a plain "no" here
        if (a[i] < icpt || (a[i] - icpt) % k != 0 || (a[i] - icpt) / k != coef) return false;
    }
    out = ClosedForm();
    out.kind = ASP_COMPRESS_CYCLE_LINEAR;
    out.cycle = cycle;
    out.coef = coef;
    out.icpt = icpt;
    return true;
}

bool detect_cycle_increase(const std::vector<u64> &a, ClosedForm &out)
{
    if (a.size() <= 2) return false;
    u64 cycle = 0;
    for (size_t i = 0; i < a.size(); i++)
        if (a[i] != a[0])
        {
            if (a[i] < a[0]) return false;
            cycle = i;
            break;
        }
    if (cycle == 0) return false; // all equal: the reference asserts here
    if (a.size() % cycle != 0) return false;
    for (size_t i = 0; i < a.size(); i++)
        if (a[i] != a[0] + i / cycle) return false;
    out = ClosedForm();
    out.kind = ASP_COMPRESS_CYCLE_INCREASE;
    out.cycle = cycle;
    out.icpt = a[0];
    return true;
}

namespace
{
std::vector<uint8_t> narrow(const std::vector<u64> &v, int dt)
{
    const int es = dtype_bytes(dt);
    std::vector<uint8_t> out(v.size() * es);
    switch (es)
    {
    case 1:
        for (size_t i = 0; i < v.size(); i++) out[i] = (uint8_t)v[i];
        break;
    case 2:
        for (size_t i = 0; i < v.size(); i++) ((uint16_t *)out.data())[i] = (uint16_t)v[i];
        break;
    case 4:
        for (size_t i = 0; i < v.size(); i++) ((uint32_t *)out.data())[i] = (uint32_t)v[i];
        break;
    default: memcpy(out.data(), v.data(), v.size() * 8);
    }
    return out;
}

TemplateArray &add_meta(TemplateData &t, int role, const std::vector<u64> &v, int dt)
{
    t.arrays.emplace_back();
    TemplateArray &a = t.arrays.back();
    a.role = role;
    a.dt = dt;
    a.len = v.size();
    a.bytes = narrow(v, dt);
    return a;
}

// dst[k*n + i] = src[i*S + k] for one strip of n TLBs of size S (row-major -> TLB-interleaved)
template <class D, class S_>
void interleave_strip(D *dst, const S_ *src, u64 n, u64 S)
{
    const u64 TB = 256;
#pragma omp parallel for schedule(static) if (n * S > (1u << 20))
    for (u64 i0 = 0; i0 < n; i0 += TB)
    {
        const u64 i1 = std::min(n, i0 + TB);
        for (u64 k = 0; k < S; k++)
            for (u64 i = i0; i < i1; i++) dst[k * n + i] = (D)src[i * S + k];
    }
}

struct NnzArrays
{
    std::vector<uint8_t> col, val;
};

void interleave_cols(uint8_t *dst, int col_dt, const u32 *src, u64 n, u64 S)
{
    switch (col_dt)
    {
    case ASP_U8: interleave_strip((uint8_t *)dst, src, n, S); break;
    case ASP_U16: interleave_strip((uint16_t *)dst, src, n, S); break;
    case ASP_U32: interleave_strip((uint32_t *)dst, src, n, S); break;
    default: interleave_strip((uint64_t *)dst, src, n, S); break;
    }
}
void interleave_vals(uint8_t *dst, int es, const uint8_t *src, u64 n, u64 S)
{
    if (es == 4) interleave_strip((uint32_t *)dst, (const uint32_t *)src, n, S);
    else interleave_strip((uint64_t *)dst, (const uint64_t *)src, n, S);
}

void add_nnz_arrays(TemplateData &t, const CompressedBlock &b, std::vector<uint8_t> &col, std::vector<uint8_t> &val, u64 n)
{
    t.arrays.emplace_back();
    TemplateArray &v = t.arrays.back();
    v.role = ASP_ARR_VAL;
    v.dt = t.val_dt;
    v.len = n;
    v.bytes.swap(val);
    t.arrays.emplace_back();
    TemplateArray &c = t.arrays.back();
    c.role = ASP_ARR_COL_INDEX;
    c.dt = b.col_dt;
    c.len = n;
    c.bytes.swap(col);
}

// global row (relative to the sub-matrix) of every TLB, in TLB order
std::vector<u64> tlb_global_rows(const CompressedBlock &b, bool &adjacent_equal)
{
    const Level &B = b.blb, &W = b.wlb, &T = b.tlb;
    std::vector<u64> rows(T.block_num);
    for (u64 i = 0; i < B.block_num; i++)
        for (u64 w = B.index.v[i]; w < B.index.v[i + 1]; w++)
        {
            const u64 base = B.first_row.v[i] + W.first_row.v[w];
            for (u64 t = W.index.v[w]; t < W.index.v[w + 1]; t++) rows[t] = base + T.first_row.v[t];
        }
    adjacent_equal = false;
    for (u64 t = 1; t < rows.size(); t++)
        if (rows[t] == rows[t - 1])
        {
            adjacent_equal = true;
            break;
        }
    return rows;
}

void common_head(const Matrix &m, const CompressedBlock &b, int type, TemplateData &t)
{
    t = TemplateData();
    t.arrays.reserve(16); // references returned by add_meta stay valid while arrays are appended
    t.template_type = type;
    t.val_dt = m.val_dt;
    t.first_row = b.min_row;
    t.first_col = b.min_col;
    t.true_nnz = b.end_coo - b.begin_coo + 1;
    t.sort_kind = m.is_sorted ? ASP_SORT_GLOBAL : ASP_SORT_NONE;
    t.n_blb = b.blb.block_num;
    t.n_wlb = b.wlb.block_num;
    t.n_tlb = b.tlb.block_num;
    // sub-matrices that do not span all columns always accumulate atomically
    t.is_atom_add = !(b.min_col == 0 && b.max_col == m.n_cols - 1);
}

void add_perm(const Matrix &m, TemplateData &t)
{
    if (!m.is_sorted) return;
    t.arrays.emplace_back();
    TemplateArray &a = t.arrays.back();
    a.role = ASP_ARR_ROW_INDEX_BEFORE_SORT;
    a.dt = m.perm_dt;
    a.len = m.n_rows;
    a.shared = m.sorted_row_index;
}

// effective unit count + host-side permutation of a row map (templates whose kernels do not read
// row_index_before_sort): rows >= the dense row count belong to COMPRESSED_ROW_PADDING
u64 effective_and_permute(const Matrix &m, const CompressedBlock &b, std::vector<u64> &rows)
{
    const u64 dense_rows = b.max_row - b.min_row + 1;
    u64 eff = rows.size();
    if (b.n_rows > dense_rows)
        for (u64 i = 0; i < rows.size(); i++)
            if (rows[i] >= dense_rows)
            {
                eff = i;
                break;
            }
    if (m.is_sorted)
        for (u64 i = 0; i < eff; i++) rows[i] = m.perm[rows[i] + b.min_row];
    return eff;
}

void try_linear_then_cycle_increase(TemplateArray &a, const std::vector<u64> &v)
{
    if (!detect_linear(v, a.comp)) detect_cycle_increase(v, a.comp);
}

// ---- DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS (direct_atom_op_warp_block_compress.cc) --------
bool init_k3(const Matrix &m, const CompressedBlock &b, TemplateData &t, std::string &err)
{
    common_head(m, b, ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS, t);
    const u64 S = b.tlb.coo_size.v[0];
    for (u64 s : b.tlb.coo_size.v)
        if (s != S)
        {
            err = "ELL-like template needs one global TLB size";
            return false;
        }
    bool adj = false;
    std::vector<u64> rows = tlb_global_rows(b, adj);
    if (adj) t.is_atom_add = true;
    const u64 n_pad = b.pad_col.size(), P = n_pad / S;
    std::vector<uint8_t> col(n_pad * dtype_bytes(b.col_dt)), val(n_pad * b.val.es);
    interleave_cols(col.data(), b.col_dt, b.pad_col.data(), P, S);
    interleave_vals(val.data(), b.val.es, b.pad_val.b.data(), P, S);
    t.effective_num = effective_and_permute(m, b, rows);
    t.tlb_size = S;
    u64 mx = 0;
    for (u64 r : rows) mx = std::max(mx, r);
    TemplateArray &rm = add_meta(t, ASP_ARR_GLOBAL_ROW_INDEX_OF_THREAD_LEVEL_BLOCK, rows, suitable_dtype(mx));
    try_linear_then_cycle_increase(rm, rows);
    add_perm(m, t);
    add_nnz_arrays(t, b, col, val, n_pad);
    return true;
}

// per-BLB view shared by the SELL-like and the row-grouped templates: TLB range and TLB size
bool blb_tlb_ranges(const CompressedBlock &b, std::vector<u64> &thr, std::vector<u64> &size, std::string &err)
{
    const Level &B = b.blb, &W = b.wlb, &T = b.tlb;
    thr.resize(B.block_num + 1);
    size.resize(B.block_num);
    for (u64 i = 0; i < B.block_num; i++)
    {
        const u64 w0 = B.index.v[i];
        thr[i] = W.index.v[w0];
        size[i] = T.coo_size.v[w0];
        for (u64 w = w0; w < B.index.v[i + 1]; w++)
            if (T.coo_size.v[w] != size[i])
            {
                err = "TLB size differs inside a BLB";
                return false;
            }
    }
    thr[B.block_num] = W.index.v[W.block_num];
    return true;
}

void interleave_per_blb(const CompressedBlock &b, const std::vector<u64> &thr, const std::vector<u64> &size, std::vector<uint8_t> &col, std::vector<uint8_t> &val)
{
    const u64 n_pad = b.pad_col.size();
    const int cb = dtype_bytes(b.col_dt), es = b.val.es;
    col.assign(n_pad * cb, 0);
    val.assign(n_pad * es, 0);
    const u64 nb = b.blb.block_num;
#pragma omp parallel for schedule(dynamic, 64)
    for (u64 i = 0; i < nb; i++)
    {
        const u64 nz0 = b.blb.coo_begin.v[i], n = thr[i + 1] - thr[i];
        interleave_cols(col.data() + nz0 * cb, b.col_dt, b.pad_col.data() + nz0, n, size[i]);
        interleave_vals(val.data() + nz0 * es, es, b.pad_val.b.data() + nz0 * es, n, size[i]);
    }
}

// ---- DIRECT_ATOM_TEMPLATE_WARP_COMPRESS (direct_atom_op_warp_compress.cc) --------------------
bool init_k2(const Matrix &m, const CompressedBlock &b, TemplateData &t, std::string &err)
{
    common_head(m, b, ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS, t);
    std::vector<u64> thr, size;
    if (!blb_tlb_ranges(b, thr, size, err)) return false;
    bool adj = false;
    std::vector<u64> rows = tlb_global_rows(b, adj);
    if (adj) t.is_atom_add = true;
    std::vector<uint8_t> col, val;
    interleave_per_blb(b, thr, size, col, val);
    t.effective_num = effective_and_permute(m, b, rows);
    u64 mx = 0;
    for (u64 r : rows) mx = std::max(mx, r);
    TemplateArray &rm = add_meta(t, ASP_ARR_GLOBAL_ROW_INDEX_OF_THREAD_LEVEL_BLOCK, rows, suitable_dtype(mx));
    try_linear_then_cycle_increase(rm, rows);
    TemplateArray &bt = add_meta(t, ASP_ARR_BLOCK_BEGIN_THREAD_INDEX_OFFSET, thr, suitable_dtype(thr.back()));
    detect_linear(thr, bt.comp);
    std::vector<u64> bnz(b.blb.coo_begin.v.begin(), b.blb.coo_begin.v.begin() + b.blb.block_num);
    TemplateArray &bn = add_meta(t, ASP_ARR_BLOCK_NZ_BEGIN_OFFSET, bnz, b.blb.coo_begin.dt);
    detect_linear(bnz, bn.comp);
    // The reference narrows this array by its LAST entry (direct_atom_op_warp_compress.cc:239, 544),
    // which is the smallest one after a descending row sort: strips
    // whose widest TLB needs more bits are then truncated (372 stored as 116). The type here is
    // wide enough for the largest entry; it equals the reference's whenever the reference is right.
    TemplateArray &ts = add_meta(t, ASP_ARR_THREAD_BLOCK_SIZE_IN_BLOCK, size, suitable_dtype(*std::max_element(size.begin(), size.end())));
    if (!detect_constant(size, ts.comp)) detect_branch(size, ts.comp);
    add_perm(m, t);
    add_nnz_arrays(t, b, col, val, b.pad_col.size());
    return true;
}

// ---- SHARED_MEMORY_TEMPLATE_WARP_COMPRESS (shared_memory_op_warp_compress.cc) ----------------
bool init_k6(const Matrix &m, const CompressedBlock &b, TemplateData &t, std::string &err)
{
    common_head(m, b, ASP_SHARED_MEMORY_TEMPLATE_WARP_COMPRESS, t);
    const Level &B = b.blb;
    std::vector<u64> thr, size;
    if (!blb_tlb_ranges(b, thr, size, err)) return false;
    // BLBs that overlap in rows (column-divided BLBs) force atomics
    u64 gmax = B.first_row.v[0] + B.row_num.v[0] - 1;
    for (u64 i = 1; i < B.block_num; i++)
    {
        if (B.first_row.v[i] <= gmax)
        {
            t.is_atom_add = true;
            break;
        }
        gmax = std::max(gmax, B.first_row.v[i] + B.row_num.v[i] - 1);
    }
    t.effective_num = b.max_row - b.min_row + 1;
    bool adj = false;
    std::vector<u64> rows = tlb_global_rows(b, adj);
    std::vector<u64> roff(b.n_rows + 1, 0);
    for (u64 r : rows) roff[r + 1]++;
    for (u64 r = 0; r < b.n_rows; r++) roff[r + 1] += roff[r];
    std::vector<uint8_t> col, val;
    interleave_per_blb(b, thr, size, col, val); // every BLB, the last one included (the reference skips it)
    TemplateArray &ro = add_meta(t, ASP_ARR_ROW_OFFSET_IN_THREAD_TMP_RESULT, roff, suitable_dtype(roff.back()));
    std::vector<u64> brow(B.first_row.v);
    brow.push_back(b.n_rows);
    TemplateArray &br = add_meta(t, ASP_ARR_BLOCK_FIRST_ROW_INDEX, brow, suitable_dtype(b.n_rows));
    TemplateArray &bt = add_meta(t, ASP_ARR_BLOCK_BEGIN_THREAD_INDEX_OFFSET, thr, suitable_dtype(thr.back()));
    TemplateArray &ts = add_meta(t, ASP_ARR_THREAD_BLOCK_SIZE_IN_BLOCK, size, b.tlb.coo_size.dt);
    std::vector<u64> bnz(B.coo_begin.v.begin(), B.coo_begin.v.begin() + B.block_num);
    TemplateArray &bn = add_meta(t, ASP_ARR_BLOCK_NZ_BEGIN_OFFSET, bnz, B.coo_begin.dt);
    detect_linear(thr, bt.comp);
    if (!detect_constant(size, ts.comp)) detect_branch(size, ts.comp);
    detect_linear(bnz, bn.comp);
    detect_linear(brow, br.comp);
    detect_linear(roff, ro.comp);
    add_perm(m, t);
    add_nnz_arrays(t, b, col, val, b.pad_col.size());
    return true;
}
// read_index[6] / staggered_padding_val_arr: inside every WLB the TLBs are taken in groups of 32 and
// element k of lane l of group g moves to g*32*S + k*32 + l (op_manager.cc:3569-3589). Identity
// when every TLB holds one non-zero.
void staggered_arrays(const CompressedBlock &b, std::vector<uint8_t> &col, std::vector<uint8_t> &val)
{
    const u64 n_pad = b.pad_col.size();
    const int cb = dtype_bytes(b.col_dt), es = b.val.es;
    col.assign(n_pad * cb, 0);
    val.assign(n_pad * es, 0);
    const Level &B = b.blb, &W = b.wlb;
    const u64 nb = B.block_num;
#pragma omp parallel for schedule(dynamic, 64)
    for (u64 i = 0; i < nb; i++)
        for (u64 w = B.index.v[i]; w < B.index.v[i + 1]; w++)
        {
            const u64 S = b.tlb.coo_size.v[w];
            const u64 base = B.coo_begin.v[i] + W.coo_begin.v[w];
            const u64 groups = (W.index.v[w + 1] - W.index.v[w]) / 32;
            for (u64 g = 0; g < groups; g++)
            {
                const u64 o = base + g * 32 * S;
                interleave_cols(col.data() + o * cb, b.col_dt, b.pad_col.data() + o, 32, S);
                interleave_vals(val.data() + o * es, es, b.pad_val.b.data() + o * es, 32, S);
            }
        }
}

std::vector<u64> first_n(const std::vector<u64> &v, u64 n) { return std::vector<u64>(v.begin(), v.begin() + n); }

// ---- DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE (direct_atom_total_warp_reduce_op.cc) ------------
bool init_k4(const Matrix &m, const CompressedBlock &b, TemplateData &t, std::string &err)
{
    common_head(m, b, ASP_DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE, t);
    const Level &B = b.blb, &W = b.wlb;
    std::vector<u64> rows(W.block_num), nz(W.block_num + 1);
    for (u64 i = 0; i < B.block_num; i++)
        for (u64 w = B.index.v[i]; w < B.index.v[i + 1]; w++)
        {
            if (W.row_num.v[w] != 1)
            {
                err = "warp-per-row template needs one row per WLB";
                return false;
            }
            rows[w] = B.first_row.v[i] + W.first_row.v[w];
            nz[w] = B.coo_begin.v[i] + W.coo_begin.v[w];
            if (w >= 1 && rows[w] == rows[w - 1]) t.is_atom_add = true;
        }
    nz[W.block_num] = b.pad_col.size();
    t.effective_num = effective_and_permute(m, b, rows);
    u64 mx = 0;
    for (u64 r : rows) mx = std::max(mx, r);
    TemplateArray &rm = add_meta(t, ASP_ARR_GLOBAL_ROW_INDEX_OF_WARP_LEVEL_BLOCK, rows, suitable_dtype(mx));
    try_linear_then_cycle_increase(rm, rows);
    TemplateArray &no = add_meta(t, ASP_ARR_GLOBAL_WARP_NZ_BEGIN_OFFSET, nz, suitable_dtype(b.pad_col.size() + 1));
    detect_linear(nz, no.comp);
    add_perm(m, t);
    std::vector<uint8_t> col, val;
    staggered_arrays(b, col, val);
    add_nnz_arrays(t, b, col, val, b.pad_col.size());
    return true;
}

// ---- SHARED_MEMORY_LONG_ROW_TEMPLATE (shared_memory_long_row_op.cc) ---------------------------
bool init_k7(const Matrix &m, const CompressedBlock &b, TemplateData &t, std::string &err)
{
    common_head(m, b, ASP_SHARED_MEMORY_LONG_ROW_TEMPLATE, t);
    const Level &B = b.blb;
    for (u64 i = 0; i < B.block_num; i++)
    {
        if (B.row_num.v[i] != 1)
        {
            err = "long-row template needs one row per BLB";
            return false;
        }
        if (i + 1 < B.block_num && B.first_row.v[i] == B.first_row.v[i + 1]) t.is_atom_add = true;
    }
    for (u64 s : b.tlb.coo_size.v)
        if (s != 1)
        {
            err = "long-row template needs TLB size 1";
            return false;
        }
    std::vector<u64> rows(B.first_row.v);
    if (m.is_sorted)
        for (u64 &r : rows) r = m.perm[r + b.min_row];
    u64 mx = 0;
    for (u64 r : rows) mx = std::max(mx, r);
    TemplateArray &rm = add_meta(t, ASP_ARR_ROW_INDEX_OF_BLOCK_LEVEL_BLOCK, rows, suitable_dtype(mx));
    try_linear_then_cycle_increase(rm, rows);
    TemplateArray &bn = add_meta(t, ASP_ARR_BLOCK_NZ_BEGIN_OFFSET, B.coo_begin.v, B.coo_begin.dt);
    detect_linear(B.coo_begin.v, bn.comp);
    add_perm(m, t);
    std::vector<uint8_t> col, val;
    staggered_arrays(b, col, val);
    add_nnz_arrays(t, b, col, val, b.pad_col.size());
    return true;
}

bool blbs_overlap_in_rows(const Level &B)
{
    u64 gmax = B.first_row.v[0] + B.row_num.v[0] - 1;
    for (u64 i = 1; i < B.block_num; i++)
    {
        if (B.first_row.v[i] <= gmax) return true;
        gmax = std::max(gmax, B.first_row.v[i] + B.row_num.v[i] - 1);
    }
    return false;
}

// ---- SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE (shared_memory_total_warp_reduce_op.cc) ---------
bool init_k8(const Matrix &m, const CompressedBlock &b, TemplateData &t, std::string &err)
{
    common_head(m, b, ASP_SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE, t);
    const Level &B = b.blb, &W = b.wlb;
    if (blbs_overlap_in_rows(B)) t.is_atom_add = true;
    t.effective_num = b.max_row - b.min_row + 1;
    std::vector<u64> roff(b.n_rows + 1, 0), nz(W.block_num + 1);
    for (u64 i = 0; i < B.block_num; i++)
        for (u64 w = B.index.v[i]; w < B.index.v[i + 1]; w++)
        {
            if (W.row_num.v[w] != 1)
            {
                err = "warp-reduce shared-memory template needs one row per WLB";
                return false;
            }
            roff[B.first_row.v[i] + W.first_row.v[w] + 1]++;
            nz[w] = B.coo_begin.v[i] + W.coo_begin.v[w];
        }
    nz[W.block_num] = b.pad_col.size();
    for (u64 r = 0; r < b.n_rows; r++) roff[r + 1] += roff[r];
    TemplateArray &ro = add_meta(t, ASP_ARR_ROW_OFFSET_IN_WARP_TMP_RESULT, roff, suitable_dtype(roff.back()));
    std::vector<u64> brow(B.first_row.v);
    brow.push_back(b.n_rows);
    TemplateArray &br = add_meta(t, ASP_ARR_BLOCK_FIRST_ROW_INDEX, brow, suitable_dtype(b.n_rows));
    TemplateArray &bw = add_meta(t, ASP_ARR_BLOCK_BEGIN_WARP_INDEX_OFFSET, B.index.v, B.index.dt);
    TemplateArray &fn = add_meta(t, ASP_ARR_GLOBAL_WARP_BLOCK_FIRST_NZ, nz, suitable_dtype(nz.back()));
    detect_linear(B.index.v, bw.comp);
    detect_linear(roff, ro.comp);
    detect_linear(brow, br.comp);
    detect_linear(nz, fn.comp);
    add_perm(m, t);
    std::vector<uint8_t> col, val;
    staggered_arrays(b, col, val);
    add_nnz_arrays(t, b, col, val, b.pad_col.size());
    return true;
}

// closed form of warp_nz_begin_offset in the 3-level templates: cycle-linear with the cycle taken
// from the linear form of block_begin_warp_index_offset (direct_atom_op.cc:1828-1890)
void try_cycle_linear_warp_nz(TemplateArray &wn, const std::vector<u64> &v, const TemplateArray &bw, const std::vector<u64> &bwv)
{
    u64 cycle = 0;
    if (bw.comp.kind == ASP_COMPRESS_LINEAR) cycle = bw.comp.coef;
    else
    {
        ClosedForm f;
        if (!detect_linear(bwv, f)) return;
        cycle = f.coef;
    }
    detect_cycle_linear(v, cycle, wn.comp);
}

// ---- DIRECT_ATOM_TEMPLATE (direct_atom_op.cc) --------------------------------------------------
bool init_k1(const Matrix &m, const CompressedBlock &b, TemplateData &t, std::string &err)
{
    common_head(m, b, ASP_DIRECT_ATOM_TEMPLATE, t);
    const Level &B = b.blb, &W = b.wlb;
    bool adj = false;
    std::vector<u64> rows = tlb_global_rows(b, adj);
    if (adj) t.is_atom_add = true;
    if (m.is_sorted)
        for (u64 &r : rows) r = m.perm[r + b.min_row]; // every TLB, padded rows included, as the reference does
    u64 mx = 0;
    for (u64 r : rows) mx = std::max(mx, r);
    TemplateArray &rm = add_meta(t, ASP_ARR_GLOBAL_ROW_INDEX_OF_THREAD_LEVEL_BLOCK, rows, suitable_dtype(mx));
    TemplateArray &bw = add_meta(t, ASP_ARR_BLOCK_BEGIN_WARP_INDEX_OFFSET, B.index.v, B.index.dt);
    TemplateArray &wt = add_meta(t, ASP_ARR_WARP_BEGIN_THREAD_INDEX_OFFSET, W.index.v, W.index.dt);
    TemplateArray &ts = add_meta(t, ASP_ARR_THREAD_BLOCK_SIZE_IN_WARP, b.tlb.coo_size.v, b.tlb.coo_size.dt);
    std::vector<u64> bnz = first_n(B.coo_begin.v, B.block_num);
    TemplateArray &bn = add_meta(t, ASP_ARR_BLOCK_NZ_BEGIN_OFFSET, bnz, B.coo_begin.dt);
    TemplateArray &wn = add_meta(t, ASP_ARR_WARP_NZ_BEGIN_OFFSET, W.coo_begin.v, W.coo_begin.dt);
    try_linear_then_cycle_increase(rm, rows);
    detect_linear(B.index.v, bw.comp);
    detect_linear(W.index.v, wt.comp);
    if (!detect_constant(b.tlb.coo_size.v, ts.comp)) detect_branch(b.tlb.coo_size.v, ts.comp);
    detect_linear(bnz, bn.comp);
    try_cycle_linear_warp_nz(wn, W.coo_begin.v, bw, B.index.v);
    add_perm(m, t);
    std::vector<uint8_t> col, val;
    staggered_arrays(b, col, val);
    add_nnz_arrays(t, b, col, val, b.pad_col.size());
    (void)err;
    return true;
}

// ---- SHARED_MEMORY_TEMPLATE (shared_memory_op.cc) ----------------------------------------------
bool init_k5(const Matrix &m, const CompressedBlock &b, TemplateData &t, std::string &err)
{
    common_head(m, b, ASP_SHARED_MEMORY_TEMPLATE, t);
    const Level &B = b.blb, &W = b.wlb;
    if (blbs_overlap_in_rows(B)) t.is_atom_add = true;
    bool adj = false;
    std::vector<u64> rows = tlb_global_rows(b, adj);
    std::vector<u64> roff(b.n_rows + 1, 0);
    for (u64 r : rows) roff[r + 1]++;
    for (u64 r = 0; r < b.n_rows; r++) roff[r + 1] += roff[r];
    // values / columns interleaved per WLB: element k of local TLB i at base + i + k*n_w
    const u64 n_pad = b.pad_col.size();
    const int cb = dtype_bytes(b.col_dt), es = b.val.es;
    std::vector<uint8_t> col(n_pad * cb), val(n_pad * es);
    for (u64 i = 0; i < B.block_num; i++)
        for (u64 w = B.index.v[i]; w < B.index.v[i + 1]; w++)
        {
            const u64 base = B.coo_begin.v[i] + W.coo_begin.v[w], n = W.index.v[w + 1] - W.index.v[w], S = b.tlb.coo_size.v[w];
            interleave_cols(col.data() + base * cb, b.col_dt, b.pad_col.data() + base, n, S);
            interleave_vals(val.data() + base * es, es, b.pad_val.b.data() + base * es, n, S);
        }
    TemplateArray &ro = add_meta(t, ASP_ARR_ROW_OFFSET_IN_THREAD_TMP_RESULT, roff, suitable_dtype(roff.back()));
    std::vector<u64> brow(B.first_row.v);
    brow.push_back(b.n_rows);
    TemplateArray &br = add_meta(t, ASP_ARR_BLOCK_FIRST_ROW_INDEX, brow, suitable_dtype(b.n_rows));
    TemplateArray &bw = add_meta(t, ASP_ARR_BLOCK_BEGIN_WARP_INDEX_OFFSET, B.index.v, B.index.dt);
    TemplateArray &wt = add_meta(t, ASP_ARR_WARP_BEGIN_THREAD_INDEX_OFFSET, W.index.v, W.index.dt);
    TemplateArray &ts = add_meta(t, ASP_ARR_THREAD_BLOCK_SIZE_IN_WARP, b.tlb.coo_size.v, b.tlb.coo_size.dt);
    std::vector<u64> bnz = first_n(B.coo_begin.v, B.block_num);
    TemplateArray &bn = add_meta(t, ASP_ARR_BLOCK_NZ_BEGIN_OFFSET, bnz, B.coo_begin.dt);
    TemplateArray &wn = add_meta(t, ASP_ARR_WARP_NZ_BEGIN_OFFSET, W.coo_begin.v, W.coo_begin.dt);
    detect_linear(B.index.v, bw.comp);
    detect_linear(W.index.v, wt.comp);
    if (!detect_constant(b.tlb.coo_size.v, ts.comp)) detect_branch(b.tlb.coo_size.v, ts.comp);
    detect_linear(bnz, bn.comp);
    try_cycle_linear_warp_nz(wn, W.coo_begin.v, bw, B.index.v);
    detect_linear(brow, br.comp);
    detect_linear(roff, ro.comp);
    add_perm(m, t);
    add_nnz_arrays(t, b, col, val, n_pad);
    (void)err;
    return true;
}

int bit_count(u64 v)
{
    int n = 0;
    while (v)
    {
        v >>= 1;
        n++;
    }
    return n;
}

// ---- UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE[_WITH_WARP_REDUCE] ---------------------------
// (unaligned_warp_reduce_same_TLB_size_op.cc:5-297, helpers :434-512 and :1332-1645)
bool init_k9(const Matrix &m, const CompressedBlock &b, bool with_warp_reduce, TemplateData &t, std::string &err)
{
    common_head(m, b, with_warp_reduce ? ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE : ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE, t);
    if (!b.tlb_is_nnz_div)
    {
        err = "CSR5-like templates need the TLB level built by the nnz division";
        return false;
    }
    const u64 S = b.tlb.coo_size.v[0];
    // rows without non-zeros become one zero at column 0; the tail is padded to whole warps by
    // repeating the last (row, column) with value 0
    std::vector<u64> row;
    std::vector<u32> col;
    row.reserve(b.col.size() + b.n_rows);
    col.reserve(b.col.size() + b.n_rows);
    std::vector<u64> src; // source position of every element, ~0 for filler
    src.reserve(b.col.size() + b.n_rows);
    u64 last_row_with_nz = 0;
    for (u64 r = 0; r < b.n_rows; r++)
        if (b.rowptr[r + 1] > b.rowptr[r]) last_row_with_nz = r;
    for (u64 r = 0; r <= last_row_with_nz; r++)
    {
        if (b.rowptr[r + 1] == b.rowptr[r])
        {
            row.push_back(r);
            col.push_back(0);
            src.push_back(~0ull);
            continue;
        }
        for (u64 k = b.rowptr[r]; k < b.rowptr[r + 1]; k++)
        {
            row.push_back(r);
            col.push_back(b.col[k]);
            src.push_back(k);
        }
    }
    const u64 wn = 32 * S;
    const u64 target = (row.size() + wn - 1) / wn * wn;
    while (row.size() < target)
    {
        row.push_back(row.back());
        col.push_back(col.back());
        src.push_back(~0ull);
    }
    const u64 n = row.size(), T = n / S, Wn = T / 32;
    // row-start flags (the first non-zero of every warp always starts a sum), first rows per warp
    std::vector<uint8_t> flag(n);
#pragma omp parallel for schedule(static) if (n > (1u << 20))
    for (u64 i = 0; i < n; i++) flag[i] = (i % wn == 0) ? 1 : (row[i] != row[i - 1]);
    std::vector<u64> wfirst(Wn);
    for (u64 w = 0; w < Wn; w++) wfirst[w] = row[w * wn];
    // per TLB: does it hold a row start, count of following start-free TLBs, first row started (relative)
    std::vector<uint8_t> has(T, 0);
    for (u64 tl = 0; tl < T; tl++)
        for (u64 k = 0; k < S; k++) has[tl] |= flag[tl * S + k];
    std::vector<u64> roff(T, 0), frow(T, 0);
    u64 max_roff = 0, max_frow = 0, last_head = 0, run = 0;
    for (u64 tl = 1; tl < T; tl++)
    {
        if (!has[tl]) run++;
        else
        {
            max_roff = std::max(max_roff, run);
            roff[last_head] = run;
            run = 0;
            last_head = tl;
        }
    }
    max_roff = std::max(max_roff, run);
    roff[last_head] = run;
    for (u64 tl = 0; tl < T; tl++)
    {
        if (has[tl])
        {
            for (u64 k = 0; k < S; k++)
                if (flag[tl * S + k])
                {
                    frow[tl] = row[tl * S + k] - wfirst[tl / 32];
                    break;
                }
        }
        else
            frow[tl] = frow[tl - 1];
        max_frow = std::max(max_frow, frow[tl]);
    }
    int bits_row = bit_count(max_frow), bits_off = bit_count(max_roff);
    if (bits_row == 0) bits_row = 1;
    if (bits_off == 0) bits_off = 1;
    const int total_bits = (int)S + bits_row + bits_off;
    if (total_bits > 64)
    {
        err = "CSR5-like: row-start flags + offsets do not fit in 64 bits";
        return false;
    }
    const int word = total_bits <= 8 ? 8 : total_bits <= 16 ? 16 : total_bits <= 32 ? 32 : 64;
    const int meta_dt = word == 8 ? ASP_U8 : word == 16 ? ASP_U16 : word == 32 ? ASP_U32 : ASP_U64;
    std::vector<u64> meta(T);
    for (u64 tl = 0; tl < T; tl++)
    {
        u64 f = 0;
        for (u64 k = 0; k < S; k++)
            if (flag[tl * S + k]) f |= 1ull << (S - 1 - k);
        u64 v = f << (word - (int)S - bits_off - bits_row + bits_off);
        v |= roff[tl];
        v <<= bits_row;
        v |= frow[tl];
        meta[tl] = v;
    }
    t.tlb_size = S;
    t.bits_word = word;
    t.bits_flag = (int)S;
    t.bits_row = bits_row;
    t.bits_off = bits_off;
    t.n_tlb = (b.col.size() + S - 1) / S;
    if (with_warp_reduce) wfirst.push_back(row.back() + 1);
    TemplateArray &fr = add_meta(t, ASP_ARR_GLOBAL_FIRST_ROW_INDEX_OF_WARP_LEVEL_BLOCK, wfirst, b.row_dt);
    try_linear_then_cycle_increase(fr, wfirst);
    add_meta(t, ASP_ARR_COMBINE_META_OF_THREAD_LEVEL_BLOCK, meta, meta_dt);
    add_perm(m, t);
    // values / columns: element k of lane l of warp w at w*32*S + k*32 + l
    const int cb = dtype_bytes(b.col_dt), es = b.val.es;
    std::vector<uint8_t> ocol(n * cb, 0), oval(n * es, 0);
#pragma omp parallel for schedule(static) if (n > (1u << 20))
    for (u64 i = 0; i < n; i++)
    {
        const u64 tl = i / S, k = i % S, w = tl / 32, lane = tl % 32;
        const u64 d = w * wn + k * 32 + lane;
        switch (cb)
        {
        case 1: ocol[d] = (uint8_t)col[i]; break;
        case 2: ((uint16_t *)ocol.data())[d] = (uint16_t)col[i]; break;
        case 4: ((uint32_t *)ocol.data())[d] = col[i]; break;
        default: ((uint64_t *)ocol.data())[d] = col[i]; break;
        }
        if (src[i] != ~0ull) memcpy(&oval[d * es], &b.val.b[src[i] * es], es);
    }
    add_nnz_arrays(t, b, ocol, oval, n);
    return true;
}
} // namespace

// ---- block-value template (this build's; no counterpart in the reference) --------------------------------
// Blocked ELL over dense r x c blocks: block rows of r consecutive rows, block columns of c consecutive columns
// (relative to the sub-matrix's first column); every block that holds a non-zero is stored in full, block rows
// are padded with zero blocks to the width of the widest one, and the block rows to an even count.
bool init_block_ell(const Matrix &m, const CompressedBlock &b, TemplateData &t, std::string &err)
{
    const u64 r = b.block_r, c = b.block_c;
    if (m.is_sorted) return err = "block_value: not for sorted matrices (a block row must be r consecutive rows of y)", false;
    if (!((r == 2 && c == 2) || (r == 3 && c == 3) || (r == 4 && c == 4))) return err = "block_value: blocks of 2 x 2, 3 x 3 or 4 x 4", false;
    const u64 width = b.max_col - b.min_col + 1;
    if (width % c) return err = "block_value: the columns of the sub-matrix are not a multiple of the block width", false;
    const u64 NBR = (b.n_rows + r - 1) / r, NB = (NBR + 1) / 2 * 2;
    // pass 1: block columns per block row (merged over its r rows), and how full the blocks are
    std::vector<u64> bptr(NBR + 1, 0);
    std::vector<u32> bcol;
    {
        std::vector<u64> cnt(NBR, 0);
#pragma omp parallel
        {
            std::vector<u32> tmp;
#pragma omp for schedule(static)
            for (int64_t br = 0; br < (int64_t)NBR; br++)
            {
                tmp.clear();
                for (u64 row = (u64)br * r; row < std::min<u64>(b.n_rows, ((u64)br + 1) * r); row++)
                    for (u64 k = b.rowptr[row]; k < b.rowptr[row + 1]; k++) tmp.push_back((u32)(b.col[k] / c));
                std::sort(tmp.begin(), tmp.end());
                cnt[br] = (u64)(std::unique(tmp.begin(), tmp.end()) - tmp.begin());
            }
        }
        for (u64 br = 0; br < NBR; br++) bptr[br + 1] = bptr[br] + cnt[br];
        bcol.resize(bptr[NBR]);
#pragma omp parallel
        {
            std::vector<u32> tmp;
#pragma omp for schedule(static)
            for (int64_t br = 0; br < (int64_t)NBR; br++)
            {
                tmp.clear();
                for (u64 row = (u64)br * r; row < std::min<u64>(b.n_rows, ((u64)br + 1) * r); row++)
                    for (u64 k = b.rowptr[row]; k < b.rowptr[row + 1]; k++) tmp.push_back((u32)(b.col[k] / c));
                std::sort(tmp.begin(), tmp.end());
                tmp.erase(std::unique(tmp.begin(), tmp.end()), tmp.end());
                std::copy(tmp.begin(), tmp.end(), bcol.begin() + bptr[br]);
            }
        }
    }
    u64 W = 0;
    for (u64 br = 0; br < NBR; br++) W = std::max(W, bptr[br + 1] - bptr[br]);
    if (W == 0) return err = "block_value: sub-matrix without non-zeros", false;
    const u64 stored = NB * W * r * c;
    if (b.nnz() == 0 || (double)stored / (double)b.nnz() > 8.0) return err = "block_value: the matrix is not made of dense blocks of this size (more than 8 stored values per non-zero)", false;
    // pass 2: the arrays
    const int es = b.val.es;
    std::vector<uint8_t> idx(NB * W * 4, 0), val(stored * (u64)es, 0);
    u32 *ip = (u32 *)idx.data();
#pragma omp parallel for schedule(static)
    for (int64_t br = 0; br < (int64_t)NBR; br++)
    {
        const u64 n = bptr[br + 1] - bptr[br];
        const u32 *bc = bcol.data() + bptr[br];
        for (u64 k = 0; k < W; k++) ip[k * NB + br] = k < n ? bc[k] : (n ? bc[n - 1] : 0); // zero blocks repeat the last block column
        for (u64 row = (u64)br * r; row < std::min<u64>(b.n_rows, ((u64)br + 1) * r); row++)
        {
            const u64 i = row - (u64)br * r;
            u64 k = 0; // the columns of a row ascend, so do its block slots
            for (u64 q = b.rowptr[row]; q < b.rowptr[row + 1]; q++)
            {
                const u32 cb = b.col[q] / (u32)c;
                while (bc[k] != cb) k++;
                const u64 j = b.col[q] - (u64)cb * c;
                memcpy(&val[(((k * r + i) * c + j) * NB + (u64)br) * es], &b.val.b[q * es], es);
            }
        }
    }
    common_head(m, b, ASP_BLOCK_ELL_TEMPLATE, t);
    t.tlb_size = W;
    t.bits_row = (int)r;
    t.bits_off = (int)c;
    t.effective_num = b.n_rows;
    t.n_blb = NBR;
    t.n_wlb = NBR;
    t.n_tlb = NB;
    t.thread_num_in_block = 128;
    t.tblock_num = (long)std::max<u64>(1, (NB / 2 + 127) / 128);
    t.arrays.emplace_back();
    TemplateArray &v = t.arrays.back();
    v.role = ASP_ARR_VAL;
    v.dt = t.val_dt;
    v.len = stored;
    v.bytes.swap(val);
    t.arrays.emplace_back();
    TemplateArray &ci = t.arrays.back();
    ci.role = ASP_ARR_COL_INDEX;
    ci.dt = ASP_U32;
    ci.len = NB * W;
    ci.bytes.swap(idx);
    return true;
}

// ---- diagonal-value template (this build's; no counterpart in the reference) ------------------------------
// DIA storage: the distinct offsets col - row of the sub-matrix (at most b.diag_max of them), values diagonal-major.
bool init_diag(const Matrix &m, const CompressedBlock &b, TemplateData &t, std::string &err)
{
    if (m.is_sorted) return err = "diag_value: not for sorted matrices (the diagonals are those of the original row order)", false;
    if (!(b.min_col == 0 && b.max_col == m.n_cols - 1)) return err = "diag_value: not for column-sliced sub-matrices", false;
    const int es = b.val.es;
    const u64 V = 16 / (u64)es, NR = (b.n_rows + V - 1) / V * V;
    const int64_t ncols = (int64_t)(b.max_col - b.min_col + 1);
    // distinct offsets; a scattered matrix leaves after a few rows
    std::set<int64_t> offs;
    for (u64 r = 0; r < b.n_rows; r++)
    {
        for (u64 k = b.rowptr[r]; k < b.rowptr[r + 1]; k++) offs.insert((int64_t)b.col[k] - (int64_t)r);
        if (offs.size() > b.diag_max) return err = "diag_value: more than " + std::to_string(b.diag_max) + " diagonals hold non-zeros", false;
    }
    if (offs.empty()) return err = "diag_value: sub-matrix without non-zeros", false;
    const std::vector<int64_t> off(offs.begin(), offs.end());
    const u64 D = off.size();
    std::vector<uint8_t> val(D * NR * (u64)es, 0);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)b.n_rows; r++)
        for (u64 k = b.rowptr[r]; k < b.rowptr[r + 1]; k++)
        {
            const u64 d = (u64)(std::lower_bound(off.begin(), off.end(), (int64_t)b.col[k] - r) - off.begin());
            memcpy(&val[(d * NR + (u64)r) * es], &b.val.b[k * es], es);
        }
    common_head(m, b, ASP_DIAG_TEMPLATE, t);
    t.tlb_size = D;
    t.effective_num = b.n_rows;
    t.n_blb = 1;
    t.n_wlb = 1;
    t.n_tlb = NR / V;
    t.thread_num_in_block = 256;
    t.tblock_num = (long)std::max<u64>(1, (NR / V + 255) / 256);
    t.arrays.emplace_back();
    TemplateArray &v = t.arrays.back();
    v.role = ASP_ARR_VAL;
    v.dt = t.val_dt;
    v.len = D * NR;
    v.bytes.swap(val);
    std::vector<u64> biased(D);
    for (u64 d = 0; d < D; d++) biased[d] = (u64)(off[d] + ncols);
    add_meta(t, ASP_ARR_COL_INDEX, biased, ASP_U64);
    return true;
}

bool init_template(const Matrix &m, size_t sub, int type, TemplateData &out, std::string &err)
{
    if (sub >= m.blocks.size())
    {
        err = "no such sub-matrix";
        return false;
    }
    const CompressedBlock &b = m.blocks[sub];
    if (type == ASP_DIAG_TEMPLATE)
    {
        if (!b.diag_max) return err = "the template D1 needs the diag_value node", false;
        return init_diag(m, b, out, err);
    }
    if (type == ASP_BLOCK_ELL_TEMPLATE)
    {
        if (!b.block_r) return err = "the template B1 needs the block_value node", false;
        return init_block_ell(m, b, out, err);
    }
    const bool csr5 = type == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE || type == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE;
    if (!csr5 && b.tlb_is_nnz_div)
    {
        err = "this template needs an ELL-style TLB level";
        return false;
    }
    if (!(b.blb.built && b.wlb.built && b.tlb.built))
    {
        err = "sub-matrix is not tiled at all three levels";
        return false;
    }
    switch (type)
    {
    case ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS: return init_k3(m, b, out, err);
    case ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS: return init_k2(m, b, out, err);
    case ASP_SHARED_MEMORY_TEMPLATE_WARP_COMPRESS: return init_k6(m, b, out, err);
    case ASP_DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE: return init_k4(m, b, out, err);
    case ASP_SHARED_MEMORY_LONG_ROW_TEMPLATE: return init_k7(m, b, out, err);
    case ASP_SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE: return init_k8(m, b, out, err);
    case ASP_DIRECT_ATOM_TEMPLATE: return init_k1(m, b, out, err);
    case ASP_SHARED_MEMORY_TEMPLATE: return init_k5(m, b, out, err);
    case ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE: return init_k9(m, b, false, out, err);
    case ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE: return init_k9(m, b, true, out, err);
    default: err = "template not implemented by the host lowering"; return false;
    }
}

} // namespace host
} // namespace asp
