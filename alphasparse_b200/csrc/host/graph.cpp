// C ABI of the host side (include/asp_b200_host.h): matrix construction, Operator Graph
// execution from a textual spec, access to the lowered templates.
#include <string.h>

#include <algorithm>
#include <stdexcept>
#include <atomic>
#include <map>
#include <memory>
#include <new>
#include <sstream>
#include <string>
#include <vector>

#include "../../../include/asp_b200_host.h"
#include "format.hpp"
#include "handles.hpp"

using namespace asp::host;

static uint64_t next_format_id()
{
    static std::atomic<uint64_t> n{0};
    return ++n;
}

asp_format::asp_format() : id(next_format_id()) {}

void asp_format::cache_from_matrix()
{
    val_dt = m->val_dt;
    n_rows = m->n_rows;
    n_cols = m->n_cols;
    perm = m->is_sorted ? m->sorted_row_index : nullptr;
    perm_dt = m->perm_dt;
    infos.assign(subs.size(), asp_sub_info());
    for (size_t i = 0; i < subs.size(); i++)
    {
        const CompressedBlock &b = m->blocks[i];
        asp_sub_info &o = infos[i];
        o.min_row = b.min_row;
        o.max_row = b.max_row;
        o.min_col = b.min_col;
        o.max_col = b.max_col;
        o.begin_coo = b.begin_coo;
        o.end_coo = b.end_coo;
        o.n_blb = b.blb.block_num;
        o.n_wlb = b.wlb.block_num;
        o.n_tlb = b.tlb.block_num;
        o.template_type = subs[i].template_type;
        o.n_arrays = (int32_t)subs[i].arrays.size();
    }
}

void asp_format::build_descs()
{
    descs.assign(subs.size(), std::vector<asp_array_desc>());
    for (size_t i = 0; i < subs.size(); i++)
    {
        for (const TemplateArray &a : subs[i].arrays)
        {
            asp_array_desc d;
            memset(&d, 0, sizeof(d));
            d.role = a.role;
            d.dtype = a.dt;
            d.host_ptr = a.data();
            d.len = a.len;
            d.compress = a.comp.kind;
            d.coef = a.comp.coef;
            d.icpt = a.comp.icpt;
            d.cycle = a.comp.cycle;
            d.n_branch = (int32_t)a.comp.val.size();
            for (size_t k = 0; k < a.comp.val.size() && k < ASP_MAX_BRANCH; k++)
            {
                d.branch_lo[k] = a.comp.lo[k];
                d.branch_hi[k] = a.comp.hi[k];
                d.branch_val[k] = a.comp.val[k];
            }
            descs[i].push_back(d);
        }
    }
}

static thread_local std::string g_host_error;
asp_status asp_host_fail(asp_status s, const std::string &msg)
{
    g_host_error = msg;
    return s;
}

namespace
{
asp_status hfail(asp_status s, const std::string &msg) { return asp_host_fail(s, msg); }

struct SubSpec
{
    std::vector<std::vector<std::string>> nodes;
    std::string templ;
    long tblock = -1, threads = -1, reduce = -1;
};

int template_of_name(const std::string &k)
{
    static const std::map<std::string, int> tab = {
        {"K1", ASP_DIRECT_ATOM_TEMPLATE},
        {"K2", ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS},
        {"K3", ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS},
        {"K4", ASP_DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE},
        {"K5", ASP_SHARED_MEMORY_TEMPLATE},
        {"K6", ASP_SHARED_MEMORY_TEMPLATE_WARP_COMPRESS},
        {"K7", ASP_SHARED_MEMORY_LONG_ROW_TEMPLATE},
        {"K8", ASP_SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE},
        {"K9", ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE},
        {"K10", ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE},
        {"EMPTY", ASP_EMPTY_TEMPLATE},
        {"B1", ASP_BLOCK_ELL_TEMPLATE}, // block-value template of this build (not one of the reference's ten)
        {"D1", ASP_DIAG_TEMPLATE},      // diagonal-value template of this build
    };
    auto it = tab.find(k);
    return it == tab.end() ? -1 : it->second;
}

bool apply_sub_node(CompressedBlock &b, const std::vector<std::string> &tok, std::string &err)
{
    auto L = [&](size_t i) -> u64 { return i < tok.size() ? strtoull(tok[i].c_str(), nullptr, 10) : 0; };
    const std::string &op = tok[0];
    // the reference inserts the default tilings of the upper levels before a lower-level node
    auto need_blb = [&]() {
        if (!b.blb.built) sep_tblock_level_row_csr(b, std::vector<u64>(1, b.n_rows));
    };
    auto need_wlb = [&]() {
        need_blb();
        if (!b.wlb.built) sep_warp_level_row_csr(b, std::vector<std::vector<u64>>());
    };
    if (op == "row_padding")
    {
        if (L(1) == 0 || L(2) == 0 || b.blb.built) return err = "row_padding needs <multiple> <row_len> and must come first", false;
        row_padding(b, L(1), L(2));
    }
    else if (op == "blb_row_evenly")
    {
        if (L(1) == 0 || b.blb.built) return err = "bad blb_row_evenly", false;
        sep_tblock_level_row_csr(b, blb_rows_evenly(b, L(1)));
    }
    else if (op == "blb_row_nnz")
    {
        if (L(1) == 0 || b.blb.built) return err = "bad blb_row_nnz", false;
        sep_tblock_level_row_csr(b, blb_rows_by_nnz_low_bound(b, L(1)));
    }
    else if (op == "blb_col_fixed")
    {
        if (L(1) == 0 || b.blb.built) return err = "bad blb_col_fixed", false;
        sep_tblock_level_col_fixed(b, L(1));
    }
    else if (op == "wlb_row_evenly")
    {
        if (L(1) == 0 || b.wlb.built) return err = "bad wlb_row_evenly", false;
        need_blb();
        sep_warp_level_row_csr(b, wlb_rows_evenly(b, L(1)));
    }
    else if (op == "wlb_col_fixed")
    {
        if (L(1) == 0 || b.wlb.built) return err = "bad wlb_col_fixed", false;
        need_blb();
        sep_warp_level_col_fixed(b, L(1));
    }
    else if (op == "tlb_row")
    {
        if (b.tlb.built) return err = "TLB level already tiled", false;
        need_wlb();
        sep_thread_level_col_ell_with_padding(b, 0);
    }
    else if (op == "tlb_col_fixed")
    {
        if (L(1) == 0 || b.tlb.built) return err = "bad tlb_col_fixed", false;
        need_wlb();
        sep_thread_level_col_ell_with_padding(b, L(1));
    }
    else if (op == "tlb_nnz")
    {
        if (L(1) == 0 || b.blb.built || b.wlb.built || b.tlb.built) return err = "tlb_nnz needs an untiled sub-matrix", false;
        need_wlb();
        sep_thread_level_acc_to_nnz(b, L(1));
    }
    else if (op == "diag_value")
    {
        // not a node of the reference: marks the sub-matrix for DIA storage (template D1); optional <max diagonals>, default 64
        if (b.blb.built || b.wlb.built || b.tlb.built || b.block_r || b.diag_max) return err = "diag_value needs an untiled sub-matrix", false;
        b.diag_max = L(1) ? L(1) : 64;
    }
    else if (op == "block_value")
    {
        // not a node of the reference: marks the sub-matrix for storage as dense <r> x <c> blocks (template B1)
        if (L(1) == 0 || L(2) == 0 || b.blb.built || b.wlb.built || b.tlb.built || b.block_r) return err = "block_value needs <r> <c> and an untiled sub-matrix", false;
        b.block_r = L(1);
        b.block_c = L(2);
    }
    else
        return err = "unknown compressed-view node " + op, false;
    return true;
}

bool apply_dense_node(Matrix &m, const std::vector<std::string> &tok, bool &compressed, std::string &err)
{
    if (tok[0] == "sort")
    {
        const u64 step = tok.size() > 1 ? strtoull(tok[1].c_str(), nullptr, 10) : 1;
        if (step == 0 || m.is_sorted || m.is_blocked) return err = "bad dense sort", false;
        dense_row_coarse_sort(m, step);
    }
    else if (tok[0] == "rowdiv_exp")
    {
        if (tok.size() < 4 || m.is_blocked) return err = "bad dense rowdiv_exp", false;
        const u64 lo = strtoull(tok[1].c_str(), nullptr, 10), hi = strtoull(tok[2].c_str(), nullptr, 10), rate = strtoull(tok[3].c_str(), nullptr, 10);
        if (lo == 0 || hi < lo || rate < 2) return err = "bad dense rowdiv_exp parameters", false;
        dense_row_div(m, row_div_position_exponential(m, lo, hi, rate));
    }
    else if (tok[0] == "rowdiv")
    {
        // DENSE_ROW_DIV with explicit positions (exe_dense_row_div_param_t: first row of every strip,
        // closed by the row count): "rowdiv p1 p2 ..." cuts [0, p1), [p1, p2), ..., [pk, n_rows)
        if (tok.size() < 2 || m.is_blocked) return err = "bad dense rowdiv", false;
        std::vector<u64> pos(1, 0);
        for (size_t i = 1; i < tok.size(); i++)
        {
            const u64 p = strtoull(tok[i].c_str(), nullptr, 10);
            if (p <= pos.back() || p >= m.n_rows) return err = "dense rowdiv positions must increase inside (0, rows)", false;
            pos.push_back(p);
        }
        pos.push_back(m.n_rows);
        dense_row_div(m, pos);
    }
    else if (tok[0] == "compress")
    {
        compress_dense_view(m);
        compressed = true;
    }
    else
        return err = "unknown dense-view node " + tok[0], false;
    return true;
}
} // namespace

extern "C" {

const char *asp_host_last_error(void) { return g_host_error.c_str(); }

asp_status asp_matrix_from_csr(uint64_t n_rows, uint64_t n_cols, const int64_t *indptr, const uint32_t *indices, const void *values, int val_dtype, asp_matrix **out)
{
    if (!out || !indptr || (!indices && indptr[n_rows] > 0) || (!values && indptr[n_rows] > 0)) return hfail(ASP_ERR_INVALID_ARG, "NULL argument");
    *out = nullptr;
    if (val_dtype != ASP_F32 && val_dtype != ASP_F64) return hfail(ASP_ERR_UNSUPPORTED, "values must be f32 or f64");
    if (n_rows == 0 || n_cols == 0 || n_cols > 0xffffffffull) return hfail(ASP_ERR_INVALID_ARG, "bad shape");
    if (indptr[0] != 0) return hfail(ASP_ERR_INVALID_ARG, "indptr[0] != 0");
    for (uint64_t r = 0; r < n_rows; r++)
    {
        if (indptr[r + 1] < indptr[r]) return hfail(ASP_ERR_INVALID_ARG, "indptr decreases");
        for (int64_t k = indptr[r]; k < indptr[r + 1]; k++)
        {
            if (indices[k] >= n_cols) return hfail(ASP_ERR_BOUNDS, "column index outside the matrix");
            if (k > indptr[r] && indices[k] < indices[k - 1]) return hfail(ASP_ERR_INVALID_ARG, "columns are not sorted inside a row");
        }
    }
    if (indptr[n_rows] == 0) return hfail(ASP_ERR_INVALID_ARG, "matrix without non-zeros");
    asp_matrix *h = new (std::nothrow) asp_matrix();
    if (!h) return hfail(ASP_ERR_ALLOC, "host allocation failed");
    try
    {
        h->m = matrix_from_csr(n_rows, n_cols, indptr, indices, values, val_dtype);
    }
    catch (const std::bad_alloc &)
    {
        delete h;
        return hfail(ASP_ERR_ALLOC, "host allocation failed");
    }
    *out = h;
    return ASP_OK;
}

asp_status asp_matrix_from_coo_file(const char *path, int val_dtype, asp_matrix **out)
{
    if (!out || !path) return hfail(ASP_ERR_INVALID_ARG, "NULL argument");
    *out = nullptr;
    if (val_dtype != ASP_F32 && val_dtype != ASP_F64) return hfail(ASP_ERR_UNSUPPORTED, "values must be f32 or f64");
    std::string err;
    std::unique_ptr<Matrix> m;
    try
    {
        m = matrix_from_coo_file(path, val_dtype, err);
    }
    catch (const std::bad_alloc &)
    {
        return hfail(ASP_ERR_ALLOC, "host allocation failed");
    }
    if (!m) return hfail(ASP_ERR_INVALID_ARG, err);
    if (m->nnz == 0) return hfail(ASP_ERR_INVALID_ARG, "matrix without non-zeros");
    asp_matrix *h = new (std::nothrow) asp_matrix();
    if (!h) return hfail(ASP_ERR_ALLOC, "host allocation failed");
    h->m = std::move(m);
    *out = h;
    return ASP_OK;
}

asp_status asp_matrix_relabel_by_column_count(const asp_matrix *m, int empty_rows_last, asp_matrix **out, uint32_t *labels, uint64_t *n_active)
{
    if (!m || !out) return hfail(ASP_ERR_INVALID_ARG, "NULL argument");
    *out = nullptr;
    const Matrix &src = *m->m;
    if (src.n_rows != src.n_cols) return hfail(ASP_ERR_INVALID_ARG, "renumbering vertices needs a square matrix");
    if (src.is_sorted || src.is_blocked || src.is_compressed) return hfail(ASP_ERR_INVALID_ARG, "renumber the matrix before any dense-view node runs");
    asp_matrix *h = new (std::nothrow) asp_matrix();
    if (!h) return hfail(ASP_ERR_ALLOC, "host allocation failed");
    try
    {
        std::vector<u32> lab;
        u64 active = 0;
        h->m = relabel_by_column_count(src, empty_rows_last != 0, lab, active);
        if (labels) memcpy(labels, lab.data(), lab.size() * sizeof(u32));
        if (n_active) *n_active = active;
    }
    catch (const std::bad_alloc &)
    {
        delete h;
        return hfail(ASP_ERR_ALLOC, "host allocation failed");
    }
    *out = h;
    return ASP_OK;
}

asp_status asp_partition_rows_by_nnz(uint64_t n_rows, const int64_t *indptr, int parts, uint64_t *bounds)
{
    if (!indptr || !bounds || parts <= 0 || n_rows == 0) return hfail(ASP_ERR_INVALID_ARG, "NULL argument or parts <= 0");
    const int64_t nnz = indptr[n_rows];
    bounds[0] = 0;
    for (int p = 1; p < parts; p++)
    {
        // first row whose offset reaches p/parts of the non-zeros; rows are never split
        const int64_t target = (int64_t)(((__int128)nnz * p) / parts);
        const int64_t *it = std::lower_bound(indptr, indptr + n_rows + 1, target);
        uint64_t r = (uint64_t)(it - indptr);
        if (r > n_rows) r = n_rows;
        if (r < bounds[p - 1]) r = bounds[p - 1];
        bounds[p] = r;
    }
    bounds[parts] = n_rows;
    return ASP_OK;
}

void asp_matrix_destroy(asp_matrix *m) { delete m; }
uint64_t asp_matrix_rows(const asp_matrix *m) { return m ? m->m->n_rows : 0; }
uint64_t asp_matrix_cols(const asp_matrix *m) { return m ? m->m->n_cols : 0; }
uint64_t asp_matrix_nnz(const asp_matrix *m) { return m ? m->m->nnz : 0; }

asp_status asp_dense_execute(const asp_matrix *in, const char *spec, asp_matrix **out)
{
    if (!in || !spec || !out) return hfail(ASP_ERR_INVALID_ARG, "NULL argument");
    *out = nullptr;
    if (in->m->is_compressed) return hfail(ASP_ERR_INVALID_ARG, "matrix is already compressed");
    try
    {
        std::unique_ptr<asp_matrix> h(new asp_matrix());
        h->m.reset(new Matrix(*in->m));
        Matrix &m = *h->m;
        bool compressed = false;
        std::istringstream f(spec);
        std::string line;
        while (std::getline(f, line))
        {
            const size_t hash = line.find('#');
            if (hash != std::string::npos) line = line.substr(0, hash);
            std::istringstream is(line);
            std::vector<std::string> tok;
            std::string w;
            while (is >> w) tok.push_back(w);
            if (tok.empty()) continue;
            if (tok[0] != "dense" || tok.size() < 2) return hfail(ASP_ERR_INVALID_ARG, "only dense-view nodes are allowed here: " + line);
            if (compressed) return hfail(ASP_ERR_INVALID_ARG, "dense-view node after compress");
            std::string err;
            if (!apply_dense_node(m, std::vector<std::string>(tok.begin() + 1, tok.end()), compressed, err)) return hfail(ASP_ERR_INVALID_ARG, err);
        }
        if (!compressed) compress_dense_view(m);
        std::vector<u32>().swap(m.col);
        std::vector<uint8_t>().swap(m.val.b);
        *out = h.release();
    }
    catch (const std::bad_alloc &)
    {
        return hfail(ASP_ERR_ALLOC, "host allocation failed");
    }
    return ASP_OK;
}

int asp_matrix_num_subs(const asp_matrix *m) { return (m && m->m->is_compressed) ? (int)m->m->blocks.size() : 0; }

asp_status asp_matrix_sub_rows(const asp_matrix *m, int sub, uint64_t *n_rows, uint64_t *nnz, uint64_t *min_row_nnz, uint64_t *max_row_nnz)
{
    if (!m || !m->m->is_compressed || sub < 0 || sub >= (int)m->m->blocks.size()) return hfail(ASP_ERR_INVALID_ARG, "bad sub-matrix id");
    const CompressedBlock &b = m->m->blocks[sub];
    u64 mn = ~0ull, mx = 0;
    for (u64 r = 0; r < b.n_rows; r++)
    {
        const u64 l = b.rowptr[r + 1] - b.rowptr[r];
        mn = std::min(mn, l);
        mx = std::max(mx, l);
    }
    if (n_rows) *n_rows = b.n_rows;
    if (nnz) *nnz = b.col.size();
    if (min_row_nnz) *min_row_nnz = mn;
    if (max_row_nnz) *max_row_nnz = mx;
    return ASP_OK;
}

asp_status asp_graph_execute(const asp_matrix *in, const char *spec, asp_format **out)
{
    if (!in || !spec || !out) return hfail(ASP_ERR_INVALID_ARG, "NULL argument");
    *out = nullptr;
    std::vector<std::vector<std::string>> dense_ops;
    std::map<long, SubSpec> subs;
    {
        std::istringstream f(spec);
        std::string line;
        while (std::getline(f, line))
        {
            const size_t h = line.find('#');
            if (h != std::string::npos) line = line.substr(0, h);
            std::istringstream is(line);
            std::vector<std::string> tok;
            std::string w;
            while (is >> w) tok.push_back(w);
            if (tok.empty()) continue;
            if (tok[0] == "dtype" || tok[0] == "fix_values") continue; // oracle-driver directives
            if (tok[0] == "dense" && tok.size() >= 2) dense_ops.push_back(std::vector<std::string>(tok.begin() + 1, tok.end()));
            else if (tok[0] == "sub" && tok.size() >= 3)
            {
                const long id = tok[1] == "all" ? -1 : atol(tok[1].c_str());
                SubSpec &s = subs[id];
                if (tok[2] == "template")
                {
                    if (tok.size() < 4) return hfail(ASP_ERR_INVALID_ARG, "template without a name");
                    s.templ = tok[3];
                    if (tok.size() > 4) s.tblock = atol(tok[4].c_str());
                    if (tok.size() > 5) s.threads = atol(tok[5].c_str());
                    if (tok.size() > 6) s.reduce = atol(tok[6].c_str());
                }
                else
                    s.nodes.push_back(std::vector<std::string>(tok.begin() + 2, tok.end()));
            }
            else
                return hfail(ASP_ERR_INVALID_ARG, "bad directive: " + line);
        }
    }
    try
    {
        std::unique_ptr<asp_format> F(new asp_format());
        auto sub_spec_of = [&](size_t i) -> const SubSpec * {
            if (subs.count((long)i)) return &subs[(long)i];
            if (subs.count(-1)) return &subs[-1];
            return nullptr;
        };
        if (in->m->is_compressed)
        {
            // the dense view has been executed already (asp_dense_execute): copy only the blocks
            // this graph lowers, the way the reference value-copies the compressed matrix per trial
            if (!dense_ops.empty()) return hfail(ASP_ERR_INVALID_ARG, "dense-view node on a matrix that is already compressed");
            const Matrix &src = *in->m;
            F->m.reset(new Matrix());
            Matrix &m = *F->m;
            m.n_rows = src.n_rows;
            m.n_cols = src.n_cols;
            m.nnz = src.nnz;
            m.val_dt = src.val_dt;
            m.is_sorted = src.is_sorted;
            m.sorted_row_index = src.sorted_row_index;
            m.perm_dt = src.perm_dt;
            m.perm = src.perm;
            m.is_blocked = src.is_blocked;
            m.is_compressed = true;
            m.ranges = src.ranges;
            m.blocks.resize(src.blocks.size());
            for (size_t i = 0; i < src.blocks.size(); i++)
            {
                const SubSpec *sp = sub_spec_of(i);
                if (!sp) return hfail(ASP_ERR_INVALID_ARG, "no spec for sub-matrix " + std::to_string(i));
                if (template_of_name(sp->templ) == ASP_EMPTY_TEMPLATE)
                {
                    CompressedBlock &b = m.blocks[i];
                    const CompressedBlock &o = src.blocks[i];
                    b.min_row = o.min_row, b.max_row = o.max_row, b.min_col = o.min_col, b.max_col = o.max_col;
                    b.begin_coo = o.begin_coo, b.end_coo = o.end_coo;
                }
                else
                    m.blocks[i] = src.blocks[i];
            }
        }
        else
        {
            F->m.reset(new Matrix(*in->m));
            Matrix &m = *F->m;
            bool compressed = false;
            for (const std::vector<std::string> &tok : dense_ops)
            {
                if (compressed) return hfail(ASP_ERR_INVALID_ARG, "dense-view node after compress");
                std::string err;
                if (!apply_dense_node(m, tok, compressed, err)) return hfail(ASP_ERR_INVALID_ARG, err);
            }
            if (!compressed) compress_dense_view(m);
            // the dense view is no longer needed once every block holds its slice
            std::vector<u32>().swap(m.col);
            std::vector<uint8_t>().swap(m.val.b);
        }
        Matrix &m = *F->m;
        const size_t nsub = m.blocks.size();
        F->subs.resize(nsub);
        for (size_t i = 0; i < nsub; i++)
        {
            const SubSpec *s = sub_spec_of(i);
            if (!s) return hfail(ASP_ERR_INVALID_ARG, "no spec for sub-matrix " + std::to_string(i));
            if (template_of_name(s->templ) == ASP_EMPTY_TEMPLATE)
            {
                F->subs[i] = TemplateData();
                continue;
            }
            CompressedBlock &b = m.blocks[i];
            std::string err;
            for (const std::vector<std::string> &tok : s->nodes)
                if (!apply_sub_node(b, tok, err)) return hfail(ASP_ERR_INVALID_ARG, err);
            const int type = template_of_name(s->templ);
            if ((b.block_r != 0) != (type == ASP_BLOCK_ELL_TEMPLATE)) return hfail(ASP_ERR_INVALID_ARG, "the block_value node and the template B1 go together");
            if ((b.diag_max != 0) != (type == ASP_DIAG_TEMPLATE)) return hfail(ASP_ERR_INVALID_ARG, "the diag_value node and the template D1 go together");
            if (!b.block_r && !b.diag_max) complete_each_level_blocking(b);
            if (type < 0) return hfail(ASP_ERR_INVALID_ARG, "unknown template " + s->templ);
            if (type == ASP_EMPTY_TEMPLATE)
            {
                F->subs[i] = TemplateData();
                continue;
            }
            if (!init_template(m, i, type, F->subs[i], err)) return hfail(ASP_ERR_UNSUPPORTED, err);
            if (s->tblock > 0) F->subs[i].tblock_num = s->tblock;
            if (s->threads > 0) F->subs[i].thread_num_in_block = s->threads;
            if (s->reduce > 0) F->subs[i].thread_num_of_row_reduce = s->reduce;
            // the tiled intermediate is not needed once the template owns its arrays
            std::vector<u32>().swap(b.pad_col);
            std::vector<uint8_t>().swap(b.pad_val.b);
            std::vector<u32>().swap(b.col);
            std::vector<uint8_t>().swap(b.val.b);
            std::vector<u64>().swap(b.tlb.first_row.v);
        }
        F->build_descs();
        F->cache_from_matrix();
        *out = F.release();
    }
    catch (const std::bad_alloc &)
    {
        return hfail(ASP_ERR_ALLOC, "host allocation failed");
    }
    catch (const std::length_error &e)
    {
        return hfail(ASP_ERR_UNSUPPORTED, std::string("graph rejected: ") + e.what());
    }
    return ASP_OK;
}

void asp_format_destroy(asp_format *f) { delete f; }
int asp_format_num_subs(const asp_format *f) { return f ? (int)f->subs.size() : 0; }
uint64_t asp_format_id(const asp_format *f) { return f ? f->id : 0; }

asp_status asp_format_global_perm(const asp_format *f, const void **ptr, int *dtype, uint64_t *len)
{
    if (!f || !ptr || !dtype || !len) return hfail(ASP_ERR_INVALID_ARG, "NULL argument");
    if (f->perm)
    {
        *ptr = f->perm->data();
        *dtype = f->perm_dt;
        *len = f->n_rows;
    }
    else
    {
        *ptr = nullptr;
        *dtype = ASP_U8;
        *len = 0;
    }
    return ASP_OK;
}

asp_status asp_format_sub_info(const asp_format *f, int sub, asp_sub_info *out)
{
    if (!f || !out || sub < 0 || sub >= (int)f->subs.size()) return hfail(ASP_ERR_INVALID_ARG, "bad sub-matrix id");
    *out = f->infos[sub];
    return ASP_OK;
}

asp_status asp_format_plan_descs(const asp_format *f, asp_plan_desc *descs)
{
    if (!f || !descs) return hfail(ASP_ERR_INVALID_ARG, "NULL argument");
    for (size_t i = 0; i < f->subs.size(); i++)
    {
        const TemplateData &t = f->subs[i];
        asp_plan_desc &d = descs[i];
        memset(&d, 0, sizeof(d));
        d.template_type = t.template_type;
        d.val_dtype = f->val_dt;
        d.n_rows = f->n_rows;
        d.n_cols = f->n_cols;
        d.first_row = t.first_row;
        d.first_col = t.first_col;
        d.true_nnz = t.true_nnz;
        d.n_arrays = (int32_t)f->descs[i].size();
        d.arrays = f->descs[i].data();
        d.effective_num = t.effective_num;
        d.tlb_size = t.tlb_size;
        d.bits_word = t.bits_word;
        d.bits_flag = t.bits_flag;
        d.bits_row = t.bits_row;
        d.bits_off = t.bits_off;
        d.is_atom_add = t.is_atom_add ? 1 : 0;
        d.sort_kind = t.sort_kind;
        d.tblock_num = t.tblock_num;
        d.thread_num_in_block = t.thread_num_in_block;
        d.thread_num_of_row_reduce = t.thread_num_of_row_reduce;
    }
    return ASP_OK;
}

double asp_format_padding_rate(const asp_format *f, int sub)
{
    if (!f || sub < 0 || sub >= (int)f->subs.size()) return 0.0;
    const TemplateData &t = f->subs[sub];
    const TemplateArray *v = t.find(ASP_ARR_VAL);
    if (!v || t.true_nnz == 0) return 0.0;
    return (double)v->len / (double)t.true_nnz;
}

} // extern "C"
