// Dense-view and compressed-view format operators (see format.hpp).
#include "format.hpp"

#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif
#include <algorithm>
#include <stdexcept>
#include <fstream>
#include <map>
#include <numeric>
#include <set>
#include <sstream>

namespace asp
{
namespace host
{

int suitable_dtype(u64 v)
{
    if (v <= 255ull) return ASP_U8;
    if (v <= 65535ull) return ASP_U16;
    if (v <= 4294967295ull) return ASP_U32;
    return ASP_U64;
}

int dtype_bytes(int dt)
{
    switch (dt)
    {
    case ASP_U8: return 1;
    case ASP_U16: return 2;
    case ASP_U32: case ASP_F32: return 4;
    default: return 8;
    }
}

const TemplateArray *TemplateData::find(int role) const
{
    for (const TemplateArray &a : arrays)
        if (a.role == role) return &a;
    return nullptr;
}

// ---------------------------------------------------------------------------------------------
// input
// ---------------------------------------------------------------------------------------------
std::unique_ptr<Matrix> matrix_from_csr(u64 n_rows, u64 n_cols, const int64_t *indptr, const u32 *indices, const void *values, int val_dt)
{
    std::unique_ptr<Matrix> m(new Matrix());
    m->n_rows = n_rows;
    m->n_cols = n_cols;
    m->nnz = (u64)indptr[n_rows];
    m->val_dt = val_dt;
    m->rowptr.resize(n_rows + 1);
    for (u64 i = 0; i <= n_rows; i++) m->rowptr[i] = (u64)indptr[i];
    m->col.assign(indices, indices + m->nnz);
    m->val.es = dtype_bytes(val_dt);
    m->val.b.assign((const uint8_t *)values, (const uint8_t *)values + m->nnz * m->val.es);
    return m;
}

// Vertices of a square matrix renumbered by how often their column occurs, most frequent first (ties keep their
// order), optionally with the vertices whose row is empty last; returns P A P^T (columns sorted inside every row).
// Not an operator of the reference: for x <- A x loops on graphs, where the numbering is free and a numbering that
// makes the often-read entries of x contiguous is worth 10-15 % of the SpMV time once x no longer fits the L2.
std::unique_ptr<Matrix> relabel_by_column_count(const Matrix &m, bool empty_rows_last, std::vector<u32> &labels, u64 &n_active)
{
    const u64 n = m.n_rows;
    std::vector<u64> cnt(n, 0);
#pragma omp parallel for schedule(static)
    for (long long k = 0; k < (long long)m.nnz; k++)
    {
#pragma omp atomic
        cnt[m.col[k]]++;
    }
    std::vector<u32> order(n);
    for (u64 i = 0; i < n; i++) order[i] = (u32)i;
    std::stable_sort(order.begin(), order.end(), [&](u32 a, u32 b) { return cnt[a] > cnt[b]; });
    n_active = 0;
    for (u64 r = 0; r < n; r++) n_active += m.rowptr[r + 1] > m.rowptr[r] ? 1 : 0;
    if (empty_rows_last) std::stable_partition(order.begin(), order.end(), [&](u32 v) { return m.rowptr[v + 1] > m.rowptr[v]; });
    labels.assign(n, 0);
    for (u64 k = 0; k < n; k++) labels[order[k]] = (u32)k;
    std::unique_ptr<Matrix> out(new Matrix());
    out->n_rows = out->n_cols = n;
    out->nnz = m.nnz;
    out->val_dt = m.val_dt;
    out->rowptr.assign(n + 1, 0);
    for (u64 k = 0; k < n; k++) out->rowptr[k + 1] = out->rowptr[k] + (m.rowptr[order[k] + 1] - m.rowptr[order[k]]);
    out->col.resize(m.nnz);
    out->val.es = m.val.es;
    out->val.b.resize(m.nnz * m.val.es);
    const size_t es = (size_t)m.val.es;
#pragma omp parallel
    {
        std::vector<std::pair<u32, u64>> row; // (new column, position in the old row)
#pragma omp for schedule(dynamic, 256)
        for (long long k = 0; k < (long long)n; k++)
        {
            const u64 b = m.rowptr[order[k]], e = m.rowptr[order[k] + 1], o = out->rowptr[k];
            row.clear();
            for (u64 j = b; j < e; j++) row.push_back({labels[m.col[j]], j});
            std::sort(row.begin(), row.end());
            for (u64 j = 0; j < row.size(); j++)
            {
                out->col[o + j] = row[j].first;
                memcpy(&out->val.b[(o + j) * es], &m.val.b[row[j].second * es], es);
            }
        }
    }
    return out;
}

// The `.mtx.coo` grammar of the reference (struct.cc:92-174): the first line that does not start with white space
// is "rows cols ..."; every other such line is "row col value", 1-based, rows non-decreasing. The reference reads it
// with getline + split + atol / stof, one line at a time; here the file is read in one piece, cut at line ends into
// one slice per thread, and the slices are parsed in parallel with strtoull / strtod.
std::unique_ptr<Matrix> matrix_from_coo_file(const std::string &path, int val_dt, std::string &err)
{
    FILE *fp = fopen(path.c_str(), "rb");
    if (!fp)
    {
        err = "cannot open " + path;
        return nullptr;
    }
    std::vector<char> buf;
    {
        fseek(fp, 0, SEEK_END);
        const long sz = ftell(fp);
        fseek(fp, 0, SEEK_SET);
        buf.resize((size_t)std::max<long>(sz, 0) + 1);
        const size_t got = sz > 0 ? fread(buf.data(), 1, (size_t)sz, fp) : 0;
        fclose(fp);
        buf.resize(got + 1);
        buf[got] = '\n'; // a last line without a line end still terminates (the numbers are parsed up to it)
    }
    const char *base = buf.data(), *end = base + buf.size();
    auto skipped = [](const char *p) { return *p == '\n' || *p == ' ' || *p == '\t' || *p == '\r'; }; // empty, or starting with white space
    auto next_line = [&](const char *p) {
        while (p < end && *p != '\n') p++;
        return p < end ? p + 1 : end;
    };
    // header
    const char *p = base;
    while (p < end && skipped(p)) p = next_line(p);
    u64 n_rows = 0, n_cols = 0;
    {
        char *q = nullptr;
        if (p >= end || !(*p >= '0' && *p <= '9'))
        {
            err = "bad header line";
            return nullptr;
        }
        n_rows = strtoull(p, &q, 10);
        const char *q2 = q;
        while (*q2 == ' ' || *q2 == '\t') q2++;
        if (!(*q2 >= '0' && *q2 <= '9'))
        {
            err = "bad header line";
            return nullptr;
        }
        n_cols = strtoull(q2, &q, 10);
        p = next_line(p);
    }
    // slices of whole lines, one per thread
    int nt = 1;
#ifdef _OPENMP
    nt = omp_get_max_threads();
#endif
    const size_t body = (size_t)(end - p);
    nt = (int)std::max<size_t>(1, std::min<size_t>((size_t)nt, body / (1u << 16) + 1));
    std::vector<const char *> cut(nt + 1);
    cut[0] = p;
    cut[nt] = end;
    for (int t = 1; t < nt; t++)
    {
        const char *c = p + body / nt * t;
        cut[t] = (c <= cut[t - 1]) ? cut[t - 1] : next_line(c - 1);
    }
    struct Part
    {
        std::vector<u64> rows;
        std::vector<u32> cols;
        std::vector<double> vals;
        std::string err;
    };
    std::vector<Part> parts(nt);
#pragma omp parallel for schedule(static, 1) num_threads(nt)
    for (int t = 0; t < nt; t++)
    {
        Part &pt = parts[t];
        const char *s = cut[t], *e = cut[t + 1];
        pt.rows.reserve((size_t)(e - s) / 12 + 16);
        pt.cols.reserve((size_t)(e - s) / 12 + 16);
        pt.vals.reserve((size_t)(e - s) / 12 + 16);
        u64 last = 0;
        while (s < e)
        {
            if (skipped(s))
            {
                s = next_line(s);
                continue;
            }
            char *q = nullptr;
            const u64 r = strtoull(s, &q, 10);
            const char *a1 = q;
            const u64 c = strtoull(a1, &q, 10);
            const char *a2 = q;
            const double v = strtod(a2, &q);
            if (a1 == s || a2 == a1 || q == a2 || r == 0 || c == 0 || r > n_rows || c > n_cols)
            {
                pt.err = "bad entry: " + std::string(s, (size_t)(next_line(s) - s - 1));
                break;
            }
            if (r < last)
            {
                pt.err = "rows are not non-decreasing";
                break;
            }
            last = r;
            pt.rows.push_back(r - 1);
            pt.cols.push_back((u32)(c - 1));
            pt.vals.push_back(v);
            s = next_line(q);
        }
    }
    u64 nnz = 0;
    for (int t = 0; t < nt; t++)
    {
        if (!parts[t].err.empty())
        {
            err = parts[t].err;
            return nullptr;
        }
        if (t > 0 && !parts[t].rows.empty())
            for (int u = t - 1; u >= 0; u--)
                if (!parts[u].rows.empty())
                {
                    if (parts[t].rows.front() < parts[u].rows.back())
                    {
                        err = "rows are not non-decreasing";
                        return nullptr;
                    }
                    break;
                }
        nnz += parts[t].rows.size();
    }
    std::unique_ptr<Matrix> m(new Matrix());
    m->n_rows = n_rows;
    m->n_cols = n_cols;
    m->nnz = nnz;
    m->val_dt = val_dt;
    m->rowptr.assign(n_rows + 1, 0);
    m->col.resize(nnz);
    m->val.es = dtype_bytes(val_dt);
    m->val.resize(nnz);
    u64 off = 0;
    for (int t = 0; t < nt; t++)
    {
        const Part &pt = parts[t];
        for (u64 r : pt.rows) m->rowptr[r + 1]++;
        std::copy(pt.cols.begin(), pt.cols.end(), m->col.begin() + off);
        if (val_dt == ASP_F64) memcpy(m->val.b.data() + off * 8, pt.vals.data(), pt.vals.size() * 8);
        else
            for (u64 i = 0; i < pt.vals.size(); i++) ((float *)m->val.b.data())[off + i] = (float)pt.vals[i];
        off += pt.rows.size();
    }
    for (u64 i = 0; i < n_rows; i++) m->rowptr[i + 1] += m->rowptr[i];
    return m;
}

// ---------------------------------------------------------------------------------------------
// dense view
// ---------------------------------------------------------------------------------------------
void dense_row_coarse_sort(Matrix &m, u64 step)
{
    const u64 R = m.n_rows;
    std::vector<u64> len(R);
    u64 mn = ~0ull, mx = 0;
    for (u64 r = 0; r < R; r++)
    {
        len[r] = m.rowptr[r + 1] - m.rowptr[r];
        mn = std::min(mn, len[r]);
        mx = std::max(mx, len[r]);
    }
    // bin low bounds (execute_dense_row_coarse_sort_fixed_param_strategy, parameter_set_strategy.cc:441):
    // step 1 -> one bin per distinct row length, the smallest bound replaced by 0
    std::vector<u64> low;
    if (step == 1)
    {
        std::vector<u64> d(len);
        std::sort(d.begin(), d.end());
        d.erase(std::unique(d.begin(), d.end()), d.end());
        for (size_t i = 0; i < d.size(); i++) low.push_back(i == 0 ? 0 : d[i]);
    }
    else
        for (u64 i = mn; i <= mx; i += step) low.push_back(i == mn ? 0 : i);
    const size_t nb = low.size();
    auto bin_of = [&](u64 l) { return (size_t)(std::upper_bound(low.begin(), low.end(), l) - low.begin()) - 1; };
    // stable counting sort of the non-empty rows by bin, largest bin first; empty rows keep their
    // order and go last
    std::vector<u64> cnt(nb + 1, 0);
    std::vector<size_t> bin(R);
    u64 n_empty = 0;
    for (u64 r = 0; r < R; r++)
    {
        if (len[r] == 0)
        {
            n_empty++;
            continue;
        }
        bin[r] = bin_of(len[r]);
        cnt[bin[r]]++;
    }
    std::vector<u64> start(nb, 0);
    u64 acc = 0;
    for (size_t b = nb; b-- > 0;)
    {
        start[b] = acc;
        acc += cnt[b];
    }
    m.perm.assign(R, 0);
    u64 epos = acc;
    for (u64 r = 0; r < R; r++)
    {
        if (len[r] == 0) m.perm[epos++] = r;
        else m.perm[start[bin[r]]++] = r;
    }
    // rewrite the dense view in the new row order
    std::vector<u64> nrp(R + 1, 0);
    for (u64 i = 0; i < R; i++) nrp[i + 1] = nrp[i] + len[m.perm[i]];
    std::vector<u32> ncol(m.nnz);
    ValBuf nval;
    nval.es = m.val.es;
    nval.b.resize(m.val.b.size());
    const int es = m.val.es;
#pragma omp parallel for schedule(dynamic, 4096)
    for (u64 i = 0; i < R; i++)
    {
        const u64 o = m.perm[i], n = len[o];
        if (n == 0) continue;
        memcpy(&ncol[nrp[i]], &m.col[m.rowptr[o]], n * sizeof(u32));
        memcpy(&nval.b[nrp[i] * es], &m.val.b[m.rowptr[o] * es], n * es);
    }
    m.rowptr.swap(nrp);
    m.col.swap(ncol);
    m.val.b.swap(nval.b);
    m.is_sorted = true;
    m.perm_dt = suitable_dtype(R);
    const int pb = dtype_bytes(m.perm_dt);
    m.sorted_row_index.reset(new std::vector<uint8_t>(R * pb));
    uint8_t *p = m.sorted_row_index->data();
    for (u64 i = 0; i < R; i++) memcpy(p + i * pb, &m.perm[i], pb); // little endian narrowing
}

std::vector<u64> row_div_position_exponential(const Matrix &m, u64 lowest, u64 highest, u64 rate)
{
    std::vector<u64> range;
    range.push_back(0);
    for (u64 b = lowest; b <= highest; b *= rate) range.push_back(b);
    if (range.back() != highest) range.push_back(highest);
    auto range_of = [&](u64 l) { return (size_t)(std::upper_bound(range.begin(), range.end(), l) - range.begin()) - 1; };
    std::vector<u64> pos;
    pos.push_back(0);
    size_t last = range_of(m.rowptr[1] - m.rowptr[0]);
    for (u64 r = 1; r < m.n_rows; r++)
    {
        const size_t cur = range_of(m.rowptr[r + 1] - m.rowptr[r]);
        if (cur != last)
        {
            pos.push_back(r);
            last = cur;
        }
    }
    pos.push_back(m.n_rows);
    return pos;
}

void dense_row_div(Matrix &m, const std::vector<u64> &pos)
{
    // strips without non-zeros are dropped (var_len_row_div, op_manager.cc:370)
    m.ranges.clear();
    for (size_t i = 0; i + 1 < pos.size(); i++)
    {
        const u64 r0 = pos[i], r1 = std::min<u64>(pos[i + 1], m.n_rows);
        if (r1 <= r0) continue;
        const u64 b = m.rowptr[r0], e = m.rowptr[r1];
        if (e <= b) continue;
        m.ranges.push_back({r0, r1 - 1, b, e - 1});
    }
    m.is_blocked = true;
}

void compress_dense_view(Matrix &m)
{
    if (!m.is_blocked && m.ranges.empty()) m.ranges.push_back({0, m.n_rows - 1, 0, m.nnz - 1});
    m.blocks.clear();
    m.blocks.resize(m.ranges.size());
    for (size_t i = 0; i < m.ranges.size(); i++)
    {
        const Matrix::BlockRange &rg = m.ranges[i];
        CompressedBlock &b = m.blocks[i];
        b.min_row = rg.min_row;
        b.max_row = rg.max_row;
        b.min_col = 0;
        b.max_col = m.n_cols - 1;
        b.begin_coo = rg.begin_coo;
        b.end_coo = rg.end_coo;
        b.n_rows = rg.max_row - rg.min_row + 1;
        b.row_dt = suitable_dtype(b.n_rows);                 // counts, not maxima: 65536 rows -> u32
        b.col_dt = suitable_dtype(b.max_col - b.min_col + 1);
        b.rowptr.resize(b.n_rows + 1);
        for (u64 r = 0; r <= b.n_rows; r++) b.rowptr[r] = m.rowptr[rg.min_row + r] - rg.begin_coo;
        const u64 n = rg.end_coo - rg.begin_coo + 1;
        b.col.assign(m.col.begin() + rg.begin_coo, m.col.begin() + rg.begin_coo + n);
        b.val.es = m.val.es;
        // every block holds ITS slice of the values; the reference copies from offset 0 for every
        // block (op_manager.cc:1077-1087), which is only right for the first one
        b.val.b.assign(m.val.b.begin() + rg.begin_coo * m.val.es, m.val.b.begin() + (rg.begin_coo + n) * m.val.es);
    }
    m.is_compressed = true;
}

// ---------------------------------------------------------------------------------------------
// compressed view
// ---------------------------------------------------------------------------------------------
void row_padding(CompressedBlock &b, u64 multiple, u64 plen)
{
    const u64 rows = b.max_row - b.min_row + 1;
    if (rows % multiple == 0) return;
    const u64 target = (rows / multiple + 1) * multiple;
    const u64 add = target - rows;
    const u64 old_nnz = b.col.size();
    b.col.resize(old_nnz + add * plen, 0); // fake rows: `plen` zeros at (relative) column 0
    b.val.b.resize((old_nnz + add * plen) * b.val.es, 0);
    b.rowptr.resize(target + 1);
    for (u64 r = rows; r < target; r++) b.rowptr[r + 1] = b.rowptr[r] + plen;
    b.n_rows = target;
    b.row_dt = suitable_dtype(target);
}

std::vector<u64> blb_rows_evenly(const CompressedBlock &b, u64 n)
{
    std::vector<u64> out(b.n_rows / n, n);
    if (b.n_rows % n) out.push_back(b.n_rows % n);
    return out;
}

std::vector<u64> blb_rows_by_nnz_low_bound(const CompressedBlock &b, u64 low)
{
    std::vector<u64> out;
    u64 rows = 0, nnz = 0;
    for (u64 r = 0; r < b.n_rows; r++)
    {
        nnz += b.rowptr[r + 1] - b.rowptr[r];
        rows++;
        if (nnz >= low)
        {
            out.push_back(rows);
            rows = 0;
            nnz = 0;
        }
    }
    if (rows > 0)
    {
        if (nnz == 0)
        {
            if (!out.empty()) out.back() += rows;
        }
        else
            out.push_back(rows);
    }
    return out;
}

void sep_tblock_level_row_csr(CompressedBlock &b, const std::vector<u64> &rows_of)
{
    Level &L = b.blb;
    L = Level();
    u64 sum = 0, mx = 0;
    for (u64 n : rows_of)
    {
        sum += n;
        mx = std::max(mx, n);
    }
    L.first_row.dt = suitable_dtype(sum + 1);
    L.row_num.dt = suitable_dtype(mx);
    L.coo_begin.dt = suitable_dtype(b.col.size());
    u64 r = 0;
    for (u64 n : rows_of)
    {
        const u64 r1 = std::min(r + n, b.n_rows);
        if (r < b.n_rows && b.rowptr[r1] > b.rowptr[r]) // blocks without non-zeros are dropped
        {
            L.first_row.v.push_back(r);
            L.row_num.v.push_back(n);
            L.coo_begin.v.push_back(b.rowptr[r]);
        }
        r += n;
    }
    L.coo_begin.v.push_back(b.col.size());
    L.block_num = L.first_row.v.size();
    L.built = true;
}

void sep_tblock_level_col_fixed(CompressedBlock &b, u64 c)
{
    // one BLB per non-empty row first (one_row_sep_tblock_level_row_csr), then every row is cut at
    // the cumulative chunk sizes of col_block_size_of_each_row and at its end
    Level &L = b.blb;
    L = Level();
    L.first_row.dt = suitable_dtype(b.n_rows + 1);
    L.row_num.dt = ASP_U8;
    L.coo_begin.dt = suitable_dtype(b.col.size());
    for (u64 r = 0; r < b.n_rows; r++)
    {
        const u64 n = b.rowptr[r + 1] - b.rowptr[r];
        if (n == 0) continue;
        const u64 full = n / c, rem = n % c;
        // nominal sizes: `full` chunks of c; remainder >= c/2 -> one more chunk; else merged into the
        // last chunk (or the only one)
        std::vector<u64> sizes(full, c);
        if (rem >= c / 2) sizes.push_back(c);
        else if (sizes.empty()) sizes.push_back(c);
        else sizes.back() = 2 * c;
        u64 beg = b.rowptr[r], k = 0, acc = 0;
        for (u64 i = 0; i < n; i++)
        {
            if (i == acc + sizes[k] - 1)
            {
                L.first_row.v.push_back(r);
                L.coo_begin.v.push_back(beg);
                beg = b.rowptr[r] + i + 1;
                acc += sizes[k];
                k++;
                if (k >= sizes.size() && i + 1 < n) k = sizes.size() - 1; // not reached with the sizes above
            }
        }
        if (beg != b.rowptr[r + 1])
        {
            L.first_row.v.push_back(r);
            L.coo_begin.v.push_back(beg);
        }
    }
    L.row_num.v.assign(L.first_row.v.size(), 1);
    L.coo_begin.v.push_back(b.col.size());
    L.block_num = L.first_row.v.size();
    L.built = true;
    b.share_row_with_other_block = true;
}

void sep_warp_level_row_csr(CompressedBlock &b, const std::vector<std::vector<u64>> &rows_of)
{
    Level &B = b.blb;
    Level &W = b.wlb;
    W = Level();
    u64 max_first_row = 0, max_coo_begin = 0, max_size = 0;
    B.index.v.assign(1, 0);
    for (u64 i = 0; i < B.block_num; i++)
    {
        const u64 br0 = B.first_row.v[i];
        const u64 c0 = B.coo_begin.v[i], c1 = B.coo_begin.v[i + 1];
        u64 made = 0;
        if (i < rows_of.size())
        {
            // WLBs that own at least one non-zero, in row order
            u64 r = 0;
            for (u64 n : rows_of[i])
            {
                const u64 g0 = std::min(br0 + r, b.n_rows), g1 = std::min(br0 + r + n, b.n_rows);
                const u64 a = std::max(b.rowptr[g0], c0), e = std::min(b.rowptr[g1], c1);
                if (e > a)
                {
                    W.first_row.v.push_back(r);
                    W.row_num.v.push_back(n);
                    W.coo_begin.v.push_back(a - c0);
                    max_first_row = std::max(max_first_row, r);
                    max_coo_begin = std::max(max_coo_begin, a - c0);
                    made++;
                }
                r += n;
            }
        }
        else
        {
            W.first_row.v.push_back(0);
            W.row_num.v.push_back(B.row_num.v[i]);
            W.coo_begin.v.push_back(0);
            made = 1;
        }
        B.index.v.push_back(B.index.v.back() + made);
    }
    W.block_num = W.first_row.v.size();
    // block sizes: distance to the next WLB of the same BLB, the last one takes the rest
    W.coo_size.v.resize(W.block_num);
    for (u64 i = 0; i < B.block_num; i++)
    {
        const u64 nnz_b = B.coo_begin.v[i + 1] - B.coo_begin.v[i];
        for (u64 w = B.index.v[i]; w < B.index.v[i + 1]; w++)
        {
            const u64 e = (w + 1 < B.index.v[i + 1]) ? W.coo_begin.v[w + 1] : nnz_b;
            W.coo_size.v[w] = e - W.coo_begin.v[w];
            max_size = std::max(max_size, W.coo_size.v[w]);
        }
    }
    B.index.dt = suitable_dtype(B.index.v.back());
    W.first_row.dt = suitable_dtype(max_first_row + 1);
    W.row_num.dt = suitable_dtype(max_size);
    W.coo_begin.dt = suitable_dtype(max_coo_begin);
    W.coo_size.dt = suitable_dtype(max_size);
    W.built = true;
}

std::vector<std::vector<u64>> wlb_rows_evenly(const CompressedBlock &b, u64 rows)
{
    std::vector<std::vector<u64>> out;
    for (u64 i = 0; i < b.blb.block_num; i++)
    {
        const u64 n = b.blb.row_num.v[i];
        std::vector<u64> v(n / rows, rows);
        if (n % rows) v.push_back(n % rows);
        out.push_back(v);
    }
    return out;
}

void sep_warp_level_col_fixed(CompressedBlock &b, u64 c)
{
    // one WLB per non-empty row of every BLB first (one_row_sep_warp_level_row_csr), then every row is
    // cut into chunks of c non-zeros, the last chunk taking what is left
    Level &B = b.blb;
    Level &W = b.wlb;
    W = Level();
    u64 max_first_row = 0, max_coo_begin = 0, max_size = 0;
    B.index.v.assign(1, 0);
    for (u64 i = 0; i < B.block_num; i++)
    {
        const u64 br0 = B.first_row.v[i], rows = B.row_num.v[i];
        const u64 c0 = B.coo_begin.v[i], c1 = B.coo_begin.v[i + 1];
        u64 made = 0;
        for (u64 r = 0; r < rows && br0 + r < b.n_rows; r++)
        {
            const u64 a = std::max(b.rowptr[br0 + r], c0), e = std::min(b.rowptr[br0 + r + 1], c1);
            for (u64 p = a; p < e; p += c)
            {
                const u64 sz = std::min(c, e - p);
                W.first_row.v.push_back(r);
                W.coo_begin.v.push_back(p - c0);
                W.coo_size.v.push_back(sz);
                max_first_row = std::max(max_first_row, r);
                if (made > 0) max_coo_begin = std::max(max_coo_begin, p - c0);
                max_size = std::max(max_size, sz);
                made++;
            }
        }
        B.index.v.push_back(B.index.v.back() + made);
    }
    W.block_num = W.first_row.v.size();
    W.row_num.v.assign(W.block_num, 1);
    B.index.dt = suitable_dtype(B.index.v.back());
    W.first_row.dt = suitable_dtype(max_first_row + 1);
    W.row_num.dt = ASP_U8;
    W.coo_begin.dt = suitable_dtype(max_coo_begin);
    W.coo_size.dt = suitable_dtype(max_size);
    W.built = true;
    b.share_row_with_other_warp = true;
}

void sep_thread_level_col_ell_with_padding(CompressedBlock &b, u64 tlb_size)
{
    Level &B = b.blb;
    Level &W = b.wlb;
    Level &T = b.tlb;
    T = Level();
    const int es = b.val.es;
    // pass 1: per WLB the TLB size, TLBs per row (rounded up, then round-robin fillers from the
    // WLB's first row until the WLB holds a multiple of 32 TLBs), padded sizes
    std::vector<u64> wlb_S(W.block_num), wlb_tlb0(W.block_num + 1, 0), wlb_pad0(W.block_num + 1, 0);
    std::vector<u64> blb_first(B.block_num + 1, 0);
    u64 max_S = 0;
    bool share_thread = tlb_size != 0;
    for (u64 i = 0; i < B.block_num; i++)
    {
        for (u64 w = B.index.v[i]; w < B.index.v[i + 1]; w++)
        {
            const u64 r0 = B.first_row.v[i] + W.first_row.v[w], rows = W.row_num.v[w];
            const u64 a = B.coo_begin.v[i] + W.coo_begin.v[w], e = a + W.coo_size.v[w];
            u64 S = tlb_size;
            if (S == 0)
            {
                for (u64 r = 0; r < rows; r++)
                {
                    const u64 lo = std::max(b.rowptr[std::min(r0 + r, b.n_rows)], a), hi = std::min(b.rowptr[std::min(r0 + r + 1, b.n_rows)], e);
                    if (hi > lo) S = std::max(S, hi - lo);
                }
            }
            u64 tl = 0;
            for (u64 r = 0; r < rows; r++)
            {
                const u64 lo = std::max(b.rowptr[std::min(r0 + r, b.n_rows)], a), hi = std::min(b.rowptr[std::min(r0 + r + 1, b.n_rows)], e);
                const u64 n = hi > lo ? hi - lo : 0;
                tl += (n + S - 1) / S;
            }
            const u64 target = (tl + 31) / 32 * 32;
            wlb_S[w] = S;
            wlb_tlb0[w + 1] = wlb_tlb0[w] + target;
            wlb_pad0[w + 1] = wlb_pad0[w] + target * S;
            max_S = std::max(max_S, S);
        }
        blb_first[i + 1] = wlb_pad0[B.index.v[i + 1]];
    }
    const u64 n_tlb = wlb_tlb0[W.block_num], n_pad = wlb_pad0[W.block_num];
    // a few long rows in an ELL-shaped strip multiply the storage: stop before materialising a
    // format that no padding gate would let through (the search bound is 4x; 64x leaves room for
    // callers with their own bound)
    if (n_pad > 64 * std::max<u64>(b.col.size(), 1024)) throw std::length_error("padded size exceeds 64x the non-zeros of the sub-matrix");
    b.pad_col.assign(n_pad, 0);
    b.pad_val.es = es;
    b.pad_val.resize(n_pad);
    T.first_row.v.resize(n_tlb);
    u64 max_thread_first_row = 0, max_w_coo_begin = 0, max_w_size = 0;
    std::vector<u64> new_w_begin(W.block_num), new_w_size(W.block_num);
    // pass 2: fill the padded arrays (row-major inside the WLB) and the per-TLB first rows
    for (u64 i = 0; i < B.block_num; i++)
    {
        for (u64 w = B.index.v[i]; w < B.index.v[i + 1]; w++)
        {
            const u64 r0 = B.first_row.v[i] + W.first_row.v[w], rows = W.row_num.v[w];
            const u64 a = B.coo_begin.v[i] + W.coo_begin.v[w], e = a + W.coo_size.v[w];
            const u64 S = wlb_S[w];
            std::vector<u64> per_row(rows);
            u64 tl = 0;
            for (u64 r = 0; r < rows; r++)
            {
                const u64 lo = std::max(b.rowptr[std::min(r0 + r, b.n_rows)], a), hi = std::min(b.rowptr[std::min(r0 + r + 1, b.n_rows)], e);
                const u64 n = hi > lo ? hi - lo : 0;
                per_row[r] = (n + S - 1) / S;
                tl += per_row[r];
            }
            const u64 target = wlb_tlb0[w + 1] - wlb_tlb0[w];
            for (u64 k = 0, rr = 0; k < target - tl; k++, rr = (rr + 1) % rows) per_row[rr]++;
            u64 out = wlb_pad0[w], t = wlb_tlb0[w];
            for (u64 r = 0; r < rows; r++)
            {
                const u64 lo = std::max(b.rowptr[std::min(r0 + r, b.n_rows)], a), hi = std::min(b.rowptr[std::min(r0 + r + 1, b.n_rows)], e);
                const u64 n = hi > lo ? hi - lo : 0;
                const u64 tgt = per_row[r] * S;
                if (n > 0)
                {
                    memcpy(&b.pad_col[out], &b.col[lo], n * sizeof(u32));
                    memcpy(&b.pad_val.b[out * es], &b.val.b[lo * es], n * es);
                    const u32 last = b.col[hi - 1];
                    for (u64 k = n; k < tgt; k++) b.pad_col[out + k] = last; // value stays 0
                }
                else
                    for (u64 k = 0; k < tgt; k++) b.pad_col[out + k] = (u32)b.min_col;
                out += tgt;
                if (per_row[r] >= 2) share_thread = true;
                for (u64 k = 0; k < per_row[r]; k++) T.first_row.v[t++] = r;
                if (per_row[r] > 0) max_thread_first_row = std::max(max_thread_first_row, r);
            }
            new_w_size[w] = target * S;
            new_w_begin[w] = (w == B.index.v[i]) ? 0 : new_w_begin[w - 1] + new_w_size[w - 1];
            if (w != B.index.v[i]) max_w_coo_begin = std::max(max_w_coo_begin, new_w_begin[w]);
            max_w_size = std::max(max_w_size, new_w_size[w]);
        }
    }
    // the BLB / WLB offsets now refer to the padded arrays (op_manager.cc:3639-3680)
    B.coo_begin.v = blb_first;
    B.coo_begin.dt = suitable_dtype(n_pad);
    W.coo_begin.v = new_w_begin;
    W.coo_begin.dt = suitable_dtype(max_w_coo_begin);
    W.coo_size.v = new_w_size;
    W.coo_size.dt = suitable_dtype(max_w_size);
    W.index.v = wlb_tlb0;
    W.index.dt = suitable_dtype(n_tlb);
    T.block_num = n_tlb;
    T.first_row.dt = suitable_dtype(max_thread_first_row + 1);
    T.coo_size.v = wlb_S;
    T.coo_size.dt = suitable_dtype(max_S);
    T.built = true;
    b.padded = true;
    b.tlb_is_nnz_div = false;
    if (share_thread) b.share_row_with_other_thread = true;
}

void sep_thread_level_acc_to_nnz(CompressedBlock &b, u64 S)
{
    // equal-nnz TLBs regardless of row boundaries; columns and values are used as they are (no padding
    // here: the CSR5-like templates pad to whole warps themselves)
    Level &T = b.tlb;
    T = Level();
    const u64 nnz = b.col.size();
    T.block_num = (nnz + S - 1) / S;
    T.coo_size.v.assign(b.wlb.block_num, S);
    T.coo_size.dt = suitable_dtype(S);
    T.built = true;
    b.tlb_is_nnz_div = true;
    b.padded = false;
}

void complete_each_level_blocking(CompressedBlock &b)
{
    if (!b.blb.built) sep_tblock_level_row_csr(b, std::vector<u64>(1, b.n_rows));
    if (!b.wlb.built) sep_warp_level_row_csr(b, std::vector<std::vector<u64>>());
    if (!b.tlb.built) sep_thread_level_col_ell_with_padding(b, 1);
}

} // namespace host
} // namespace asp
