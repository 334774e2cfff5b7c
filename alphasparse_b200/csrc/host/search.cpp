// The search loop over Operator Graphs (the reference's search_strategy.cc stop rule, the whitelist
// strategies of whilte_list_path_impl.cc:3411-4579 and the launch sweeps of
// default_auto_tuner.cc:449-2030), written against the public host C ABI and a timing callback, so
// that the same loop runs with the GPU as the timer or, in the CPU tests, with a model of it.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "../../../include/asp_b200_host.h"

namespace
{
struct Launch
{
    int64_t threads, reduce;
};

struct Candidate
{
    std::string name;
    std::vector<std::string> nodes; // compressed-view node lines without the "sub <id>" prefix
    std::string templ;              // "K1" .. "K10"
    std::vector<Launch> launches;

    std::string lines(int sub) const
    {
        std::string s;
        const std::string pre = "sub " + std::to_string(sub) + " ";
        for (const std::string &n : nodes) s += pre + n + "\n";
        s += pre + "template " + templ;
        return s;
    }
};

// register_integer_independ_param_to_enumerater semantics: lo, lo + step, ... while <= hi
std::vector<int64_t> integer_range(int64_t lo, int64_t hi, int64_t step)
{
    std::vector<int64_t> v;
    for (int64_t x = lo; x <= hi; x += step) v.push_back(x);
    return v;
}

int64_t ceil32(int64_t v) { return (v + 31) / 32 * 32; }

std::vector<Launch> cross(const std::vector<int64_t> &threads, const std::vector<int64_t> &reduces)
{
    std::vector<Launch> l;
    for (int64_t t : threads)
        for (int64_t r : reduces) l.push_back({t, r});
    return l;
}

// ---- the reference's node-parameter grids (whilte_list_path_impl.cc), one function per strategy ------------
// `mode`: 1 = quick (one or two points per strategy, short launch sweeps), 0 = the reference's grids plus the
// extensions of this build (marked below), 2 = the reference's grids exactly (what the enumeration test compares
// with the reference's own tuner). In modes 0 and 2 the launch sweep of a point is derived from the lowered
// format (reference_launches), as default_auto_tuner.cc does; Candidate::launches is then only the fallback.
std::vector<Candidate> reference_candidates(int64_t mn, int64_t mx, uint64_t rows, uint64_t nnz, bool is_sorted, bool extensions)
{
    std::vector<Candidate> out;
    const std::vector<Launch> none;
    auto S = [](int64_t v) { return std::to_string(v); };
    if (extensions && !is_sorted)
    {
        // (extension, "strategy 0") the block-value operator: dense r x c blocks with one block-column index each.
        // Matrices that are not made of such blocks fail the lowering or the padding gate.
        for (int64_t rc : {3, 2, 4})
            out.push_back({"S0_B1_" + S(rc) + "x" + S(rc), {"block_value " + S(rc) + " " + S(rc)}, "B1", cross({128}, {1})});
        // (extension) DIA storage for matrices on a few diagonals
        if (mx <= 64) out.push_back({"S0_D1", {"diag_value 64"}, "D1", cross({128, 256}, {1})});
    }
    if (mn >= 128)
    {
        // strategy 8 (:2838-2867): BLB_COL_DIV(c), c = 128, 256, ... <= min(4096, ceil32(max))
        int64_t hi = std::min<int64_t>(4096, ceil32(mx));
        hi = std::max<int64_t>(hi, 128);
        for (int64_t c = 128; c <= hi; c *= 2) out.push_back({"S8_K7_c" + S(c), {"blb_col_fixed " + S(c)}, "K7", none});
    }
    if (mx <= 512)
    {
        // strategy 1 (:228): ROW_PADDING(m, 1) -> BLB_ROW_DIV(evenly m) -> TLB_ROW_DIV, m = 64 .. 256 step 64
        for (int64_t mm : integer_range(64, 256, 64))
            out.push_back({"S1_K2_m" + S(mm), {"row_padding " + S(mm) + " 1", "blb_row_evenly " + S(mm), "tlb_row"}, "K2", none});
        // strategy 5 (:1806-1813): ROW_PADDING(32, 1) -> TLB_ROW_DIV
        out.push_back({"S5_K3", {"row_padding 32 1", "tlb_row"}, "K3", none});
    }
    if (!is_sorted)
    {
        // strategy 9 (:3119-3176): TLB_NNZ_DIV(s), s = 2 .. clamp(floor(nnz / rows), 2, 32) in steps of a quarter of the range
        int64_t avg = rows ? (int64_t)(nnz / rows) : 2;
        avg = std::min<int64_t>(32, std::max<int64_t>(2, avg));
        const int64_t step = std::max<int64_t>(1, (avg - 2) / 4);
        std::set<int64_t> ss;
        for (int64_t v : integer_range(2, avg, step)) ss.insert(v);
        if (extensions)
        {
            // (extension) long rows make the 2..avg range too narrow for the loads of a thread to cover the memory latency
            if (mx > 512) ss.insert(8), ss.insert(16);
            ss.insert(32);
        }
        for (int64_t v : ss)
        {
            out.push_back({"S9_K9_s" + S(v), {"tlb_nnz " + S(v)}, "K9", none});
            out.push_back({"S9_K10_s" + S(v), {"tlb_nnz " + S(v)}, "K10", none});
        }
    }
    if (mn >= 30 && mx <= 512)
    {
        // strategy 4 (:1483-1520): WLB_COL_DIV(c), c = 32 .. (first grid point >= max) in steps of ceil32((max - min) / 3)
        int64_t step = (mx - mn) / 3;
        if (step % 32) step = (step / 32 + 1) * 32;
        step = std::max<int64_t>(32, step);
        int64_t up = 32;
        while (up < mx) up += step;
        for (int64_t c : integer_range(32, up, step)) out.push_back({"S4_K4_c" + S(c), {"wlb_col_fixed " + S(c)}, "K4", none});
    }
    if (mn >= 32 && mx <= 1024)
    {
        // strategy 6 (:2093-2127): ROW_PADDING(m, min row nnz) -> BLB_ROW_DIV(evenly m) -> WLB_COL_DIV(c), m = 2, 4 (fastest), c = 32 .. F step 32
        int64_t F = mx / 2;
        if (F % 32) F = (F / 32 + 1) * 32;
        F = std::max<int64_t>(32, std::min<int64_t>(128, F));
        for (int64_t c : integer_range(32, F, 32))
            for (int64_t mm : {2, 4})
                out.push_back({"S6_K8_m" + S(mm) + "_c" + S(c), {"row_padding " + S(mm) + " " + S(mn), "blb_row_evenly " + S(mm), "wlb_col_fixed " + S(c)}, "K8", none});
        // strategy 7 (:2481-2530): BLB_ROW_DIV(nnz >= b) -> WLB_COL_DIV(c), b = 128, 512, 896; c = 32 .. ceil32(min(b / 2, max / 2, 128)) step 32
        for (int64_t bb : integer_range(128, 1024, 384))
        {
            int64_t U = std::min<int64_t>(std::min<int64_t>(bb / 2, mx / 2), 128);
            if (U % 32) U = (U / 32 + 1) * 32;
            for (int64_t c = 32; c <= U; c += 32)
                out.push_back({"S7_K8_b" + S(bb) + "_c" + S(c), {"blb_row_nnz " + S(bb), "wlb_col_fixed " + S(c)}, "K8", none});
        }
    }
    if (mx <= 1024)
    {
        // strategy 2 (:613-643): ROW_PADDING(m, min row nnz) -> BLB_ROW_DIV(evenly m) -> TLB_COL_DIV(c), m = 32, 64 (fastest), c = 1 .. min(16, ceil(max / 2)) step 3
        const int64_t F = std::min<int64_t>(16, (mx + 1) / 2);
        for (int64_t c : integer_range(1, F, 3))
            for (int64_t mm : {32, 64})
                out.push_back({"S2_K6_m" + S(mm) + "_c" + S(c), {"row_padding " + S(mm) + " " + S(std::max<int64_t>(1, mn)), "blb_row_evenly " + S(mm), "tlb_col_fixed " + S(c)}, "K6", none});
        // strategy 3 (:1072-1110): BLB_ROW_DIV(nnz >= b) -> TLB_COL_DIV(c), b = 128, 512, 896; c = 1, 1 + max(1, b / 192), ... <= min(max(1, b / 64), max / 2 (+1 when max is even))
        const int64_t maxcol = mx / 2 + ((mx % 2 == 0) ? 1 : 0);
        for (int64_t bb : integer_range(128, 1024, 384))
        {
            const int64_t up = std::max<int64_t>(1, bb / 64), st = std::max<int64_t>(1, bb / 192);
            for (int64_t c = 1; c <= up && c <= maxcol; c += st)
                out.push_back({"S3_K6_b" + S(bb) + "_c" + S(c), {"blb_row_nnz " + S(bb), "tlb_col_fixed " + S(c)}, "K6", none});
        }
    }
    return out;
}

std::vector<Candidate> compressed_candidates(uint64_t mn_, uint64_t mx_, double avg, bool is_sorted, bool quick)
{
    const int64_t mn = (int64_t)mn_, mx = (int64_t)mx_;
    std::vector<Candidate> out;
    const std::vector<int64_t> T3 = quick ? std::vector<int64_t>{128, 256} : integer_range(32, 256, 32);
    const std::vector<int64_t> T2 = {128, 256};
    if (!is_sorted)
        for (int64_t rc : {3, 2, 4}) // the block-value operator of this build (see reference_candidates)
            out.push_back({"S0_B1_" + std::to_string(rc) + "x" + std::to_string(rc), {"block_value " + std::to_string(rc) + " " + std::to_string(rc)}, "B1", cross({128}, {1})});
    if (!is_sorted && mx <= 64) out.push_back({"S0_D1", {"diag_value 64"}, "D1", cross({128, 256}, {1})}); // DIA storage (see reference_candidates)
    if (mn >= 128)
    {
        // strategy 8: BLB_COL_DIV(c) -> long-row template; c = 128 .. min(4096, ceil32(max)), doubling
        std::vector<int64_t> cs;
        for (int64_t c = 128; c <= std::min<int64_t>(4096, ceil32(mx)); c *= 2) cs.push_back(c);
        const size_t from = (quick && cs.size() > 2) ? cs.size() - 2 : 0;
        for (size_t i = from; i < cs.size(); i++)
        {
            const int64_t c = cs[i];
            std::set<int64_t> th = {std::min<int64_t>(1024, std::max<int64_t>(32, c / 16)), std::min<int64_t>(1024, std::max<int64_t>(64, c / 8)),
                                    std::min<int64_t>(1024, std::max<int64_t>(64, c / 4))};
            out.push_back({"S8_K7_c" + std::to_string(c), {"blb_col_fixed " + std::to_string(c)}, "K7", cross(std::vector<int64_t>(th.begin(), th.end()), {1})});
        }
    }
    if (mx <= 512)
    {
        out.push_back({"S5_K3", {"row_padding 32 1", "tlb_row"}, "K3", cross(T3, {1})});
        for (int64_t mm : (quick ? std::vector<int64_t>{128, 256} : std::vector<int64_t>{64, 128, 192, 256}))
            out.push_back({"S1_K2_m" + std::to_string(mm), {"row_padding " + std::to_string(mm) + " 1", "blb_row_evenly " + std::to_string(mm), "tlb_row"}, "K2", cross(T2, {1})});
    }
    if (!is_sorted)
    {
        // strategy 9: TLB_NNZ_DIV(s) -> CSR5-like templates, s = 2 .. min(avg, 32); rows of any length
        const int64_t hi = (int64_t)std::max(2.0, std::min(avg, 32.0));
        std::set<int64_t> ss;
        if (quick) ss = {2, std::max<int64_t>(2, hi / 2), hi};
        else
        {
            int64_t step = std::max<int64_t>(1, (hi - 2) / 3);
            for (int64_t v : integer_range(2, hi, step)) ss.insert(v);
        }
        if (mx > 512)
        {
            ss.insert(8);
            ss.insert(16);
        }
        for (int64_t s : ss)
        {
            // (third launch parameter of the CSR5-like templates: 1 = rows stored one by one, 2 = staged write-out)
            out.push_back({"S9_K9_s" + std::to_string(s), {"tlb_nnz " + std::to_string(s)}, "K9", cross(T2, {1, 2})});
            out.push_back({"S9_K10_s" + std::to_string(s), {"tlb_nnz " + std::to_string(s)}, "K10", cross(T2, {1, 2})});
        }
    }
    if (mn >= 30 && mx <= 512)
    {
        // strategy 4: WLB_COL_DIV(c) -> warp per row chunk; c from 32 up past the longest row
        const int64_t step = std::max<int64_t>(32, ceil32(std::max<int64_t>(1, (mx - mn) / 3)));
        const std::vector<int64_t> cs = integer_range(32, ceil32(mx) + step, step);
        std::vector<int64_t> use = cs;
        if (quick && !cs.empty()) use = {cs.front(), cs.back()}; // (the same value twice when there is one)
        for (int64_t c : use)
            out.push_back({"S4_K4_c" + std::to_string(c), {"wlb_col_fixed " + std::to_string(c)}, "K4", cross(quick ? T2 : integer_range(32, 512, 64), {1})});
    }
    if (mn >= 32 && mx <= 1024)
    {
        std::vector<int64_t> cs = integer_range(32, std::min<int64_t>(128, ceil32((mx + 1) / 2)), 32);
        if (cs.empty()) cs = {32};
        const std::vector<int64_t> use = quick ? std::vector<int64_t>{cs.back()} : cs;
        for (int64_t mm : (quick ? std::vector<int64_t>{4} : std::vector<int64_t>{2, 4}))
            for (int64_t c : use)
                out.push_back({"S6_K8_m" + std::to_string(mm) + "_c" + std::to_string(c),
                               {"row_padding " + std::to_string(mm) + " 1", "blb_row_evenly " + std::to_string(mm), "wlb_col_fixed " + std::to_string(c)}, "K8", cross(T2, {1, 4})});
        for (int64_t bb : (quick ? std::vector<int64_t>{512} : std::vector<int64_t>{128, 512, 896}))
            for (int64_t c : use)
                out.push_back({"S7_K8_b" + std::to_string(bb) + "_c" + std::to_string(c), {"blb_row_nnz " + std::to_string(bb), "wlb_col_fixed " + std::to_string(c)}, "K8", cross(T2, {1, 4})});
    }
    if (mx <= 1024)
    {
        const std::vector<int64_t> cs = integer_range(1, std::min<int64_t>(16, std::max<int64_t>(1, (mx + 1) / 2)), 3);
        std::vector<int64_t> use = cs;
        if (quick && cs.size() > 2) use = {cs[0], cs[1]};
        for (int64_t mm : (quick ? std::vector<int64_t>{64} : std::vector<int64_t>{32, 64}))
            for (int64_t c : use)
                out.push_back({"S2_K6_m" + std::to_string(mm) + "_c" + std::to_string(c),
                               {"row_padding " + std::to_string(mm) + " 1", "blb_row_evenly " + std::to_string(mm), "tlb_col_fixed " + std::to_string(c)}, "K6", cross(T2, {1, 4})});
        if (!quick)
            for (int64_t bb : {128, 512, 896})
                for (int64_t c : cs)
                    out.push_back({"S3_K6_b" + std::to_string(bb) + "_c" + std::to_string(c), {"blb_row_nnz " + std::to_string(bb), "tlb_col_fixed " + std::to_string(c)}, "K6", cross(T2, {1, 4, 16})});
    }
    return out;
}

// ---- the reference's launch sweeps (default_auto_tuner.cc), derived from the lowered format ----------------
struct ArrView
{
    const asp_array_desc *d = nullptr;
    uint64_t len() const { return d ? d->len : 0; }
    uint64_t get(uint64_t i) const
    {
        switch (d->compress)
        {
        case ASP_COMPRESS_NONE:
            switch (d->dtype)
            {
            case ASP_U8: return ((const uint8_t *)d->host_ptr)[i];
            case ASP_U16: return ((const uint16_t *)d->host_ptr)[i];
            case ASP_U32: return ((const uint32_t *)d->host_ptr)[i];
            default: return ((const uint64_t *)d->host_ptr)[i];
            }
        case ASP_COMPRESS_LINEAR: return i * d->coef + d->icpt;
        case ASP_COMPRESS_CONSTANT: return d->icpt;
        case ASP_COMPRESS_CYCLE_LINEAR: return (i % d->cycle) * d->coef + d->icpt;
        case ASP_COMPRESS_CYCLE_INCREASE: return i / d->cycle + d->icpt;
        default:
        {
            uint64_t v = d->branch_val[0];
            for (int b = 1; b < d->n_branch; b++)
                if (i > d->branch_hi[b - 1]) v = d->branch_val[b];
            return v;
        }
        }
    }
};
ArrView role_of(const asp_plan_desc &d, int role)
{
    ArrView v;
    for (int i = 0; i < d.n_arrays; i++)
        if (d.arrays[i].role == role) v.d = &d.arrays[i];
    return v;
}
// smallest and largest difference of consecutive entries of a CSR-like offset array
void min_max_diff(const ArrView &a, uint64_t init_min, uint64_t &mn, uint64_t &mx)
{
    mn = init_min;
    mx = 0;
    for (uint64_t i = 0; i + 1 < a.len(); i++)
    {
        const uint64_t d = a.get(i + 1) - a.get(i);
        mn = std::min(mn, d);
        mx = std::max(mx, d);
    }
}
// thread_num_in_block from `lo` to `hi` in at most `parts` steps that are multiples of 32
std::vector<int64_t> thread_range(uint64_t lo, uint64_t hi, uint64_t parts)
{
    uint64_t step = (hi - lo) / parts;
    if (step % 32) step = (step / 32 + 1) * 32;
    step = std::max<uint64_t>(32, step);
    return integer_range((int64_t)lo, (int64_t)hi, (int64_t)step);
}
uint64_t floor32_clamped(uint64_t v) { return std::min<uint64_t>(1024, std::max<uint64_t>(32, v / 32 * 32)); }

// false: the reference skips the template on this format altogether
bool reference_launches(int templ, const asp_plan_desc &d, const asp_sub_info &info, uint64_t max_tblock, std::vector<Launch> &out)
{
    out.clear();
    uint64_t mn = 0, mx = 0;
    switch (templ)
    {
    case ASP_DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS: // :465
        out = cross(integer_range(32, 256, 32), {1});
        return true;
    case ASP_DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE: // :849
        out = cross(integer_range(32, 512, 64), {1});
        return true;
    case ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE: // :1911-1925 registers (0, 256, 64) and skips 0
        out = cross(integer_range(64, 256, 64), {1});
        return true;
    case ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE: // :1749-1798
    {
        uint64_t lo = std::max<uint64_t>(32, info.n_tlb / (max_tblock - 1));
        if (lo % 32) lo = (lo / 32 + 1) * 32;
        if (lo > 512) return false;
        out = cross(thread_range(lo, 512, 4), {1});
        return true;
    }
    case ASP_DIRECT_ATOM_TEMPLATE_WARP_COMPRESS: // :587-700: from the TLBs per BLB
    {
        min_max_diff(role_of(d, ASP_ARR_BLOCK_BEGIN_THREAD_INDEX_OFFSET), 9999999, mn, mx);
        const uint64_t hi = std::min<uint64_t>(1024, (mx + 31) / 32 * 32), lo = floor32_clamped(mn);
        if (lo > hi) return false;
        out = cross(thread_range(lo, hi, 8), {1});
        return true;
    }
    case ASP_SHARED_MEMORY_LONG_ROW_TEMPLATE: // :970-1110: from the non-zeros per BLB (the upper end is rounded DOWN there)
    {
        min_max_diff(role_of(d, ASP_ARR_BLOCK_NZ_BEGIN_OFFSET), 9999999999999999ull, mn, mx);
        const uint64_t hi = floor32_clamped(mx), lo = floor32_clamped(mn);
        if (lo > hi) return false;
        out = cross(thread_range(lo, hi, 8), {1});
        return true;
    }
    case ASP_SHARED_MEMORY_TEMPLATE_WARP_COMPRESS: // :1215-1360: TLBs per BLB in 4 steps; row reduce 1, 4, 16 up to the most partials of a row
    {
        min_max_diff(role_of(d, ASP_ARR_BLOCK_BEGIN_THREAD_INDEX_OFFSET), 4096, mn, mx);
        if (mx > 1024) return false; // "too many (> 1024) TLB in BLB" (whilte_list_path_impl.cc:798, 1220): strategies 2 and 3 drop the point
        uint64_t rmn = 0, rmx = 0;
        min_max_diff(role_of(d, ASP_ARR_ROW_OFFSET_IN_THREAD_TMP_RESULT), ~0ull, rmn, rmx);
        const uint64_t hi = std::min<uint64_t>(1024, (mx + 31) / 32 * 32), lo = floor32_clamped(mn);
        if (lo > hi) return false;
        std::vector<int64_t> red;
        for (uint64_t r = 1; r <= 32 && r <= rmx; r *= 4) red.push_back((int64_t)r);
        out = cross(thread_range(lo, hi, 4), red);
        return true;
    }
    case ASP_SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE: // :1495-1625: WLBs per BLB x 32 in 8 steps; row reduce 1, 2, 4, ... up to the most partials of a row
    {
        min_max_diff(role_of(d, ASP_ARR_BLOCK_BEGIN_WARP_INDEX_OFFSET), 1024, mn, mx);
        uint64_t rmn = 0, rmx = 0;
        min_max_diff(role_of(d, ASP_ARR_ROW_OFFSET_IN_WARP_TMP_RESULT), ~0ull, rmn, rmx);
        const uint64_t hi = std::min<uint64_t>(1024, mx * 32), lo = std::min<uint64_t>(1024, std::max<uint64_t>(32, mn * 32));
        if (lo > hi) return false;
        std::vector<int64_t> red;
        for (uint64_t r = 1; r <= 32 && r <= rmx; r *= 2) red.push_back((int64_t)r);
        out = cross(thread_range(lo, hi, 8), red);
        return true;
    }
    case ASP_BLOCK_ELL_TEMPLATE:
        out = cross({128}, {1});
        return true;
    case ASP_DIAG_TEMPLATE:
        out = cross({128, 256}, {1});
        return true;
    default: return false; // the two 3-level templates are not reachable from the whitelist strategies
    }
}

std::vector<std::string> dense_strategies(bool quick)
{
    std::vector<std::string> out = {"dense compress", "dense rowdiv_exp 32 4096 4\ndense compress"};
    std::vector<std::pair<int, int>> g3;
    if (quick) g3 = {{128, 8}};
    else
        for (int mn : {512, 128, 32})
            for (int r : {4, 8, 16}) g3.push_back({mn, r});
    for (auto &p : g3) out.push_back("dense sort 1\ndense rowdiv_exp " + std::to_string(p.first) + " 4096 " + std::to_string(p.second) + "\ndense compress");
    return out;
}

int template_id(const std::string &k)
{
    static const char *names[] = {"K1", "K2", "K3", "K5", "K6", "K7", "K8", "K4", "K9", "K10"}; // asp_template_type order
    for (int i = 0; i < 10; i++)
        if (k == names[i]) return i;
    if (k == "B1") return ASP_BLOCK_ELL_TEMPLATE;
    if (k == "D1") return ASP_DIAG_TEMPLATE;
    return -1;
}

int64_t derive_tblock(int templ, uint64_t n_tlb, uint64_t n_wlb, uint64_t n_blb, int64_t threads)
{
    // one CTA per BLB for the CTA-per-BLB templates, ceil(units / threads) otherwise
    uint64_t n;
    switch (templ)
    {
    case 0: case 1: case 3: case 4: case 5: case 6: n = n_blb; break; // K1 K2 K5 K6 K7 K8
    case 7: n = (32 * n_wlb + (uint64_t)threads - 1) / (uint64_t)threads; break; // K4
    case ASP_BLOCK_ELL_TEMPLATE: n = (n_tlb / 2 + (uint64_t)threads - 1) / (uint64_t)threads; break; // a thread owns two block rows
    case ASP_DIAG_TEMPLATE: n = (n_tlb + (uint64_t)threads - 1) / (uint64_t)threads; break;            // n_tlb counts the threads' row groups
    default: n = (n_tlb + (uint64_t)threads - 1) / (uint64_t)threads; break;      // K3 K9 K10
    }
    return (int64_t)std::max<uint64_t>(1, std::min<uint64_t>(n, 2147483647ull));
}

// search_strategy.cc:5-80
struct StopRule
{
    uint64_t remain = 10, struggle;
    double limit, best = 0;
    std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
    StopRule(uint64_t s, double l) : struggle(s), limit(l) {}
    bool out_of_time() const { return limit > 0 && std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() >= limit; }
    bool go_on(double gflops)
    {
        if (gflops > best)
        {
            remain = (uint64_t)std::max(5.0, std::min(25.0, std::floor((gflops - best) * 5)));
            best = gflops;
        }
        else if (remain > 0) remain--;
        else if (struggle > 0) struggle--;
        else return false;
        return !out_of_time();
    }
};

struct Pick
{
    Candidate cand;
    Launch launch;
    float ms;
};

struct FormatDeleter
{
    void operator()(asp_format *f) const { asp_format_destroy(f); }
};
struct MatrixDeleter
{
    void operator()(asp_matrix *m) const { asp_matrix_destroy(m); }
};
typedef std::unique_ptr<asp_format, FormatDeleter> FormatPtr;
typedef std::unique_ptr<asp_matrix, MatrixDeleter> MatrixPtr;

std::string one_line(std::string s)
{
    size_t p = 0;
    while ((p = s.find('\n', p)) != std::string::npos) s.replace(p, 1, " | ");
    return s;
}

thread_local std::string g_text;
} // namespace

struct asp_search_result
{
    std::string dense;
    std::vector<std::string> sub_spec, sub_name;
    std::vector<Launch> launch;
    float ms = 0;
    std::vector<std::string> trials;
};

extern "C" {

const char *asp_search_candidates(uint64_t mn, uint64_t mx, double avg, int is_sorted, int quick)
{
    g_text.clear();
    // quick: 1 = the short table, 0 = the long table of this build (both carry their own launch lists), 2 = the
    // reference's node grids exactly (launches are derived from the lowered format, so none are listed)
    const std::vector<Candidate> cands = quick == 2 ? reference_candidates((int64_t)mn, (int64_t)mx, 1000, (uint64_t)(avg * 1000.0 + 0.5), is_sorted != 0, false)
                                                    : compressed_candidates(mn, mx, avg, is_sorted != 0, quick != 0);
    for (const Candidate &c : cands)
    {
        g_text += c.name + " ; " + c.templ + " ; ";
        for (size_t i = 0; i < c.nodes.size(); i++) g_text += (i ? "|" : "") + c.nodes[i];
        g_text += " ; ";
        for (size_t i = 0; i < c.launches.size(); i++) g_text += (i ? "," : "") + std::to_string(c.launches[i].threads) + ":" + std::to_string(c.launches[i].reduce);
        g_text += "\n";
    }
    return g_text.c_str();
}

int64_t asp_search_derive_tblock(int template_type, uint64_t n_tlb, uint64_t n_wlb, uint64_t n_blb, int64_t threads)
{
    return derive_tblock(template_type, n_tlb, n_wlb, n_blb, threads > 0 ? threads : 1);
}

asp_status asp_search(const asp_matrix *m, const asp_search_options *opt_, asp_time_fn time_fn, void *time_user, asp_search_result **out)
{
    if (!m || !time_fn || !out) return ASP_ERR_INVALID_ARG;
    *out = nullptr;
    asp_search_options opt = {};
    if (opt_) opt = *opt_;
    else
    {
        opt.quick = 1;
        opt.struggle_step_num = -1;
    }
    if (opt.warmup <= 0) opt.warmup = 2;
    if (opt.reps <= 0) opt.reps = 10;
    if (opt.max_subs <= 0) opt.max_subs = 5;
    const double pad_bound = opt.padding_rate_up_bound > 0 ? opt.padding_rate_up_bound : 4.0;
    auto log = [&](const std::string &s) {
        if (opt.log_fn) opt.log_fn(opt.log_user, s.c_str());
    };
    const uint64_t total_nnz = asp_matrix_nnz(m);
    // checkpoint: points timed by an earlier, interrupted run of the same search (key: the trial line without its time)
    std::map<std::string, float> done;
    FILE *ckpt = nullptr;
    struct CloseFile
    {
        FILE *&f;
        ~CloseFile()
        {
            if (f) fclose(f);
        }
    } close_ckpt{ckpt};
    if (opt.checkpoint_path && opt.checkpoint_path[0])
    {
        if (FILE *in = fopen(opt.checkpoint_path, "r"))
        {
            char line[1024];
            while (fgets(line, sizeof line, in))
            {
                // "<dense> ; sub <i> ; <name> ; threads ; reduce ; ms ; padding"
                std::string s(line);
                size_t p5 = std::string::npos, pos = 0;
                int semis = 0;
                size_t p6 = std::string::npos;
                while ((pos = s.find(" ; ", pos)) != std::string::npos)
                {
                    semis++;
                    if (semis == 5) p5 = pos;
                    if (semis == 6) p6 = pos;
                    pos += 3;
                }
                if (semis != 6) continue; // a line cut off by the interruption
                const float ms = (float)atof(s.substr(p5 + 3, p6 - p5 - 3).c_str());
                if (ms > 0) done[s.substr(0, p5)] = ms;
            }
            fclose(in);
            log("checkpoint: " + std::to_string(done.size()) + " timed points taken from " + opt.checkpoint_path);
        }
        ckpt = fopen(opt.checkpoint_path, "a");
    }

    std::unique_ptr<asp_search_result> best;
    std::vector<std::string> trials;
    for (const std::string &dense : dense_strategies(opt.quick == 1))
    {
        asp_matrix *cm_raw = nullptr;
        if (asp_dense_execute(m, dense.c_str(), &cm_raw) != ASP_OK) continue;
        MatrixPtr cm(cm_raw);
        const int n = asp_matrix_num_subs(cm.get());
        // the reference abandons row divisions that give too many strips or no split at all
        if (n <= 0 || n > opt.max_subs || (n == 1 && dense.find("rowdiv") != std::string::npos)) continue;
        log("dense view: " + one_line(dense) + " -> " + std::to_string(n) + " sub-matrices");
        const bool is_sorted = dense.find("sort") != std::string::npos;
        std::vector<Pick> picks;
        bool ok = true;
        for (int sub = 0; sub < n && ok; sub++)
        {
            uint64_t rows = 0, nnz = 0, mn = 0, mx = 0;
            if (asp_matrix_sub_rows(cm.get(), sub, &rows, &nnz, &mn, &mx) != ASP_OK)
            {
                ok = false;
                break;
            }
            std::string others;
            for (int j = 0; j < n; j++)
                if (j != sub) others += "\nsub " + std::to_string(j) + " template EMPTY";
            std::unique_ptr<StopRule> rule;
            if (opt.struggle_step_num >= 0) rule.reset(new StopRule((uint64_t)opt.struggle_step_num, opt.time_limit_s));
            bool have = false, stop = false;
            Pick bestp{};
            const std::vector<Candidate> cands = opt.quick == 1 ? compressed_candidates(mn, mx, rows ? (double)nnz / (double)rows : 0.0, is_sorted, true)
                                                                : reference_candidates((int64_t)mn, (int64_t)mx, rows, nnz, is_sorted, opt.quick == 0);
            for (const Candidate &cand : cands)
            {
                // names start with "S<k>_": the whitelist strategy the point belongs to
                if (opt.strategy_mask && !(opt.strategy_mask & (1u << (cand.name[1] - '0')))) continue;
                asp_format *f_raw = nullptr;
                if (asp_graph_execute(cm.get(), (cand.lines(sub) + others).c_str(), &f_raw) != ASP_OK)
                {
                    log("  sub " + std::to_string(sub) + " " + cand.name + ": graph rejected (" + asp_host_last_error() + ")");
                    continue;
                }
                FormatPtr f(f_raw);
                const double rate = asp_format_padding_rate(f.get(), sub);
                if (rate > pad_bound) continue;
                asp_sub_info info;
                if (asp_format_sub_info(f.get(), sub, &info) != ASP_OK) continue;
                const int tid = template_id(cand.templ);
                std::vector<Launch> launches = cand.launches;
                if (opt.quick != 1)
                {
                    // the launch sweep the reference derives from the lowered format (default_auto_tuner.cc:449-2030);
                    // its 65535-CTA grid cap only survives in the exact mode
                    std::vector<asp_plan_desc> descs(n);
                    if (asp_format_plan_descs(f.get(), descs.data()) != ASP_OK) continue;
                    if (!reference_launches(tid, descs[sub], info, opt.quick == 2 ? 65535 : 2147483647ull, launches)) continue;
                    if (opt.quick == 0 && (tid == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE || tid == ASP_UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE))
                    {
                        // (extension) the staged write-out of the CSR5-like kernels, as the third launch parameter
                        const size_t n0 = launches.size();
                        for (size_t q = 0; q < n0; q++)
                            if (launches[q].threads <= 256) launches.push_back({launches[q].threads, 2});
                    }
                }
                if (opt.prune_gbs > 0 && have)
                {
                    // sound pruning: the kernel has to read every byte of the format at least once
                    std::vector<asp_plan_desc> descs(n);
                    uint64_t bytes = 0;
                    if (asp_format_plan_descs(f.get(), descs.data()) == ASP_OK)
                        for (int a = 0; a < descs[sub].n_arrays; a++)
                        {
                            const asp_array_desc &ad = descs[sub].arrays[a];
                            if (ad.compress != ASP_COMPRESS_NONE) continue; // replaced by a closed form: never read
                            static const uint64_t es[] = {1, 2, 4, 8, 4, 8};    // asp_dtype order: u8 u16 u32 u64 f32 f64
                            bytes += ad.len * es[ad.dtype < 6 ? ad.dtype : 2];
                        }
                    const uint64_t min_bytes = opt.prune_min_bytes ? opt.prune_min_bytes : (256ull << 20);
                    const double bound_ms = (double)bytes / (opt.prune_gbs * 1e6);
                    if (bytes >= min_bytes && bound_ms > bestp.ms)
                    {
                        char buf[256];
                        snprintf(buf, sizeof buf, "  sub %d %s: not timed, %.0f MB cannot be read in under %.1f us", sub, cand.name.c_str(), bytes * 1e-6, bestp.ms * 1e3);
                        log(buf);
                        continue;
                    }
                }
                for (const Launch &l : launches)
                {
                    std::vector<int64_t> tb(n, 1), th(n, 32), rd(n, 1);
                    tb[sub] = derive_tblock(tid, info.n_tlb, info.n_wlb, info.n_blb, l.threads);
                    th[sub] = l.threads;
                    rd[sub] = l.reduce;
                    float ms = 0;
                    char key[512];
                    snprintf(key, sizeof key, "%s ; sub %d ; %s ; %lld ; %lld", one_line(dense).c_str(), sub, cand.name.c_str(), (long long)l.threads, (long long)l.reduce);
                    const auto was = done.find(key);
                    if (was != done.end()) ms = was->second;
                    else if (time_fn(time_user, f.get(), tb.data(), th.data(), rd.data(), opt.warmup, opt.reps, &ms) != 0 || !(ms > 0))
                    {
                        log("  sub " + std::to_string(sub) + " " + cand.name + " threads=" + std::to_string(l.threads) + ": cannot run");
                        continue;
                    }
                    char buf[512];
                    snprintf(buf, sizeof buf, "%s ; sub %d ; %s ; %lld ; %lld ; %.6f ; %.4f", one_line(dense).c_str(), sub, cand.name.c_str(), (long long)l.threads,
                             (long long)l.reduce, ms, rate);
                    trials.push_back(buf);
                    if (ckpt && was == done.end())
                    {
                        fprintf(ckpt, "%s\n", buf);
                        fflush(ckpt);
                    }
                    snprintf(buf, sizeof buf, "  sub %d [%llu rows, nnz/row %llu..%llu] %s threads=%lld reduce=%lld: %.1f us", sub, (unsigned long long)rows, (unsigned long long)mn,
                             (unsigned long long)mx, cand.name.c_str(), (long long)l.threads, (long long)l.reduce, ms * 1e3);
                    log(buf);
                    if (!have || ms < bestp.ms)
                    {
                        bestp = {cand, l, ms};
                        have = true;
                    }
                    if (rule && !rule->go_on(2.0 * (double)nnz * 1e-6 / ms))
                    {
                        stop = true;
                        break;
                    }
                }
                if (stop)
                {
                    log("  sub " + std::to_string(sub) + ": search budget used up after " + cand.name);
                    break;
                }
            }
            if (!have) ok = false;
            else picks.push_back(bestp);
        }
        if (!ok || (int)picks.size() != n) continue;
        // the whole matrix with the per-strip winners
        std::string spec;
        for (int i = 0; i < n; i++) spec += (i ? "\n" : "") + picks[i].cand.lines(i);
        asp_format *f_raw = nullptr;
        if (asp_graph_execute(cm.get(), spec.c_str(), &f_raw) != ASP_OK) continue;
        FormatPtr f(f_raw);
        std::vector<int64_t> tb(n), th(n), rd(n);
        for (int i = 0; i < n; i++)
        {
            asp_sub_info info;
            if (asp_format_sub_info(f.get(), i, &info) != ASP_OK) ok = false;
            tb[i] = derive_tblock(template_id(picks[i].cand.templ), info.n_tlb, info.n_wlb, info.n_blb, picks[i].launch.threads);
            th[i] = picks[i].launch.threads;
            rd[i] = picks[i].launch.reduce;
        }
        float ms = 0;
        if (!ok || time_fn(time_user, f.get(), tb.data(), th.data(), rd.data(), opt.warmup, std::max(opt.reps, 20), &ms) != 0 || !(ms > 0)) continue;
        char buf[160];
        snprintf(buf, sizeof buf, "  whole matrix: %.1f us  %.1f GFLOP/s", ms * 1e3, 2.0 * (double)total_nnz * 1e-6 / ms);
        log(buf);
        if (!best || ms < best->ms)
        {
            best.reset(new asp_search_result());
            best->dense = dense;
            best->ms = ms;
            for (int i = 0; i < n; i++)
            {
                best->sub_spec.push_back(picks[i].cand.lines(i));
                best->sub_name.push_back(picks[i].cand.name);
                best->launch.push_back(picks[i].launch);
            }
        }
    }
    if (!best) return ASP_ERR_UNSUPPORTED;
    best->trials.swap(trials);
    *out = best.release();
    return ASP_OK;
}

void asp_search_result_destroy(asp_search_result *r) { delete r; }
const char *asp_search_result_dense(const asp_search_result *r) { return r ? r->dense.c_str() : ""; }
int asp_search_result_num_subs(const asp_search_result *r) { return r ? (int)r->sub_spec.size() : 0; }
const char *asp_search_result_sub_spec(const asp_search_result *r, int i) { return (r && i >= 0 && i < (int)r->sub_spec.size()) ? r->sub_spec[i].c_str() : ""; }
const char *asp_search_result_sub_name(const asp_search_result *r, int i) { return (r && i >= 0 && i < (int)r->sub_name.size()) ? r->sub_name[i].c_str() : ""; }
asp_status asp_search_result_sub_launch(const asp_search_result *r, int i, int64_t *threads, int64_t *reduce)
{
    if (!r || i < 0 || i >= (int)r->launch.size() || !threads || !reduce) return ASP_ERR_INVALID_ARG;
    *threads = r->launch[i].threads;
    *reduce = r->launch[i].reduce;
    return ASP_OK;
}
float asp_search_result_ms(const asp_search_result *r) { return r ? r->ms : 0.f; }
int asp_search_result_num_trials(const asp_search_result *r) { return r ? (int)r->trials.size() : 0; }
const char *asp_search_result_trial(const asp_search_result *r, int i) { return (r && i >= 0 && i < (int)r->trials.size()) ? r->trials[i].c_str() : ""; }

} // extern "C"
