// Binary file of a lowered format: everything asp_plan_group_create needs, so that a matrix tuned once
// is uploaded later without its Operator Graph being executed again. The reference keeps the same
// information as a directory of text files next to the generated program (store_code_builder_data,
// code_builder.cc:2429-2517); this is its counterpart for the C ABI.
//
// Layout (little endian): magic "ASPFMT1\0"; header {val_dt, perm_dt: i32; n_rows, n_cols, n_subs,
// perm_bytes: u64}; the global row permutation (perm_bytes); per sub-matrix: the scalars of its
// template, its asp_sub_info, the array count, and per array {role, dt, len, closed form, flag
// "is the shared permutation", payload bytes unless shared}.
#include <stdio.h>
#include <string.h>

#include <memory>
#include <string>
#include <vector>

#include "handles.hpp"

using namespace asp::host;

namespace
{
const char MAGIC[8] = {'A', 'S', 'P', 'F', 'M', 'T', '1', 0};

struct File
{
    FILE *f = nullptr;
    ~File()
    {
        if (f) fclose(f);
    }
};

template <class T>
bool put(FILE *f, const T &v)
{
    return fwrite(&v, sizeof(T), 1, f) == 1;
}
template <class T>
bool get(FILE *f, T &v)
{
    return fread(&v, sizeof(T), 1, f) == 1;
}

struct SubScalars
{
    int32_t template_type, val_dt, bits_word, bits_flag, bits_row, bits_off, is_atom_add, sort_kind;
    uint64_t first_row, first_col, true_nnz, effective_num, tlb_size, n_blb, n_wlb, n_tlb;
    int64_t tblock_num, thread_num_in_block, thread_num_of_row_reduce;
};

struct ArrayHead
{
    int32_t role, dt, kind, n_branch, shared_perm, pad;
    uint64_t len, coef, icpt, cycle, payload_bytes;
    uint64_t lo[ASP_MAX_BRANCH], hi[ASP_MAX_BRANCH], val[ASP_MAX_BRANCH];
};
} // namespace

extern "C" {

asp_status asp_format_save(const asp_format *f, const char *path)
{
    if (!f || !path) return asp_host_fail(ASP_ERR_INVALID_ARG, "NULL argument");
    File out;
    out.f = fopen(path, "wb");
    if (!out.f) return asp_host_fail(ASP_ERR_INVALID_ARG, std::string("cannot create ") + path);
    bool ok = fwrite(MAGIC, 1, 8, out.f) == 8;
    const int32_t val_dt = f->val_dt, perm_dt = f->perm_dt;
    const uint64_t n_subs = f->subs.size(), perm_bytes = f->perm ? f->perm->size() : 0;
    ok = ok && put(out.f, val_dt) && put(out.f, perm_dt) && put(out.f, f->n_rows) && put(out.f, f->n_cols) && put(out.f, n_subs) && put(out.f, perm_bytes);
    if (perm_bytes) ok = ok && fwrite(f->perm->data(), 1, perm_bytes, out.f) == perm_bytes;
    for (size_t i = 0; i < f->subs.size() && ok; i++)
    {
        const TemplateData &t = f->subs[i];
        SubScalars s;
        memset(&s, 0, sizeof(s));
        s.template_type = t.template_type, s.val_dt = t.val_dt, s.bits_word = t.bits_word, s.bits_flag = t.bits_flag, s.bits_row = t.bits_row;
        s.bits_off = t.bits_off, s.is_atom_add = t.is_atom_add ? 1 : 0, s.sort_kind = t.sort_kind;
        s.first_row = t.first_row, s.first_col = t.first_col, s.true_nnz = t.true_nnz, s.effective_num = t.effective_num, s.tlb_size = t.tlb_size;
        s.n_blb = t.n_blb, s.n_wlb = t.n_wlb, s.n_tlb = t.n_tlb;
        s.tblock_num = t.tblock_num, s.thread_num_in_block = t.thread_num_in_block, s.thread_num_of_row_reduce = t.thread_num_of_row_reduce;
        const uint64_t n_arrays = t.arrays.size();
        ok = ok && put(out.f, s) && put(out.f, f->infos[i]) && put(out.f, n_arrays);
        for (const TemplateArray &a : t.arrays)
        {
            ArrayHead h;
            memset(&h, 0, sizeof(h));
            h.role = a.role, h.dt = a.dt, h.kind = a.comp.kind, h.n_branch = (int32_t)a.comp.val.size();
            h.shared_perm = (a.shared && f->perm && a.shared.get() == f->perm.get()) ? 1 : 0;
            h.len = a.len, h.coef = a.comp.coef, h.icpt = a.comp.icpt, h.cycle = a.comp.cycle;
            const std::vector<uint8_t> &bytes = a.shared ? *a.shared : a.bytes;
            h.payload_bytes = h.shared_perm ? 0 : bytes.size();
            for (int k = 0; k < h.n_branch && k < ASP_MAX_BRANCH; k++) h.lo[k] = a.comp.lo[k], h.hi[k] = a.comp.hi[k], h.val[k] = a.comp.val[k];
            ok = ok && put(out.f, h);
            if (h.payload_bytes) ok = ok && fwrite(bytes.data(), 1, h.payload_bytes, out.f) == h.payload_bytes;
        }
    }
    if (!ok) return asp_host_fail(ASP_ERR_INVALID_ARG, std::string("write to ") + path + " failed");
    return ASP_OK;
}

asp_status asp_format_load(const char *path, asp_format **out)
{
    if (!path || !out) return asp_host_fail(ASP_ERR_INVALID_ARG, "NULL argument");
    *out = nullptr;
    File in;
    in.f = fopen(path, "rb");
    if (!in.f) return asp_host_fail(ASP_ERR_INVALID_ARG, std::string("cannot open ") + path);
    char magic[8];
    if (fread(magic, 1, 8, in.f) != 8 || memcmp(magic, MAGIC, 8) != 0) return asp_host_fail(ASP_ERR_INVALID_ARG, std::string(path) + " is not a format file of this library");
    try
    {
        std::unique_ptr<asp_format> F(new asp_format());
        int32_t val_dt = 0, perm_dt = 0;
        uint64_t n_subs = 0, perm_bytes = 0;
        bool ok = get(in.f, val_dt) && get(in.f, perm_dt) && get(in.f, F->n_rows) && get(in.f, F->n_cols) && get(in.f, n_subs) && get(in.f, perm_bytes);
        if (!ok || n_subs > (1u << 20) || (val_dt != ASP_F32 && val_dt != ASP_F64)) return asp_host_fail(ASP_ERR_INVALID_ARG, "corrupt header");
        F->val_dt = val_dt;
        F->perm_dt = perm_dt;
        if (perm_bytes)
        {
            if (perm_bytes != F->n_rows * (uint64_t)dtype_bytes(perm_dt)) return asp_host_fail(ASP_ERR_INVALID_ARG, "corrupt permutation");
            F->perm = std::make_shared<std::vector<uint8_t>>(perm_bytes);
            ok = fread(F->perm->data(), 1, perm_bytes, in.f) == perm_bytes;
        }
        F->subs.resize(n_subs);
        F->infos.resize(n_subs);
        for (uint64_t i = 0; i < n_subs && ok; i++)
        {
            SubScalars s;
            uint64_t n_arrays = 0;
            ok = get(in.f, s) && get(in.f, F->infos[i]) && get(in.f, n_arrays);
            if (!ok || n_arrays > 64) return asp_host_fail(ASP_ERR_INVALID_ARG, "corrupt sub-matrix record");
            if (s.template_type < 0 || s.template_type > ASP_DIAG_TEMPLATE || (s.template_type != ASP_EMPTY_TEMPLATE && s.val_dt != val_dt) || s.sort_kind < ASP_SORT_NONE || s.sort_kind > ASP_SORT_LOCAL)
                return asp_host_fail(ASP_ERR_INVALID_ARG, "corrupt sub-matrix record: template, value type or sort kind out of range");
            if (s.first_row >= F->n_rows || s.first_col >= F->n_cols) return asp_host_fail(ASP_ERR_INVALID_ARG, "corrupt sub-matrix record: first row / column outside the matrix");
            TemplateData &t = F->subs[i];
            t.template_type = s.template_type, t.val_dt = s.val_dt, t.bits_word = s.bits_word, t.bits_flag = s.bits_flag, t.bits_row = s.bits_row;
            t.bits_off = s.bits_off, t.is_atom_add = s.is_atom_add != 0, t.sort_kind = s.sort_kind;
            t.first_row = s.first_row, t.first_col = s.first_col, t.true_nnz = s.true_nnz, t.effective_num = s.effective_num, t.tlb_size = s.tlb_size;
            t.n_blb = s.n_blb, t.n_wlb = s.n_wlb, t.n_tlb = s.n_tlb;
            t.tblock_num = (long)s.tblock_num, t.thread_num_in_block = (long)s.thread_num_in_block, t.thread_num_of_row_reduce = (long)s.thread_num_of_row_reduce;
            t.arrays.resize(n_arrays);
            for (uint64_t k = 0; k < n_arrays && ok; k++)
            {
                ArrayHead h;
                ok = get(in.f, h);
                if (!ok || h.n_branch < 0 || h.n_branch > ASP_MAX_BRANCH) return asp_host_fail(ASP_ERR_INVALID_ARG, "corrupt array record");
                if (h.role < 0 || h.role >= ASP_ARR_ROLE_COUNT || h.dt < ASP_U8 || h.dt > ASP_F64 || h.kind < ASP_COMPRESS_NONE || h.kind > ASP_COMPRESS_CYCLE_INCREASE)
                    return asp_host_fail(ASP_ERR_INVALID_ARG, "corrupt array record: role, element type or closed-form kind out of range");
                if ((h.kind == ASP_COMPRESS_CYCLE_LINEAR || h.kind == ASP_COMPRESS_CYCLE_INCREASE) && h.cycle == 0)
                    return asp_host_fail(ASP_ERR_INVALID_ARG, "corrupt array record: cycle of length 0");
                TemplateArray &a = t.arrays[k];
                a.role = h.role, a.dt = h.dt, a.len = h.len;
                a.comp.kind = h.kind, a.comp.coef = h.coef, a.comp.icpt = h.icpt, a.comp.cycle = h.cycle;
                for (int b = 0; b < h.n_branch; b++) a.comp.lo.push_back(h.lo[b]), a.comp.hi.push_back(h.hi[b]), a.comp.val.push_back(h.val[b]);
                if (h.shared_perm)
                {
                    if (!F->perm) return asp_host_fail(ASP_ERR_INVALID_ARG, "array refers to a permutation the file does not hold");
                    if (h.len != F->n_rows || h.dt != perm_dt) return asp_host_fail(ASP_ERR_INVALID_ARG, "array refers to the shared permutation with another length or element type");
                    a.shared = F->perm;
                }
                else
                {
                    // the payload may be shorter than len * element size only for arrays replaced by a closed form
                    if (h.payload_bytes > (1ull << 40) || h.len > (1ull << 40)) return asp_host_fail(ASP_ERR_INVALID_ARG, "corrupt array size");
                    // an array that is loaded element by element must be there in full; one that a closed form replaces may be
                    // stored or not, but never longer than it claims to be
                    const uint64_t full = h.len * (uint64_t)dtype_bytes(h.dt);
                    if ((h.kind == ASP_COMPRESS_NONE && h.payload_bytes != full) || h.payload_bytes > full)
                        return asp_host_fail(ASP_ERR_INVALID_ARG, "array payload does not match its length and element type");
                    a.bytes.resize(h.payload_bytes);
                    if (h.payload_bytes) ok = fread(a.bytes.data(), 1, h.payload_bytes, in.f) == h.payload_bytes;
                }
            }
        }
        if (!ok) return asp_host_fail(ASP_ERR_INVALID_ARG, std::string(path) + " is truncated");
        F->build_descs();
        *out = F.release();
    }
    catch (const std::bad_alloc &)
    {
        return asp_host_fail(ASP_ERR_ALLOC, "host allocation failed");
    }
    return ASP_OK;
}

} // extern "C"
