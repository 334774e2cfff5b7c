// Definitions of the opaque handles of include/asp_b200_host.h, shared by the translation units that
// implement them.
#ifndef ASP_HOST_HANDLES_HPP
#define ASP_HOST_HANDLES_HPP
#include <memory>
#include <string>
#include <vector>

#include "../../../include/asp_b200_host.h"
#include "format.hpp"

struct asp_matrix
{
    std::unique_ptr<asp::host::Matrix> m;
};

struct asp_format
{
    uint64_t id;                          // unique per process: addresses are reused, ids are not
    std::unique_ptr<asp::host::Matrix> m; // the transformed copy; absent in a format loaded from a file
    std::vector<asp::host::TemplateData> subs;
    std::vector<std::vector<asp_array_desc>> descs;
    // what the accessors report, cached so that a loaded format (no Matrix) answers the same way
    int val_dt = ASP_F32;
    uint64_t n_rows = 0, n_cols = 0;
    std::shared_ptr<std::vector<uint8_t>> perm; // global row permutation (new -> old), null when unsorted
    int perm_dt = ASP_U8;
    std::vector<asp_sub_info> infos;
    asp_format();
    void cache_from_matrix(); // fills the cached fields from m and subs
    void build_descs();       // C-ABI descriptors over the template arrays
};

asp_status asp_host_fail(asp_status s, const std::string &msg);
#endif
