// asp_search with the GPU as the timer: a trial's format is uploaded once, its launch parameters are
// swept in place, and asp_time measures it (replaces the reference's emit + nvcc + run per trial).
#include <vector>

#include "../../include/asp_b200.h"
#include "../../include/asp_b200_host.h"

namespace
{
struct GpuTimer
{
    asp_ctx *ctx;
    uint64_t cached = 0; // asp_format_id of the uploaded format
    std::vector<asp_plan *> plans;

    void drop()
    {
        for (asp_plan *p : plans)
            if (p) asp_plan_destroy(p);
        plans.clear();
        cached = 0;
    }
    ~GpuTimer() { drop(); }
};

int time_on_gpu(void *user, const asp_format *fmt, const int64_t *tblock, const int64_t *threads, const int64_t *reduce, int warmup, int reps, float *ms)
{
    GpuTimer *t = static_cast<GpuTimer *>(user);
    const int n = asp_format_num_subs(fmt);
    if (n <= 0) return 1;
    if (t->cached != asp_format_id(fmt))
    {
        t->drop();
        std::vector<asp_plan_desc> descs(n);
        if (asp_format_plan_descs(fmt, descs.data()) != ASP_OK) return 1;
        t->plans.assign(n, nullptr);
        if (asp_plan_group_create(t->ctx, descs.data(), n, t->plans.data()) != ASP_OK)
        {
            t->plans.clear();
            return 1;
        }
        t->cached = asp_format_id(fmt);
    }
    std::vector<asp_plan_desc> descs(n);
    if (asp_format_plan_descs(fmt, descs.data()) != ASP_OK) return 1;
    for (int i = 0; i < n; i++)
    {
        if (descs[i].template_type == ASP_EMPTY_TEMPLATE) continue;
        if (asp_plan_set_launch(t->plans[i], tblock[i], threads[i], reduce[i]) != ASP_OK) return 1;
    }
    float gflops = 0;
    return asp_time(t->ctx, t->plans.data(), n, warmup, reps, 2, 0.0, ms, &gflops) == ASP_OK ? 0 : 1;
}
} // namespace

extern "C" asp_status asp_search_gpu(asp_ctx *ctx, const void *matrix, const void *options, void **result)
{
    if (!ctx || !matrix || !result) return ASP_ERR_INVALID_ARG;
    GpuTimer timer{ctx};
    asp_search_result *r = nullptr;
    const asp_status st = asp_search(static_cast<const asp_matrix *>(matrix), static_cast<const asp_search_options *>(options), time_on_gpu, &timer, &r);
    *result = r;
    return st;
}
