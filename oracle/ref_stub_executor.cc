// Test infrastructure (oracle side): replacement for the reference's executor.cc.
// The reference's executor writes text files, shells out to nvcc and runs a.out
// (executor.cc:6-260). The format oracle only needs the host-side format building, so the
// five entry points of executor.hpp:12-22 are satisfied with stubs that report "not run".
#include "executor.hpp"

bool part_execute_code_builder(code_builder_t *, vector<int>, float &time_ms, float &gflops, string, string, bool)
{
    time_ms = 0; gflops = 0; return false;
}
bool part_execute_code_builder(code_builder_t *, vector<int>, float &time_ms, float &gflops, string, string, bool, bool)
{
    time_ms = 0; gflops = 0; return false;
}
bool execute_code_builder(code_builder_t *, float &time_ms, float &gflops, string, string, bool)
{
    time_ms = 0; gflops = 0; return false;
}
bool compile_spmv_code(string) { return false; }
bool execute_binary(string, float &t, float &g) { t = 0; g = 0; return false; }
