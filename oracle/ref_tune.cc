// Test infrastructure (oracle side). NOT part of the product.
//
// Drives the UNMODIFIED tuner of the reference over one matrix, linked with oracle/ref_shim_executor.cc in
// place of the reference's executor.cc: the reference's own whitelist strategies
// (find_best_path_of_white_list_strategy1..9, whilte_list_path_impl.cc) or its rule dispatcher
// (find_best_path_of_compressed_sub_matrix, whilte_list_path_impl.cc:3411) enumerate their graphs and launch
// parameters exactly as they always did, and every trial they hand to executor.hpp:12-22 is timed by the
// hand-written kernels behind the C ABI (or, with ASP_SHIM_NO_GPU=1, only recorded).
//
// Usage: ref_tune <matrix.mtx.coo> <float|double> <1..9|all>
// Prints one line per strategy run: "strategy <k> ms <best time> gflops <best gflops> template <type>".
#include <cstdio>
#include <cstdlib>
#include <string>

#include "default_auto_tuner.hpp"

int main(int argc, char **argv)
{
    if (argc < 4)
    {
        fprintf(stderr, "usage: %s <matrix.mtx.coo> <float|double> <1..9|all>\n", argv[0]);
        return 2;
    }
    const std::string mtx = argv[1], which = argv[3];
    const data_type vt = std::string(argv[2]) == "double" ? DOUBLE : FLOAT;
    // dense view: input + compress, the pattern of the reference's own drivers (main.cc:368-443)
    dense_begin_memory_cache_input_file_direct_param_strategy_t in = get_begin_memory_cache_input_file_direct_param_strategy_from_coo_file(mtx, vt);
    exe_dense_sub_graph_t dg;
    param_strategy_of_sub_graph_t dp;
    add_a_exe_node_and_param_strategy_to_exe_dense_sub_graph(&dg, &dp, BEGIN_MEMORY_CACHE_INPUT_FILE, DENSE_BEGIN_MEMORY_CACHE_INPUT_FILE_DIRECT_PARAM_STRATEGY, &in);
    compress_none_param_strategy_t cs;
    add_a_exe_node_and_param_strategy_to_exe_dense_sub_graph(&dg, &dp, COMPRESS, COMPRESS_NONE_PARAM_STRATEGY, &cs);
    sparse_struct_t *matrix = execute_dense_matrix_exe_graph_with_param_strategy(&dg, &dp);
    float t = 0, g = 0;
    compressed_sub_block_exe_graph_and_template_t best;
    if (which == "all") best = find_best_path_of_compressed_sub_matrix(matrix, 0, t, g, NULL, NULL);
    else
    {
        switch (atoi(which.c_str()))
        {
        case 1: best = find_best_path_of_white_list_strategy1(matrix, 0, t, g, NULL, NULL); break;
        case 2: best = find_best_path_of_white_list_strategy2(matrix, 0, t, g, NULL, NULL); break;
        case 3: best = find_best_path_of_white_list_strategy3(matrix, 0, t, g, NULL, NULL); break;
        case 4: best = find_best_path_of_white_list_strategy4(matrix, 0, t, g, NULL, NULL); break;
        case 5: best = find_best_path_of_white_list_strategy5(matrix, 0, t, g, NULL, NULL); break;
        case 6: best = find_best_path_of_white_list_strategy6(matrix, 0, t, g, NULL, NULL); break;
        case 7: best = find_best_path_of_white_list_strategy7(matrix, 0, t, g, NULL, NULL); break;
        case 8: best = find_best_path_of_white_list_strategy8(matrix, 0, t, g, NULL, NULL); break;
        case 9: best = find_best_path_of_white_list_strategy9(matrix, 0, t, g, NULL, NULL); break;
        default: fprintf(stderr, "no such strategy\n"); return 2;
        }
    }
    printf("strategy %s ms %g gflops %g template %d\n", which.c_str(), (double)t, (double)g, (int)best.temp_node.type);
    return 0;
}
