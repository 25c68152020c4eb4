/*
 * odezza_ref_shim.c - test infrastructure: makes the reference's own fixed-shape CPU rollout scorer
 * callable from the tests.
 *
 * The reference holds one host-side scorer for RK4 rollouts, o_cpu_score
 * (projects/odezza/research/ast_tools/o_ast_engine_benchmark.c:368-434), a static function of its
 * engine benchmark: 4 states, 3 trajectories, 8 observations 0.05 apart, right-hand sides in the
 * engine's own bytecode evaluated by o_ast_cpu_evaluate (o_ast_cpu.c:111-209).  This file includes
 * that benchmark source where it lies (the Makefile passes its directory with -I; nothing is
 * copied), renames its main() out of the way, and exports one wrapper around the static function.
 * Unused code of the benchmark (which calls the engine's GPU library) is dropped by the linker's
 * section garbage collection, so the result depends on libm only.  Built into oracle/_ref/ by
 * `make odezza`; only the tests load it, to pin oracle/secant_oracle.c::so_rk4_score.
 */
#define main o_ast_engine_benchmark_main_unused
#include "o_ast_engine_benchmark.c"
#undef main

__attribute__((visibility("default")))
float so_ref_o_cpu_score(const uint8_t* const* programs, const size_t* byte_counts, size_t rhs_count, const float* constants,
                         uint32_t permutation, const float* reference, uint32_t steps_per_observation) {
    OdezzaScoringRhs rhs[O_STATE_COUNT];
    OdezzaScoringSystem system;
    size_t i;
    if (rhs_count != O_STATE_COUNT) return -1.0f;
    memset(rhs, 0, sizeof(rhs));
    for (i = 0; i < rhs_count; ++i) {
        rhs[i].state_index = (uint8_t)i;
        rhs[i].program.bytes = programs[i];
        rhs[i].program.byte_count = byte_counts[i];
    }
    system.rhs = rhs;
    system.rhs_count = rhs_count;
    return o_cpu_score(&system, 0u, constants, permutation, reference, steps_per_observation);
}
