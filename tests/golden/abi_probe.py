"""Shared by make_abi_layout.py and tests/test_abi_layout.py: builds and runs a small C
program that prints sizeof/offsetof of every public struct of a Secant header as JSON."""
import json
import os
import subprocess
import tempfile

STRUCTS = {
    "SecantAstProgramList": ["items", "count"],
    "SecantAstProgramSet": ["routines", "asts"],
    "SecantDeviceMatrixF32": ["address", "num_elements", "leading_dimension"],
    "SecantConstHostMatrixF32": ["data", "num_elements", "leading_dimension"],
    "SecantHostMatrixF32": ["data", "num_elements", "leading_dimension"],
    "SecantDeviceConstantBanks": ["address", "num_elements", "bank_stride"],
    "SecantConstHostConstantBanks": ["data", "num_elements", "bank_stride"],
    "SecantCubinRecipeHeader": ["struct_size", "version", "shape", "flags"],
    "SecantCubinMaterializeRecipe": ["header", "num_kernels", "asts_per_kernel", "num_inputs", "patch_capacity_instructions"],
    "SecantCubinSSERecipe": ["header", "num_kernels", "asts_per_kernel", "num_inputs", "num_targets", "tile_rows",
                             "threads_per_block", "patch_capacity_instructions"],
    "SecantCubinAffineStatsRecipe": ["header", "num_kernels", "asts_per_kernel", "num_inputs", "num_targets", "tile_rows",
                                     "threads_per_block", "patch_capacity_instructions"],
    "SecantCubinGramStatsRecipe": ["header", "num_kernels", "asts_per_kernel", "num_inputs", "num_targets", "tile_rows",
                                   "threads_per_block", "patch_capacity_instructions"],
    "SecantCubinToggleSSERecipe": ["header", "num_kernels", "asts_per_kernel", "num_inputs", "num_constants", "num_targets",
                                   "tile_rows", "threads_per_block", "patch_capacity_instructions"],
    "SecantCubinRunHeader": ["struct_size", "version", "shape", "flags"],
    "SecantCubinMaterializeRun": ["header", "programs", "input", "num_rows", "output", "output_module_stride"],
    "SecantCubinSSERun": ["header", "programs", "input", "targets", "num_rows", "num_targets", "output"],
    "SecantCubinAffineStatsRun": ["header", "programs", "input", "targets", "num_rows", "num_targets", "ast_stats"],
    "SecantCubinGramStatsRun": ["header", "programs", "input", "targets", "num_rows", "num_targets", "statistics"],
    "SecantCubinToggleSSERun": ["header", "programs", "input", "targets", "constants", "num_rows", "num_targets",
                                "num_banks", "toggle_bits", "output"],
    "SecantCpuRunHeader": ["struct_size", "version", "shape", "flags"],
    "SecantCpuMaterializeRun": ["header", "programs", "num_inputs", "input", "num_rows", "output"],
    "SecantCpuSSERun": ["header", "programs", "num_inputs", "num_targets", "input", "targets", "num_rows", "output"],
    "SecantCpuAffineStatsRun": ["header", "programs", "num_inputs", "num_targets", "input", "targets", "num_rows", "ast_stats"],
    "SecantCpuGramStatsRun": ["header", "programs", "asts_per_cohort", "num_inputs", "num_targets", "input", "targets",
                              "num_rows", "statistics"],
    "SecantCpuToggleSSERun": ["header", "programs", "num_inputs", "num_constants", "input", "targets", "constants",
                              "num_rows", "num_targets", "num_banks", "toggle_bits", "output"],
    "SecantCubinRunnerOptions": ["struct_size", "version", "flags", "reserved", "num_workers", "num_streams"],
    "SecantCubinPlanInfo": ["struct_size", "version", "shape", "flags", "cubin_size"],
    "SecantRunnerStats": ["struct_size", "version", "flags", "reserved", "num_modules", "num_asts", "modules_loaded",
                          "compile_window_seconds", "compile_critical_seconds", "compile_work_seconds",
                          "module_load_seconds", "completion_wait_seconds", "module_unload_seconds", "runtime_seconds",
                          "total_seconds"],
}
CONSTANTS = [
    "SECANT_RESULT_COUNT", "SECANT_ERROR_COMPLETION_UNKNOWN", "SECANT_ERROR_BAD_PROGRAM", "SECANT_ERROR_UNSUPPORTED_VERSION",
    "SECANT_AST_INSTRUCTION_TYPE_COLUMN_F32", "SECANT_AST_INSTRUCTION_TYPE_AFFINE_BANK_F32",
    "SECANT_AST_INSTRUCTION_TYPE_TOGGLE4_F32", "SECANT_AST_INSTRUCTION_TYPE_EXP_F32", "SECANT_AST_INSTRUCTION_TYPE_TANH_F32",
    "SECANT_AST_INSTRUCTION_TYPE_FMA_U32", "SECANT_AST_INSTRUCTION_TYPE_ONE_PAST_LAST", "SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32",
    "SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32", "SECANT_CUBIN_RUN_VERSION_3", "SECANT_RUNNER_STATS_VERSION_1",
    "SECANT_AST_MAX_PROGRAM_INSTRUCTIONS", "SECANT_AST_MAX_STACK_DEPTH", "SECANT_AST_MAX_INPUTS", "SECANT_AST_MAX_ROUTINES",
]


def probe(header_name, include_dir):
    lines = ["#include <stdio.h>", "#include <stddef.h>", f'#include "{header_name}"', "int main(void) {", 'printf("{");']
    first = True
    for name, fields in STRUCTS.items():
        sep = "" if first else ","
        first = False
        lines.append(f'printf("{sep}\\"{name}\\": {{\\"sizeof\\": %zu", sizeof({name}));')
        for f in fields:
            lines.append(f'printf(", \\"{f}\\": %zu", offsetof({name}, {f}));')
        lines.append('printf("}");')
    for c in CONSTANTS:
        lines.append(f'printf(", \\"{c}\\": %lld", (long long)({c}));')
    # widths of every opcode byte value, so the two decoders are compared exhaustively
    lines.append('printf(", \\"instruction_sizes\\": [");')
    lines.append("for (int op = 0; op < 256; ++op) { unsigned char b[10] = {0}; b[0] = (unsigned char)op; "
                 'printf("%s%zu", op ? "," : "", secant_ast_instruction_size_get(b)); }')
    lines.append('printf("]}\\n"); return 0; }')
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "probe.c")
        exe = os.path.join(tmp, "probe")
        with open(src, "w") as f:
            f.write("\n".join(lines))
        subprocess.run(["gcc", "-std=c99", "-I", include_dir, src, "-o", exe], check=True)
        return json.loads(subprocess.run([exe], check=True, capture_output=True, text=True).stdout)
