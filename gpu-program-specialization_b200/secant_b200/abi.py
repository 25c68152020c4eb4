"""ctypes mirror of include/secant_b200.h.

Only declarations live here: structure layouts, constants and the loader of
libsecant_b200.so.  The layouts are the reference's (projects/secant/secant.h:245-679);
tests/test_abi_layout.py checks every size and field offset against values recorded from
the reference header.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "libsecant_b200.so")

# result codes (secant.h:92-131)
RESULT_NAMES = [
    "SUCCESS", "INVALID_VALUE", "OVERFLOW", "INSUFFICIENT_BUFFER", "FORMAT", "ALLOCATION_FAILED", "COMPILE_FAILED",
    "PARSE_FAILED", "SKELETON_NOT_FOUND", "BAD_PROGRAM", "STACK_OVERFLOW", "STACK_UNDERFLOW", "TOO_MANY_ARGS",
    "UNSUPPORTED_OP", "ROUTINE_IDX_OUT_OF_BOUNDS", "ROUTINE_ARG_IDX_OUT_OF_BOUNDS", "ROUTINE_DEPTH_EXCEEDED",
    "INSUFFICIENT_PATCH_SPACE", "REGISTER_OVERFLOW", "UNSUPPORTED_ARCHITECTURE", "INVALID_STATE", "UNSUPPORTED_SHAPE",
    "UNEXPECTED_INSTRUCTION", "BACKEND_UNAVAILABLE", "BAD_BINARY", "BAD_PATCH_SITE", "FUNCTION_NOT_FOUND",
    "PATCH_SITE_NOT_FOUND", "REGISTER_COUNT_NOT_FOUND", "THREAD_FAILED", "DRIVER_FAILED", "EAGER_LOADING_REQUIRED",
    "UNSUPPORTED_VERSION", "COMPLETION_UNKNOWN",
]
for _i, _n in enumerate(RESULT_NAMES):
    globals()[_n if _n == "SUCCESS" else "ERROR_" + _n] = _i

SHAPE_MATERIALIZE, SHAPE_SSE, SHAPE_AFFINE_STATS, SHAPE_GRAM_STATS, SHAPE_TOGGLE_SSE = 1, 2, 5, 6, 10
RECIPE_VERSION = RUN_VERSION = CPU_RUN_VERSION = 3
OPTIONS_VERSION = PLAN_INFO_VERSION = STATS_VERSION = 1

_sz = C.c_size_t
_u32 = C.c_uint32


class ProgramList(C.Structure):
    _fields_ = [("items", C.POINTER(C.POINTER(C.c_uint8))), ("count", _sz)]


class ProgramSet(C.Structure):
    _fields_ = [("routines", ProgramList), ("asts", ProgramList)]


class DeviceMatrix(C.Structure):
    _fields_ = [("address", C.c_size_t), ("num_elements", _sz), ("leading_dimension", _sz)]


class HostMatrix(C.Structure):
    _fields_ = [("data", C.POINTER(C.c_float)), ("num_elements", _sz), ("leading_dimension", _sz)]


class DeviceBanks(C.Structure):
    _fields_ = [("address", C.c_size_t), ("num_elements", _sz), ("bank_stride", _sz)]


class HostBanks(C.Structure):
    _fields_ = [("data", C.POINTER(C.c_float)), ("num_elements", _sz), ("bank_stride", _sz)]


class Header(C.Structure):
    _fields_ = [("struct_size", _u32), ("version", _u32), ("shape", _u32), ("flags", _u32)]


class MaterializeRecipe(C.Structure):
    _fields_ = [("header", Header), ("num_kernels", _sz), ("asts_per_kernel", _sz), ("num_inputs", _sz),
                ("patch_capacity_instructions", _sz)]


class TiledRecipe(C.Structure):  # static SSE / affine stats / Gram stats
    _fields_ = [("header", Header), ("num_kernels", _sz), ("asts_per_kernel", _sz), ("num_inputs", _sz),
                ("num_targets", _sz), ("tile_rows", _sz), ("threads_per_block", _sz),
                ("patch_capacity_instructions", _sz)]


class ToggleRecipe(C.Structure):
    _fields_ = [("header", Header), ("num_kernels", _sz), ("asts_per_kernel", _sz), ("num_inputs", _sz),
                ("num_constants", _sz), ("num_targets", _sz), ("tile_rows", _sz), ("threads_per_block", _sz),
                ("patch_capacity_instructions", _sz)]


class MaterializeRun(C.Structure):
    _fields_ = [("header", Header), ("programs", ProgramSet), ("input", DeviceMatrix), ("num_rows", _sz),
                ("output", DeviceMatrix), ("output_module_stride", _sz)]


class StaticRun(C.Structure):  # SSE / affine stats / Gram stats runs share one layout
    _fields_ = [("header", Header), ("programs", ProgramSet), ("input", DeviceMatrix), ("targets", DeviceMatrix),
                ("num_rows", _sz), ("num_targets", _sz), ("output", DeviceMatrix)]


class ToggleRun(C.Structure):
    _fields_ = [("header", Header), ("programs", ProgramSet), ("input", DeviceMatrix), ("targets", DeviceMatrix),
                ("constants", DeviceBanks), ("num_rows", _sz), ("num_targets", _sz), ("num_banks", _sz),
                ("toggle_bits", _u32), ("output", DeviceMatrix)]


class ToggleRunExt(C.Structure):  # SecantB200ToggleSSERun
    _fields_ = [("base", ToggleRun), ("program_bank_stride", _sz), ("first_program_index", _sz)]


class CpuMaterializeRun(C.Structure):
    _fields_ = [("header", Header), ("programs", ProgramSet), ("num_inputs", _sz), ("input", HostMatrix),
                ("num_rows", _sz), ("output", HostMatrix)]


class CpuStaticRun(C.Structure):
    _fields_ = [("header", Header), ("programs", ProgramSet), ("num_inputs", _sz), ("num_targets", _sz),
                ("input", HostMatrix), ("targets", HostMatrix), ("num_rows", _sz), ("output", HostMatrix)]


class CpuGramRun(C.Structure):
    _fields_ = [("header", Header), ("programs", ProgramSet), ("asts_per_cohort", _sz), ("num_inputs", _sz),
                ("num_targets", _sz), ("input", HostMatrix), ("targets", HostMatrix), ("num_rows", _sz),
                ("statistics", HostMatrix)]


class CpuToggleRun(C.Structure):
    _fields_ = [("header", Header), ("programs", ProgramSet), ("num_inputs", _sz), ("num_constants", _sz),
                ("input", HostMatrix), ("targets", HostMatrix), ("constants", HostBanks), ("num_rows", _sz),
                ("num_targets", _sz), ("num_banks", _sz), ("toggle_bits", _u32), ("output", HostMatrix)]


class RunnerOptions(C.Structure):
    _fields_ = [("struct_size", _u32), ("version", _u32), ("flags", _u32), ("reserved", _u32), ("num_workers", _sz),
                ("num_streams", _sz)]


class PlanInfo(C.Structure):
    _fields_ = [("struct_size", _u32), ("version", _u32), ("shape", _u32), ("flags", _u32), ("cubin_size", _sz)]


class RunnerStats(C.Structure):
    _fields_ = [("struct_size", _u32), ("version", _u32), ("flags", _u32), ("reserved", _u32), ("num_modules", _sz),
                ("num_asts", _sz), ("modules_loaded", _sz), ("compile_window_seconds", C.c_double),
                ("compile_critical_seconds", C.c_double), ("compile_work_seconds", C.c_double),
                ("module_load_seconds", C.c_double), ("completion_wait_seconds", C.c_double),
                ("module_unload_seconds", C.c_double), ("runtime_seconds", C.c_double), ("total_seconds", C.c_double)]


class Rk4Run(C.Structure):  # SecantB200Rk4Run
    _fields_ = [("struct_size", _u32), ("version", _u32), ("flags", _u32), ("reserved", _u32), ("programs", ProgramSet),
                ("num_systems", _sz), ("num_states", _sz), ("num_constants", _sz), ("constants", DeviceBanks),
                ("system_bank_stride", _sz), ("num_banks", _sz), ("toggle_bits", _u32), ("reserved2", _u32),
                ("reference", DeviceMatrix), ("num_trajectories", _sz), ("points_per_trajectory", _sz),
                ("times", C.c_size_t), ("steps_per_observation", _sz), ("output", DeviceMatrix),
                ("trajectory_offsets", C.c_size_t), ("total_points", _sz), ("allow_missing_observations", _u32),
                ("reserved3", _u32), ("sampled_parameters", C.c_size_t), ("uniform_pool", C.c_size_t),
                ("normal_pool", C.c_size_t), ("rng_pool_size", C.c_uint64), ("integrated_intervals", C.c_size_t)]


class SampledParameter(C.Structure):  # SecantB200SampledParameter, layout of the reference's OdezzaSampledParameter
    _fields_ = [("offset", C.c_uint64), ("stride", _u32), ("distribution", _u32), ("scale", C.c_float), ("shift", C.c_float),
                ("lower", C.c_float), ("upper", C.c_float)]


class Winner(C.Structure):  # SecantB200Winner
    _fields_ = [("mse", C.c_float), ("reserved", _u32), ("score_index", C.c_uint64)]


class Score(C.Structure):  # SecantB200Score, layout of the reference consumer's SRScore
    _fields_ = [("sse", C.c_float), ("reserved", _u32), ("configuration", C.c_uint64), ("valid_configurations", C.c_uint64)]


def init_header(struct, version, shape):
    struct.header.struct_size = C.sizeof(struct)
    struct.header.version = version
    struct.header.shape = shape
    struct.header.flags = 0
    return struct


def runner_options(num_workers=1, num_streams=1):
    o = RunnerOptions()
    o.struct_size = C.sizeof(o)
    o.version = OPTIONS_VERSION
    o.num_workers = num_workers
    o.num_streams = num_streams
    return o


def runner_stats():
    s = RunnerStats()
    s.struct_size = C.sizeof(s)
    s.version = STATS_VERSION
    return s


# every symbol include/secant_b200.h and include/secant_b200_ext.h declare
EXPORTED = {
    "secant_result_to_string": (C.c_char_p, [C.c_int32]),
    "secant_cuda_target_stats_f32_source_get": (C.c_char_p, [C.POINTER(_sz)]),
    "secant_cubin_recipe_validate": (C.c_int32, [C.c_void_p]),
    "secant_cubin_source_size": (C.c_int32, [C.c_void_p, C.POINTER(_sz)]),
    "secant_cubin_source_write": (C.c_int32, [C.c_void_p, C.c_char_p, _sz]),
    "secant_cubin_plan_storage_size": (C.c_int32, [C.c_void_p, C.c_void_p, _sz, C.POINTER(_sz)]),
    "secant_cubin_plan_init": (C.c_int32, [C.c_void_p, C.c_void_p, _sz, C.c_void_p, _sz, C.POINTER(C.c_void_p)]),
    "secant_cubin_plan_info_get": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "secant_cubin_plan_recipe_get": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "secant_cubin_specialize_into": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, _sz]),
    "secant_cubin_runner_create": (C.c_int32, [C.c_void_p, C.c_void_p, _sz, C.c_void_p, C.POINTER(C.c_void_p)]),
    "secant_cubin_runner_run_batch": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p), _sz, C.c_void_p]),
    "secant_cubin_runner_run": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "secant_cubin_runner_destroy": (C.c_int32, [C.c_void_p]),
    "secant_cpu_run": (C.c_int32, [C.c_void_p]),
    "secant_b200_runner_create": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    "secant_b200_population_create": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(C.c_void_p)]),
    "secant_b200_population_run": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "secant_b200_population_run_batch": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p), _sz, C.c_void_p]),
    "secant_b200_population_num_ops": (C.c_uint64, [C.c_void_p]),
    "secant_b200_population_destroy": (C.c_int32, [C.c_void_p]),
    "secant_b200_runner_set_scratch_limit": (C.c_int32, [C.c_void_p, C.c_size_t]),
    "secant_b200_runner_set_math": (C.c_int32, [C.c_void_p, C.c_uint32]),
    "secant_b200_grouped_topk": (C.c_int32, [C.c_size_t, _sz, _sz, C.c_uint32, C.c_uint32, C.c_uint32, C.c_size_t, C.c_size_t,
                                 C.c_void_p]),
    "secant_b200_rk4_score": (C.c_int32, [C.c_void_p]),
    "secant_b200_release_cached_memory": (C.c_int32, []),
    "secant_b200_best_config": (C.c_int32, [C.c_size_t, _sz, _sz, _sz, C.c_size_t, C.c_void_p]),
    "secant_b200_topk": (C.c_int32, [C.c_size_t, _sz, _sz, C.c_size_t, C.c_size_t, C.c_void_p]),
    "secant_b200_topk_scratch_elements": (_sz, [_sz, _sz]),
    "secant_b200_topk_static": (C.c_int32, [C.c_size_t, _sz, _sz, C.c_size_t, C.c_size_t, C.c_void_p]),
    "secant_b200_fp32_peak_probe": (C.c_int32, [C.c_double, C.POINTER(C.c_double)]),
    "secant_b200_runner_last_error": (C.c_char_p, [C.c_void_p]),
    "secant_b200_kernel_launch_count": (C.c_uint64, []),
    "secant_b200_row_stream_bytes": (C.c_uint64, []),
}

_lib = None


def load():
    """Loads libsecant_b200.so; raises if the library has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `make -C {os.path.dirname(LIB_PATH)}`")
        lib = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in EXPORTED.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def result_name(code):
    return RESULT_NAMES[code] if 0 <= code < len(RESULT_NAMES) else f"UNKNOWN({code})"


class SecantError(RuntimeError):
    def __init__(self, code, what=""):
        super().__init__(f"{what}: SECANT_{'ERROR_' if code else ''}{result_name(code)}")
        self.code = code


def check(code, what=""):
    if code != SUCCESS:  # noqa: F821 (defined through globals())
        raise SecantError(code, what)
