"""ctypes mirror of include/odezza_b200.h: the ODE engine's scoring handle, random pools and score
reducer (projects/odezza/core/odezza.h:236-518) as libsecant_b200.so provides them.

Layouts and names are the reference's; the small classes below only keep the buffers a launch
points at alive and turn result codes into exceptions.  Device memory is the caller's (torch
tensors in the tests): every address is passed as an integer, as the C interface takes it.
"""
import ctypes as C

from . import abi

RESULT_NAMES = [
    "SUCCESS", "INVALID_ARGUMENT", "INSUFFICIENT_BUFFER", "OVERFLOW", "FORMAT", "ALLOCATION", "IO", "UNSUPPORTED", "COMPILATION",
    "COMPILER", "AST", "SPECIALIZATION_CAPACITY", "REGISTER_PRESSURE", "STATE_LAYOUT", "QUEUE_FULL", "CUDA", "THREAD", "BUSY",
    "CUDA_UNFENCED",
]
for _i, _n in enumerate(RESULT_NAMES):
    globals()[_n if _n == "SUCCESS" else "ERROR_" + _n] = _i

# right-hand-side bytecode (projects/odezza/core/odezza.h:70-96)
OP = {
    "RET": 0x80, "STATE": 0x81, "CONSTANT": 0x82, "LIT": 0x83, "TOG2": 0x84, "TOG4": 0x85, "ADD": 0x90, "SUB": 0x91, "MUL": 0x92,
    "DIV": 0x93, "NEG": 0x94, "SQRT": 0x95, "RCP": 0x96, "ABS": 0x97, "MIN": 0x98, "MAX": 0x99, "FMA": 0x9A, "SIN": 0x9B,
    "COS": 0x9C, "EX2": 0x9D, "LG2": 0x9E, "RSQRT": 0x9F, "TANH": 0xA0, "EXP": 0xA1, "LOG": 0xA2,
}
BY_SYSTEM, BY_SYSTEM_PERMUTATION, GLOBAL = 0, 1, 2
RNG_UNIFORM, RNG_NORMAL = 1, 2

_sz, _u32, _u64, _ptr = C.c_size_t, C.c_uint32, C.c_uint64, C.c_uint64  # CUdeviceptr is 64 bits wide


class AstProgram(C.Structure):
    _fields_ = [("bytes", C.POINTER(C.c_uint8)), ("byte_count", _sz)]


class ScoringRhs(C.Structure):
    _fields_ = [("state_index", C.c_uint8), ("program", AstProgram)]


class ScoringSystem(C.Structure):
    _fields_ = [("rhs", C.POINTER(ScoringRhs)), ("rhs_count", _sz)]


class CreateInfo(C.Structure):
    _fields_ = [("sm_version", _u32), ("state_count", _sz), ("state_capacity", _sz), ("constant_count", _u32),
                ("constant_capacity", _u32), ("fixed_rhs", C.POINTER(ScoringRhs)), ("fixed_rhs_count", _sz),
                ("system_capacity", _u32), ("shared_patch_capacity", _u32), ("system_patch_capacity", _u32),
                ("worker_count", _u32), ("cubin_slots_per_worker", _u32)]


class SampledParameter(C.Structure):
    _fields_ = [("offset", _u64), ("stride", _u32), ("distribution", _u32), ("scale", C.c_float), ("shift", C.c_float),
                ("lower", C.c_float), ("upper", C.c_float)]


class Launch(C.Structure):
    _fields_ = [("constant_banks_device", _ptr), ("constant_bank_count", _u32), ("active_toggle_count", _u32),
                ("trajectory_offsets_device", _ptr), ("trajectory_times_device", _ptr), ("reference_data_device", _ptr),
                ("trajectory_count", _u32), ("trajectory_point_count", _u32), ("steps_per_observation", _u32),
                ("mse_output_device", _ptr), ("sampled_parameters_device", _ptr), ("uniform_pool_device", _ptr),
                ("normal_pool_device", _ptr), ("rng_pool_size", _u64), ("allow_missing_observations", _u32),
                ("input_ready_event", C.c_void_p), ("profile_timing", _u32)]


class RunReport(C.Structure):
    _fields_ = [("system_count", _sz), ("module_count", _sz), ("configuration_count", _u64), ("total_seconds", C.c_double),
                ("queue_wait_seconds", C.c_double), ("cubin_reset_seconds", C.c_double), ("specialization_seconds", C.c_double),
                ("module_load_seconds", C.c_double), ("function_lookup_seconds", C.c_double), ("launch_seconds", C.c_double),
                ("completion_wait_seconds", C.c_double), ("module_unload_seconds", C.c_double), ("gpu_sum_seconds", C.c_double),
                ("gpu_active_seconds", C.c_double), ("gpu_span_seconds", C.c_double), ("profiled_modules", _u64),
                ("maximum_register_count", _u32), ("maximum_shared_memory_bytes", _u32)]


class PipelineStats(C.Structure):
    _fields_ = [(n, _u64) for n in ("submitted_ticket_count", "completed_ticket_count", "cubin_reset_count", "cubin_reset_byte_count",
                                    "specialization_failure_count", "cuda_failure_count", "worker_slot_wait_count")] + \
               [(n, _u32) for n in ("peak_pending_ticket_count", "peak_ready_slot_count", "peak_inflight_module_count")] + \
               [(n, C.c_double) for n in ("cubin_reset_seconds", "specialization_seconds", "module_load_seconds",
                                          "function_lookup_seconds", "launch_seconds", "completion_wait_seconds",
                                          "module_unload_seconds", "cuda_resource_create_seconds")]


class RngPoolInfo(C.Structure):
    _fields_ = [("seed", _u64), ("stream", _u64), ("sample_base", _u64), ("size", _u64), ("distributions", _u32)]


class RngPoolView(C.Structure):
    _fields_ = [("uniform_device", _ptr), ("normal_device", _ptr), ("info", RngPoolInfo), ("uniform_seconds", C.c_double),
                ("normal_seconds", C.c_double)]


class ScoreWinner(C.Structure):
    _fields_ = [("mse", C.c_float), ("reserved", _u32), ("score_index", _u64)]


class ScoreCounts(C.Structure):
    _fields_ = [("valid", _u64), ("invalid", _u64), ("negative", _u64)]


class ScoreIndex(C.Structure):
    _fields_ = [("system_index", _u64), ("configuration_index", _u64), ("bank_index", _u64), ("permutation", _u32)]


class ReductionSize(C.Structure):
    _fields_ = [("configuration_count", _u64), ("score_count", _u64), ("group_count", _u64), ("tiles_per_group", _u32),
                ("workspace_bytes", _sz), ("winner_bytes", _sz), ("count_bytes", _sz)]


class ReductionReport(C.Structure):
    _fields_ = [("kernel_seconds", C.c_double), ("group_count", _u64), ("score_count", _u64)]


_r, _vp = C.c_int32, C.c_void_p
# every symbol include/odezza_b200.h declares
EXPORTED = {
    "odezza_scoring_pipeline_create": (_r, [_vp, C.POINTER(_vp)]),
    "odezza_scoring_pipeline_destroy": (_r, [_vp]),
    "odezza_scoring_pipeline_workspace_requirements": (_r, [_vp, C.POINTER(_sz), C.POINTER(_sz)]),
    "odezza_scoring_pipeline_run": (_r, [_vp, _vp, _sz, _vp, _vp, _sz, _vp]),
    "odezza_scoring_pipeline_write_error": (_r, [_vp, C.c_char_p, _sz, C.POINTER(_sz)]),
    "o_scoring_pipeline_stats": (_r, [_vp, _vp]),
    "odezza_philox4x32": (_r, [C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32)]),
    "odezza_rng_uniform": (_r, [_u64, _u64, _u64, C.POINTER(C.c_float)]),
    "odezza_rng_pool_create": (_r, [_u32, _vp, C.POINTER(_vp)]),
    "odezza_rng_pool_view": (_r, [_vp, _vp]),
    "odezza_rng_pool_write_error": (_r, [_vp, C.c_char_p, _sz]),
    "odezza_rng_pool_destroy": (_r, [_vp]),
    "odezza_sampled_parameter_validate": (_r, [_vp, _u32, _vp]),
    "odezza_score_reducer_create": (_r, [_u32, _u32, C.POINTER(_vp)]),
    "odezza_score_reducer_set_k": (_r, [_vp, _u32]),
    "odezza_score_reducer_destroy": (_r, [_vp]),
    "odezza_score_reducer_write_error": (_r, [_vp, C.c_char_p, _sz]),
    "odezza_score_reduction_requirements": (_r, [_vp, _sz, C.c_int, _u32, _vp]),
    "odezza_score_decode_index": (_r, [_vp, _sz, _u64, _vp]),
    "odezza_score_reducer_run": (_r, [_vp, _vp, _sz, C.c_int, _ptr, _sz, _ptr, _sz, _ptr, _sz, _vp]),
    "odezza_score_reducer_gather": (_r, [_vp, _vp, _sz, C.c_int, _u32, _ptr, _sz, _ptr, _sz]),
}

_bound = False


def load():
    """libsecant_b200.so with the engine entry points typed."""
    global _bound
    lib = abi.load()
    if not _bound:
        for name, (restype, argtypes) in EXPORTED.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        _bound = True
    return lib


def result_name(code):
    return RESULT_NAMES[code] if 0 <= code < len(RESULT_NAMES) else f"UNKNOWN({code})"


class EngineError(RuntimeError):
    def __init__(self, code, what=""):
        super().__init__(f"{what}: ODEZZA_{'ERROR_' if code else ''}{result_name(code)}")
        self.code = code


def check(code, what=""):
    if code:
        raise EngineError(code, what)


def _program(code):
    buf = (C.c_uint8 * len(code)).from_buffer_copy(bytes(code))
    return buf, AstProgram(C.cast(buf, C.POINTER(C.c_uint8)), len(code))


def rhs_array(pairs):
    """[(state index, program bytes)] -> (ScoringRhs array, objects that must outlive it)."""
    keep, arr = [], (ScoringRhs * max(1, len(pairs)))()
    for i, (state, code) in enumerate(pairs):
        buf, prog = _program(code)
        keep.append(buf)
        arr[i].state_index = state
        arr[i].program = prog
    return arr, keep


def systems_array(systems):
    """[[(state index, program bytes), ...] per system] -> (ScoringSystem array, keep-alive list)."""
    keep, arr = [], (ScoringSystem * len(systems))()
    for i, pairs in enumerate(systems):
        rhs, alive = rhs_array(pairs)
        keep += [rhs, alive]
        arr[i].rhs = C.cast(rhs, C.POINTER(ScoringRhs))
        arr[i].rhs_count = len(pairs)
    return arr, keep


class ScoringPipeline:
    """odezza_scoring_pipeline_create / run / destroy."""

    def __init__(self, states, constants=0, fixed=(), sm_version=100, system_capacity=1, check_result=True):
        self.lib = load()
        info = CreateInfo()
        info.sm_version = sm_version
        info.state_count = info.state_capacity = states
        info.constant_count = info.constant_capacity = constants
        self._fixed, self._keep = rhs_array(list(fixed))
        info.fixed_rhs = C.cast(self._fixed, C.POINTER(ScoringRhs)) if fixed else None
        info.fixed_rhs_count = len(fixed)
        info.system_capacity = system_capacity
        info.shared_patch_capacity, info.system_patch_capacity = 64, 128
        info.worker_count, info.cubin_slots_per_worker = 1, 2
        self.handle = C.c_void_p()
        self.created = self.lib.odezza_scoring_pipeline_create(C.byref(info), C.byref(self.handle))
        if check_result:
            check(self.created, "odezza_scoring_pipeline_create: " + self.error())
        size, alignment = C.c_size_t(), C.c_size_t()
        self.workspace = None
        if self.created == 0:
            check(self.lib.odezza_scoring_pipeline_workspace_requirements(self.handle, C.byref(size), C.byref(alignment)))
            self.workspace = (C.c_uint64 * ((size.value + 7) // 8))()
            self.workspace_size = size.value

    def error(self):
        if not self.handle:
            return ""
        buf, n = C.create_string_buffer(1024), C.c_size_t()
        self.lib.odezza_scoring_pipeline_write_error(self.handle, buf, len(buf), C.byref(n))
        return buf.value.decode()

    def run(self, systems, launch, count=None):
        """Returns (result code, RunReport)."""
        arr, keep = systems_array(systems)
        report = RunReport()
        code = self.lib.odezza_scoring_pipeline_run(self.handle, arr, len(systems) if count is None else count, C.byref(launch),
                                                    self.workspace, self.workspace_size, C.byref(report))
        del keep
        return code, report

    def stats(self):
        s = PipelineStats()
        check(self.lib.o_scoring_pipeline_stats(self.handle, C.byref(s)))
        return s

    def close(self):
        if self.handle:
            check(self.lib.odezza_scoring_pipeline_destroy(self.handle))
            self.handle = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
