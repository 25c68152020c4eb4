"""Runner: the reference's create / run / destroy call sequence over torch device memory.

torch is used for device allocations, streams and (in the benchmark) torch.distributed
only; every evaluation goes through the C-ABI of libsecant_b200.so.  Method names and
argument meaning follow the reference run descriptors (projects/secant/secant.h:418-540):
matrices are [column][row] float32, outputs are caller-visible tensors the library clears
and writes.
"""
import ctypes as C

import torch

from . import abi

_SHAPE_RECIPE = {
    abi.SHAPE_MATERIALIZE: abi.MaterializeRecipe,
    abi.SHAPE_SSE: abi.TiledRecipe,
    abi.SHAPE_AFFINE_STATS: abi.TiledRecipe,
    abi.SHAPE_GRAM_STATS: abi.TiledRecipe,
    abi.SHAPE_TOGGLE_SSE: abi.ToggleRecipe,
}


def make_recipe(shape, num_inputs, num_targets=1, num_constants=0, num_kernels=8, asts_per_kernel=None):
    r = abi.init_header(_SHAPE_RECIPE[shape](), abi.RECIPE_VERSION, shape)
    r.num_kernels = num_kernels
    r.asts_per_kernel = asts_per_kernel or (8 if shape == abi.SHAPE_TOGGLE_SSE else 4)
    r.num_inputs = num_inputs
    r.patch_capacity_instructions = 2048
    if shape != abi.SHAPE_MATERIALIZE:
        r.num_targets = num_targets
        r.tile_rows = 128
        r.threads_per_block = 128
    if shape == abi.SHAPE_TOGGLE_SSE:
        r.num_constants = num_constants
    return r


def _matrix(t, leading_dimension=None):
    m = abi.DeviceMatrix()
    if t is not None:
        m.address = t.data_ptr()
        m.num_elements = t.numel()
        m.leading_dimension = leading_dimension if leading_dimension is not None else (t.shape[-1] if t.dim() else 1)
    return m


class Runner:
    """One runner handle for one kernel shape, bound to torch's current CUDA context."""

    def __init__(self, shape, num_inputs, num_targets=1, num_constants=0, workers=1, streams=1, via_plan=False,
                 num_kernels=8, asts_per_kernel=None):
        if not torch.cuda.is_available():
            raise RuntimeError("a CUDA device is required: this library has no CPU fallback")
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # make sure torch's primary context is current on this thread
        self.lib = abi.load()
        self.shape = shape
        self.num_inputs, self.num_targets, self.num_constants = num_inputs, num_targets, num_constants
        self.recipe = make_recipe(shape, num_inputs, num_targets, num_constants, num_kernels, asts_per_kernel)
        self.handle = C.c_void_p()
        options = abi.runner_options(workers, streams)
        if via_plan:
            # the reference sequence: source -> (caller compiles) -> plan -> runner
            size = C.c_size_t()
            abi.check(self.lib.secant_cubin_source_size(C.byref(self.recipe), C.byref(size)), "source_size")
            self._source = C.create_string_buffer(size.value)
            abi.check(self.lib.secant_cubin_source_write(C.byref(self.recipe), self._source, size.value), "source_write")
            self._cubin = C.create_string_buffer(self._source.raw, size.value)  # stands in for the compiled binary
            need = C.c_size_t()
            abi.check(self.lib.secant_cubin_plan_storage_size(C.byref(self.recipe), self._cubin, size.value, C.byref(need)),
                      "plan_storage_size")
            self._plan_storage = C.create_string_buffer(need.value)
            self._plan = C.c_void_p()
            abi.check(self.lib.secant_cubin_plan_init(C.byref(self.recipe), self._cubin, size.value, self._plan_storage,
                                                      need.value, C.byref(self._plan)), "plan_init")
            abi.check(self.lib.secant_cubin_runner_create(self._plan, self._cubin, size.value, C.byref(options),
                                                          C.byref(self.handle)), "runner_create")
        else:
            abi.check(self.lib.secant_b200_runner_create(C.byref(self.recipe), C.byref(options), C.byref(self.handle)),
                      "secant_b200_runner_create")
        self.stats = abi.runner_stats()

    # -- request builders -------------------------------------------------------
    def toggle_request(self, packed, x, y, banks, num_banks, toggle_bits, out, out_ld=None, bank_stride=None,
                       program_bank_stride=0, first_program_index=0):
        ext = abi.ToggleRunExt()
        run = ext.base
        abi.init_header(run, abi.RUN_VERSION, abi.SHAPE_TOGGLE_SSE)
        run.header.struct_size = C.sizeof(ext)
        packed.fill(run.programs)
        run.input = _matrix(x)
        run.targets = _matrix(y)
        if banks is not None and self.num_constants:
            run.constants.address = banks.data_ptr()
            run.constants.num_elements = banks.numel()
            run.constants.bank_stride = bank_stride if bank_stride is not None else banks.shape[-1]
        run.num_rows = y.shape[-1]
        run.num_targets = y.shape[0]
        run.num_banks = num_banks
        run.toggle_bits = toggle_bits
        run.output = _matrix(out, out_ld if out_ld is not None else out.shape[-1])
        ext.program_bank_stride = program_bank_stride
        ext.first_program_index = first_program_index
        return ext

    def static_request(self, packed, x, y, out, out_ld=None):
        run = abi.init_header(abi.StaticRun(), abi.RUN_VERSION, self.shape)
        packed.fill(run.programs)
        run.input = _matrix(x)
        run.targets = _matrix(y)
        run.num_rows = x.shape[-1]
        run.num_targets = y.shape[0]
        run.output = _matrix(out, out_ld if out_ld is not None else out.shape[-1])
        return run

    def materialize_request(self, packed, x, out, out_ld=None):
        run = abi.init_header(abi.MaterializeRun(), abi.RUN_VERSION, abi.SHAPE_MATERIALIZE)
        packed.fill(run.programs)
        run.input = _matrix(x)
        run.num_rows = x.shape[-1]
        run.output = _matrix(out, out_ld if out_ld is not None else out.shape[-1])
        return run

    # -- execution --------------------------------------------------------------
    def run(self, request, check=True):
        code = self.lib.secant_cubin_runner_run(self.handle, C.byref(request), C.byref(self.stats))
        if check:
            abi.check(code, "secant_cubin_runner_run: " + self.last_error())
        return code

    def run_batch(self, requests, check=True):
        ptrs = (C.c_void_p * len(requests))(*[C.addressof(r) for r in requests])
        code = self.lib.secant_cubin_runner_run_batch(self.handle, ptrs, len(requests), C.byref(self.stats))
        if check:
            abi.check(code, "secant_cubin_runner_run_batch: " + self.last_error())
        return code

    def last_error(self):
        return (self.lib.secant_b200_runner_last_error(self.handle) or b"").decode()

    # -- conveniences -------------------------------------------------------------
    def toggle_sse(self, packed, x, y, banks, num_banks, toggle_bits, **kw):
        configs = num_banks << toggle_bits
        out = torch.empty((len(packed.asts), y.shape[0], configs), dtype=torch.float32, device=y.device)
        self.run(self.toggle_request(packed, x, y, banks, num_banks, toggle_bits, out, **kw))
        return out

    def sse(self, packed, x, y):
        out = torch.empty((len(packed.asts), y.shape[0]), dtype=torch.float32, device=x.device)
        self.run(self.static_request(packed, x, y, out))
        return out

    def affine_stats(self, packed, x, y):
        out = torch.empty((len(packed.asts), 2 + y.shape[0]), dtype=torch.float32, device=x.device)
        self.run(self.static_request(packed, x, y, out))
        return out

    def gram_stats(self, packed, x, y):
        """[cohort][A sums | A x A Gram matrix | A x T cross sums], A = the recipe's programs per kernel."""
        cohort = self.recipe.asts_per_kernel
        cohorts = (len(packed.asts) + cohort - 1) // cohort
        out = torch.full((cohorts, cohort * (1 + cohort + y.shape[0])), float("nan"), dtype=torch.float32, device=x.device)
        self.run(self.static_request(packed, x, y, out))
        return out

    def materialize(self, packed, x):
        out = torch.empty((len(packed.asts), x.shape[-1]), dtype=torch.float32, device=x.device)
        self.run(self.materialize_request(packed, x, out))
        return out

    def set_math(self, fast):
        """fast=True selects the approximate division / transcendental functions of the reference's GPU kernels."""
        abi.check(self.lib.secant_b200_runner_set_math(self.handle, 1 if fast else 0), "secant_b200_runner_set_math")

    def set_scratch_limit(self, nbytes):
        """Caps the device scratch one launch may use for per-split partial sums (0 = default)."""
        abi.check(self.lib.secant_b200_runner_set_scratch_limit(self.handle, C.c_size_t(nbytes)), "set_scratch_limit")

    def population(self, packed, toggle_bits=0):
        return Population(self, packed, toggle_bits)

    def destroy(self):
        if self.handle:
            abi.check(self.lib.secant_cubin_runner_destroy(self.handle), "runner_destroy")
            self.handle = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.destroy()


class Population:
    """Programs validated, encoded and uploaded once; scored many times (extension API)."""

    def __init__(self, runner, packed, toggle_bits=0):
        self.runner = runner
        self.packed = packed
        self.handle = C.c_void_p()
        pset = abi.ProgramSet()
        packed.fill(pset)
        abi.check(runner.lib.secant_b200_population_create(runner.handle, C.byref(pset), toggle_bits, C.byref(self.handle)),
                  "secant_b200_population_create")
        self.num_ops = runner.lib.secant_b200_population_num_ops(self.handle)

    def run(self, request, check=True):
        code = self.runner.lib.secant_b200_population_run(self.handle, C.byref(request), C.byref(self.runner.stats))
        if check:
            abi.check(code, "secant_b200_population_run: " + self.runner.last_error())
        return code

    def destroy(self):
        if self.handle:
            abi.check(self.runner.lib.secant_b200_population_destroy(self.handle), "population_destroy")
            self.handle = C.c_void_p()


# ---- device-side reductions over score grids (extension API) -----------------------------

from .sharding import SCORE_BYTES, record_fields as score_fields  # noqa: E402,F401  (the record layout lives with the combine step)

assert SCORE_BYTES == C.sizeof(abi.Score)


def best_config(scores, out=None):
    """Best configuration of every vector of a [vectors][configurations] float32 CUDA tensor.
    Returns a uint8 tensor of SecantB200Score records (24 bytes each); score_fields() views it."""
    lib = abi.load()
    flat = scores.reshape(-1, scores.shape[-1])
    assert flat.is_cuda and flat.dtype == torch.float32 and flat.stride(-1) == 1
    if out is None:
        out = torch.empty(flat.shape[0] * SCORE_BYTES, dtype=torch.uint8, device=scores.device)
    stream = torch.cuda.current_stream().cuda_stream
    abi.check(lib.secant_b200_best_config(flat.data_ptr(), flat.shape[0], flat.shape[1], flat.stride(0), out.data_ptr(),
                                          C.c_void_p(stream)), "secant_b200_best_config")
    return out


def topk(scores, k):
    """Indices (int64, UINT64_MAX shows as -1) and values of the k best scores of a 1-D float32
    CUDA tensor under (valid first, score ascending, index ascending)."""
    lib = abi.load()
    scores = scores.contiguous()
    idx = torch.empty(k, dtype=torch.int64, device=scores.device)
    val = torch.empty(k, dtype=torch.float32, device=scores.device)
    stream = torch.cuda.current_stream().cuda_stream
    abi.check(lib.secant_b200_topk(scores.data_ptr(), scores.numel(), k, idx.data_ptr(), val.data_ptr(), C.c_void_p(stream)),
              "secant_b200_topk")
    return idx, val


def rk4_score(packed, num_states, reference, times, constants=None, num_constants=0, num_banks=1, toggle_bits=0,
              steps_per_observation=1, points_per_trajectory=None, offsets=None, allow_missing=False, sampled=None,
              integrated=None):
    """Fixed-step RK4 rollout scores [system][configuration] (extension API).

    packed: num_systems * num_states right-hand-side programs, system-major.
    Uniform form: reference is a CUDA tensor [state][trajectories * points], times a CUDA tensor
    [points].  Ragged form (offsets given: CUDA int32/uint32 tensor [trajectories + 1]): reference
    is [state][concatenated points], times is [concatenated points]; with allow_missing NaN
    reference values after a trajectory's first point are unobserved.
    constants: CUDA tensor [system][bank][slot] or None.
    sampled: (descriptors, uniform_pool, normal_pool) instead of constants - a CUDA uint8 tensor
    holding abi.SampledParameter[system][constant] and two CUDA float pools of equal size.
    integrated: optional CUDA int64 tensor of one element, incremented by the (trajectory, observation
    interval) pairs that were integrated (candidates that are already invalid are not integrated on)."""
    lib = abi.load()
    run = abi.Rk4Run()
    run.struct_size, run.version = C.sizeof(run), abi.RUN_VERSION
    packed.fill(run.programs)
    systems = len(packed.asts) // num_states
    run.num_systems, run.num_states, run.num_constants = systems, num_states, num_constants
    if constants is not None and num_constants:
        run.constants.address, run.constants.num_elements, run.constants.bank_stride = (
            constants.data_ptr(), constants.numel(), constants.shape[-1])
    run.num_banks, run.toggle_bits = num_banks, toggle_bits
    run.reference = _matrix(reference)
    if offsets is not None:
        run.trajectory_offsets = offsets.data_ptr()
        run.num_trajectories = offsets.numel() - 1
        run.total_points = times.numel()
        run.allow_missing_observations = 1 if allow_missing else 0
    else:
        points = points_per_trajectory or times.numel()
        run.num_trajectories = reference.shape[-1] // points
        run.points_per_trajectory = points
    if sampled is not None:
        descriptors, uniform_pool, normal_pool = sampled
        run.sampled_parameters = descriptors.data_ptr()
        run.uniform_pool, run.normal_pool = uniform_pool.data_ptr(), normal_pool.data_ptr()
        run.rng_pool_size = uniform_pool.numel()
    run.times = times.data_ptr()
    run.steps_per_observation = steps_per_observation
    if integrated is not None:
        run.integrated_intervals = integrated.data_ptr()
    out = torch.empty((systems, num_banks << toggle_bits), dtype=torch.float32, device=reference.device)
    run.output = _matrix(out)
    abi.check(lib.secant_b200_rk4_score(C.byref(run)), "secant_b200_rk4_score")
    return out


def grouped_topk(scores, num_systems, num_banks, toggle_bits, grouping, k):
    """Top-k per group of a contiguous [system][configuration] CUDA score grid (extension API).
    Returns (mse [group][k] float32, score_index [group][k] int64 with -1 for unfilled ranks,
    counts [group][3] int64 = valid, invalid, negative)."""
    lib = abi.load()
    perms = 1 << toggle_bits
    groups = num_systems if grouping == 0 else num_systems * perms if grouping == 1 else 1
    winners = torch.empty((groups, k, 2), dtype=torch.int64, device=scores.device)     # 16-byte records
    counts = torch.empty((groups, 3), dtype=torch.int64, device=scores.device)
    abi.check(lib.secant_b200_grouped_topk(scores.data_ptr(), num_systems, num_banks, toggle_bits, grouping, k,
                                           winners.data_ptr(), counts.data_ptr(), torch.cuda.current_stream().cuda_stream),
              "secant_b200_grouped_topk")
    mse = winners.view(torch.float32)[:, :, 0].clone()          # first 4 bytes of every 16-byte record
    return mse, winners[:, :, 1].clone(), counts
