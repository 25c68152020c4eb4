"""Shared helpers of the test-suite: library loaders and thin call wrappers.

Three native libraries are involved:
  * libsecant_b200.so            the product (C-ABI), via secant_b200.abi.load()
  * libsecant_b200_testhooks.so  host-only encoder/validator hooks for CPU tests
  * oracle/libsecant_oracle.so   the CPU restatement of the reference evaluator (checker)
and, only on a machine that holds the reference checkout and ran `make -C oracle ref`,
  * oracle/_ref/libsecant_ref.so the reference's own host evaluator, compiled unmodified.
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "gpu-program-specialization_b200")
if PKG not in sys.path:
    sys.path.insert(0, PKG)

from secant_b200 import abi, programs  # noqa: E402

F32P = C.POINTER(C.c_float)
F64P = C.POINTER(C.c_double)
U8P = C.POINTER(C.c_uint8)
U64P = C.POINTER(C.c_uint64)


def _build(target_dir, args):
    subprocess.run(["make", "-C", target_dir] + args, check=True, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE)


_oracle = None


def oracle():
    """The CPU restatement (oracle/secant_oracle.c), built on demand with gcc."""
    global _oracle
    if _oracle is None:
        path = os.path.join(ROOT, "oracle", "libsecant_oracle.so")
        if not os.path.exists(path):
            _build(os.path.join(ROOT, "oracle"), ["all"])
        _oracle = C.CDLL(path)
    return _oracle


_hooks = None


def hooks():
    global _hooks
    if _hooks is None:
        path = os.path.join(PKG, "libsecant_b200_testhooks.so")
        if not os.path.exists(path):
            _build(PKG, ["testhooks"])
        _hooks = C.CDLL(path)
    return _hooks


def reference_lib():
    """The reference's own evaluator, or None when it was not built on this machine."""
    path = os.path.join(ROOT, "oracle", "_ref", "libsecant_ref.so")
    return C.CDLL(path) if os.path.exists(path) else None


def fptr(a):
    return a.ctypes.data_as(F32P) if a is not None else None


def blob_args(packed):
    """(routine_blob, routine_off, n_routines, ast_blob, ast_off, n_asts) ctypes arguments."""
    rb = (C.c_uint8 * max(1, len(packed.routine_blob))).from_buffer_copy(packed.routine_blob or b"\0")
    ab = (C.c_uint8 * max(1, len(packed.ast_blob))).from_buffer_copy(packed.ast_blob or b"\0")
    return (rb, packed.routine_off.ctypes.data_as(U64P), C.c_size_t(len(packed.routines)), ab,
            packed.ast_off.ctypes.data_as(U64P), C.c_size_t(len(packed.asts)))


def oracle_materialize(packed, x):
    """x: [inputs][rows] float32 -> [asts][rows]."""
    F, N = x.shape
    out = np.zeros((len(packed.asts), N), dtype=np.float32)
    r = oracle().so_materialize(*blob_args(packed), C.c_size_t(F), fptr(x), C.c_size_t(N), C.c_size_t(N), fptr(out),
                                C.c_size_t(N))
    return r, out


def oracle_sse(packed, x, y, want64=True):
    """Static SSE [asts][targets] (accumulated from zero); returns (code, f32, f64)."""
    F, N = x.shape
    T = y.shape[0]
    out = np.zeros((len(packed.asts), T), dtype=np.float32)
    out64 = np.zeros((len(packed.asts), T), dtype=np.float64)
    r = oracle().so_sse(*blob_args(packed), C.c_size_t(F), C.c_size_t(T), fptr(x), C.c_size_t(N), fptr(y), C.c_size_t(N),
                        C.c_size_t(N), fptr(out), C.c_size_t(T), out64.ctypes.data_as(F64P) if want64 else None)
    return r, out, out64


def oracle_gram_stats(packed, x, y, cohort):
    """Gram statistics [cohorts][A + A*A + A*T] of programs in consecutive cohorts of `cohort`
    (accumulated from zero); returns (code, f32, f64)."""
    F, N = x.shape
    T = y.shape[0]
    cohorts = (len(packed.asts) + cohort - 1) // cohort
    width = cohort * (1 + cohort + T)
    out = np.zeros((cohorts, width), dtype=np.float32)
    out64 = np.zeros((cohorts, width), dtype=np.float64)
    r = oracle().so_gram_stats(*blob_args(packed), C.c_size_t(cohort), C.c_size_t(F), C.c_size_t(T), fptr(x), C.c_size_t(N), fptr(y),
                               C.c_size_t(N), C.c_size_t(N), fptr(out), C.c_size_t(width), out64.ctypes.data_as(F64P))
    return r, out, out64


def reference_gram_stats(lib, packed, x, y, cohort):
    """The same through the reference's own host evaluator (secant_cpu_run, Gram-statistics shape)."""
    from secant_b200 import abi
    F, N = x.shape
    T = y.shape[0]
    cohorts = (len(packed.asts) + cohort - 1) // cohort
    width = cohort * (1 + cohort + T)
    out = np.zeros((cohorts, width), dtype=np.float32)
    run = abi.init_header(abi.CpuGramRun(), abi.CPU_RUN_VERSION, abi.SHAPE_GRAM_STATS)
    packed.fill(run.programs)
    run.asts_per_cohort, run.num_inputs, run.num_targets, run.num_rows = cohort, F, T, N
    run.input, run.targets, run.statistics = host_matrix(x, N), host_matrix(y, N), host_matrix(out, width)
    return lib.secant_cpu_run(C.byref(run)), out


def oracle_toggle_sse(packed, x, y, banks, num_constants, toggle_bits, bank_stride=None, program_bank_stride=0,
                      out=None, out_ld=None):
    """Toggle SSE [asts][targets][configs]; banks: [banks][stride] (or per program)."""
    F, N = (x.shape if x is not None and x.size else (0, y.shape[1]))
    T = y.shape[0]
    A = len(packed.asts)
    if program_bank_stride:
        nb = banks.shape[1]
    else:
        nb = banks.shape[0] if banks is not None else 1
    if bank_stride is None:
        bank_stride = banks.shape[-1] if (banks is not None and num_constants) else 0
    configs = nb << toggle_bits
    if out_ld is None:
        out_ld = configs
    if out is None:
        out = np.zeros((A, T, out_ld), dtype=np.float32)
    out64 = np.zeros((A, T, out_ld), dtype=np.float64)
    nconst_elems = banks.size if banks is not None else 0
    r = oracle().so_toggle_sse(*blob_args(packed), C.c_size_t(F), C.c_size_t(num_constants), fptr(x) if F else None,
                               C.c_size_t(x.size if F else 0), C.c_size_t(N), fptr(y), C.c_size_t(y.size), C.c_size_t(N),
                               fptr(banks) if nconst_elems else None, C.c_size_t(nconst_elems), C.c_size_t(bank_stride),
                               C.c_size_t(program_bank_stride), C.c_size_t(N), C.c_size_t(T), C.c_size_t(nb),
                               C.c_uint32(toggle_bits), fptr(out), C.c_size_t(out.size), C.c_size_t(out_ld),
                               out64.ctypes.data_as(F64P))
    return r, out, out64


def oracle_toggle_materialize(packed, x, banks, num_constants, toggle_bits, configuration, program_bank_stride=0):
    F, N = x.shape
    out = np.zeros((len(packed.asts), N), dtype=np.float32)
    stride = banks.shape[-1] if (banks is not None and num_constants) else 0
    r = oracle().so_toggle_materialize(*blob_args(packed), C.c_size_t(F), C.c_size_t(num_constants), fptr(x), C.c_size_t(N),
                                       fptr(banks) if banks is not None else None, C.c_size_t(stride),
                                       C.c_size_t(program_bank_stride), C.c_uint32(toggle_bits), C.c_size_t(configuration),
                                       C.c_size_t(N), fptr(out), C.c_size_t(N))
    return r, out


# ---- the reference's own evaluator through its public structs (only where built) ----

def host_matrix(a, ld):
    m = abi.HostMatrix()
    m.data = fptr(a)
    m.num_elements = a.size
    m.leading_dimension = ld
    return m


def reference_toggle_sse(lib, packed, x, y, banks, num_constants, toggle_bits, out_ld=None):
    run = abi.init_header(abi.CpuToggleRun(), abi.CPU_RUN_VERSION, abi.SHAPE_TOGGLE_SSE)
    packed.fill(run.programs)
    F, N = x.shape
    T = y.shape[0]
    nb = banks.shape[0] if banks is not None else 1
    configs = nb << toggle_bits
    out_ld = out_ld or configs
    out = np.zeros((len(packed.asts), T, out_ld), dtype=np.float32)
    run.num_inputs = F
    run.num_constants = num_constants
    run.input = host_matrix(x, N)
    run.targets = host_matrix(y, N)
    if banks is not None and num_constants:
        run.constants.data = fptr(banks)
        run.constants.num_elements = banks.size
        run.constants.bank_stride = banks.shape[1]
    run.num_rows = N
    run.num_targets = T
    run.num_banks = nb
    run.toggle_bits = toggle_bits
    run.output = host_matrix(out, out_ld)
    lib.secant_cpu_run.restype = C.c_int32
    code = lib.secant_cpu_run(C.byref(run))
    return code, out


def reference_materialize(lib, packed, x):
    run = abi.init_header(abi.CpuMaterializeRun(), abi.CPU_RUN_VERSION, abi.SHAPE_MATERIALIZE)
    packed.fill(run.programs)
    F, N = x.shape
    out = np.zeros((len(packed.asts), N), dtype=np.float32)
    run.num_inputs = F
    run.input = host_matrix(x, N)
    run.num_rows = N
    run.output = host_matrix(out, N)
    lib.secant_cpu_run.restype = C.c_int32
    code = lib.secant_cpu_run(C.byref(run))
    return code, out


def reference_sse(lib, packed, x, y):
    run = abi.init_header(abi.CpuStaticRun(), abi.CPU_RUN_VERSION, abi.SHAPE_SSE)
    packed.fill(run.programs)
    F, N = x.shape
    T = y.shape[0]
    out = np.zeros((len(packed.asts), T), dtype=np.float32)
    run.num_inputs = F
    run.num_targets = T
    run.input = host_matrix(x, N)
    run.targets = host_matrix(y, N)
    run.num_rows = N
    run.output = host_matrix(out, T)
    lib.secant_cpu_run.restype = C.c_int32
    code = lib.secant_cpu_run(C.byref(run))
    return code, out


def row_sensitivity(packed, x, banks, num_constants, toggle_bits, configuration, program_bank_stride=0, ulps=2):
    """Per-row values of one configuration plus how far they move when every transcendental
    result is shifted by +-`ulps` units in the last place: (values, sensitivity), [asts][rows].
    Rows whose finiteness changes under the shift get an infinite sensitivity."""
    lib = oracle()
    code, base = oracle_toggle_materialize(packed, x, banks, num_constants, toggle_bits, configuration, program_bank_stride)
    assert code == 0, code
    sens = np.zeros(base.shape, dtype=np.float64)
    try:
        for shift in (ulps, -ulps):
            lib.so_set_ulp_shift(shift)
            _, moved = oracle_toggle_materialize(packed, x, banks, num_constants, toggle_bits, configuration, program_bank_stride)
            with np.errstate(invalid="ignore", over="ignore"):
                d = np.abs(moved.astype(np.float64) - base.astype(np.float64))
            unstable = np.isfinite(moved) != np.isfinite(base)
            d[unstable] = np.inf
            d[~np.isfinite(base) & ~unstable] = 0.0
            sens = np.maximum(sens, d)
    finally:
        lib.so_set_ulp_shift(0)
    return base, sens


def sse_slack(packed, x, y, banks, num_constants, toggle_bits, program_bank_stride=0, out_ld=None, ulps=2):
    """Allowed deviation of each SSE bin caused by transcendental results that differ by up to
    `ulps` units in the last place: sum over rows of 2*|err|*s + s*s, s = row sensitivity."""
    T, N = y.shape
    if program_bank_stride:
        nb = banks.shape[1]
    else:
        nb = banks.shape[0] if (banks is not None and num_constants) else 1
    configs = nb << toggle_bits
    out_ld = out_ld or configs
    slack = np.zeros((len(packed.asts), T, out_ld), dtype=np.float64)
    xx = x if (x is not None and x.size) else np.zeros((1, N), dtype=np.float32)
    for cfg in range(configs):
        base, sens = row_sensitivity(packed, xx, banks, num_constants, toggle_bits, cfg, program_bank_stride, ulps)
        for t in range(T):
            with np.errstate(invalid="ignore", over="ignore"):
                err = np.abs(base.astype(np.float64) - y[t].astype(np.float64)[None, :])
                term = 2.0 * err * sens + sens * sens
            term[np.isnan(term)] = np.inf
            term[sens == 0] = 0.0
            slack[:, t, cfg] = term.sum(axis=1)
    return slack


def oracle_rk4(packed, num_states, reference, num_trajectories, times, constants=None, substeps=1, toggle_bits=0,
               permutation=0, want64=False, offsets=None, allow_missing=False):
    """RK4 rollout scores of the CPU restatement, one per system (single bank per system).
    With offsets (uint32[num_trajectories + 1]) the ragged form: times and reference are per
    concatenated point."""
    systems = len(packed.asts) // num_states
    K = constants.shape[1] if constants is not None else 0
    scores = np.zeros(systems, dtype=np.float32)
    scores64 = np.zeros(systems, dtype=np.float64)
    if offsets is not None:
        offsets = np.ascontiguousarray(offsets, dtype=np.uint32)
        code = oracle().so_rk4_score_ragged(*blob_args(packed)[:5], C.c_size_t(systems), C.c_size_t(num_states), C.c_size_t(K),
                                            fptr(constants) if K else None, C.c_size_t(K), fptr(reference),
                                            C.c_size_t(len(offsets) - 1), offsets.ctypes.data_as(C.POINTER(C.c_uint32)),
                                            C.c_size_t(len(times)), C.c_int(1 if allow_missing else 0), fptr(times),
                                            C.c_size_t(substeps), C.c_uint32(toggle_bits), C.c_uint32(permutation),
                                            fptr(scores), scores64.ctypes.data_as(F64P))
        return (code, scores, scores64) if want64 else (code, scores)
    code = oracle().so_rk4_score(*blob_args(packed)[:5], C.c_size_t(systems), C.c_size_t(num_states), C.c_size_t(K),
                                 fptr(constants) if K else None, C.c_size_t(K), fptr(reference), C.c_size_t(num_trajectories),
                                 C.c_size_t(len(times)), fptr(times), C.c_size_t(substeps), C.c_uint32(toggle_bits),
                                 C.c_uint32(permutation), fptr(scores), scores64.ctypes.data_as(F64P))
    if want64:
        return code, scores, scores64
    return code, scores


def sampled_constants(descriptors, uniform_pool, normal_pool, num_banks):
    """Explicit [system][bank][constant] table of sampled coefficients: the rule of the reference
    engine (projects/odezza/core/o_sampled_constants_source.h:32-44) restated in float32 numpy.
    descriptors: [system][constant] tuples (offset, stride, distribution, scale, shift, lower, upper)."""
    systems, K = len(descriptors), len(descriptors[0])
    out = np.zeros((systems, num_banks, K), dtype=np.float32)
    size = len(uniform_pool)
    for i in range(systems):
        for k in range(K):
            offset, stride, dist, scale, shift, lower, upper = descriptors[i][k]
            for b in range(num_banks):
                if dist == 0:
                    out[i, b, k] = np.float32(shift)
                    continue
                delta = b * stride
                pool = uniform_pool if dist == 1 else normal_pool if dist == 2 else None
                if offset >= size or delta >= size - offset or pool is None:
                    out[i, b, k] = np.nan
                    continue
                v = np.float32(np.float32(pool[offset + delta]) * np.float32(scale)) + np.float32(shift)
                out[i, b, k] = min(np.float32(upper), max(np.float32(lower), np.float32(v)))
    return out


def sse_reference_parallel(packed, x, y, banks, num_constants, toggle_bits, program_bank_stride=0, threads=None, ulps=2):
    """(want64, slack) of a toggle-SSE run like oracle_toggle_sse() and sse_slack(), with the programs
    spread over host threads (the checker is a single-threaded C loop that releases the GIL).
    The shift of the math results is one global of the checker library, so the three passes
    (plain, +ulps, -ulps) run one after the other, each on all threads."""
    from concurrent.futures import ThreadPoolExecutor
    lib = oracle()
    A = len(packed.asts)
    T, N = y.shape
    threads = threads or min(A, os.cpu_count() or 1)
    bounds = np.linspace(0, A, threads + 1).astype(int)
    spans = [(int(a), int(b)) for a, b in zip(bounds[:-1], bounds[1:]) if b > a]
    subs = [packed.subset(range(a, b)) for a, b in spans]
    tables = [banks[a:b] if program_bank_stride else banks for a, b in spans]
    if program_bank_stride:
        nb = banks.shape[1]
    else:
        nb = banks.shape[0] if (banks is not None and num_constants) else 1
    configs = nb << toggle_bits
    xx = x if (x is not None and x.size) else np.zeros((1, N), dtype=np.float32)

    def rows_of(i):
        out = np.empty((spans[i][1] - spans[i][0], configs, N), dtype=np.float32)
        for cfg in range(configs):
            code, vals = oracle_toggle_materialize(subs[i], xx, tables[i], num_constants, toggle_bits, cfg, program_bank_stride)
            assert code == 0, code
            out[:, cfg, :] = vals
        return out

    def run_pass(shift):
        lib.so_set_ulp_shift(shift)
        try:
            with ThreadPoolExecutor(max_workers=len(spans)) as pool:
                return list(pool.map(rows_of, range(len(spans))))
        finally:
            lib.so_set_ulp_shift(0)

    base = np.concatenate(run_pass(0))                      # [program][configuration][row]
    sens = np.zeros(base.shape, dtype=np.float64)
    for shift in (ulps, -ulps):
        moved = np.concatenate(run_pass(shift))
        with np.errstate(invalid="ignore", over="ignore"):
            d = np.abs(moved.astype(np.float64) - base.astype(np.float64))
        unstable = np.isfinite(moved) != np.isfinite(base)
        d[unstable] = np.inf
        d[~np.isfinite(base) & ~unstable] = 0.0
        np.maximum(sens, d, out=sens)
    want64 = np.zeros((A, T, configs), dtype=np.float64)
    slack = np.zeros((A, T, configs), dtype=np.float64)
    for t in range(T):
        with np.errstate(invalid="ignore", over="ignore"):
            err = (base - y[t][None, None, :]).astype(np.float64)   # the residual is a float32 subtraction, as in the evaluators
            want64[:, t, :] = (err * err).sum(axis=2)
            term = 2.0 * np.abs(err) * sens + sens * sens
        term[np.isnan(term)] = np.inf
        term[sens == 0] = 0.0
        slack[:, t, :] = term.sum(axis=2)
    return want64, slack
