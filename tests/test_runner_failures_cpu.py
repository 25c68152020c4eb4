"""Failure paths of the runner without a GPU: the production host pipeline (csrc/runner.cpp),
compiled against a deterministic model of the CUDA runtime (tests/fake_cuda), with every runtime
call, allocation site and worker-thread start failed once in create, run and destroy, and the
compound cases of the reference's own suite: completion unknown makes a handle destroy-only, a
failed construction with failed clean-up returns an owned destroy-only handle, a bad program
leaves the handle usable, wrong context, run and destroy during a run
(projects/secant/tests/runner_failure_test.c:414-575, tests/support/fake_cuda/cuda.h:27-63).
The model also checks stream order: no launch before the upload of its records, no buffer
overwritten or freed while a launch may still use it.
"""
import ctypes as C
import os
import subprocess
import threading
import time

import numpy as np
import pytest

import support as S
from secant_b200 import abi, programs as P
from secant_b200.runner import make_recipe

PKG = S.PKG
_lib = None


def fake():
    global _lib
    if _lib is None:
        path = os.path.join(PKG, "libsecant_b200_fakecuda.so")
        subprocess.run(["make", "-C", PKG, "fakecuda"], check=True, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE)
        lib = C.CDLL(path)
        for name in ("secant_cubin_runner_create", "secant_cubin_runner_run_batch", "secant_cubin_runner_run",
                     "secant_cubin_runner_destroy", "secant_b200_runner_create", "secant_cubin_plan_storage_size",
                     "secant_cubin_plan_init", "secant_cubin_source_size", "secant_cubin_source_write",
                     "secant_b200_population_create", "secant_b200_population_run", "secant_b200_population_destroy"):
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = abi.EXPORTED[name]
        lib.fake_arm.argtypes = [C.c_char_p, C.c_uint, C.c_int]
        lib.fake_calls.argtypes = [C.c_char_p]
        lib.fake_calls.restype = C.c_uint
        lib.fake_call_names.argtypes = [C.c_char_p, C.c_size_t]
        lib.fake_call_names.restype = C.c_size_t
        lib.fake_device_buffer.argtypes = [C.c_size_t]
        lib.fake_device_buffer.restype = C.c_void_p
        lib.fake_device_release.argtypes = [C.c_void_p]
        lib.fake_last_violation.restype = C.c_char_p
        _lib = lib
    return _lib


def state(lib):
    out = (C.c_uint * 6)()
    lib.fake_state(out)
    return dict(zip(("allocations", "streams", "events", "violations", "launches", "threads"), list(out)))


def call_names(lib):
    buf = C.create_string_buffer(4096)
    lib.fake_call_names(buf, 4096)
    return [n for n in buf.value.decode().split("\n") if n]


class Harness:
    """A toggle-SSE request over buffers of the model's device memory."""
    ROWS, BANKS, BITS, K, F = 300, 5, 2, 4, 3

    def __init__(self, lib, programs=6000):
        self.lib = lib
        self.pop = P.random_population(11, programs, 16, self.F, self.K, 1.0, toggle_bits=self.BITS, ops=P.ARITHMETIC_OPS)
        self.recipe = make_recipe(abi.SHAPE_TOGGLE_SSE, self.F, 1, self.K)
        configs = self.BANKS << self.BITS
        self.sizes = dict(x=self.F * self.ROWS, y=self.ROWS, banks=self.BANKS * self.K, out=programs * configs)
        self.buffers = {k: lib.fake_device_buffer(4 * n) for k, n in self.sizes.items()}
        run = abi.init_header(abi.ToggleRun(), abi.RUN_VERSION, abi.SHAPE_TOGGLE_SSE)
        self.pop.fill(run.programs)
        for field, key, ld in (("input", "x", self.ROWS), ("targets", "y", self.ROWS), ("output", "out", configs)):
            m = getattr(run, field)
            m.address, m.num_elements, m.leading_dimension = self.buffers[key], self.sizes[key], ld
        run.constants.address, run.constants.num_elements, run.constants.bank_stride = self.buffers["banks"], self.sizes["banks"], self.K
        run.num_rows, run.num_targets, run.num_banks, run.toggle_bits = self.ROWS, 1, self.BANKS, self.BITS
        self.run = run
        self.stats = abi.runner_stats()

    def release(self):
        for p in self.buffers.values():
            self.lib.fake_device_release(p)

    def create(self, workers=3, streams=2):
        handle = C.c_void_p()
        options = abi.runner_options(workers, streams)
        code = self.lib.secant_b200_runner_create(C.byref(self.recipe), C.byref(options), C.byref(handle))
        return code, handle

    def execute(self, handle):
        return self.lib.secant_cubin_runner_run(handle, C.byref(self.run), C.byref(self.stats))


@pytest.fixture()
def world():
    lib = fake()
    lib.fake_reset()
    before = state(lib)
    h = Harness(lib)
    yield lib, h
    h.release()
    lib.fake_reset()
    after = state(lib)
    assert after["allocations"] == before["allocations"], "device or pinned memory left behind"
    assert after["streams"] == before["streams"] and after["events"] == before["events"]


def expected(name):
    if name == "alloc":
        return abi.ERROR_ALLOCATION_FAILED
    if name == "thread":
        return abi.ERROR_THREAD_FAILED
    if name == "cuCtxGetCurrent":
        return abi.ERROR_INVALID_STATE
    if name == "encode":
        return abi.ERROR_BAD_PROGRAM
    if name == "cudaMalloc:scratch":
        return abi.ERROR_ALLOCATION_FAILED
    return abi.ERROR_DRIVER_FAILED


def test_a_healthy_runner_orders_its_work(world):
    lib, h = world
    code, r = h.create()
    assert code == 0
    for _ in range(3):
        assert h.execute(r) == 0
        s = state(lib)
        assert s["violations"] == 0, lib.fake_last_violation()
    assert s["launches"] >= 6 and s["threads"] == 3          # two program batches per run
    assert h.stats.num_asts == 6000 and h.stats.modules_loaded == h.stats.num_modules > 0
    assert lib.secant_cubin_runner_destroy(r) == 0
    assert state(lib)["violations"] == 0, lib.fake_last_violation()


@pytest.mark.parametrize("phase", ["create", "run", "destroy"])
def test_every_call_fails_once(world, phase):
    """Independently fails every operation a successful create / run / destroy reaches."""
    lib, h = world
    # which calls, and how often, does the healthy phase make
    lib.fake_reset()
    r = None
    if phase != "create":
        code, r = h.create()
        assert code == 0
    if phase == "destroy":
        assert h.execute(r) == 0
    lib.fake_reset()
    if phase == "create":
        code, r = h.create()
        assert code == 0
    elif phase == "run":
        assert h.execute(r) == 0
    else:
        assert lib.secant_cubin_runner_destroy(r) == 0
        r = None
    counts = {n: lib.fake_calls(n.encode()) for n in call_names(lib)}
    if r:
        assert lib.secant_cubin_runner_destroy(r) == 0
    assert counts, "the phase made no call the model saw"
    tried = 0
    for name, calls in counts.items():
        for n in range(1, calls + 1):
            lib.fake_reset()
            r = None
            if phase != "create":
                code, r = h.create()
                assert code == 0
            if phase == "destroy":
                assert h.execute(r) == 0
            lib.fake_reset()
            lib.fake_arm(name.encode(), n, 0)
            tried += 1
            if phase == "create":
                handle = C.c_void_p()
                code, handle = h.create()
                assert code != 0, (name, n)
                assert code == expected(name), (name, n, abi.result_name(code))
                r = handle if handle.value else None      # a handle is only returned when clean-up failed as well
                assert r is None, (name, n)
            elif phase == "run":
                code = h.execute(r)
                assert code != 0, (name, n)
                lib.fake_reset()
                again = h.execute(r)
                if code == abi.ERROR_COMPLETION_UNKNOWN:
                    assert again == abi.ERROR_INVALID_STATE, (name, n)           # destroy-only handle
                else:
                    allowed = (expected(name), abi.ERROR_ALLOCATION_FAILED) if name == "cudaMalloc" else (expected(name),)
                    assert code in allowed, (name, n, abi.result_name(code))
                    assert again == 0, (name, n, abi.result_name(again))        # the handle recovers
            else:
                code = lib.secant_cubin_runner_destroy(r)
                assert code != 0, (name, n)
                assert code in (expected(name), abi.ERROR_COMPLETION_UNKNOWN), (name, n, abi.result_name(code))
                lib.fake_reset()
                if name == "cuCtxGetCurrent":       # refused before anything was shut down
                    assert h.execute(r) == 0, (name, n)
                else:                               # shut down, never reusable
                    assert h.execute(r) == abi.ERROR_INVALID_STATE, (name, n)
            assert state(lib)["violations"] == 0, (name, n, lib.fake_last_violation())
            lib.fake_reset()
            if r:
                assert lib.secant_cubin_runner_destroy(r) == 0, (name, n)
    assert tried >= 10


def test_completion_unknown_makes_the_handle_destroy_only(world):
    """A wait that reports an error leaves device work in an unknown state: the call answers
    COMPLETION_UNKNOWN, later runs are refused, destroy keeps failing while the streams cannot be
    drained and succeeds once they can (projects/secant/secant.h:1142-1159)."""
    lib, h = world
    code, r = h.create()
    assert code == 0
    lib.fake_arm(b"cudaEventSynchronize", 1, 1)
    assert h.execute(r) == abi.ERROR_COMPLETION_UNKNOWN
    assert h.execute(r) == abi.ERROR_INVALID_STATE
    lib.fake_arm(b"cudaStreamSynchronize", 1, 1)
    assert lib.secant_cubin_runner_destroy(r) == abi.ERROR_COMPLETION_UNKNOWN
    live = state(lib)
    assert live["streams"] and live["allocations"] > 4            # nothing was released under running work
    lib.fake_reset()
    assert lib.secant_cubin_runner_destroy(r) == 0
    assert state(lib)["violations"] == 0, lib.fake_last_violation()


def test_failed_construction_with_failed_cleanup_returns_an_owned_handle(world):
    lib, h = world
    lib.fake_arm(b"cudaEventCreate", 2, 0)
    lib.fake_arm(b"cudaStreamSynchronize", 1, 0)
    code, r = h.create()
    assert code == abi.ERROR_DRIVER_FAILED and r.value
    assert h.execute(r) == abi.ERROR_INVALID_STATE
    lib.fake_reset()
    assert lib.secant_cubin_runner_destroy(r) == 0


def test_bad_program_found_while_encoding_leaves_the_handle_usable(world):
    lib, h = world
    code, r = h.create()
    assert code == 0
    lib.fake_arm(b"encode", 2, 0)
    assert h.execute(r) == abi.ERROR_BAD_PROGRAM
    assert h.execute(r) == 0
    # a preflight failure touches nothing and reports zero counters
    bad = P.PackedPrograms([P.col(9) + P.RET])
    bad.fill(h.run.programs)
    launches = state(lib)["launches"]
    assert h.execute(r) == abi.ERROR_BAD_PROGRAM
    assert state(lib)["launches"] == launches and h.stats.num_modules == 0 and h.stats.total_seconds == 0
    h.pop.fill(h.run.programs)
    assert h.execute(r) == 0
    assert lib.secant_cubin_runner_destroy(r) == 0
    assert state(lib)["violations"] == 0, lib.fake_last_violation()


def test_wrong_context_is_refused_for_run_and_destroy(world):
    lib, h = world
    code, r = h.create()
    assert code == 0
    lib.fake_set_context(2)
    assert h.execute(r) == abi.ERROR_INVALID_STATE
    assert lib.secant_cubin_runner_destroy(r) == abi.ERROR_INVALID_STATE
    lib.fake_set_context(0)
    assert h.execute(r) == abi.ERROR_INVALID_STATE
    lib.fake_set_context(1)
    assert h.execute(r) == 0
    assert lib.secant_cubin_runner_destroy(r) == 0
    lib.fake_set_context(0)
    code, none = h.create()
    assert code == abi.ERROR_INVALID_STATE and not none.value
    lib.fake_set_context(1)


def test_run_and_destroy_during_a_run_are_refused(world):
    lib, h = world
    code, r = h.create(workers=1)
    assert code == 0
    results = []
    lib.fake_hold_encoding(1)                              # the worker parks inside the first batch
    t = threading.Thread(target=lambda: results.append(h.execute(r)))
    t.start()
    deadline = time.time() + 20
    while not lib.fake_encoding_entered() and time.time() < deadline:
        time.sleep(0.001)
    try:
        assert lib.fake_encoding_entered()
        assert lib.secant_cubin_runner_run(r, C.byref(h.run), None) == abi.ERROR_INVALID_STATE
        assert lib.secant_cubin_runner_destroy(r) == abi.ERROR_INVALID_STATE
    finally:
        lib.fake_hold_encoding(0)
        t.join()
    assert results == [0]
    assert h.execute(r) == 0
    assert lib.secant_cubin_runner_destroy(r) == 0


def test_a_population_keeps_its_runner_alive(world):
    lib, h = world
    code, r = h.create()
    assert code == 0
    pop = C.c_void_p()
    assert lib.secant_b200_population_create(r, C.byref(h.run.programs), h.BITS, C.byref(pop)) == 0
    assert lib.secant_b200_population_run(pop, C.byref(h.run), C.byref(h.stats)) == 0
    assert lib.secant_cubin_runner_destroy(r) == abi.ERROR_INVALID_STATE      # the population points at the runner
    assert lib.secant_b200_population_destroy(pop) == 0
    assert lib.secant_cubin_runner_destroy(r) == 0
    assert state(lib)["violations"] == 0, lib.fake_last_violation()
