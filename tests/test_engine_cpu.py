"""The ODE engine interface (include/odezza_b200.h) as far as it runs without a GPU: exported symbols,
the host-side Philox replay, descriptor validation, reduction layout arithmetic, and the scoring
handle's creation and launch validation, which answer before any CUDA call is made.  Expected
codes are the reference's (projects/odezza/core/o_scoring_pipeline.c:477-523 and 1541-1594,
o_philox.c:44-71, o_score_reduce.c:62-116; its own tests tests/o_scoring_cuda_test.c:188-205,
tests/o_score_reduce_test.c:118-124, tests/o_philox_test.c:101-104)."""
import ctypes as C
import os
import re
import struct

import numpy as np

from secant_b200 import engine as E

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
M32 = 0xFFFFFFFF


def test_library_exports_every_engine_symbol():
    lib = E.load()
    text = open(os.path.join(ROOT, "include", "odezza_b200.h")).read()
    declared = set(re.findall(r"ODEZZA_DEC\s+[\w\s\*]+?\b(o\w+)\s*\(", text))
    assert len(declared) == 21
    for name in declared:
        assert hasattr(lib, name), name
    assert declared == set(E.EXPORTED)


def philox4x32(counter, key):
    """Philox4x32-10 restated (Salmon, Moraes, Dror, Shaw: Parallel random numbers: as easy as 1, 2, 3, SC'11)."""
    c, k = list(counter), list(key)
    for _ in range(10):
        p0, p1 = 0xD2511F53 * c[0], 0xCD9E8D57 * c[2]
        c = [(p1 >> 32) ^ c[1] ^ k[0], p1 & M32, (p0 >> 32) ^ c[3] ^ k[1], p0 & M32]
        k = [(k[0] + 0x9E3779B9) & M32, (k[1] + 0xBB67AE85) & M32]
    return c


def uniform_sample(seed, stream, sample):
    words = philox4x32([(sample // 4) & M32, (sample // 4) >> 32, (stream << 1) & M32, (stream << 1) >> 32], [seed & M32, seed >> 32])
    return np.float32((np.float32(words[sample % 4] >> 9) + np.float32(0.5)) * np.float32(2.0 ** -23))


def lib_philox(counter, key):
    out = (C.c_uint32 * 4)()
    assert E.load().odezza_philox4x32((C.c_uint32 * 4)(*counter), (C.c_uint32 * 2)(*key), out) == 0
    return list(out)


def test_philox_known_answers_and_uniform_replay():
    # the generator's published known-answer vectors; the first is the one the reference test holds
    # (projects/odezza/tests/o_philox_test.c:101-104)
    vectors = [([0, 0, 0, 0], [0, 0], [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]),
               ([M32] * 4, [M32] * 2, [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]),
               ([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0],
                [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1])]
    for counter, key, want in vectors:
        assert philox4x32(counter, key) == want
        assert lib_philox(counter, key) == want
    rng = np.random.default_rng(5)
    for _ in range(200):
        counter, key = [int(v) for v in rng.integers(0, 1 << 32, 4)], [int(v) for v in rng.integers(0, 1 << 32, 2)]
        assert lib_philox(counter, key) == philox4x32(counter, key)
    lib = E.load()
    assert lib.odezza_philox4x32(None, (C.c_uint32 * 2)(), (C.c_uint32 * 4)()) == E.ERROR_INVALID_ARGUMENT
    out = C.c_float()
    for seed, stream, sample in [(20260906, 37, 7), (0, 0, 0), ((1 << 64) - 1, (1 << 63) - 1, (1 << 64) - 1), (12345, 2, (1 << 34) + 3)]:
        assert lib.odezza_rng_uniform(seed, stream, sample, C.byref(out)) == 0
        assert np.float32(out.value) == uniform_sample(seed, stream, sample)
        assert 0.0 < out.value < 1.0
    assert lib.odezza_rng_uniform(1, 1 << 63, 0, C.byref(out)) == E.ERROR_INVALID_ARGUMENT      # the stream is doubled into the counter
    assert lib.odezza_rng_uniform(1, 1, 0, None) == E.ERROR_INVALID_ARGUMENT


def test_sampled_parameter_validation():
    lib = E.load()
    pool = E.RngPoolInfo(1, 2, 0, 1000, 3)

    def code(p, banks=10, info=pool):
        return lib.odezza_sampled_parameter_validate(C.byref(info) if info else None, banks, C.byref(p) if p else None)
    ok = E.SampledParameter(10, 3, 1, 2.0, -0.5, -0.5, 4.0)
    assert code(ok) == 0
    assert code(E.SampledParameter(0, 0, 0, 0, 0.1, 0.1, 0.1)) == 0                       # a fixed value inside its bounds
    assert code(E.SampledParameter(0, 0, 0, 0, 0.2, 0.1, 0.1)) == E.ERROR_INVALID_ARGUMENT
    assert code(E.SampledParameter(10, 3, 3, 1, 0, 0, 1)) == E.ERROR_INVALID_ARGUMENT      # no such distribution
    assert code(E.SampledParameter(10, 0, 1, 1, 0, 0, 1)) == E.ERROR_INVALID_ARGUMENT      # zero stride
    assert code(E.SampledParameter(1000, 1, 1, 1, 0, 0, 1)) == E.ERROR_INVALID_ARGUMENT    # offset outside the pool
    assert code(E.SampledParameter(973, 3, 1, 1, 0, 0, 1)) == E.ERROR_INVALID_ARGUMENT     # bank 9 at 1000
    assert code(E.SampledParameter(972, 3, 1, 1, 0, 0, 1)) == 0                            # bank 9 at 999
    assert code(E.SampledParameter(10, 3, 1, float("inf"), 0, 0, 1)) == E.ERROR_INVALID_ARGUMENT
    assert code(E.SampledParameter(10, 3, 1, 1, 0, 2, 1)) == E.ERROR_INVALID_ARGUMENT      # lower above upper
    assert code(E.SampledParameter(10, 3, 2, 1, 0, 0, 1), info=E.RngPoolInfo(1, 2, 0, 1000, 1)) == E.ERROR_INVALID_ARGUMENT
    assert code(ok, banks=0) == E.ERROR_INVALID_ARGUMENT
    assert code(None) == E.ERROR_INVALID_ARGUMENT and code(ok, info=None) == E.ERROR_INVALID_ARGUMENT
    assert code(ok, info=E.RngPoolInfo(1, 2, 0, 0, 3)) == E.ERROR_INVALID_ARGUMENT


def requirements(banks, bits, systems, grouping, k):
    launch = E.Launch()
    launch.constant_bank_count, launch.active_toggle_count = banks, bits
    size = E.ReductionSize()
    return E.load().odezza_score_reduction_requirements(C.byref(launch), systems, grouping, k, C.byref(size)), size


def test_reduction_layout_and_index_decoding():
    lib = E.load()
    launch = E.Launch()
    launch.constant_bank_count, launch.active_toggle_count = 3, 32
    index = E.ScoreIndex()
    assert lib.odezza_score_decode_index(C.byref(launch), 2, (5 << 32) + M32, C.byref(index)) == 0
    assert (index.system_index, index.bank_index, index.permutation, index.configuration_index) == (1, 2, M32, (2 << 32) + M32)
    assert lib.odezza_score_decode_index(C.byref(launch), 2, 6 << 32, C.byref(index)) == E.ERROR_INVALID_ARGUMENT
    size = E.ReductionSize()
    assert lib.odezza_score_reduction_requirements(C.byref(launch), (1 << 64) - 1, E.GLOBAL, 1, C.byref(size)) == E.ERROR_OVERFLOW
    launch.active_toggle_count = 33
    assert lib.odezza_score_decode_index(C.byref(launch), 1, 0, C.byref(index)) == E.ERROR_INVALID_ARGUMENT
    for k in (0, 257):
        assert requirements(3, 1, 2, E.GLOBAL, k)[0] == E.ERROR_INVALID_ARGUMENT
    assert requirements(3, 1, 2, 3, 1)[0] == E.ERROR_INVALID_ARGUMENT
    assert requirements(0, 1, 2, E.GLOBAL, 1)[0] == E.ERROR_INVALID_ARGUMENT
    # sizes: tiles of 2048 scores; one level of partial winners and counts, two when a group spans several tiles
    for banks, bits, systems, k in [(3, 0, 3, 1), (1027, 2, 33, 17), (2049, 1, 3, 256), (65537, 1, 2, 4), (1048577, 0, 2, 256)]:
        configs = banks << bits
        for grouping, groups in ((E.BY_SYSTEM, systems), (E.BY_SYSTEM_PERMUTATION, systems << bits), (E.GLOBAL, 1)):
            code, s = requirements(banks, bits, systems, grouping, k)
            assert code == 0
            elements = systems * configs // groups
            tiles = 1 + (elements - 1) // 2048
            partial = groups * tiles * (16 * k + 24)
            assert (s.configuration_count, s.score_count, s.group_count, s.tiles_per_group) == (configs, systems * configs, groups, tiles)
            assert (s.winner_bytes, s.count_bytes) == (groups * k * 16, groups * 24)
            assert s.workspace_bytes == partial * (2 if tiles > 1 else 1)


def lit(v):
    return bytes([E.OP["LIT"]]) + struct.pack("<f", v)


RET = bytes([E.OP["RET"]])


def constant_slope(v):
    return lit(v) + RET


def reference_launch(**changes):
    """The launch of the reference's scoring test with made-up device addresses (never dereferenced here)."""
    l = E.Launch()
    l.constant_bank_count, l.trajectory_count, l.trajectory_point_count, l.steps_per_observation = 3, 2, 5, 2
    l.trajectory_offsets_device, l.trajectory_times_device, l.reference_data_device, l.mse_output_device = 0x1000, 0x2000, 0x3000, 0x4000
    for name, value in changes.items():
        setattr(l, name, value)
    return l


def test_scoring_handle_creation_rules():
    one = [(0, constant_slope(1.0))]
    with E.ScoringPipeline(1) as p:
        assert p.created == 0 and p.workspace_size > 0 and p.error() == ""
        assert p.stats().submitted_ticket_count == 0
    for kwargs, want in [(dict(states=0), E.ERROR_INVALID_ARGUMENT), (dict(states=1, system_capacity=0), E.ERROR_INVALID_ARGUMENT),
                         (dict(states=1, sm_version=90), E.ERROR_UNSUPPORTED), (dict(states=9), E.ERROR_UNSUPPORTED),
                         (dict(states=2, constants=129), E.ERROR_UNSUPPORTED),
                         (dict(states=1, fixed=one + one), E.ERROR_INVALID_ARGUMENT),               # more fixed sides than states
                         (dict(states=2, fixed=one + one), E.ERROR_STATE_LAYOUT),                   # the same state twice
                         (dict(states=2, fixed=[(2, constant_slope(1.0))]), E.ERROR_STATE_LAYOUT),
                         (dict(states=2, fixed=[(0, lit(1) + lit(2) + bytes([E.OP["TOG2"], 0]) + RET)]), E.ERROR_AST),
                         (dict(states=2, fixed=[(0, bytes([E.OP["STATE"], 2]) + RET)]), E.ERROR_AST)]:
        p = E.ScoringPipeline(check_result=False, **kwargs)
        assert p.created == want, kwargs
        assert p.handle and p.error() != ""                                    # a diagnostic handle: message and destroy only
        size = C.c_size_t()
        assert p.lib.odezza_scoring_pipeline_workspace_requirements(p.handle, C.byref(size), C.byref(size)) == E.ERROR_BUSY
        assert p.lib.odezza_scoring_pipeline_run(p.handle, None, 1, None, None, 0, None) == E.ERROR_INVALID_ARGUMENT
        p.close()
    lib = E.load()
    assert lib.odezza_scoring_pipeline_create(None, None) == E.ERROR_INVALID_ARGUMENT
    assert lib.odezza_scoring_pipeline_destroy(None) == E.ERROR_INVALID_ARGUMENT
    n = C.c_size_t()
    with E.ScoringPipeline(1) as p:
        assert lib.odezza_scoring_pipeline_write_error(p.handle, None, 0, C.byref(n)) == 0 and n.value == 0
        assert lib.odezza_scoring_pipeline_write_error(p.handle, C.create_string_buffer(1), 0, C.byref(n)) == E.ERROR_INSUFFICIENT_BUFFER


def test_launches_are_rejected_before_any_work():
    """The rejection matrix of projects/odezza/tests/o_scoring_cuda_test.c:188-205 and the argument
    rules before it: every rejected launch leaves the ticket counters alone and reports nothing."""
    systems = [[(0, constant_slope(float(s + 1)))] for s in range(3)]
    big = (1 << 64) - 4
    with E.ScoringPipeline(1) as p:
        def rejected(launch, want, count=None):
            before = p.stats().submitted_ticket_count
            code, report = p.run(systems, launch, count)
            assert code == want, (E.result_name(code), E.result_name(want), p.error())
            assert p.stats().submitted_ticket_count == before
            assert report.module_count == 0 and report.configuration_count == 0 and p.error() != ""
        rejected(reference_launch(mse_output_device=big), E.ERROR_OVERFLOW)
        rejected(reference_launch(reference_data_device=big), E.ERROR_OVERFLOW)
        rejected(reference_launch(trajectory_times_device=0x2001), E.ERROR_OVERFLOW)
        rejected(reference_launch(trajectory_point_count=M32), E.ERROR_OVERFLOW)
        rejected(reference_launch(constant_bank_count=128, active_toggle_count=32), E.ERROR_UNSUPPORTED)
        rejected(reference_launch(active_toggle_count=33), E.ERROR_INVALID_ARGUMENT)
        rejected(reference_launch(), E.ERROR_OVERFLOW, count=((1 << 64) - 1) // C.sizeof(E.ScoringSystem) + 1)
        for field in ("constant_bank_count", "reference_data_device", "trajectory_offsets_device", "trajectory_times_device",
                      "trajectory_count", "steps_per_observation", "mse_output_device"):
            rejected(reference_launch(**{field: 0}), E.ERROR_INVALID_ARGUMENT)
        rejected(reference_launch(trajectory_count=6), E.ERROR_INVALID_ARGUMENT)          # more trajectories than points
        rejected(reference_launch(allow_missing_observations=2), E.ERROR_INVALID_ARGUMENT)
        rejected(reference_launch(profile_timing=2), E.ERROR_INVALID_ARGUMENT)
        rejected(reference_launch(), E.ERROR_INVALID_ARGUMENT, count=0)
        # programs are checked before the device is touched: a truncated program, a bad index, a toggle over a computed value
        for bad in (constant_slope(1.0)[:1], bytes([E.OP["STATE"], 1]) + RET, bytes([E.OP["CONSTANT"], 0]) + RET,
                    lit(1) + lit(2) + bytes([E.OP["ADD"]]) + lit(3) + bytes([E.OP["TOG2"], 0]) + RET, lit(float("inf")) + RET,
                    lit(1) + RET + RET, lit(1) + lit(2) + RET, bytes([0x8F]) + RET):
            before = p.stats()
            code, report = p.run([[(0, bad)]] + systems[1:], reference_launch(active_toggle_count=1))
            assert code == E.ERROR_AST, bad.hex()
            after = p.stats()
            assert after.submitted_ticket_count == before.submitted_ticket_count
            assert after.specialization_failure_count == before.specialization_failure_count + 1
            assert report.system_count == 0 and report.configuration_count == 0
        # a system must define every state that is not fixed, once
        for bad_system in ([], [(0, constant_slope(1.0)), (0, constant_slope(2.0))], [(1, constant_slope(1.0))]):
            code, _ = p.run([bad_system], reference_launch())
            assert code == E.ERROR_STATE_LAYOUT
        # the workspace is checked like the reference's: present, 8-byte aligned, large enough
        arr, keep = E.systems_array(systems)
        launch = reference_launch()
        for workspace, size in ((None, p.workspace_size), (p.workspace, p.workspace_size - 1),
                                (C.cast(C.addressof(p.workspace) + 4, C.c_void_p), p.workspace_size)):
            assert p.lib.odezza_scoring_pipeline_run(p.handle, arr, 3, C.byref(launch), workspace, size, None) == E.ERROR_INVALID_ARGUMENT
    with E.ScoringPipeline(2, constants=2) as p:
        code, _ = p.run([[(0, constant_slope(1.0)), (1, constant_slope(1.0))]], reference_launch())   # constants without a table or descriptors
        assert code == E.ERROR_INVALID_ARGUMENT
        sampled = reference_launch(sampled_parameters_device=0x5000, rng_pool_size=0, uniform_pool_device=0x6000)
        assert p.run([[(0, constant_slope(1.0)), (1, constant_slope(1.0))]], sampled)[0] == E.ERROR_INVALID_ARGUMENT
        sampled = reference_launch(sampled_parameters_device=0x5004, rng_pool_size=16, uniform_pool_device=0x6000)
        assert p.run([[(0, constant_slope(1.0)), (1, constant_slope(1.0))]], sampled)[0] == E.ERROR_INVALID_ARGUMENT


def test_reference_handle_contract_test_passes():
    """projects/odezza/tests/o_scoring_pipeline_test.c (a failed creation keeps a diagnostic handle
    with a message, refuses the workspace query, can be destroyed), compiled unmodified against the
    reference header and linked against this library (oracle/Makefile, target engine-tests); it
    needs no device."""
    import subprocess
    import pytest
    binary = os.path.join(ROOT, "oracle", "_ref", "o_scoring_pipeline_test")
    if not os.path.exists(binary):
        pytest.skip("oracle/_ref/o_scoring_pipeline_test is built only where the reference checkout exists")
    done = subprocess.run([binary], capture_output=True, text=True, timeout=60)
    assert done.returncode == 0, (done.stdout, done.stderr)
    assert "verified" in done.stdout
