"""The ODE engine interface (include/odezza_b200.h) on the device.

Two kinds of evidence.  (1) The reference engine's own tests of its scoring handle, random pools
and score reducer (projects/odezza/tests/o_scoring_cuda_test.c, o_philox_test.c,
o_score_reduce_test.c), compiled unmodified against the reference's headers and linked against
this library (oracle/Makefile, target `engine-tests`), with the argument sets of the reference's
build (projects/odezza/CMakeLists.txt:198-200).  (2) Seeded cases through the same entry points
checked against the CPU restatement: rollout scores against oracle/secant_oracle.c::so_rk4_score
(itself pinned on the reference's host scorer, tests/test_rk4_cpu.py), pools against a Python
restatement of the generator, reductions against a sort on the host."""
import ctypes as C
import os
import struct
import subprocess

import numpy as np
import pytest
import torch

import support as S
from secant_b200 import engine as E, programs as P
from test_engine_cpu import uniform_sample
from test_rk4_cpu import FLT_MAX, to_engine_bytecode

pytestmark = pytest.mark.gpu
REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle", "_ref")


def run_reference_test(name, *args, timeout=900):
    binary = os.path.join(REF, name)
    if not os.path.exists(binary):
        pytest.skip(f"oracle/_ref/{name} is built only where the reference checkout exists")
    done = subprocess.run([binary, *args], capture_output=True, text=True, timeout=timeout)
    assert done.returncode == 0, (done.stdout[-1500:], done.stderr[-1500:])
    return done.stdout


@pytest.mark.parametrize("args", [("1", "0", "1"), ("8", "8", "1"), ("8", "8", "8")])
def test_reference_scoring_test_passes(cuda, args):
    out = run_reference_test("o_scoring_cuda_test", *args)
    assert "all scores and invalid data verified" in out


def test_reference_pool_test_passes(cuda):
    out = run_reference_test("o_philox_test")
    assert '"sampled_vs_explicit_scores":"bitwise_equal"' in out


def test_reference_reducer_test_passes(cuda):
    out = run_reference_test("o_score_reduce_test", timeout=1800)
    assert "score reducer checks passed" in out


# ---- seeded cases against the CPU restatement ------------------------------------------------------

def dev(a):
    return torch.tensor(np.ascontiguousarray(a), device="cuda")


def launch_for(offsets, times, reference, out, banks, nb, bits, steps, allow_missing=False):
    l = E.Launch()
    l.constant_banks_device = banks.data_ptr() if banks is not None else 0
    l.constant_bank_count, l.active_toggle_count = nb, bits
    l.trajectory_offsets_device, l.trajectory_times_device = offsets.data_ptr(), times.data_ptr()
    l.reference_data_device, l.mse_output_device = reference.data_ptr(), out.data_ptr()
    l.trajectory_count, l.trajectory_point_count = offsets.numel() - 1, times.numel()
    l.steps_per_observation = steps
    l.allow_missing_observations = 1 if allow_missing else 0
    return l


def test_scores_match_the_cpu_restatement(cuda):
    """40 candidate systems of 2 states, 3 coefficients, 3 banks, 1 toggle bit, ragged trajectories:
    state 1's right-hand side is fixed at creation, state 0's comes with every candidate.  Every
    (system, bank, permutation) score against the CPU restatement; the same candidates with both
    sides supplied per system must give identical bits."""
    S_, K, nb, bits, n_sys = 2, 3, 3, 1, 40
    ops = [(P.op("ADD"), 2), (P.op("SUB"), 2), (P.op("MUL"), 2), (P.op("SIN"), 1), (P.op("COS"), 1), (P.op("TANH"), 1)]
    raw = P.random_population(31, n_sys, 14, S_, K, 1.0, toggle_bits=bits, ops=ops)
    moving = [a[:-1] + P.op("TANH") + P.col(0) + P.op("SUB") + P.RET for a in raw.asts]          # contracting
    fixed = P.bank(1) + P.col(0) + P.op("MUL") + P.col(1) + P.op("SUB") + P.RET                  # y' = c1 x - y
    pop = P.PackedPrograms([prog for a in moving for prog in (a, fixed)], raw.routines)
    rng = np.random.default_rng(32)
    lengths = rng.integers(2, 25, size=37)
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.uint32)
    times = np.concatenate([np.cumsum(rng.uniform(0.02, 0.07, size=n)) for n in lengths]).astype(np.float32)
    reference = rng.uniform(-1, 1, size=(S_, int(offsets[-1]))).astype(np.float32)
    banks = rng.normal(0, 1, size=(n_sys, nb, K)).astype(np.float32)
    d_off, d_t, d_ref, d_banks = torch.tensor(offsets.astype(np.int32), device="cuda"), dev(times), dev(reference), dev(banks)
    out = torch.full((n_sys, nb << bits), float("nan"), device="cuda")
    launch = launch_for(d_off, d_t, d_ref, out, d_banks, nb, bits, 2)
    with E.ScoringPipeline(S_, K, fixed=[(1, to_engine_bytecode(fixed))]) as pipe:
        code, report = pipe.run([[(0, to_engine_bytecode(a))] for a in moving], launch)
        assert code == 0, pipe.error()
        assert (report.system_count, report.configuration_count, report.module_count) == (n_sys, n_sys * (nb << bits), 1)
        stats = pipe.stats()
        assert stats.submitted_ticket_count == stats.completed_ticket_count == 1
    got = out.cpu().numpy()
    for cfg in range(nb << bits):
        code, want, want64 = S.oracle_rk4(pop, S_, reference, len(lengths), times, np.ascontiguousarray(banks[:, cfg >> bits, :]), 2, bits,
                                          cfg & 1, want64=True, offsets=offsets)
        assert code == 0
        assert np.allclose(got[:, cfg], want64, rtol=2e-4, atol=1e-6), cfg
    again = torch.full_like(out, float("nan"))
    launch.mse_output_device = again.data_ptr()
    with E.ScoringPipeline(S_, K) as pipe:
        systems = [[(1, to_engine_bytecode(fixed)), (0, to_engine_bytecode(a))] for a in moving]     # any order of states
        code, _ = pipe.run(systems, launch)
        assert code == 0, pipe.error()
    assert np.array_equal(again.cpu().numpy().view(np.uint32), got.view(np.uint32))


def test_a_run_larger_than_one_batch_and_timing_report(cuda):
    """20,000 one-state systems (more than one internal batch): dx/dt = slope with the closed form of
    the reference's test, 0.4375 * (slope - 1)^2 on its five-point layout."""
    n_sys = 20000
    offsets = torch.tensor([0, 3, 5], dtype=torch.int32, device="cuda")
    times = dev(np.array([0.0, 0.25, 1.0, 0.0, 0.5], dtype=np.float32))
    reference = dev(np.array([[1.0, 1.25, 2.0, 2.0, 2.5]], dtype=np.float32))
    out = torch.full((n_sys, 1), float("nan"), device="cuda")
    slopes = 1.0 + (np.arange(n_sys) % 64).astype(np.float32) / 8
    launch = launch_for(offsets, times, reference, out, None, 1, 0, 2)
    launch.profile_timing = 1
    with E.ScoringPipeline(1) as pipe:
        code, report = pipe.run([[(0, bytes([E.OP["LIT"]]) + struct.pack("<f", float(s)) + bytes([E.OP["RET"]]))] for s in slopes], launch)
        assert code == 0, pipe.error()
        assert report.system_count == n_sys and report.module_count == 2 and report.profiled_modules == 2
        assert 0 < report.gpu_span_seconds <= report.total_seconds
    assert np.allclose(out.cpu().numpy()[:, 0], 0.4375 * (slopes - 1) ** 2, atol=1e-5)


class DeviceFloats:
    """A float32 range of device memory that is not torch's, viewable as a tensor."""

    def __init__(self, address, count):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (address, False), "version": 2}


def download(address, count):
    return torch.as_tensor(DeviceFloats(address, count), device="cuda").cpu().numpy().copy()


def test_pools_are_reproducible_sample_for_sample(cuda):
    lib = E.load()
    info = E.RngPoolInfo(20260906, 37, 7, 300007, 3)
    pool, view = C.c_void_p(), E.RngPoolView()
    E.check(lib.odezza_rng_pool_create(100, C.byref(info), C.byref(pool)))
    E.check(lib.odezza_rng_pool_view(pool, C.byref(view)))
    uniform, normal = download(view.uniform_device, info.size), download(view.normal_device, info.size)
    picks = np.concatenate([np.arange(64), np.random.default_rng(1).integers(0, info.size, 500), [info.size - 1]])
    for i in picks:
        assert uniform[i] == uniform_sample(info.seed, info.stream, info.sample_base + int(i)), i
    assert uniform.min() > 0 and uniform.max() < 1
    # the normal plane: Box-Muller over the uniform samples of the odd domain, pairs inside a block of four
    first = info.sample_base // 4 * 4
    for i in picks[:200]:
        sample = info.sample_base + int(i)
        pair = (sample - first) // 2 * 2 + first
        u0, u1 = (float(uniform_sample_domain(info.seed, 2 * info.stream + 1, s)) for s in (pair, pair + 1))
        radius, angle = np.sqrt(-2.0 * np.log(u0)), 2.0 * np.pi * u1
        want = radius * (np.cos(angle) if sample == pair else np.sin(angle))
        assert abs(normal[i] - want) <= 4e-6 * max(1.0, abs(want)), (i, normal[i], want)
    assert abs(normal.mean()) < 0.01 and abs(normal.var() - 1) < 0.02
    # a pool that starts 13 samples later is a slice of the first one
    part_info = E.RngPoolInfo(info.seed, info.stream, info.sample_base + 13, 39, 3)
    part, part_view = C.c_void_p(), E.RngPoolView()
    E.check(lib.odezza_rng_pool_create(100, C.byref(part_info), C.byref(part)))
    E.check(lib.odezza_rng_pool_view(part, C.byref(part_view)))
    for device, whole in ((part_view.uniform_device, uniform), (part_view.normal_device, normal)):
        assert np.array_equal(download(device, 39).view(np.uint32), whole[13:52].view(np.uint32))
    E.check(lib.odezza_rng_pool_destroy(part))
    E.check(lib.odezza_rng_pool_destroy(pool))
    assert lib.odezza_rng_pool_create(100, C.byref(E.RngPoolInfo(1, 1, 0, 0, 3)), C.byref(pool)) == E.ERROR_INVALID_ARGUMENT


def uniform_sample_domain(seed, domain, sample):
    from test_engine_cpu import philox4x32
    m = 0xFFFFFFFF
    words = philox4x32([(sample // 4) & m, (sample // 4) >> 32, domain & m, domain >> 32], [seed & m, seed >> 32])
    return np.float32((np.float32(words[sample % 4] >> 9) + np.float32(0.5)) * np.float32(2.0 ** -23))


def host_reduction(scores, systems, banks, bits, grouping, k):
    configs = banks << bits
    flat = scores.reshape(-1)
    if grouping == E.GLOBAL:
        groups = [np.arange(flat.size)]
    elif grouping == E.BY_SYSTEM:
        groups = [np.arange(s * configs, (s + 1) * configs) for s in range(systems)]
    else:
        groups = [s * configs + np.arange(banks) * (1 << bits) + p for s in range(systems) for p in range(1 << bits)]
    winners, counts = [], []
    for index in groups:
        v = flat[index]
        ok = (v >= 0) & (v < FLT_MAX)
        negative = np.isfinite(v) & (v < 0)
        counts.append((int(ok.sum()), int((~ok).sum()), int(negative.sum())))
        keys = np.where(v[ok] == 0, np.float32(0), v[ok])
        order = np.lexsort((index[ok], keys))[:k]
        rows = [(v[ok][o], int(index[ok][o])) for o in order]
        winners.append(rows + [(FLT_MAX, (1 << 64) - 1)] * (k - len(rows)))
    return winners, counts


@pytest.mark.parametrize("systems,banks,bits,k", [(3, 3, 0, 1), (33, 1027, 2, 17), (3, 70001, 1, 256), (2, 300017, 0, 4)])
def test_reducer_and_gather_match_a_host_sort(cuda, systems, banks, bits, k):
    lib = E.load()
    rng = np.random.default_rng(systems * 7 + banks)
    configs = banks << bits
    scores = (rng.integers(0, 5000, size=(systems, configs)) / 8).astype(np.float32)               # many exact ties
    flat = scores.reshape(-1)
    for value, every in ((np.nan, 37), (np.inf, 41), (FLT_MAX, 43), (-1.0, 47), (-0.0, 29)):
        flat[::every] = value
    flat[:configs // 2] = np.nan
    constants = rng.normal(0, 1, size=(systems, banks, 2)).astype(np.float32)
    d_scores, d_constants = dev(scores), dev(constants)
    launch = E.Launch()
    launch.constant_bank_count, launch.active_toggle_count = banks, bits
    launch.mse_output_device, launch.constant_banks_device = d_scores.data_ptr(), d_constants.data_ptr()
    reducer = C.c_void_p()
    E.check(lib.odezza_score_reducer_create(100, k, C.byref(reducer)))
    for grouping in (E.BY_SYSTEM, E.BY_SYSTEM_PERMUTATION, E.GLOBAL):
        size = E.ReductionSize()
        E.check(lib.odezza_score_reduction_requirements(C.byref(launch), systems, grouping, k, C.byref(size)))
        workspace = torch.zeros(size.workspace_bytes // 8 + 1, dtype=torch.int64, device="cuda")
        winners = torch.zeros(size.winner_bytes // 8, dtype=torch.int64, device="cuda")
        counts = torch.zeros(size.count_bytes // 8, dtype=torch.int64, device="cuda")
        rows = torch.zeros(size.group_count * k * 2, dtype=torch.float32, device="cuda")
        args = (reducer, C.byref(launch), systems, grouping)
        report = E.ReductionReport()
        assert lib.odezza_score_reducer_run(*args, workspace.data_ptr(), size.workspace_bytes - 1, winners.data_ptr(), size.winner_bytes,
                                            counts.data_ptr(), size.count_bytes, None) == E.ERROR_INSUFFICIENT_BUFFER
        assert lib.odezza_score_reducer_run(*args, workspace.data_ptr(), size.workspace_bytes, workspace.data_ptr(), size.winner_bytes,
                                            counts.data_ptr(), size.count_bytes, None) == E.ERROR_INVALID_ARGUMENT
        E.check(lib.odezza_score_reducer_run(*args, workspace.data_ptr(), size.workspace_bytes, winners.data_ptr(), size.winner_bytes,
                                             counts.data_ptr(), size.count_bytes, C.byref(report)))
        assert (report.group_count, report.score_count) == (size.group_count, systems * configs) and report.kernel_seconds > 0
        E.check(lib.odezza_score_reducer_gather(*args, 2, winners.data_ptr(), size.winner_bytes, rows.data_ptr(), rows.numel() * 4))
        raw = winners.cpu().numpy().view(np.uint32).reshape(-1, k, 4)
        got_mse, got_index = raw[:, :, 0].view(np.float32), raw[:, :, 2].astype(np.uint64) | (raw[:, :, 3].astype(np.uint64) << 32)
        got_counts = counts.cpu().numpy().reshape(-1, 3)
        got_rows = rows.cpu().numpy().reshape(-1, k, 2)
        want, want_counts = host_reduction(scores, systems, banks, bits, grouping, k)
        assert got_counts.tolist() == [list(c) for c in want_counts]
        for g, group in enumerate(want):
            assert got_index[g].tolist() == [i for _, i in group], (grouping, g)
            assert np.array_equal(got_mse[g].view(np.uint32), np.array([m for m, _ in group], dtype=np.float32).view(np.uint32))
            assert np.all(raw[g, :, 1] == 0)
            for rank, (_, index) in enumerate(group):
                if index == (1 << 64) - 1:
                    assert np.isnan(got_rows[g, rank]).all()
                else:
                    decoded = E.ScoreIndex()
                    E.check(lib.odezza_score_decode_index(C.byref(launch), systems, index, C.byref(decoded)))
                    assert np.array_equal(got_rows[g, rank], constants[decoded.system_index, decoded.bank_index])
        # the plain entry point (one CTA per group, no scratch) selects the same winners
        plain = torch.zeros_like(winners)
        plain_counts = torch.zeros_like(counts)
        assert lib.secant_b200_grouped_topk(d_scores.data_ptr(), systems, banks, bits, grouping, k, plain.data_ptr(), plain_counts.data_ptr(), None) == 0
        torch.cuda.synchronize()
        assert torch.equal(plain, winners) and torch.equal(plain_counts, counts)
    E.check(lib.odezza_score_reducer_destroy(reducer))


# ---- the reference's own pools, run beside this library's -----------------------------------------

def reference_engine():
    """oracle/_ref/libodezza_engine_ref.so: the reference's o_philox.c (kernels compiled with NVRTC at
    run time), built by `make -C oracle engine-ref`."""
    path = os.path.join(REF, "libodezza_engine_ref.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libodezza_engine_ref.so is built only where the reference checkout exists")
    lib = C.CDLL(path)
    for name, (restype, argtypes) in E.EXPORTED.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
    return lib


def pool_planes(lib, info):
    pool, view = C.c_void_p(), E.RngPoolView()
    code = lib.odezza_rng_pool_create(100, C.byref(info), C.byref(pool))
    if code:
        buf = C.create_string_buffer(2048)
        lib.odezza_rng_pool_write_error(pool, buf, len(buf))
        raise AssertionError((E.result_name(code), buf.value.decode()[-800:]))
    E.check(lib.odezza_rng_pool_view(pool, C.byref(view)))
    planes = download(view.uniform_device, info.size), download(view.normal_device, info.size)
    E.check(lib.odezza_rng_pool_destroy(pool))
    return planes


def test_pools_equal_the_reference_pools_bit_for_bit(cuda):
    """Both planes, sample for sample, against the reference's own pool kernels on the same device
    (projects/odezza/core/o_philox.cu, compiled by the reference with --fmad=false): an odd sample
    base, a size that is no multiple of four, and a second stream and seed."""
    ref = reference_engine()
    mine = E.load()
    for info in (E.RngPoolInfo(20260906, 37, 7, 1048583, 3), E.RngPoolInfo(1, 0, 0, 4099, 3), E.RngPoolInfo((1 << 64) - 3, 12345, (1 << 40) + 2, 70001, 3)):
        got, want = pool_planes(mine, info), pool_planes(ref, info)
        for plane in range(2):
            assert np.array_equal(got[plane].view(np.uint32), want[plane].view(np.uint32)), (info.seed, "uniform normal".split()[plane])
