"""The reference's own consumer of the runner API running against this library.

oracle/_ref/secant_sr_cuda_test is the reference's projects/secant-sr/toggle/tests/cuda_test.c
with its CUDA adapter (projects/secant-sr/toggle/src/cuda.c: the create sequence at :290-321,
the scoring loop at :411-429) and search library, compiled unmodified and linked against
libsecant_b200.so in place of the reference's runner libraries (recipe: oracle/Makefile,
target `consumer`).  It compiles the source this library hands out with NVRTC, builds a plan and a
runner from the result, scores 129 programs in 7 partial batches with 3-bit toggles and 5 banks,
reduces them with its own kernel and compares every score with the reference host evaluator;
it also checks ties, all-invalid programs, a malformed program and a repeated call."""
import os
import subprocess

import pytest

BINARY = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle", "_ref", "secant_sr_cuda_test")


@pytest.mark.gpu
def test_reference_consumer_passes_against_the_drop_in(cuda):
    if not os.path.exists(BINARY):
        pytest.skip("oracle/_ref/secant_sr_cuda_test is built only where the reference checkout exists")
    done = subprocess.run([BINARY], capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    assert "CUDA SR adapter: CPU agreement" in done.stdout


SEARCH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle", "_ref", "secant_sr_search")


def _search(backend, extra=()):
    import json
    args = [SEARCH, "--backend", backend, "--problem", "nguyen1", "--population", "256", "--generations", "6", "--banks", "16",
            "--constants", "4", "--toggle-bits", "4", "--seed", "7", "--rows", "512", "--validation-rows", "256", *extra]
    env = dict(os.environ, CUDA_MODULE_LOADING="EAGER")
    done = subprocess.run(args, capture_output=True, text=True, timeout=600, env=env)
    events = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    return done, events


@pytest.mark.gpu
def test_reference_search_driver_runs_on_the_drop_in(cuda):
    """The reference's search driver (projects/secant-sr/toggle/src/main.c, README.md:68-79) with its
    CUDA backend, compiled unmodified against this library (oracle/Makefile, target `search`):
    populations are scored through secant_cubin_runner_run_toggle_sse, coefficient refinement through
    secant_sr_cuda_score_banks (projects/secant-sr/toggle/src/cuda.c:368-489).  The driver replays its
    winner on the host evaluator and fails when the two scores disagree; the first generation, scored
    from the same seeded population on both backends, must report the same best error."""
    if not os.path.exists(SEARCH):
        pytest.skip("oracle/_ref/secant_sr_search is built only where the reference checkout exists")
    gpu, gpu_events = _search("cuda")
    assert gpu.returncode == 0, gpu.stderr[-2000:]
    cpu, cpu_events = _search("cpu")
    assert cpu.returncode == 0, cpu.stderr[-2000:]
    first = lambda events: next(e for e in events if e.get("event") == "generation")
    g, c = first(gpu_events), first(cpu_events)
    assert g["configurations"] == c["configurations"] and g["finite_configurations"] == c["finite_configurations"]
    assert abs(g["best_mse"] - c["best_mse"]) <= 2e-4 * abs(c["best_mse"]) + 1e-9, (g, c)
    assert any(e.get("event") == "result" for e in gpu_events)
    # the refinement path: new coefficient banks proposed and scored for a fixed set of programs
    refined, events = _search("cuda", ("--refine-rounds", "2", "--refine-budget", "32"))
    assert refined.returncode == 0, refined.stderr[-2000:]
    assert any(e.get("event") == "result" for e in events)


REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle", "_ref")


@pytest.mark.gpu
def test_reference_runner_test_passes_against_the_drop_in(cuda):
    """The reference's own GPU test of the runner API (projects/secant/tests/toggle_cuda_test.c,
    compiled unmodified with the reference host evaluator and linked against this library:
    oracle/Makefile, target `secant-tests`; oracle/secant_runner_test_shim.c calls its parts): the
    fixture toggles with 1 and 3 programs per kernel (partial batches, ties, repeated and batched
    runs, a malformed program), seeded random programs with 1, 8 and 32 programs per kernel, and
    the four static shapes (materialize, SSE, affine statistics, Gram statistics), each compared
    with the reference host evaluator.  The edge part (no columns, no constants, no toggles, a
    toggle inside a routine) compares its scores too and then looks for the machine-code bytes of one
    instruction in what secant_cubin_specialize_into() wrote, which a library that patches no machine
    code cannot show: the process must end exactly there."""
    binary = os.path.join(REF, "secant_toggle_cuda_test")
    if not os.path.exists(binary):
        pytest.skip("oracle/_ref/secant_toggle_cuda_test is built only where the reference checkout exists")
    env = dict(os.environ, CUDA_MODULE_LOADING="EAGER")
    done = subprocess.run([binary], capture_output=True, text=True, timeout=600, env=env)
    assert done.returncode == 0, (done.stdout[-1500:], done.stderr[-1500:])
    assert "static shape 3 passed" in done.stdout and "random toggles (packed=32)" in done.stdout
    assert "scores of the toggle, random and static parts agree" in done.stdout
    edge = subprocess.run([binary, "edge"], capture_output=True, text=True, timeout=600, env=env)
    assert edge.returncode == 1 and edge.stderr.strip().endswith("toggle_cuda_test.c:521: found"), (edge.stdout[-800:], edge.stderr[-800:])
    assert "mismatch" not in edge.stderr
