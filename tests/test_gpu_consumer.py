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
