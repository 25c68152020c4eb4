"""Generates tests/golden/reference_vectors.npz by running the REFERENCE's own host
evaluator (projects/secant/s_cpu.c, compiled unmodified into oracle/_ref/libsecant_ref.so by
`make -C oracle ref`) on small inputs.  Run it on a machine that has the reference checkout:

    make -C oracle ref && python tests/golden/make_golden.py

The fixture programs, inputs and bank values restate the reference's tests
(projects/secant/tests/toggle_fixture.h:34-56, tests/toggle_test.c:44-72 and :179-199,
tests/cpu_test.c:39-76 and :112-118); every expected value in the file was produced by the
reference library, none by this repository's code.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import support as S  # noqa: E402
from secant_b200 import programs as P  # noqa: E402

ref = S.reference_lib()
if ref is None:
    raise SystemExit("oracle/_ref/libsecant_ref.so is missing: run `make -C oracle ref` first")

out = {}


def save_programs(prefix, packed):
    out[prefix + "_ast_blob"] = np.frombuffer(packed.ast_blob, dtype=np.uint8)
    out[prefix + "_ast_off"] = packed.ast_off[: len(packed.asts)]
    out[prefix + "_routine_blob"] = np.frombuffer(packed.routine_blob or b"", dtype=np.uint8)
    out[prefix + "_routine_off"] = packed.routine_off[: len(packed.routines)]


# ---- 1. the seven toggle fixture programs (toggle_fixture.h:34-56) -------------------
col, bank, tog2, tog4, lit_bits, op, RET = P.col, P.bank, P.tog2, P.tog4, P.lit_bits, P.op, P.RET
fixture = P.PackedPrograms([
    col(0) + col(1) + tog2(0) + bank(0) + op("MUL") + RET,
    col(2) + bank(1) + tog2(1) + col(0) + bank(0) + tog2(0) + op("ADD") + RET,
    col(0) + bank(0) + col(2) + bank(1) + tog4(0, 2) + RET,
    bank(0) + bank(1) + tog2(2) + bank(1) + bank(0) + tog2(2) + op("SUB") + RET,
    col(0) + bank(0) + tog2(0) + col(1) + bank(1) + tog2(1) + op("MUL") + col(2) + bank(0) + tog2(2) + op("ADD") + RET,
    lit_bits(0x3F800000) + bank(1) + tog2(1) + RET,
    bank(0) + bank(1) + col(0) + col(1) + tog4(2, 0) + bank(0) + op("ADD") + RET,
])
x = (np.arange(3 * 17, dtype=np.float32) * np.float32(0.013) - np.float32(0.3)).reshape(3, 17)
y = (np.arange(2 * 17, dtype=np.float32) * np.float32(0.007)).reshape(2, 17)
banks_flat = (np.arange(38, dtype=np.float32) * np.float32(0.01) - np.float32(0.6))
banks_flat = np.concatenate([banks_flat, np.zeros(1, dtype=np.float32)])  # 13 banks, stride 3 (last one padded)
banks = banks_flat.reshape(13, 3)
save_programs("fixture", fixture)
out["fixture_x"], out["fixture_y"], out["fixture_banks"] = x, y, banks
for pass_idx in range(2):
    b = banks if pass_idx == 0 else (banks + np.float32(0.137)).astype(np.float32)
    code, sse = S.reference_toggle_sse(ref, fixture, x, y, b, 2, 3, out_ld=109)
    assert code == 0, code
    out[f"fixture_sse_pass{pass_idx}"] = sse
# error cases of toggle_test.c:96-134, as (programs, toggle_bits) -> result code
code, _ = S.reference_toggle_sse(ref, fixture, x, y, banks, 2, 2, out_ld=109)
out["fixture_bits2_code"] = np.int32(code)
bad_programs = P.PackedPrograms([
    bytes([0xB7, 0]) + RET,
    col(0) + col(1) + op("ADD") + bank(0) + tog2(0) + RET,
    col(0) + col(1) + bank(0) + bank(1) + tog4(0, 0) + RET,
])
codes = []
for i in range(3):
    c, _ = S.reference_toggle_sse(ref, bad_programs.subset([i]), x, y, banks, 2, 3)
    codes.append(c)
save_programs("bad", bad_programs)
out["bad_codes"] = np.array(codes, dtype=np.int32)

# ---- 2. affine bank leaf (toggle_test.c:179-199) ------------------------------------
affine = P.PackedPrograms([P.affine(0, 2.0, 3.0) + col(0) + tog2(0) + RET])
ax = np.array([[5.0]], dtype=np.float32)
ay = np.array([[0.0]], dtype=np.float32)
ab = np.array([[-0.25], [0.5]], dtype=np.float32)
code, sse = S.reference_toggle_sse(ref, affine, ax, ay, ab, 1, 1)
assert code == 0
save_programs("affine", affine)
out["affine_x"], out["affine_y"], out["affine_banks"], out["affine_sse"] = ax, ay, ab, sse

# ---- 3. static programs with a routine (cpu_test.c:39-76, 112-118) -------------------
arg, lit = P.arg, P.lit
safe_div = arg(0) + arg(1) + op("MUL") + arg(1) + arg(1) + op("MUL") + lit_bits(0x358637BD) + op("ADD") + op("RCP") + op("MUL") + RET
static = P.PackedPrograms([col(0) + col(1) + op("ADD") + RET, col(2) + op("SIN") + RET, col(0) + col(1) + P.routine(0) + RET],
                          [safe_div])
rows = np.arange(17, dtype=np.float32)
sx = np.stack([np.float32(0.5) + np.float32(0.1) * rows, np.float32(1.25) + np.float32(0.03) * rows,
               np.float32(-0.75) + np.float32(0.07) * rows]).astype(np.float32)
sy = np.stack([np.float32(0.2) * rows, np.float32(1.0) - np.float32(0.04) * rows]).astype(np.float32)
code, mat = S.reference_materialize(ref, static, sx)
assert code == 0
code, sse = S.reference_sse(ref, static, sx, sy)
assert code == 0
save_programs("static", static)
out["static_x"], out["static_y"], out["static_materialize"], out["static_sse"] = sx, sy, mat, sse

# ---- 4. seeded random populations through the reference ------------------------------
pop = P.random_population(424242, 129, 24, 3, 4, 1.0, toggle_bits=3)
rx = np.stack([P.uniform(5, c, 97, -0.75, 0.75) for c in range(3)])
ry = np.stack([P.uniform(6, c, 97, -1, 1) for c in range(2)])
rb = np.stack([P.uniform(7, b, 4, -1, 1) for b in range(5)])
code, sse = S.reference_toggle_sse(ref, pop, rx, ry, rb, 4, 3)
assert code == 0
save_programs("random", pop)
out["random_x"], out["random_y"], out["random_banks"], out["random_sse"] = rx, ry, rb, sse

c1 = P.random_population(1, 64, 15, 4, 0, 1.0)
cx = np.stack([P.uniform(1, c, 512, -1, 1) for c in range(4)])
cy = (cx[0] * cx[1] + np.sin(cx[2]) + P.normal(1, 99, 512, 0.01))[None, :].astype(np.float32)
code, mat = S.reference_materialize(ref, c1, cx)
assert code == 0
code, sse = S.reference_sse(ref, c1, cx, cy)
assert code == 0
save_programs("c1", c1)
out["c1_x"], out["c1_y"], out["c1_materialize"], out["c1_sse"] = cx, cy, mat, sse

path = os.path.join(HERE, "reference_vectors.npz")
np.savez_compressed(path, **out)
print("wrote", path, os.path.getsize(path), "bytes")
