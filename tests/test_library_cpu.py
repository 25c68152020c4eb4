"""What can be checked of the shipped library without a GPU: it loads, exports every symbol
the headers declare, and its GPU-free entry points (result names, recipe validation, source
and plan shims, program validation, request validation) answer with the reference's result
codes (projects/secant/s_cubin_api.c:31-72, s_cubin_runner.c:33-241, s_cpu.c:919-937)."""
import ctypes as C
import re
import os

import numpy as np

import support as S
from secant_b200 import abi, programs as P
from secant_b200.runner import make_recipe

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    lib = abi.load()
    declared = set()
    for header in ("secant_b200.h", "secant_b200_ext.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        declared |= set(re.findall(r"SECANT_DEC\s+[\w\s\*]+?\b(secant_\w+)\s*\(", text))
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), name
    assert declared == set(abi.EXPORTED)


def test_result_names_and_cpu_entry():
    lib = abi.load()
    assert lib.secant_result_to_string(0) == b"SECANT_SUCCESS"
    assert lib.secant_result_to_string(9) == b"SECANT_ERROR_BAD_PROGRAM"
    assert lib.secant_result_to_string(33) == b"SECANT_ERROR_COMPLETION_UNKNOWN"
    assert lib.secant_result_to_string(34) == b"SECANT_ERROR_UNKNOWN"
    size = C.c_size_t()
    src = lib.secant_cuda_target_stats_f32_source_get(C.byref(size))
    assert b"secant_cuda_target_stats_f32" in src and size.value == len(src) + 1
    # the host entry validates the header like the reference, then reports that no host backend exists
    run = abi.init_header(abi.CpuToggleRun(), abi.CPU_RUN_VERSION, abi.SHAPE_TOGGLE_SSE)
    assert lib.secant_cpu_run(C.byref(run)) == abi.ERROR_BACKEND_UNAVAILABLE
    run.header.version = 2
    assert lib.secant_cpu_run(C.byref(run)) == abi.ERROR_UNSUPPORTED_VERSION
    run.header.version = 3
    run.header.shape = 77
    assert lib.secant_cpu_run(C.byref(run)) == abi.ERROR_UNSUPPORTED_SHAPE
    run.header.shape = abi.SHAPE_TOGGLE_SSE
    run.header.flags = 1
    assert lib.secant_cpu_run(C.byref(run)) == abi.ERROR_INVALID_VALUE
    assert lib.secant_cpu_run(None) == abi.ERROR_INVALID_VALUE


def test_recipe_validation_and_source_plan_shims():
    lib = abi.load()
    r = make_recipe(abi.SHAPE_TOGGLE_SSE, 3, 2, 8)
    r.num_kernels, r.asts_per_kernel, r.tile_rows = 3, 32, 31
    r.patch_capacity_instructions = 256
    assert lib.secant_cubin_recipe_validate(C.byref(r)) == 0
    size = C.c_size_t()
    assert lib.secant_cubin_source_size(C.byref(r), C.byref(size)) == 0 and size.value > 0
    buf = C.create_string_buffer(size.value)
    assert lib.secant_cubin_source_write(C.byref(r), buf, size.value - 1) == abi.ERROR_INSUFFICIENT_BUFFER
    assert lib.secant_cubin_source_write(C.byref(r), buf, size.value) == 0
    assert buf.value.count(b"__global__") == 3 and b"secant_cubin_toggle_sse_002" in buf.value
    for version in (1, 2):
        r.header.version = version
        assert lib.secant_cubin_source_size(C.byref(r), C.byref(size)) == abi.ERROR_UNSUPPORTED_VERSION
    r.header.version = 3
    for field, value in (("asts_per_kernel", 33), ("num_targets", 0), ("threads_per_block", 100), ("num_kernels", 65536),
                         ("tile_rows", 4000)):
        bad = make_recipe(abi.SHAPE_TOGGLE_SSE, 3, 2, 8)
        setattr(bad, field, value)
        assert lib.secant_cubin_recipe_validate(C.byref(bad)) == abi.ERROR_INVALID_VALUE, field
    bad = make_recipe(abi.SHAPE_TOGGLE_SSE, 3, 2, 8)
    bad.header.shape = 99
    assert lib.secant_cubin_recipe_validate(C.byref(bad)) == abi.ERROR_UNSUPPORTED_SHAPE
    bad = make_recipe(abi.SHAPE_SSE, 3, 2)
    bad.threads_per_block = 1024
    assert lib.secant_cubin_recipe_validate(C.byref(bad)) == abi.ERROR_UNSUPPORTED_SHAPE
    # plan: storage is caller-owned and may be unaligned; the plan reports shape, size and recipe back
    cubin = C.create_string_buffer(b"\x7fELF-not-inspected", 64)
    need = C.c_size_t()
    assert lib.secant_cubin_plan_storage_size(C.byref(r), cubin, 64, C.byref(need)) == 0
    storage = C.create_string_buffer(need.value + 1)
    plan = C.c_void_p()
    assert lib.secant_cubin_plan_init(C.byref(r), cubin, 64, C.addressof(storage) + 1, need.value, C.byref(plan)) == 0
    assert lib.secant_cubin_plan_init(C.byref(r), cubin, 64, storage, 8, C.byref(plan)) == abi.ERROR_INSUFFICIENT_BUFFER
    assert not plan.value
    assert lib.secant_cubin_plan_init(C.byref(r), cubin, 64, C.addressof(storage) + 1, need.value, C.byref(plan)) == 0
    info = abi.PlanInfo()
    info.struct_size, info.version = C.sizeof(info), abi.PLAN_INFO_VERSION
    assert lib.secant_cubin_plan_info_get(plan, C.byref(info)) == 0
    assert info.shape == abi.SHAPE_TOGGLE_SSE and info.cubin_size == 64
    back = abi.init_header(abi.ToggleRecipe(), abi.RECIPE_VERSION, abi.SHAPE_TOGGLE_SSE)
    assert lib.secant_cubin_plan_recipe_get(plan, C.byref(back)) == 0
    assert (back.num_kernels, back.asts_per_kernel, back.num_constants, back.tile_rows) == (3, 32, 8, 31)
    wrong = abi.init_header(abi.TiledRecipe(), abi.RECIPE_VERSION, abi.SHAPE_SSE)
    assert lib.secant_cubin_plan_recipe_get(plan, C.byref(wrong)) == abi.ERROR_UNSUPPORTED_SHAPE
    # "specialize" validates programs and leaves the binary alone
    good = P.PackedPrograms([P.col(0) + P.bank(7) + P.tog2(31) + P.RET])
    pset = abi.ProgramSet()
    good.fill(pset)
    image = C.create_string_buffer(cubin.raw, 64)
    assert lib.secant_cubin_specialize_into(plan, C.byref(pset), image, 64) == 0 and image.raw == cubin.raw
    assert lib.secant_cubin_specialize_into(plan, C.byref(pset), image, 63) == abi.ERROR_INSUFFICIENT_BUFFER
    assert lib.secant_cubin_specialize_into(plan, C.byref(pset), image, 65) == abi.ERROR_INVALID_VALUE
    under = P.PackedPrograms([P.col(0) + P.op("MUL") + P.RET])
    under.fill(pset)
    assert lib.secant_cubin_specialize_into(plan, C.byref(pset), image, 64) == abi.ERROR_STACK_UNDERFLOW
    # runner creation is refused before any device work for a mismatching binary size
    runner = C.c_void_p()
    opts = abi.runner_options(1, 1)
    assert lib.secant_cubin_runner_create(plan, cubin, 63, C.byref(opts), C.byref(runner)) == abi.ERROR_INVALID_VALUE
    opts.num_workers = 0
    assert lib.secant_cubin_runner_create(plan, cubin, 64, C.byref(opts), C.byref(runner)) == abi.ERROR_INVALID_VALUE
    assert lib.secant_cubin_runner_destroy(None) == 0


def fake_matrix(address, elements, ld):
    m = abi.DeviceMatrix()
    m.address, m.num_elements, m.leading_dimension = address, elements, ld
    return m


def toggle_request(packed, rows=17, banks=13, bits=3, stride=3, out_ld=109, bank_elements=38):
    run = abi.init_header(abi.ToggleRun(), abi.RUN_VERSION, abi.SHAPE_TOGGLE_SSE)
    packed.fill(run.programs)
    n = len(packed.asts)
    run.input = fake_matrix(0x10000, 3 * rows, rows)
    run.targets = fake_matrix(0x20000, 2 * rows, rows)
    run.constants.address, run.constants.num_elements, run.constants.bank_stride = 0x30000, bank_elements, stride
    run.num_rows, run.num_targets, run.num_banks, run.toggle_bits = rows, 2, banks, bits
    run.output = fake_matrix(0x40000, n * 2 * out_ld, out_ld)
    return run


def validate(recipe, *runs):
    ptrs = (C.c_void_p * len(runs))(*[C.addressof(r) for r in runs])
    return S.hooks().sbt_validate_runs(C.byref(recipe), ptrs, C.c_size_t(len(runs)))


def test_request_validation_order_and_codes():
    fx = P.PackedPrograms([P.col(0) + P.col(1) + P.tog2(0) + P.bank(0) + P.op("MUL") + P.RET,
                           P.bank(0) + P.bank(1) + P.tog2(2) + P.RET])
    recipe = make_recipe(abi.SHAPE_TOGGLE_SSE, 3, 2, 2)
    assert validate(recipe, toggle_request(fx)) == 0
    r = toggle_request(fx); r.header.version = 2
    assert validate(recipe, r) == abi.ERROR_UNSUPPORTED_VERSION
    r = toggle_request(fx); r.header.flags = 4
    assert validate(recipe, r) == abi.ERROR_INVALID_VALUE
    r = toggle_request(fx); r.header.shape = abi.SHAPE_SSE
    assert validate(recipe, r) == abi.ERROR_UNSUPPORTED_SHAPE
    r = toggle_request(fx); r.header.struct_size -= 8
    assert validate(recipe, r) == abi.ERROR_INVALID_VALUE
    assert validate(recipe, toggle_request(fx, bits=2)) == abi.ERROR_BAD_PROGRAM          # program uses bit 2
    assert validate(recipe, toggle_request(fx, bank_elements=37)) == abi.ERROR_INSUFFICIENT_BUFFER
    assert validate(recipe, toggle_request(fx, stride=1)) == abi.ERROR_INVALID_VALUE
    assert validate(recipe, toggle_request(fx, out_ld=103)) == abi.ERROR_INVALID_VALUE    # fewer than 104 configurations
    assert validate(recipe, toggle_request(fx, banks=0)) == abi.ERROR_INVALID_VALUE
    assert validate(recipe, toggle_request(fx, bits=33)) == abi.ERROR_INVALID_VALUE
    r = toggle_request(fx); r.output.address = r.input.address + 8
    assert validate(recipe, r) == abi.ERROR_INVALID_VALUE                                   # output overlaps input
    r = toggle_request(fx); r.output.address += 2
    assert validate(recipe, r) == abi.ERROR_INVALID_VALUE                                   # misaligned device address
    r = toggle_request(fx); r.num_targets = 1
    assert validate(recipe, r) == abi.ERROR_INVALID_VALUE                                   # toggle runs use the recipe's target count
    r = toggle_request(fx); r.input.leading_dimension = 16
    assert validate(recipe, r) == abi.ERROR_INVALID_VALUE
    r = toggle_request(fx); r.num_banks = 2 ** 62
    assert validate(recipe, r) == abi.ERROR_OVERFLOW
    # batches: same program arrays everywhere, outputs disjoint from everything
    a, b = toggle_request(fx), toggle_request(fx)
    b.output.address = 0x80000
    assert validate(recipe, a, b) == 0
    b.output.address = a.output.address + 64
    assert validate(recipe, a, b) == abi.ERROR_INVALID_VALUE
    other = P.PackedPrograms(fx.asts)
    c = toggle_request(other); c.output.address = 0x80000
    assert validate(recipe, a, c) == abi.ERROR_INVALID_VALUE
    # the minimum toggle_bits over the entries bounds the programs
    d = toggle_request(fx, bits=2, out_ld=109); d.output.address = 0x80000
    assert validate(recipe, a, d) == abi.ERROR_BAD_PROGRAM
    # zero constants allow a null bank address but no stride
    nz = P.PackedPrograms([P.lit(2.0) + P.RET])
    recipe0 = make_recipe(abi.SHAPE_TOGGLE_SSE, 3, 2, 0)
    r0 = toggle_request(nz, banks=1, bits=0, stride=0, out_ld=1, bank_elements=0)
    r0.constants.address = 0
    assert validate(recipe0, r0) == 0
    r0.constants.bank_stride = 1
    assert validate(recipe0, r0) == abi.ERROR_INVALID_VALUE


def test_extension_fields_default_to_reference_behaviour():
    fx = P.PackedPrograms([P.bank(0) + P.RET, P.bank(1) + P.RET])
    recipe = make_recipe(abi.SHAPE_TOGGLE_SSE, 3, 2, 2)
    ext = abi.ToggleRunExt()
    plain = toggle_request(fx)
    C.memmove(C.addressof(ext), C.addressof(plain), C.sizeof(abi.ToggleRun))
    ext.base.header.struct_size = C.sizeof(ext)
    assert validate(recipe, ext) == 0                       # zeros: one shared table, as in the reference
    ext.program_bank_stride = 39
    assert validate(recipe, ext) == abi.ERROR_INSUFFICIENT_BUFFER  # two tables no longer fit in 38 elements
    ext.base.constants.num_elements = 39 + 38
    assert validate(recipe, ext) == 0


def test_reference_header_tests_pass_against_this_include_directory():
    """projects/secant/tests/c_header_test.c and cpp_header_test.cpp (descriptor layouts and
    initialisers, bytecode encoders, the entry points that need no device), compiled unmodified
    against include/ of this repository - where secant.h and secant_instructions.h forward to
    secant_b200.h - as C99 with -Wpedantic -Werror and as C++17, and linked against the library
    (oracle/Makefile, target header-tests)."""
    import subprocess
    import pytest
    ran = 0
    for name in ("secant_c_header_test", "secant_cpp_header_test"):
        binary = os.path.join(ROOT, "oracle", "_ref", name)
        if os.path.exists(binary):
            assert subprocess.run([binary], timeout=60).returncode == 0, name
            ran += 1
    if not ran:
        pytest.skip("oracle/_ref/secant_*_header_test are built only where the reference checkout exists")
