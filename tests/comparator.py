"""Compiled-topology comparator: a measuring stick, not part of the product path.

The reference scores a population with kernels whose body is machine code patched into a
compiled template (projects/secant/s_cubin_generate_toggle_sse.c:339-386).  Running patched
machine code written for another GPU generation is not an option here, so this module answers
the question "how fast is the reference's KERNEL DESIGN on this GPU when a compiler writes the
program bodies": it generates CUDA source with the same topology

  * grid.x = row tiles, grid.y = blocks of configurations, one THREAD per configuration;
  * the (inputs + targets) x tile_rows tile staged in shared memory by the CTA;
  * the coefficient bank of the thread's configuration in registers;
  * A programs per kernel, each with its own squared-error accumulator per target;
  * one atomicAdd per (program, target, configuration) and tile;

and, where the reference leaves a patchable island, plain expression code for each program.
The source is compiled with NVRTC at run time (the reference control experiment does the same,
projects/secant/docs/BENCHMARKS.md:123-128) and launched through the driver API on torch's
stream.  Compile time is reported separately: avoiding it is the reason the reference patches
machine code, and the reason this repository interprets records instead.

Two math modes: "fast" uses the reference's compile flags (--use_fast_math --fmad=false,
projects/secant/tests/toggle_cuda_test.c:74), "accurate" drops --use_fast_math so that
division and the transcendental functions have the accuracy of the product kernel.
"""
import ctypes as C
import struct
import time

import numpy as np

from secant_b200.programs import OP, _WIDTH

_BINARY = {OP["ADD"]: "__fadd_rn({a}, {b})", OP["SUB"]: "__fsub_rn({a}, {b})", OP["MUL"]: "__fmul_rn({a}, {b})",
           OP["DIV"]: "({a} / {b})", OP["MIN"]: "fminf({a}, {b})", OP["MAX"]: "fmaxf({a}, {b})"}
_UNARY = {OP["NEG"]: "(-{a})", OP["SQRT"]: "sqrtf({a})", OP["RCP"]: "(1.0f / {a})", OP["ABS"]: "fabsf({a})",
          OP["SIN"]: "sinf({a})", OP["COS"]: "cosf({a})", OP["EX2"]: "exp2f({a})", OP["LG2"]: "log2f({a})",
          OP["RSQRT"]: "(1.0f / sqrtf({a}))", OP["TANH"]: "tanhf({a})", OP["EXP"]: "expf({a})", OP["LOG"]: "logf({a})"}


class _Body:
    """Straight-line single-assignment code for one program (routines inlined, arguments bound once)."""

    def __init__(self, routines, num_inputs, tag):
        self.routines, self.num_inputs, self.tag = routines, num_inputs, tag
        self.lines, self.count = [], 0

    def _emit(self, expr):
        name = f"v{self.tag}_{self.count}"
        self.count += 1
        self.lines.append(f"   const float {name} = {expr};")
        return name

    def run(self, code, args=(), depth=0):
        if depth > 8:
            raise ValueError("routine nesting deeper than the reference allows")
        stack, at = [], 0
        while True:
            o = code[at]
            if o == OP["RET"]:
                if len(stack) != 1:
                    raise ValueError("program does not leave exactly one value")
                return stack[0]
            if o == OP["COL"]:
                stack.append(f"input{code[at + 1]}")
            elif o == OP["BANK"]:
                stack.append(f"input{self.num_inputs + code[at + 1]}")
            elif o == OP["LIT"]:
                stack.append(f"__int_as_float(0x{struct.unpack('<I', code[at + 1:at + 5])[0]:08x})")
            elif o == OP["AFFINE"]:
                scale, offset = struct.unpack("<II", code[at + 2:at + 10])
                stack.append(self._emit(f"__fadd_rn(__fmul_rn(input{self.num_inputs + code[at + 1]}, "
                                        f"__int_as_float(0x{scale:08x})), __int_as_float(0x{offset:08x}))"))
            elif o == OP["ARG"]:
                stack.append(args[code[at + 1]])
            elif o == OP["TOG2"]:
                b = stack.pop()
                a = stack.pop()
                stack.append(self._emit(f"((permutation >> {code[at + 1]}) & 1u) ? {b} : {a}"))
            elif o == OP["TOG4"]:
                leaves = [stack.pop() for _ in range(4)][::-1]
                b0, b1 = code[at + 1], code[at + 2]
                lo = f"(((permutation >> {b0}) & 1u) ? {leaves[1]} : {leaves[0]})"
                hi = f"(((permutation >> {b0}) & 1u) ? {leaves[3]} : {leaves[2]})"
                stack.append(self._emit(f"((permutation >> {b1}) & 1u) ? {hi} : {lo}"))
            elif o == OP["ROUTINE"]:
                body = self.routines[code[at + 1]]
                arity = _routine_arity(body)
                bound = [stack.pop() for _ in range(arity)][::-1]
                stack.append(self.run(body, bound, depth + 1))
            elif o == OP["FMA"]:
                c = stack.pop()
                b = stack.pop()
                a = stack.pop()
                stack.append(self._emit(f"fmaf({a}, {b}, {c})"))
            elif o in _BINARY:
                b = stack.pop()
                a = stack.pop()
                stack.append(self._emit(_BINARY[o].format(a=a, b=b)))
            elif o in _UNARY:
                stack.append(self._emit(_UNARY[o].format(a=stack.pop())))
            else:
                raise ValueError(f"opcode 0x{o:02x} has no expression form")
            at += _WIDTH.get(o, 1)


def _routine_arity(code):
    at, arity = 0, 0
    while code[at] != OP["RET"]:
        if code[at] == OP["ARG"]:
            arity = max(arity, code[at + 1] + 1)
        at += _WIDTH.get(code[at], 1)
    return arity


def generate_source(packed, first, count, asts_per_kernel, num_inputs, num_constants, num_targets, tile_rows,
                    threads_per_block):
    """CUDA source scoring programs [first, first + count): ceil(count / asts_per_kernel) kernels
    named secant_compiled_toggle_sse_NNN with the reference template's parameter list."""
    cols = num_inputs + num_targets
    out = ["// configuration = bank * 2^toggle_bits + permutation"]
    kernels = (count + asts_per_kernel - 1) // asts_per_kernel
    for k in range(kernels):
        out.append(f'extern "C" __global__ __launch_bounds__({threads_per_block}) void secant_compiled_toggle_sse_{k:03d}(\n'
                   " const float *input, unsigned long long input_ld, const float *targets, unsigned long long target_ld,\n"
                   " const float *banks, unsigned long long bank_stride,\n"
                   " unsigned long long num_rows, unsigned long long num_configurations, unsigned int toggle_bits,\n"
                   " float *output, unsigned long long output_ld) {")
        out.append(f" __shared__ float tile[{cols * tile_rows}];")
        out.append(f" const unsigned long long row_start = (unsigned long long)blockIdx.x * {tile_rows};")
        out.append(f" for (unsigned int i = threadIdx.x; i < {cols * tile_rows}; i += blockDim.x) {{")
        out.append(f"  const unsigned int col = i / {tile_rows}, row = i % {tile_rows};")
        out.append("  const unsigned long long absolute_row = row_start + row;")
        out.append(f"  tile[i] = absolute_row >= num_rows ? 0.f : (col < {num_inputs} ? input[col * input_ld + absolute_row]"
                   f" : targets[(col - {num_inputs}) * target_ld + absolute_row]);")
        out.append(" }\n __syncthreads();")
        out.append(" #pragma unroll 1")
        out.append(" for (unsigned long long configuration = (unsigned long long)blockIdx.y * blockDim.x + threadIdx.x;")
        out.append("      configuration < num_configurations; configuration += (unsigned long long)gridDim.y * blockDim.x) {")
        out.append("  const unsigned int permutation = (unsigned int)configuration;")
        out.append("  const unsigned long long bank = configuration >> toggle_bits;")
        for c in range(num_constants):
            out.append(f"  const float input{num_inputs + c} = banks[bank * bank_stride + {c}];")
        here = range(first + k * asts_per_kernel, min(first + count, first + (k + 1) * asts_per_kernel))
        for a in here:
            for t in range(num_targets):
                out.append(f"  float sse_{a - first}_{t} = 0.f;")
        out.append("  #pragma unroll 1")
        out.append(f"  for (unsigned int row = 0; row < {tile_rows} && row_start + row < num_rows; ++row) {{")
        for c in range(num_inputs):
            out.append(f"   const float input{c} = tile[{c * tile_rows} + row];")
        for t in range(num_targets):
            out.append(f"   const float target{t} = tile[{(num_inputs + t) * tile_rows} + row];")
        for a in here:
            body = _Body(packed.routines, num_inputs, a - first)
            value = body.run(packed.asts[a])
            out.extend(body.lines)
            for t in range(num_targets):
                out.append(f"   {{ const float err = __fsub_rn(target{t}, {value}); sse_{a - first}_{t} = fmaf(err, err, sse_{a - first}_{t}); }}")
        out.append("  }")
        for a in here:
            for t in range(num_targets):
                out.append(f"  atomicAdd(output + {(a - first) * num_targets + t}ull * output_ld + configuration, sse_{a - first}_{t});")
        out.append(" }\n}")
    return "\n".join(out) + "\n", kernels


def _check(result, what):
    code = result[0]
    if int(code) != 0:
        raise RuntimeError(f"{what} failed: {code}")
    return result[1:] if len(result) > 2 else (result[1] if len(result) == 2 else None)


def compile_cubin(source, arch, fast_math):
    """NVRTC: source -> cubin for `arch` (for example "sm_100a").  Returns (cubin bytes, seconds)."""
    from cuda.bindings import nvrtc
    t0 = time.perf_counter()
    prog = _check(nvrtc.nvrtcCreateProgram(source.encode(), b"secant_compiled.cu", 0, [], []), "nvrtcCreateProgram")
    flags = [f"--gpu-architecture={arch}".encode(), b"--std=c++14", b"--fmad=false"]
    if fast_math:
        flags.append(b"--use_fast_math")
    status = nvrtc.nvrtcCompileProgram(prog, len(flags), flags)[0]
    if int(status) != 0:
        size = _check(nvrtc.nvrtcGetProgramLogSize(prog), "nvrtcGetProgramLogSize")
        log = b" " * size
        nvrtc.nvrtcGetProgramLog(prog, log)
        raise RuntimeError("NVRTC: " + log.decode(errors="replace")[:2000])
    size = _check(nvrtc.nvrtcGetCUBINSize(prog), "nvrtcGetCUBINSize")
    cubin = b" " * size
    _check(nvrtc.nvrtcGetCUBIN(prog, cubin), "nvrtcGetCUBIN")
    nvrtc.nvrtcDestroyProgram(prog)
    return cubin, time.perf_counter() - t0


class CompiledPopulation:
    """Programs [first, first + count) of `packed` compiled into modules of kernels x asts_per_kernel
    programs (the reference's recipe capacity), ready to score on the current CUDA device."""

    def __init__(self, packed, num_inputs, num_constants, num_targets=1, first=0, count=None, num_kernels=8,
                 asts_per_kernel=8, tile_rows=128, threads_per_block=128, fast_math=True):
        import torch
        from cuda.bindings import driver
        self.driver, self.torch = driver, torch
        count = len(packed.asts) - first if count is None else count
        self.first, self.count = first, count
        self.num_inputs, self.num_constants, self.num_targets = num_inputs, num_constants, num_targets
        self.tile_rows, self.threads, self.asts_per_kernel = tile_rows, threads_per_block, asts_per_kernel
        major, minor = torch.cuda.get_device_capability()
        arch = f"sm_{major}{minor}{'a' if major >= 9 else ''}"
        self.modules, self.compile_seconds, self.load_seconds = [], 0.0, 0.0
        capacity = num_kernels * asts_per_kernel
        torch.zeros(1, device="cuda")  # torch's primary context is current from here on
        for base in range(first, first + count, capacity):
            n = min(capacity, first + count - base)
            source, kernels = generate_source(packed, base, n, asts_per_kernel, num_inputs, num_constants, num_targets,
                                              tile_rows, threads_per_block)
            cubin, seconds = compile_cubin(source, arch, fast_math)
            self.compile_seconds += seconds
            t0 = time.perf_counter()
            module = _check(driver.cuModuleLoadData(cubin), "cuModuleLoadData")
            functions = [_check(driver.cuModuleGetFunction(module, f"secant_compiled_toggle_sse_{k:03d}".encode()),
                                "cuModuleGetFunction") for k in range(kernels)]
            self.load_seconds += time.perf_counter() - t0
            self.modules.append((module, functions, base, n))

    def score(self, x, y, banks, num_banks, toggle_bits, out):
        """Adds squared errors into `out` ([count][targets][configurations], zeroed by the caller)
        for shared banks [bank][slot]; returns the number of kernel launches."""
        driver, torch = self.driver, self.torch
        rows = x.shape[-1]
        configs = num_banks << toggle_bits
        grid_x = (rows + self.tile_rows - 1) // self.tile_rows
        grid_y = min(65535, (configs + self.threads - 1) // self.threads)
        stream = torch.cuda.current_stream().cuda_stream
        out_ld = out.shape[-1]
        bank_stride = banks.shape[-1] if banks is not None else 0
        launches = 0
        for _, functions, base, n in self.modules:
            for fn in functions:
                dst = out.data_ptr() + (base - self.first) * self.num_targets * out_ld * 4  # kernels index from the module base
                values = (x.data_ptr(), x.shape[-1], y.data_ptr(), y.shape[-1], banks.data_ptr() if banks is not None else 0,
                          bank_stride, rows, configs, toggle_bits, dst, out_ld)
                types = (C.c_void_p, C.c_ulonglong, C.c_void_p, C.c_ulonglong, C.c_void_p, C.c_ulonglong, C.c_ulonglong,
                         C.c_ulonglong, C.c_uint, C.c_void_p, C.c_ulonglong)
                _check(driver.cuLaunchKernel(fn, grid_x, grid_y, 1, self.threads, 1, 1, 0, stream, (values, types), 0),
                       "cuLaunchKernel")
                launches += 1
        return launches

    def close(self):
        for module, _, _, _ in self.modules:
            self.driver.cuModuleUnload(module)
        self.modules = []
