"""Python host mirror of the Secant C API for the B200-native evaluator.

abi       ctypes declarations of include/secant_b200.h and the library loader
programs  bytecode builders and the seeded synthetic workloads
runner    Runner: the reference's create / run / destroy sequence over torch device memory
"""
from . import abi, programs  # noqa: F401
