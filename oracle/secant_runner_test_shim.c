/*
 * secant_runner_test_shim.c - test infrastructure: runs the parts of the reference's own GPU test of
 * the runner API one by one.
 *
 * projects/secant/tests/toggle_cuda_test.c is included where it lies (the Makefile passes its
 * directory with -I; nothing is copied) with its main() renamed out of the way.  Its main() runs
 * toggle_test, edge_test, random_test and static_test in a row and every failed check exits the
 * process.  One check at the end of edge_test searches the buffer secant_cubin_specialize_into()
 * wrote for the machine-code bytes of one instruction ("bit 31 encoding"); a library that patches no
 * machine code has nothing to show there, so the test as shipped never reaches random_test and
 * static_test.  This driver calls the same static functions:
 *   (no argument)  toggle_test(1), toggle_test(3), random_test(1), random_test(8), random_test(32),
 *                  static_test() - everything that compares scores with the reference host evaluator;
 *   edge           edge_test() alone: its score comparisons run first, then the machine-code check
 *                  ends the process with its message, which the caller of this binary expects.
 */
#define main secant_toggle_cuda_test_main_unused
#include "toggle_cuda_test.c"
#undef main

int main(int argc, char **argv) {
    CUdevice device;
    CUcontext context;
    CUDA(cuInit(0));
    CUDA(cuDeviceGet(&device, 0));
    CUDA(cuDevicePrimaryCtxRetain(&context, device));
    CUDA(cuCtxSetCurrent(context));
    if (argc > 1 && !strcmp(argv[1], "edge")) {
        edge_test();
    } else {
        toggle_test(1);
        toggle_test(3);
        random_test(1);
        random_test(8);
        random_test(32);
        static_test();
        puts("scores of the toggle, random and static parts agree with the reference host evaluator");
    }
    CUDA(cuDevicePrimaryCtxRelease(device));
    return 0;
}
