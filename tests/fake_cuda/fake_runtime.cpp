/*
 * fake_runtime.cpp - a deterministic model of the CUDA runtime for host-only failure tests of the
 * runner (csrc/runner.cpp), linked in place of cudart by the Makefile target `fakecuda`.
 *
 * What it models
 *   - every runtime entry point the runner calls, with a per-name call counter and a fault table:
 *     fake_arm(name, n, sticky) makes the n-th call of `name` from now on return an error (sticky:
 *     every call from the n-th on);
 *   - device and pinned allocations, streams and events as counted resources, so a test can ask
 *     whether everything was released;
 *   - stream order as vector clocks: every stream operation advances its stream, an event records
 *     the clock of its stream, a wait merges it, a host synchronisation merges it into what the
 *     host knows to be complete.  A launch marks the device buffers it reads or writes (the program
 *     records, the partial-sum scratch) as in use until its position; overwriting or freeing a
 *     buffer before the host knows that position to be complete is recorded as a violation;
 *   - the evaluator launch itself (launch_eval is stubbed here: no kernel exists in this build),
 *     the current-context query, and two hooks of the production code: worker-thread creation and
 *     program encoding can be told to fail.
 * Plays the role of the reference's fake driver and fault hooks
 * (projects/secant/tests/support/fake_cuda/cuda.h:27-63, tests/runner_failure_test.c:414-575).
 */
#include "evaluator.cuh"

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <map>
#include <mutex>
#include <new>
#include <string>
#include <vector>

namespace {

typedef std::map<const void*, uint64_t> Clock; /* stream -> position */

void merge(Clock& into, const Clock& from) {
    for (const auto& kv : from)
        if (into[kv.first] < kv.second) into[kv.first] = kv.second;
}

struct Allocation { size_t bytes; bool pinned; Clock busy; Clock written; };

struct Fault { unsigned calls = 0, fail_at = 0; bool sticky = false; };

struct World {
    std::mutex mutex;
    std::map<std::string, Fault> faults;
    std::map<void*, Allocation> allocations;
    std::map<const void*, Clock> streams;   /* live streams and their clocks */
    std::map<const void*, Clock> events;    /* live events and the clock they recorded */
    Clock host;                             /* what the host knows to be complete */
    unsigned violations = 0, launches = 0, threads_started = 0;
    void* context = reinterpret_cast<void*>(0x1234);
    bool no_context = false;
    std::string last_violation;
    std::atomic<bool> hold_encode{false}, entered_encode{false};
} world;

/* Counts the call and decides whether it fails.  Caller holds the mutex. */
bool failing(const char* name) {
    Fault& f = world.faults[name];
    ++f.calls;
    if (!f.fail_at) return false;
    if (f.calls == f.fail_at || (f.sticky && f.calls > f.fail_at)) return true;
    return false;
}
#define FAKE_ENTER(name)                              \
    std::lock_guard<std::mutex> lock(world.mutex);    \
    if (failing(name)) return cudaErrorUnknown

bool complete(const Clock& busy) {
    for (const auto& kv : busy) {
        const auto it = world.host.find(kv.first);
        if (it == world.host.end() || it->second < kv.second) return false;
    }
    return true;
}

Allocation* owner_of(const void* p) {
    for (auto& kv : world.allocations) {
        const char* base = static_cast<const char*>(kv.first);
        if (p >= base && p < base + kv.second.bytes) return &kv.second;
    }
    return nullptr;
}

void violation(const char* what) {
    ++world.violations;
    world.last_violation = what;
}

/* one more operation on a stream: returns the stream's clock after it */
Clock& advance(cudaStream_t stream) {
    Clock& c = world.streams[stream];
    ++c[stream];
    return c;
}

int fake_ctx_get_current(void** ctx) {
    std::lock_guard<std::mutex> lock(world.mutex);
    if (failing("cuCtxGetCurrent")) return 999;
    *ctx = world.no_context ? nullptr : world.context;
    return 0;
}

}  // namespace

extern "C" {

cudaError_t cudaGetDevice(int* device) { FAKE_ENTER("cudaGetDevice"); *device = 0; return cudaSuccess; }
cudaError_t cudaDeviceGetAttribute(int* value, enum cudaDeviceAttr attr, int) {
    FAKE_ENTER("cudaDeviceGetAttribute");
    *value = attr == cudaDevAttrMultiProcessorCount ? 148 : 232448;
    return cudaSuccess;
}
cudaError_t cudaGetDriverEntryPoint(const char* symbol, void** entry, unsigned long long, cudaDriverEntryPointQueryResult* status) {
    std::lock_guard<std::mutex> lock(world.mutex);
    const bool known = !std::strcmp(symbol, "cuCtxGetCurrent");
    *entry = known ? reinterpret_cast<void*>(&fake_ctx_get_current) : nullptr;
    *status = known ? cudaDriverEntryPointSuccess : cudaDriverEntryPointSymbolNotFound;
    return cudaSuccess;
}
cudaError_t cudaGetLastError(void) { return cudaSuccess; }
const char* cudaGetErrorString(cudaError_t error) { return error == cudaSuccess ? "no error" : "injected failure"; }

cudaError_t cudaMalloc(void** ptr, size_t bytes) {
    FAKE_ENTER("cudaMalloc");
    void* p = std::malloc(bytes ? bytes : 1);
    if (!p) return cudaErrorMemoryAllocation;
    world.allocations[p] = Allocation{bytes, false, {}, {}};
    *ptr = p;
    return cudaSuccess;
}
cudaError_t cudaFree(void* ptr) {
    FAKE_ENTER("cudaFree");
    if (!ptr) return cudaSuccess; /* context initialisation idiom */
    const auto it = world.allocations.find(ptr);
    if (it == world.allocations.end() || it->second.pinned) { violation("cudaFree of an unknown pointer"); return cudaErrorInvalidValue; }
    if (!complete(it->second.busy)) violation("device buffer freed while a launch may still use it");
    world.allocations.erase(it);
    std::free(ptr);
    return cudaSuccess;
}
cudaError_t cudaHostAlloc(void** ptr, size_t bytes, unsigned) {
    FAKE_ENTER("cudaHostAlloc");
    void* p = std::malloc(bytes ? bytes : 1);
    if (!p) return cudaErrorMemoryAllocation;
    world.allocations[p] = Allocation{bytes, true, {}, {}};
    *ptr = p;
    return cudaSuccess;
}
cudaError_t cudaFreeHost(void* ptr) {
    FAKE_ENTER("cudaFreeHost");
    const auto it = world.allocations.find(ptr);
    if (it == world.allocations.end() || !it->second.pinned) { violation("cudaFreeHost of an unknown pointer"); return cudaErrorInvalidValue; }
    if (!complete(it->second.busy)) violation("pinned buffer freed while a copy may still read it");
    world.allocations.erase(it);
    std::free(ptr);
    return cudaSuccess;
}
cudaError_t cudaMemcpyAsync(void* dst, const void* src, size_t bytes, enum cudaMemcpyKind, cudaStream_t stream) {
    FAKE_ENTER("cudaMemcpyAsync");
    Allocation* d = owner_of(dst);
    Allocation* s = owner_of(src);
    if (!d || !s || d->bytes < bytes || s->bytes < bytes) { violation("copy outside an allocation"); return cudaErrorInvalidValue; }
    if (!complete(d->busy)) violation("program records overwritten while a launch may still read them");
    const Clock& now = advance(stream);
    merge(s->busy, now); /* the pinned source is read until the copy has run */
    d->written = now;    /* readers must be ordered after this position */
    std::memcpy(dst, src, bytes);
    return cudaSuccess;
}
cudaError_t cudaMemset2DAsync(void*, size_t, int, size_t, size_t, cudaStream_t stream) {
    FAKE_ENTER("cudaMemset2DAsync");
    advance(stream);
    return cudaSuccess;
}
cudaError_t cudaStreamCreateWithFlags(cudaStream_t* stream, unsigned) {
    FAKE_ENTER("cudaStreamCreateWithFlags");
    *stream = reinterpret_cast<cudaStream_t>(std::malloc(8));
    world.streams[*stream] = Clock();
    return cudaSuccess;
}
cudaError_t cudaStreamDestroy(cudaStream_t stream) {
    FAKE_ENTER("cudaStreamDestroy");
    if (!world.streams.erase(stream)) { violation("cudaStreamDestroy of an unknown stream"); return cudaErrorInvalidValue; }
    std::free(stream);
    return cudaSuccess;
}
cudaError_t cudaStreamSynchronize(cudaStream_t stream) {
    FAKE_ENTER("cudaStreamSynchronize");
    const auto it = world.streams.find(stream);
    if (it == world.streams.end()) { violation("cudaStreamSynchronize of an unknown stream"); return cudaErrorInvalidValue; }
    merge(world.host, it->second);
    return cudaSuccess;
}
cudaError_t cudaStreamWaitEvent(cudaStream_t stream, cudaEvent_t event, unsigned) {
    FAKE_ENTER("cudaStreamWaitEvent");
    const auto e = world.events.find(event);
    if (e == world.events.end() || !world.streams.count(stream)) { violation("wait on an unknown stream or event"); return cudaErrorInvalidValue; }
    merge(world.streams[stream], e->second);
    return cudaSuccess;
}
cudaError_t cudaEventCreateWithFlags(cudaEvent_t* event, unsigned) {
    FAKE_ENTER("cudaEventCreate");
    *event = reinterpret_cast<cudaEvent_t>(std::malloc(8));
    world.events[*event] = Clock();
    return cudaSuccess;
}
cudaError_t cudaEventCreate(cudaEvent_t* event) { return cudaEventCreateWithFlags(event, 0); }
cudaError_t cudaEventDestroy(cudaEvent_t event) {
    FAKE_ENTER("cudaEventDestroy");
    if (!world.events.erase(event)) { violation("cudaEventDestroy of an unknown event"); return cudaErrorInvalidValue; }
    std::free(event);
    return cudaSuccess;
}
cudaError_t cudaEventRecord(cudaEvent_t event, cudaStream_t stream) {
    FAKE_ENTER("cudaEventRecord");
    if (!world.events.count(event) || !world.streams.count(stream)) { violation("record on an unknown stream or event"); return cudaErrorInvalidValue; }
    world.events[event] = advance(stream);
    return cudaSuccess;
}
cudaError_t cudaEventSynchronize(cudaEvent_t event) {
    FAKE_ENTER("cudaEventSynchronize");
    const auto e = world.events.find(event);
    if (e == world.events.end()) { violation("cudaEventSynchronize of an unknown event"); return cudaErrorInvalidValue; }
    merge(world.host, e->second);
    return cudaSuccess;
}
cudaError_t cudaEventElapsedTime(float* ms, cudaEvent_t start, cudaEvent_t stop) {
    FAKE_ENTER("cudaEventElapsedTime");
    if (!complete(world.events[start]) || !complete(world.events[stop])) violation("elapsed time of an event the host has not waited for");
    *ms = 1.0f;
    return cudaSuccess;
}

/* ---- hooks of the production code (runner.cpp, compiled with SECANT_B200_FAULT_HOOKS) ---- */
int secant_b200_fault_hook(const char* site) {
    if (!std::strcmp(site, "encode")) { /* a test may park the worker here to catch a run in the act */
        world.entered_encode.store(true);
        while (world.hold_encode.load()) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    std::lock_guard<std::mutex> lock(world.mutex);
    if (!std::strcmp(site, "thread") && !failing("thread")) { ++world.threads_started; return 0; }
    if (!std::strcmp(site, "thread")) return 1;
    return failing(site) ? 1 : 0;
}

/* ---- control surface for the tests ---- */
#define FAKE_EXPORT __attribute__((visibility("default")))
FAKE_EXPORT void fake_reset(void) {
    std::lock_guard<std::mutex> lock(world.mutex);
    world.faults.clear();
    world.violations = 0;
    world.launches = 0;
    world.no_context = false;
    world.context = reinterpret_cast<void*>(0x1234);
    world.last_violation.clear();
}
FAKE_EXPORT void fake_arm(const char* name, unsigned nth, int sticky) {
    std::lock_guard<std::mutex> lock(world.mutex);
    Fault& f = world.faults[name];
    f.fail_at = f.calls + nth;
    f.sticky = sticky != 0;
}
FAKE_EXPORT unsigned fake_calls(const char* name) {
    std::lock_guard<std::mutex> lock(world.mutex);
    return world.faults[name].calls;
}
/* names of the calls made since the last reset, separated by newlines */
FAKE_EXPORT size_t fake_call_names(char* out, size_t capacity) {
    std::lock_guard<std::mutex> lock(world.mutex);
    std::string all;
    for (const auto& kv : world.faults)
        if (kv.second.calls) all += kv.first + "\n";
    if (out && capacity) {
        std::strncpy(out, all.c_str(), capacity - 1);
        out[capacity - 1] = 0;
    }
    return all.size();
}
/* what[0..5] = live allocations, live streams, live events, violations, launches, worker threads started */
FAKE_EXPORT void fake_state(unsigned* what) {
    std::lock_guard<std::mutex> lock(world.mutex);
    what[0] = (unsigned)world.allocations.size();
    what[1] = (unsigned)world.streams.size();
    what[2] = (unsigned)world.events.size();
    what[3] = world.violations;
    what[4] = world.launches;
    what[5] = world.threads_started;
}
FAKE_EXPORT const char* fake_last_violation(void) { return world.last_violation.c_str(); }
FAKE_EXPORT void fake_set_context(int which) { /* 0: none, n: context n */
    std::lock_guard<std::mutex> lock(world.mutex);
    world.no_context = which == 0;
    world.context = reinterpret_cast<void*>((uintptr_t)0x1234 + (uintptr_t)which - 1);
}
FAKE_EXPORT void fake_hold_encoding(int on) { world.entered_encode.store(false); world.hold_encode.store(on != 0); }
FAKE_EXPORT int fake_encoding_entered(void) { return world.entered_encode.load() ? 1 : 0; }
FAKE_EXPORT void* fake_device_buffer(size_t bytes) { /* stands for a caller's device allocation */
    void* p = nullptr;
    return cudaMalloc(&p, bytes) == cudaSuccess ? p : nullptr;
}
FAKE_EXPORT void fake_device_release(void* p) { cudaFree(p); }

}  // extern "C"

/* ---- the evaluator's launch interface, without kernels ---- */
namespace sb {

cudaError_t configure_kernels() {
    std::lock_guard<std::mutex> lock(world.mutex);
    return failing("configure_kernels") ? cudaErrorUnknown : cudaSuccess;
}

cudaError_t launch_eval(const DeviceBatch& batch, const EvalProblem&, const LaunchPlan& plan, float* partial, cudaStream_t stream,
                        unsigned* launches) {
    std::lock_guard<std::mutex> lock(world.mutex);
    *launches = 0;
    if (failing("launch_eval")) return cudaErrorUnknown;
    Allocation* records = owner_of(batch.programs);
    if (!records) { violation("launch with program records outside any device allocation"); return cudaErrorInvalidValue; }
    if (plan.partial_elements) {
        Allocation* scratch = owner_of(partial);
        if (!scratch || scratch->bytes < plan.partial_elements * sizeof(float)) {
            violation("launch with too little scratch for its partial sums");
            return cudaErrorInvalidValue;
        }
        merge(scratch->busy, advance(stream));
    }
    const Clock& now = advance(stream);
    for (const auto& kv : records->written) { /* ordered by an event the stream waited on, or known complete by the host */
        const auto it = now.find(kv.first);
        const auto known = world.host.find(kv.first);
        const bool by_stream = it != now.end() && it->second >= kv.second;
        const bool by_host = known != world.host.end() && known->second >= kv.second;
        if (!by_stream && !by_host) { violation("launch not ordered after the upload of its program records"); break; }
    }
    merge(records->busy, now);
    ++world.launches;
    *launches = 2;
    return cudaSuccess;
}

cudaError_t launch_rk4(const DeviceBatch&, const Rk4Problem&, size_t, unsigned, cudaStream_t) { return cudaErrorUnknown; }

cudaError_t launch_gram(const float* predictions, size_t prediction_ld, uint32_t, const float*, size_t, uint32_t, uint32_t, uint32_t batch_programs,
                        float*, size_t, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(world.mutex);
    if (failing("launch_gram")) return cudaErrorUnknown;
    Allocation* scratch = owner_of(predictions);
    if (!scratch || scratch->bytes < (size_t)batch_programs * prediction_ld * sizeof(float)) {
        violation("statistics launch with too little scratch for its predictions");
        return cudaErrorInvalidValue;
    }
    merge(scratch->busy, advance(stream));
    ++world.launches;
    return cudaSuccess;
}

}  // namespace sb
