/*
 * runner.cpp - the blocking bulk runner: validate, clear, encode -> upload -> evaluate.
 *
 * Mirrors the reference runner's contract (projects/secant/s_cubin_runner.c:243-352,
 * s_runner_pipeline.c:320-427) with a different pipeline underneath.  The reference
 * specializes machine code on worker threads, loads one CUDA module per program batch,
 * launches it, waits and unloads it, so the GPU idles between modules.  Here worker
 * threads encode program batches into records, the calling thread copies each batch to
 * the device through pinned memory on a copy stream, and the resident evaluator kernel
 * of batch k runs while batch k+1 is being encoded and uploaded.  Nothing is loaded or
 * unloaded, so the "module" counters of the statistics count program batches.
 */
#include "evaluator.cuh"
#include "internal.h"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

/* Fault hooks: in the host-only test build (Makefile target `fakecuda`) the named sites ask the test
 * harness whether to fail; in the product they compile to nothing. */
#ifdef SECANT_B200_FAULT_HOOKS
extern "C" int secant_b200_fault_hook(const char* site);
#define SB_FAULT(site) (secant_b200_fault_hook(site) != 0)
#else
#define SB_FAULT(site) false
#endif

namespace sb {

std::atomic<uint64_t> g_kernel_launches{0};
std::atomic<uint64_t> g_row_stream_bytes{0};
void note_kernel_launches(unsigned n) { g_kernel_launches.fetch_add(n); }

namespace {

double now_seconds() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

/* cuCtxGetCurrent without linking the driver library: the library must load on machines
 * that have no GPU driver at all. */
void* current_context(bool* ok) {
    typedef int (*GetCurrentFn)(void**);
    static GetCurrentFn fn = nullptr;
    static bool resolved = false;
    if (!resolved) {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &entry, cudaEnableDefault, &status) == cudaSuccess &&
            status == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<GetCurrentFn>(entry);
        resolved = true;
    }
    void* ctx = nullptr;
    *ok = fn && fn(&ctx) == 0;
    return ctx;
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

enum SlotState { SLOT_FREE = 0, SLOT_ENCODING, SLOT_READY, SLOT_IN_FLIGHT };

struct Slot {
    EncodedBatch enc;
    SlotState state = SLOT_FREE;
    size_t batch = 0;              /* batch index held */
    size_t first_program = 0;
    SecantResult status = SECANT_SUCCESS;
    double encode_seconds = 0;
    void* pinned = nullptr;
    size_t pinned_cap = 0;
    void* device = nullptr;
    size_t device_cap = 0;
    cudaEvent_t uploaded = nullptr;
    std::vector<cudaEvent_t> done;  /* one per compute stream */
    std::vector<char> used;         /* which compute streams this batch touched */
};

}  // namespace
}  // namespace sb

using namespace sb;

constexpr size_t kDefaultScratchFloats = (size_t)1 << 28; /* 1 GiB of per-split partial sums per launch */

struct SecantCubinRunnerImpl {
    SecantCubinPlan owned_plan;     /* used when created straight from a recipe */
    const SecantCubinPlan* plan = nullptr;
    void* context = nullptr;
    int device = 0, sm_count = 0;
    size_t smem_limit = 0;
    std::vector<cudaStream_t> streams;
    std::vector<void*> scratch;      /* per compute stream: partial sums of the launch in flight */
    std::vector<size_t> scratch_cap;
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev_cleared = nullptr, ev_start = nullptr, ev_stop = nullptr;
    std::vector<Slot> slots;
    std::vector<std::thread> workers;
    std::vector<double> worker_seconds;
    std::mutex mutex;
    std::condition_variable cv_work, cv_ready;
    /* current job, guarded by mutex */
    bool job_active = false;
    const SecantAstProgramSet* job_programs = nullptr;
    const uint8_t* job_arity = nullptr;
    ProgramRules job_rules;
    size_t job_batch_size = 0, job_num_batches = 0, job_next_batch = 0;
    bool job_abort = false;
    /* handle state */
    bool active = false, failed = false, shutdown = false;
    size_t populations = 0;        /* device-resident populations created from this runner and not yet destroyed */
    size_t scratch_limit = kDefaultScratchFloats; /* secant_b200_runner_set_scratch_limit */
    uint32_t fast_math = 0;        /* secant_b200_runner_set_math */
    std::string last_error;
};


/* A population kept on the device: programs validated, encoded and uploaded once, then
 * scored any number of times (new data, new coefficient banks) without touching the host
 * copies again. */
struct SecantB200PopulationImpl {
    SecantCubinRunnerImpl* runner = nullptr;
    std::vector<uint8_t> ast_bytes, routine_bytes;
    std::vector<const uint8_t*> ast_ptrs, routine_ptrs;
    SecantAstProgramSet set{};
    unsigned toggle_bits = 0;
    struct Resident { void* device = nullptr; std::vector<DeviceBatch> views; size_t first = 0; };
    std::vector<Resident> batches;
    uint64_t total_ops = 0;
};

namespace {

void worker_main(SecantCubinRunnerImpl* r, size_t worker_index) {
    std::unique_lock<std::mutex> lock(r->mutex);
    for (;;) {
        Slot* slot = nullptr;
        r->cv_work.wait(lock, [&] {
            if (r->shutdown) return true;
            if (!r->job_active || r->job_abort || r->job_next_batch >= r->job_num_batches) return false;
            for (auto& s : r->slots)
                if (s.state == SLOT_FREE) { slot = &s; return true; }
            return false;
        });
        if (r->shutdown) return;
        const size_t batch = r->job_next_batch++;
        slot->state = SLOT_ENCODING;
        slot->batch = batch;
        const SecantAstProgramSet* programs = r->job_programs;
        const uint8_t* arity = r->job_arity;
        const ProgramRules rules = r->job_rules;
        const size_t first = batch * r->job_batch_size;
        const size_t count = std::min(r->job_batch_size, programs->asts.count - first);
        lock.unlock();

        const double begin = now_seconds();
        SecantResult status = SECANT_SUCCESS;
        try { /* an allocation failure inside the encoder must reach the caller as a result code */
            slot->enc.clear();
            slot->enc.programs.reserve(count);
            for (size_t i = 0; i < count && status == SECANT_SUCCESS; ++i) {
                status = encode_program(programs->asts.items[first + i], programs->routines, arity, rules, slot->enc);
                if (status == SECANT_SUCCESS) slot->enc.programs.back().index = (uint32_t)(first + i);
            }
        } catch (...) {
            status = SECANT_ERROR_ALLOCATION_FAILED;
        }
        if (SB_FAULT("encode")) status = SECANT_ERROR_BAD_PROGRAM;
        const double spent = now_seconds() - begin;

        lock.lock();
        slot->first_program = first;
        slot->status = status;
        slot->encode_seconds = spent;
        slot->state = SLOT_READY;
        r->worker_seconds[worker_index] += spent;
        r->cv_ready.notify_all();
    }
}

SecantResult cuda_fail(SecantCubinRunnerImpl* r, cudaError_t e, const char* what) {
    char text[256];
    std::snprintf(text, sizeof(text), "%s: %s", what, cudaGetErrorString(e));
    r->last_error = text;
    return SECANT_ERROR_DRIVER_FAILED;
}
#define SB_CUDA(call, what) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return cuda_fail(r, e_, what); } while (0)

SecantResult runner_init(SecantCubinRunnerImpl* r, const SecantCubinRunnerOptions* options) {
    bool ok = false;
    SB_CUDA(cudaGetDevice(&r->device), "cudaGetDevice");
    SB_CUDA(cudaFree(nullptr), "context initialisation");
    r->context = current_context(&ok);
    if (!ok || !r->context) { r->last_error = "no current CUDA context"; return SECANT_ERROR_INVALID_STATE; }
    int value = 0;
    SB_CUDA(cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, r->device), "device attributes");
    r->sm_count = value;
    SB_CUDA(cudaDeviceGetAttribute(&value, cudaDevAttrMaxSharedMemoryPerBlockOptin, r->device), "device attributes");
    r->smem_limit = (size_t)value;
    SB_CUDA(configure_kernels(), "kernel attributes");
    r->streams.resize(options->num_streams);
    for (auto& s : r->streams) SB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreate");
    r->scratch.assign(r->streams.size(), nullptr);
    r->scratch_cap.assign(r->streams.size(), 0);
    SB_CUDA(cudaStreamCreateWithFlags(&r->copy_stream, cudaStreamNonBlocking), "cudaStreamCreate");
    SB_CUDA(cudaEventCreateWithFlags(&r->ev_cleared, cudaEventDisableTiming), "cudaEventCreate");
    SB_CUDA(cudaEventCreate(&r->ev_start), "cudaEventCreate");
    SB_CUDA(cudaEventCreate(&r->ev_stop), "cudaEventCreate");
    r->slots.resize(options->num_workers + 2); /* same slot budget as the reference: workers + 2 */
    for (auto& s : r->slots) {
        SB_CUDA(cudaEventCreateWithFlags(&s.uploaded, cudaEventDisableTiming), "cudaEventCreate");
        s.done.resize(r->streams.size());
        s.used.assign(r->streams.size(), 0);
        for (auto& e : s.done) SB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
    }
    r->worker_seconds.assign(options->num_workers, 0.0);
    try {
        for (size_t i = 0; i < options->num_workers; ++i) {
            if (SB_FAULT("thread")) throw std::bad_alloc();
            r->workers.emplace_back(worker_main, r, i);
        }
    } catch (...) {
        r->last_error = "worker thread creation failed";
        return SECANT_ERROR_THREAD_FAILED;
    }
    return SECANT_SUCCESS;
}

/* Stops the workers, waits for the streams and releases everything the runner owns.  May be
 * called again after a failure: a resource is forgotten only once its release has succeeded, so a
 * second destroy retries what the first could not free. */
SecantResult runner_teardown(SecantCubinRunnerImpl* r) {
    {
        std::lock_guard<std::mutex> lock(r->mutex);
        r->shutdown = true;
    }
    r->cv_work.notify_all();
    for (auto& t : r->workers)
        if (t.joinable()) t.join();
    r->workers.clear();
    SecantResult result = SECANT_SUCCESS;
    auto ok = [&](cudaError_t e) {
        if (e == cudaSuccess || e == cudaErrorCudartUnloading) return true;
        result = SECANT_ERROR_DRIVER_FAILED;
        return false;
    };
    for (auto& s : r->streams) if (s) ok(cudaStreamSynchronize(s));
    if (r->copy_stream) ok(cudaStreamSynchronize(r->copy_stream));
    if (result != SECANT_SUCCESS) return SECANT_ERROR_COMPLETION_UNKNOWN; /* nothing is released under work that may still run */
    for (auto& s : r->slots) {
        if (s.pinned && ok(cudaFreeHost(s.pinned))) { s.pinned = nullptr; s.pinned_cap = 0; }
        if (s.device && ok(cudaFree(s.device))) { s.device = nullptr; s.device_cap = 0; }
        if (s.uploaded && ok(cudaEventDestroy(s.uploaded))) s.uploaded = nullptr;
        for (auto& e : s.done) if (e && ok(cudaEventDestroy(e))) e = nullptr;
    }
    for (size_t k = 0; k < r->scratch.size(); ++k)
        if (r->scratch[k] && ok(cudaFree(r->scratch[k]))) { r->scratch[k] = nullptr; r->scratch_cap[k] = 0; }
    for (auto& s : r->streams) if (s && ok(cudaStreamDestroy(s))) s = nullptr;
    if (r->copy_stream && ok(cudaStreamDestroy(r->copy_stream))) r->copy_stream = nullptr;
    if (r->ev_cleared && ok(cudaEventDestroy(r->ev_cleared))) r->ev_cleared = nullptr;
    if (r->ev_start && ok(cudaEventDestroy(r->ev_start))) r->ev_start = nullptr;
    if (r->ev_stop && ok(cudaEventDestroy(r->ev_stop))) r->ev_stop = nullptr;
    return result;
}

SecantResult options_validate(const SecantCubinRunnerOptions* options) {
    if (!options || options->struct_size < sizeof(*options)) return SECANT_ERROR_INVALID_VALUE;
    if (options->version != SECANT_CUBIN_RUNNER_OPTIONS_VERSION_1) return SECANT_ERROR_UNSUPPORTED_VERSION;
    if (options->flags || options->reserved || !options->num_workers || !options->num_streams ||
        options->num_workers > 256 || options->num_streams > 1024)
        return SECANT_ERROR_INVALID_VALUE;
    return SECANT_SUCCESS;
}

SecantResult create_common(SecantCubinRunnerImpl* r, const SecantCubinRunnerOptions* options, SecantCubinRunner* out) {
    const SecantResult result = runner_init(r, options);
    if (result != SECANT_SUCCESS) {
        if (runner_teardown(r) != SECANT_SUCCESS) { /* keep ownership: destroy-only handle */
            r->failed = true;
            *out = r;
            return result;
        }
        delete r;
        return result;
    }
    *out = r;
    return SECANT_SUCCESS;
}

/* Programs whose per-warp working set (spill slots, constant table, hoisted row values) is larger
 * than this are launched separately, so that the shared-memory budget of the common case is not
 * sized by rare programs. */
constexpr unsigned kLightSlots = 2, kLightTable = 8, kLightHoisted = 4;

bool is_light(const SbProgram& p) { return p.n_slots <= kLightSlots && p.n_cst <= kLightTable && p.n_hoisted <= kLightHoisted; }

/* scheduling weight of a program: one row pass over sixteen bank groups */
uint64_t schedule_cost(const SbProgram& p) {
    const uint64_t main_part = p.cost & 0xffffu, prelude = p.cost >> 16;
    return main_part * ((p.flags & SB_PROG_BANK_INDEPENDENT) ? 1u : 16u) + prelude;
}

/* Copies an encoded batch into the slot's pinned buffer, grows the device buffer when
 * needed, and enqueues the upload.  Layout: programs | insns | patches | affines | lits. */
SecantResult upload_batch(SecantCubinRunnerImpl* r, Slot& s, std::vector<DeviceBatch>* views) {
    EncodedBatch& e = s.enc;
    /* light programs first, heavy ones after them; SbProgram::index keeps their place in the run */
    std::stable_partition(e.programs.begin(), e.programs.end(), is_light);
    /* inside each group, costly programs first: every CTA takes a strided subset, so its queue runs
     * from its costliest item to its cheapest and its warps finish a tile close together */
    const auto light_end = std::find_if(e.programs.begin(), e.programs.end(), [](const SbProgram& p) { return !is_light(p); });
    const auto by_cost = [](const SbProgram& a, const SbProgram& b) { return schedule_cost(a) > schedule_cost(b); };
    std::stable_sort(e.programs.begin(), light_end, by_cost);
    std::stable_sort(light_end, e.programs.end(), by_cost);
    const size_t num_light = (size_t)(light_end - e.programs.begin());
    const size_t o_prog = 0;
    const size_t o_insn = align256(o_prog + e.programs.size() * sizeof(SbProgram));
    const size_t o_patch = align256(o_insn + e.insns.size() * sizeof(SbInsn));
    const size_t o_aff = align256(o_patch + e.patches.size() * sizeof(SbPatch));
    const size_t o_lit = align256(o_aff + e.affines.size() * sizeof(SbAffine));
    const size_t total = align256(o_lit + e.lits.size() * sizeof(float) + 16);
    if (s.pinned_cap < total) {
        if (s.pinned) SB_CUDA(cudaFreeHost(s.pinned), "cudaFreeHost");
        s.pinned = nullptr; s.pinned_cap = 0;
        SB_CUDA(cudaHostAlloc(&s.pinned, total + total / 2, cudaHostAllocDefault), "cudaHostAlloc");
        s.pinned_cap = total + total / 2;
    }
    if (s.device_cap < total) {
        if (s.device) SB_CUDA(cudaFree(s.device), "cudaFree");
        s.device = nullptr; s.device_cap = 0;
        SB_CUDA(cudaMalloc(&s.device, total + total / 2), "cudaMalloc");
        s.device_cap = total + total / 2;
    }
    char* h = static_cast<char*>(s.pinned);
    std::memcpy(h + o_prog, e.programs.data(), e.programs.size() * sizeof(SbProgram));
    std::memcpy(h + o_insn, e.insns.data(), e.insns.size() * sizeof(SbInsn));
    if (!e.patches.empty()) std::memcpy(h + o_patch, e.patches.data(), e.patches.size() * sizeof(SbPatch));
    if (!e.affines.empty()) std::memcpy(h + o_aff, e.affines.data(), e.affines.size() * sizeof(SbAffine));
    if (!e.lits.empty()) std::memcpy(h + o_lit, e.lits.data(), e.lits.size() * sizeof(float));
    SB_CUDA(cudaMemcpyAsync(s.device, s.pinned, total, cudaMemcpyHostToDevice, r->copy_stream), "program upload");
    SB_CUDA(cudaEventRecord(s.uploaded, r->copy_stream), "cudaEventRecord");
    const char* d = static_cast<const char*>(s.device);
    views->clear();
    const size_t bounds[3] = {0, num_light, e.programs.size()};
    for (int k = 0; k < 2; ++k) {
        if (bounds[k] == bounds[k + 1]) continue;
        DeviceBatch db;
        std::memset(&db, 0, sizeof(db));
        db.insns = reinterpret_cast<const SbInsn*>(d + o_insn);
        db.patches = reinterpret_cast<const SbPatch*>(d + o_patch);
        db.affines = reinterpret_cast<const SbAffine*>(d + o_aff);
        db.lits = reinterpret_cast<const float*>(d + o_lit);
        db.programs = reinterpret_cast<const SbProgram*>(d + o_prog) + bounds[k];
        db.num_programs = (uint32_t)(bounds[k + 1] - bounds[k]);
        db.max_insn = 1;
        for (size_t i = bounds[k]; i < bounds[k + 1]; ++i) {
            const SbProgram& p = e.programs[i];
            db.max_insn = std::max<uint32_t>(db.max_insn, p.n_insn);
            db.max_extra = std::max<uint32_t>(db.max_extra, (uint32_t)p.n_affine + p.n_lits);
            db.max_slots = std::max<uint32_t>(db.max_slots, p.n_slots);
            db.max_hoisted = std::max<uint32_t>(db.max_hoisted, p.n_hoisted);
            db.max_cst = std::max<uint32_t>(db.max_cst, p.n_cst);
            db.max_btmp = std::max<uint32_t>(db.max_btmp, p.n_btmp);
            db.uses_scratch |= (p.flags & SB_PROG_USES_SCRATCH) ? 1u : 0u;
        }
        views->push_back(db);
    }
    return SECANT_SUCCESS;
}

EvalProblem make_problem(const SecantCubinPlan& plan, const UnpackedRun& run, size_t first_program) {
    EvalProblem p;
    std::memset(&p, 0, sizeof(p));
    p.input = reinterpret_cast<const float*>(run.input.address);
    p.input_ld = run.input.leading_dimension;
    p.num_inputs = (uint32_t)plan.num_inputs;
    p.targets = reinterpret_cast<const float*>(run.targets.address);
    p.targets_ld = run.targets.leading_dimension;
    p.num_targets = (uint32_t)run.num_targets;
    p.banks = reinterpret_cast<const float*>(run.banks.address);
    p.bank_stride = run.banks.bank_stride;
    p.program_bank_stride = run.program_bank_stride;
    p.first_program = first_program;
    p.num_constants = (uint32_t)plan.num_constants;
    p.num_banks = (uint32_t)run.num_banks;
    p.toggle_bits = run.toggle_bits;
    p.num_rows = run.rows;
    p.output = reinterpret_cast<float*>(run.output.address);
    switch (plan.shape) {
    case SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32:
        p.mode = EVAL_MATERIALIZE; p.out_program_stride = run.output.leading_dimension; p.out_target_stride = 0; break;
    case SECANT_KERNEL_SHAPE_STATIC_SSE_F32:
        p.mode = EVAL_SSE; p.out_program_stride = run.output.leading_dimension; p.out_target_stride = 1; break;
    case SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32:
        p.mode = EVAL_AFFINE_STATS; p.out_program_stride = run.output.leading_dimension; p.out_target_stride = 1; break;
    case SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32: /* predictions are materialized into scratch; launch_gram_batch() places them */
        p.mode = EVAL_MATERIALIZE; p.output = nullptr; p.out_program_stride = 0; p.out_target_stride = 0; break;
    default:
        p.mode = EVAL_SSE;
        p.out_program_stride = run.num_targets * run.output.leading_dimension;
        p.out_target_stride = run.output.leading_dimension;
        break;
    }
    return p;
}

/* Per-stream scratch for the evaluator's per-split partial sums.  Launches on one stream run in
 * order, so the evaluator and the kernel that folds its partial sums may reuse the buffer of the
 * launch before them; growing it waits for the stream first. */
SecantResult stream_scratch(SecantCubinRunnerImpl* r, size_t k, size_t elements, float** out) {
    const size_t bytes = elements * sizeof(float);
    if (elements > SIZE_MAX / sizeof(float)) return SECANT_ERROR_OVERFLOW;
    if (r->scratch_cap[k] < bytes) {
        SB_CUDA(cudaStreamSynchronize(r->streams[k]), "cudaStreamSynchronize");
        if (r->scratch[k]) SB_CUDA(cudaFree(r->scratch[k]), "cudaFree");
        r->scratch[k] = nullptr; r->scratch_cap[k] = 0;
        const size_t want = bytes + bytes / 4;
        if (cudaMalloc(&r->scratch[k], want) != cudaSuccess) {
            (void)cudaGetLastError();
            r->last_error = "no device memory for the partial sums of a launch";
            return SECANT_ERROR_ALLOCATION_FAILED;
        }
        r->scratch_cap[k] = want;
    }
    *out = static_cast<float*>(r->scratch[k]);
    return SECANT_SUCCESS;
}

/* Enqueues the evaluation of one device-resident batch for every run entry, spreading
 * entries over the compute streams.  `after` (optional) is an event each stream waits on
 * first; `done`/`used` (optional) receive one completion event per touched stream. */
SecantResult launch_batch(SecantCubinRunnerImpl* r, const DeviceBatch& db, const std::vector<UnpackedRun>& runs,
                          size_t* stream_cursor, cudaEvent_t after, std::vector<cudaEvent_t>* done, std::vector<char>* used) {
    const SecantCubinPlan& plan = *r->plan;
    for (size_t e = 0; e < runs.size(); ++e) {
        const size_t k = (*stream_cursor)++ % r->streams.size();
        cudaStream_t stream = r->streams[k];
        EvalProblem prob = make_problem(plan, runs[e], 0); /* SbProgram::index already places every program in the run */
        prob.fast_math = r->fast_math;
        if (runs[e].program_bank_stride)
            prob.banks = reinterpret_cast<const float*>(runs[e].banks.address) + runs[e].first_program_index * runs[e].program_bank_stride;
        const LaunchPlan lp = plan_launch(db, prob, r->sm_count, r->smem_limit, r->scratch_limit);
        if (!lp.ok) {
            r->last_error = lp.overflow ? "configuration count beyond the evaluator's 32-bit item index" : "program batch does not fit shared memory";
            return lp.overflow ? SECANT_ERROR_OVERFLOW : SECANT_ERROR_REGISTER_OVERFLOW;
        }
        float* partial = nullptr;
        if (lp.partial_elements) {
            const SecantResult a = stream_scratch(r, k, lp.partial_elements, &partial);
            if (a != SECANT_SUCCESS) return a;
        }
        unsigned launches = 0;
        cudaError_t ce = after ? cudaStreamWaitEvent(stream, after, 0) : cudaSuccess;
        if (ce == cudaSuccess) ce = launch_eval(db, prob, lp, partial, stream, &launches);
        g_kernel_launches.fetch_add(launches);
        if (launches)
            g_row_stream_bytes.fetch_add((uint64_t)lp.num_groups * (prob.num_inputs + (prob.mode == EVAL_MATERIALIZE ? 0u : prob.num_targets)) *
                                         (uint64_t)prob.num_rows * sizeof(float));
        if (ce == cudaSuccess && done) ce = cudaEventRecord((*done)[k], stream);
        if (ce != cudaSuccess) return cuda_fail(r, ce, "kernel launch");
        if (used) (*used)[k] = 1;
    }
    return SECANT_SUCCESS;
}

/* The static Gram shape: the predictions of the batch's programs are materialized for a range of
 * rows into the stream's scratch by the evaluator (every view of the batch), then reduced to the
 * cohorts' statistics, range after range on one stream, so every statistic is added to in row
 * order.  first_program is the batch's first program and a multiple of the cohort size. */
SecantResult launch_gram_batch(SecantCubinRunnerImpl* r, const std::vector<DeviceBatch>& views, const std::vector<UnpackedRun>& runs,
                               size_t first_program, size_t batch_programs, size_t* stream_cursor, cudaEvent_t after,
                               std::vector<cudaEvent_t>* done, std::vector<char>* used) {
    const SecantCubinPlan& plan = *r->plan;
    const size_t cohort = plan.asts_per_kernel;
    for (size_t e = 0; e < runs.size(); ++e) {
        const UnpackedRun& run = runs[e];
        const size_t k = (*stream_cursor)++ % r->streams.size();
        cudaStream_t stream = r->streams[k];
        /* rows per range: what the scratch limit leaves for this batch, between 128 and 16,384 */
        const size_t fit = r->scratch_limit / batch_programs;
        const size_t range = std::min<size_t>(run.rows, std::max<size_t>(128, std::min<size_t>(16384, fit)));
        float* scratch = nullptr;
        const SecantResult a = stream_scratch(r, k, batch_programs * range, &scratch);
        if (a != SECANT_SUCCESS) return a;
        cudaError_t ce = after ? cudaStreamWaitEvent(stream, after, 0) : cudaSuccess;
        for (size_t r0 = 0; r0 < run.rows && ce == cudaSuccess; r0 += range) {
            const size_t rows_now = std::min(range, run.rows - r0);
            for (const DeviceBatch& db : views) {
                EvalProblem prob = make_problem(plan, run, 0);
                prob.fast_math = r->fast_math;
                prob.input += r0;
                prob.num_rows = rows_now;
                /* SbProgram::index is the program's position in the run: shift the base so that the batch's first program lands on row 0 */
                prob.output = reinterpret_cast<float*>(reinterpret_cast<uintptr_t>(scratch) - first_program * range * sizeof(float));
                prob.out_program_stride = range;
                const LaunchPlan lp = plan_launch(db, prob, r->sm_count, r->smem_limit, r->scratch_limit);
                if (!lp.ok) {
                    r->last_error = "program batch does not fit shared memory";
                    return lp.overflow ? SECANT_ERROR_OVERFLOW : SECANT_ERROR_REGISTER_OVERFLOW;
                }
                unsigned launches = 0;
                ce = launch_eval(db, prob, lp, nullptr, stream, &launches);
                g_kernel_launches.fetch_add(launches);
                if (ce != cudaSuccess) break;
            }
            if (ce == cudaSuccess)
                ce = launch_gram(scratch, range, (uint32_t)rows_now, reinterpret_cast<const float*>(run.targets.address) + r0,
                                 run.targets.leading_dimension, (uint32_t)run.num_targets, (uint32_t)cohort, (uint32_t)batch_programs,
                                 reinterpret_cast<float*>(run.output.address) + (first_program / cohort) * run.output.leading_dimension,
                                 run.output.leading_dimension, stream);
        }
        if (ce == cudaSuccess && done) ce = cudaEventRecord((*done)[k], stream);
        if (ce != cudaSuccess) return cuda_fail(r, ce, "kernel launch");
        if (used) (*used)[k] = 1;
    }
    return SECANT_SUCCESS;
}

/* Waits for everything the runner has enqueued; false (and a destroy-only handle) when a wait fails. */
bool drain_streams(SecantCubinRunnerImpl* r) {
    bool ok = true;
    for (auto& s : r->streams) ok = (cudaStreamSynchronize(s) == cudaSuccess) && ok;
    ok = (cudaStreamSynchronize(r->copy_stream) == cudaSuccess) && ok;
    if (!ok) r->failed = true;
    return ok;
}

/* Waits until every compute stream that touched the slot has finished with it. */
SecantResult retire_slot(SecantCubinRunnerImpl* r, Slot& s, bool* unknown) {
    SecantResult result = SECANT_SUCCESS;
    for (size_t k = 0; k < s.done.size(); ++k) {
        if (!s.used[k]) continue;
        const cudaError_t e = cudaEventSynchronize(s.done[k]);
        if (e != cudaSuccess) { result = cuda_fail(r, e, "waiting for a batch"); *unknown = true; }
        s.used[k] = 0;
    }
    return result;
}

SecantResult execute(SecantCubinRunnerImpl* r, const std::vector<UnpackedRun>& runs, const ProgramRules& rules,
                     SecantRunnerStats* stats) {
    const SecantCubinPlan& plan = *r->plan;
    const SecantAstProgramSet& programs = runs[0].programs;
    const size_t P = programs.asts.count;
    uint8_t arity[SECANT_AST_MAX_ROUTINES];
    SecantResult result = routine_arities(programs.routines, arity);
    if (result != SECANT_SUCCESS) return result;
    if ((uint64_t)P > 0xffffffffull) return SECANT_ERROR_OVERFLOW;

    const double t_begin = now_seconds();
    size_t batch_size = (P + 3) / 4;
    if (batch_size < 4096) batch_size = 4096;
    const bool gram = plan.shape == SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32;
    if (gram) batch_size = (batch_size + plan.asts_per_kernel - 1) / plan.asts_per_kernel * plan.asts_per_kernel; /* whole cohorts */
    if (batch_size > P) batch_size = P;
    const size_t num_batches = (P + batch_size - 1) / batch_size;
    const bool accumulate = plan.shape != SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32;

    /* clear the active output bins only; padding between vectors is preserved */
    SB_CUDA(cudaEventRecord(r->ev_start, r->streams[0]), "cudaEventRecord");
    if (accumulate)
        for (const auto& run : runs)
            SB_CUDA(cudaMemset2DAsync(reinterpret_cast<void*>(run.output.address), run.output.leading_dimension * sizeof(float), 0,
                                      run.output_width * sizeof(float), run.output_count, r->streams[0]),
                    "clearing output");
    SB_CUDA(cudaEventRecord(r->ev_cleared, r->streams[0]), "cudaEventRecord");
    for (size_t k = 1; k < r->streams.size(); ++k) SB_CUDA(cudaStreamWaitEvent(r->streams[k], r->ev_cleared, 0), "cudaStreamWaitEvent");

    {
        std::lock_guard<std::mutex> lock(r->mutex);
        for (auto& s : r->slots) { s.state = SLOT_FREE; std::fill(s.used.begin(), s.used.end(), 0); }
        std::fill(r->worker_seconds.begin(), r->worker_seconds.end(), 0.0);
        r->job_programs = &programs;
        r->job_arity = arity;
        r->job_rules = rules;
        r->job_batch_size = batch_size;
        r->job_num_batches = num_batches;
        r->job_next_batch = 0;
        r->job_abort = false;
        r->job_active = true;
    }
    r->cv_work.notify_all();
    /* Whatever way this function is left (a result code or an exception from a container), the
     * workers must be off this job first: they read `arity`, `programs` and `rules`, which live in
     * the caller's frames. */
    struct JobGuard {
        SecantCubinRunnerImpl* r;
        ~JobGuard() {
            std::unique_lock<std::mutex> lock(r->mutex);
            r->job_abort = true;
            r->cv_ready.wait(lock, [&] {
                for (auto& s : r->slots)
                    if (s.state == SLOT_ENCODING) return false;
                return true;
            });
            r->job_active = false;
        }
    } job_guard{r};

    bool unknown = false;
    size_t launched_batches = 0, stream_cursor = 0;
    double upload_seconds = 0, wait_seconds = 0, encode_sum = 0;
    std::vector<Slot*> in_flight;
    for (size_t b = 0; b < num_batches && result == SECANT_SUCCESS; ++b) {
        Slot* slot = nullptr;
        {
            std::unique_lock<std::mutex> lock(r->mutex);
            r->cv_ready.wait(lock, [&] {
                for (auto& s : r->slots)
                    if (s.state == SLOT_READY && s.batch == b) { slot = &s; return true; }
                return false;
            });
            slot->state = SLOT_IN_FLIGHT;
        }
        encode_sum += slot->encode_seconds;
        result = slot->status;
        if (result != SECANT_SUCCESS) break;
        std::vector<DeviceBatch> views;
        const double t_up = now_seconds();
        result = upload_batch(r, *slot, &views);
        upload_seconds += now_seconds() - t_up;
        if (result != SECANT_SUCCESS) break;
        if (gram) {
            const size_t first = b * batch_size;
            result = launch_gram_batch(r, views, runs, first, std::min(batch_size, P - first), &stream_cursor, slot->uploaded, &slot->done,
                                       &slot->used);
        } else {
            for (const DeviceBatch& db : views) {
                result = launch_batch(r, db, runs, &stream_cursor, slot->uploaded, &slot->done, &slot->used);
                if (result != SECANT_SUCCESS) break;
            }
        }
        in_flight.push_back(slot);
        ++launched_batches;
        /* recycle the oldest batch once two are queued behind it, so workers always find a slot */
        while (in_flight.size() > 2 || (result != SECANT_SUCCESS && !in_flight.empty())) {
            Slot* old = in_flight.front();
            in_flight.erase(in_flight.begin());
            const double t_wait = now_seconds();
            const SecantResult w = retire_slot(r, *old, &unknown);
            wait_seconds += now_seconds() - t_wait;
            if (result == SECANT_SUCCESS) result = w;
            {
                std::lock_guard<std::mutex> lock(r->mutex);
                old->state = SLOT_FREE;
            }
            r->cv_work.notify_all();
        }
    }
    /* stop the workers' job, then drain what is still running */
    {
        std::unique_lock<std::mutex> lock(r->mutex);
        r->job_abort = true;
        r->cv_ready.wait(lock, [&] {
            for (auto& s : r->slots)
                if (s.state == SLOT_ENCODING) return false;
            return true;
        });
        r->job_active = false;
    }
    const double t_wait = now_seconds();
    for (Slot* s : in_flight) {
        const SecantResult w = retire_slot(r, *s, &unknown);
        if (result == SECANT_SUCCESS) result = w;
    }
    /* join all compute streams into stream 0 for the device-time interval */
    if (!unknown) {
        cudaError_t ce = cudaSuccess;
        for (size_t k = 1; k < r->streams.size() && ce == cudaSuccess; ++k) {
            ce = cudaEventRecord(r->ev_cleared, r->streams[k]);
            if (ce == cudaSuccess) ce = cudaStreamWaitEvent(r->streams[0], r->ev_cleared, 0);
        }
        if (ce == cudaSuccess) ce = cudaEventRecord(r->ev_stop, r->streams[0]);
        if (ce == cudaSuccess) ce = cudaEventSynchronize(r->ev_stop);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(r->copy_stream);
        float ms = 0;
        if (ce == cudaSuccess) ce = cudaEventElapsedTime(&ms, r->ev_start, r->ev_stop);
        if (ce != cudaSuccess) { const SecantResult w = cuda_fail(r, ce, "completion"); unknown = true; if (result == SECANT_SUCCESS) result = w; }
        stats->runtime_seconds = ms * 1e-3;
    }
    wait_seconds += now_seconds() - t_wait;
    {
        std::lock_guard<std::mutex> lock(r->mutex);
        for (auto& s : r->slots) s.state = SLOT_FREE;
        double critical = 0;
        for (double w : r->worker_seconds) critical = w > critical ? w : critical;
        stats->compile_critical_seconds = critical;
    }
    /* module counts in the reference's unit, a recipe-capacity worth of programs (callers such as
     * projects/secant/tests/toggle_cuda_test.c:245 check them); batches here are much larger */
    {
        const size_t capacity = std::max<size_t>(1, r->plan->num_kernels * r->plan->asts_per_kernel);
        const size_t launched_programs = std::min<size_t>(P, launched_batches * batch_size);
        stats->num_modules = (P + capacity - 1) / capacity;
        stats->modules_loaded = (launched_programs + capacity - 1) / capacity;
    }
    stats->num_asts = P;
    stats->compile_work_seconds = encode_sum;
    stats->compile_window_seconds = now_seconds() - t_begin - wait_seconds;
    stats->module_load_seconds = upload_seconds;
    stats->completion_wait_seconds = wait_seconds;
    stats->module_unload_seconds = 0;
    if (unknown) {
        r->failed = true;
        return SECANT_ERROR_COMPLETION_UNKNOWN;
    }
    return result;
}

}  // namespace

extern "C" {

SecantResult secant_cubin_runner_create(const SecantCubinPlan* plan, const void* cubin, size_t cubin_size,
                                        const SecantCubinRunnerOptions* options, SecantCubinRunner* runner_ret) {
    if (!runner_ret) return SECANT_ERROR_INVALID_VALUE;
    *runner_ret = nullptr;
    if (!plan || plan->magic != kPlanMagic || !cubin || cubin_size != plan->cubin_size || !options ||
        options->struct_size < sizeof(*options))
        return SECANT_ERROR_INVALID_VALUE;
    const SecantResult o = options_validate(options);
    if (o != SECANT_SUCCESS) return o;
    SecantCubinRunnerImpl* r = SB_FAULT("alloc") ? nullptr : new (std::nothrow) SecantCubinRunnerImpl();
    if (!r) return SECANT_ERROR_ALLOCATION_FAILED;
    r->plan = plan;
    return create_common(r, options, runner_ret);
}

SecantResult secant_b200_runner_create(const SecantCubinRecipeHeader* recipe, const SecantCubinRunnerOptions* options,
                                       SecantCubinRunner* runner_ret) {
    if (!runner_ret) return SECANT_ERROR_INVALID_VALUE;
    *runner_ret = nullptr;
    const SecantResult v = recipe_validate(recipe);
    if (v != SECANT_SUCCESS) return v;
    const SecantResult o = options_validate(options);
    if (o != SECANT_SUCCESS) return o;
    SecantCubinRunnerImpl* r = SB_FAULT("alloc") ? nullptr : new (std::nothrow) SecantCubinRunnerImpl();
    if (!r) return SECANT_ERROR_ALLOCATION_FAILED;
    plan_fill(&r->owned_plan, recipe, 0);
    r->plan = &r->owned_plan;
    return create_common(r, options, runner_ret);
}

SecantResult secant_cubin_runner_run_batch(SecantCubinRunner r, const SecantCubinRunHeader* const* headers, size_t count,
                                           SecantRunnerStats* stats) {
    SecantRunnerStats measured = secant_runner_stats_init();
    const double begin = now_seconds();
    if (stats) {
        if (stats->struct_size < sizeof(*stats) || stats->flags || stats->reserved) return SECANT_ERROR_INVALID_VALUE;
        if (stats->version != SECANT_RUNNER_STATS_VERSION_1) return SECANT_ERROR_UNSUPPORTED_VERSION;
        measured.struct_size = stats->struct_size;
        std::memcpy(stats, &measured, sizeof(measured)); /* zero counters, trailing bytes untouched */
    }
    if (!r || !headers || !count || count > SIZE_MAX / sizeof(UnpackedRun)) return SECANT_ERROR_INVALID_VALUE;
    bool ok = false;
    void* ctx = current_context(&ok);
    if (!ok || ctx != r->context) return SECANT_ERROR_INVALID_STATE;
    {
        std::lock_guard<std::mutex> lock(r->mutex);
        if (r->active || r->failed || r->shutdown) return SECANT_ERROR_INVALID_STATE;
        r->active = true;
    }
    SecantResult result = SECANT_SUCCESS;
    std::vector<UnpackedRun> runs;
    try {
        if (SB_FAULT("alloc")) throw std::bad_alloc();
        runs.resize(count);
    } catch (...) {
        result = SECANT_ERROR_ALLOCATION_FAILED;
    }
    for (size_t i = 0; result == SECANT_SUCCESS && i < count; ++i) result = run_unpack(*r->plan, headers[i], &runs[i]);
    ProgramRules rules;
    if (result == SECANT_SUCCESS) result = runs_validate(*r->plan, runs.data(), count, &rules);
    if (result == SECANT_SUCCESS) {
        try {
            result = execute(r, runs, rules, &measured);
        } catch (const std::bad_alloc&) {
            /* work already enqueued still reads the caller's buffers: wait for it before handing them back */
            result = drain_streams(r) ? SECANT_ERROR_ALLOCATION_FAILED : SECANT_ERROR_COMPLETION_UNKNOWN;
        }
    }
    {
        std::lock_guard<std::mutex> lock(r->mutex);
        r->active = false;
    }
    if (measured.num_modules) measured.total_seconds = now_seconds() - begin;
    if (stats) std::memcpy(stats, &measured, sizeof(measured));
    return result;
}

SecantResult secant_cubin_runner_run(SecantCubinRunner r, const SecantCubinRunHeader* run, SecantRunnerStats* stats) {
    return secant_cubin_runner_run_batch(r, &run, 1, stats);
}

SecantResult secant_cubin_runner_destroy(SecantCubinRunner r) {
    if (!r) return SECANT_SUCCESS;
    bool ok = false;
    void* ctx = current_context(&ok);
    if (r->context && (!ok || ctx != r->context)) return SECANT_ERROR_INVALID_STATE;
    {
        std::lock_guard<std::mutex> lock(r->mutex);
        if (r->active || r->populations) return SECANT_ERROR_INVALID_STATE; /* populations hold a pointer to their runner */
    }
    const SecantResult result = runner_teardown(r);
    if (result != SECANT_SUCCESS) { r->failed = true; return result; }
    delete r;
    return SECANT_SUCCESS;
}

const char* secant_b200_runner_last_error(SecantCubinRunner r) { return r ? r->last_error.c_str() : ""; }

uint64_t secant_b200_kernel_launch_count(void) { return g_kernel_launches.load(); }
uint64_t secant_b200_row_stream_bytes(void) { return g_row_stream_bytes.load(); }

}  // extern "C"

/* ---- device-resident populations ------------------------------------------------------ */

namespace {

size_t program_length(const SecantAstInstruction* code) {
    size_t at = 0;
    for (size_t n = 0; n < SECANT_AST_MAX_PROGRAM_INSTRUCTIONS; ++n) {
        const size_t width = secant_ast_instruction_size_get(code + at);
        if (!width) return 0;
        const bool last = code[at] == SECANT_AST_INSTRUCTION_TYPE_RETURN_F32;
        at += width;
        if (last) return at;
    }
    return 0;
}

SecantResult copy_programs(const SecantAstProgramList& list, std::vector<uint8_t>* bytes, std::vector<const uint8_t*>* ptrs) {
    std::vector<size_t> offsets(list.count);
    for (size_t i = 0; i < list.count; ++i) {
        if (!list.items[i]) return SECANT_ERROR_BAD_PROGRAM;
        const size_t n = program_length(list.items[i]);
        if (!n) return SECANT_ERROR_BAD_PROGRAM;
        offsets[i] = bytes->size();
        bytes->insert(bytes->end(), list.items[i], list.items[i] + n);
    }
    ptrs->resize(list.count);
    for (size_t i = 0; i < list.count; ++i) (*ptrs)[i] = bytes->data() + offsets[i];
    return SECANT_SUCCESS;
}

SecantResult execute_resident(SecantCubinRunnerImpl* r, SecantB200PopulationImpl* pop, const std::vector<UnpackedRun>& runs,
                              SecantRunnerStats* stats) {
    const SecantCubinPlan& plan = *r->plan;
    const bool accumulate = plan.shape != SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32;
    SB_CUDA(cudaEventRecord(r->ev_start, r->streams[0]), "cudaEventRecord");
    if (accumulate)
        for (const auto& run : runs)
            SB_CUDA(cudaMemset2DAsync(reinterpret_cast<void*>(run.output.address), run.output.leading_dimension * sizeof(float), 0,
                                      run.output_width * sizeof(float), run.output_count, r->streams[0]),
                    "clearing output");
    SB_CUDA(cudaEventRecord(r->ev_cleared, r->streams[0]), "cudaEventRecord");
    for (size_t k = 1; k < r->streams.size(); ++k) SB_CUDA(cudaStreamWaitEvent(r->streams[k], r->ev_cleared, 0), "cudaStreamWaitEvent");
    size_t cursor = 0;
    SecantResult result = SECANT_SUCCESS;
    for (auto& b : pop->batches) {
        for (const DeviceBatch& db : b.views) {
            result = launch_batch(r, db, runs, &cursor, nullptr, nullptr, nullptr);
            if (result != SECANT_SUCCESS) break;
        }
        if (result != SECANT_SUCCESS) break;
    }
    const double t_wait = now_seconds();
    cudaError_t ce = cudaSuccess;
    for (size_t k = 1; k < r->streams.size() && ce == cudaSuccess; ++k) {
        ce = cudaEventRecord(r->ev_cleared, r->streams[k]);
        if (ce == cudaSuccess) ce = cudaStreamWaitEvent(r->streams[0], r->ev_cleared, 0);
    }
    if (ce == cudaSuccess) ce = cudaEventRecord(r->ev_stop, r->streams[0]);
    if (ce == cudaSuccess) ce = cudaEventSynchronize(r->ev_stop);
    float ms = 0;
    if (ce == cudaSuccess) ce = cudaEventElapsedTime(&ms, r->ev_start, r->ev_stop);
    stats->completion_wait_seconds = now_seconds() - t_wait;
    stats->runtime_seconds = ms * 1e-3;
    {
        const size_t capacity = std::max<size_t>(1, r->plan->num_kernels * r->plan->asts_per_kernel);
        stats->num_modules = stats->modules_loaded = (pop->set.asts.count + capacity - 1) / capacity;
    }
    stats->num_asts = pop->set.asts.count;
    if (ce != cudaSuccess) {
        cuda_fail(r, ce, "completion");
        r->failed = true;
        return SECANT_ERROR_COMPLETION_UNKNOWN;
    }
    return result;
}

}  // namespace

extern "C" {

SecantResult secant_b200_population_create(SecantCubinRunner r, const SecantAstProgramSet* programs, uint32_t toggle_bits,
                                           SecantB200Population* population_ret) {
    if (!population_ret) return SECANT_ERROR_INVALID_VALUE;
    *population_ret = nullptr;
    if (!r || !programs || !programs->asts.count || !programs->asts.items || toggle_bits > 32u ||
        programs->routines.count > SECANT_AST_MAX_ROUTINES || (programs->routines.count && !programs->routines.items) ||
        (uint64_t)programs->asts.count > 0xffffffffull)
        return SECANT_ERROR_INVALID_VALUE;
    bool ok = false;
    void* ctx = current_context(&ok);
    if (!ok || ctx != r->context) return SECANT_ERROR_INVALID_STATE;
    const SecantCubinPlan& plan = *r->plan;
    if (plan.shape == SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32) return SECANT_ERROR_UNSUPPORTED_SHAPE; /* cohorts go through the run entry points */
    ProgramRules rules;
    rules.num_columns = plan.num_inputs;
    rules.num_constants = plan.num_constants;
    rules.banks_allowed = plan.shape == SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32;
    rules.toggle_bits = rules.banks_allowed ? toggle_bits : 0;
    rules.split_parts = true;
    rules.hoist_bank = true;
    rules.hoist_row = rules.banks_allowed; /* a population is usually scored against many banks */
    for (size_t i = 0; i < programs->routines.count; ++i) {
        const SecantResult s = preflight(programs->routines.items[i], rules);
        if (s != SECANT_SUCCESS) return s;
    }
    for (size_t i = 0; i < programs->asts.count; ++i) {
        const SecantResult s = preflight(programs->asts.items[i], rules);
        if (s != SECANT_SUCCESS) return s;
    }
    uint8_t arity[SECANT_AST_MAX_ROUTINES];
    SecantResult result = routine_arities(programs->routines, arity);
    if (result != SECANT_SUCCESS) return result;
    SecantB200PopulationImpl* pop = new (std::nothrow) SecantB200PopulationImpl();
    if (!pop) return SECANT_ERROR_ALLOCATION_FAILED;
    pop->runner = r;
    pop->toggle_bits = toggle_bits;
    try {
        result = copy_programs(programs->routines, &pop->routine_bytes, &pop->routine_ptrs);
        if (result == SECANT_SUCCESS) result = copy_programs(programs->asts, &pop->ast_bytes, &pop->ast_ptrs);
        pop->set.routines.items = pop->routine_ptrs.data();
        pop->set.routines.count = pop->routine_ptrs.size();
        pop->set.asts.items = pop->ast_ptrs.data();
        pop->set.asts.count = pop->ast_ptrs.size();
        const size_t P = programs->asts.count;
        size_t batch_size = (P + 3) / 4;
        if (batch_size < 4096) batch_size = 4096;
        if (batch_size > P) batch_size = P;
        Slot staging; /* reuses the upload helper; its buffers are handed to the population */
        for (size_t first = 0; first < P && result == SECANT_SUCCESS; first += batch_size) {
            const size_t count = std::min(batch_size, P - first);
            staging.enc.clear();
            for (size_t i = 0; i < count && result == SECANT_SUCCESS; ++i) {
                result = encode_program(programs->asts.items[first + i], programs->routines, arity, rules, staging.enc);
                if (result == SECANT_SUCCESS) staging.enc.programs.back().index = (uint32_t)(first + i);
            }
            if (result != SECANT_SUCCESS) break;
            for (const auto& p : staging.enc.programs) pop->total_ops += p.n_ops;
            if (!staging.uploaded && cudaEventCreateWithFlags(&staging.uploaded, cudaEventDisableTiming) != cudaSuccess) {
                result = SECANT_ERROR_DRIVER_FAILED;
                break;
            }
            SecantB200PopulationImpl::Resident res;
            result = upload_batch(r, staging, &res.views);
            if (result != SECANT_SUCCESS) break;
            if (cudaStreamSynchronize(r->copy_stream) != cudaSuccess) { result = SECANT_ERROR_DRIVER_FAILED; break; }
            res.device = staging.device; /* keep this allocation; the next batch gets a new one */
            res.first = first;
            staging.device = nullptr;
            staging.device_cap = 0;
            pop->batches.push_back(res);
        }
        if (staging.pinned) cudaFreeHost(staging.pinned);
        if (staging.device) cudaFree(staging.device);
        if (staging.uploaded) cudaEventDestroy(staging.uploaded);
    } catch (const std::bad_alloc&) {
        result = SECANT_ERROR_ALLOCATION_FAILED;
    }
    if (result != SECANT_SUCCESS) {
        for (auto& b : pop->batches) cudaFree(b.device);
        delete pop;
        return result;
    }
    {
        std::lock_guard<std::mutex> lock(r->mutex);
        ++r->populations;
    }
    *population_ret = pop;
    return SECANT_SUCCESS;
}

SecantResult secant_b200_population_run_batch(SecantB200Population pop, const SecantCubinRunHeader* const* headers, size_t count,
                                              SecantRunnerStats* stats) {
    SecantRunnerStats measured = secant_runner_stats_init();
    const double begin = now_seconds();
    if (stats) {
        if (stats->struct_size < sizeof(*stats) || stats->flags || stats->reserved) return SECANT_ERROR_INVALID_VALUE;
        if (stats->version != SECANT_RUNNER_STATS_VERSION_1) return SECANT_ERROR_UNSUPPORTED_VERSION;
        measured.struct_size = stats->struct_size;
        std::memcpy(stats, &measured, sizeof(measured));
    }
    if (!pop || !headers || !count) return SECANT_ERROR_INVALID_VALUE;
    SecantCubinRunnerImpl* r = pop->runner;
    bool ok = false;
    void* ctx = current_context(&ok);
    if (!ok || ctx != r->context) return SECANT_ERROR_INVALID_STATE;
    {
        std::lock_guard<std::mutex> lock(r->mutex);
        if (r->active || r->failed || r->shutdown) return SECANT_ERROR_INVALID_STATE;
        r->active = true;
    }
    SecantResult result = SECANT_SUCCESS;
    std::vector<UnpackedRun> runs;
    try {
        runs.resize(count);
    } catch (...) {
        std::lock_guard<std::mutex> lock(r->mutex);
        r->active = false;
        return SECANT_ERROR_ALLOCATION_FAILED;
    }
    bool same_bits = true;
    for (size_t i = 0; result == SECANT_SUCCESS && i < count; ++i) {
        /* the request's program views are replaced by the population's own */
        alignas(16) unsigned char copy[sizeof(SecantB200ToggleSSERun) + 64];
        const SecantCubinRunHeader* h = headers[i];
        if (!h || h->struct_size < sizeof(*h) + sizeof(SecantAstProgramSet)) { result = SECANT_ERROR_INVALID_VALUE; break; }
        const size_t n = std::min<size_t>(h->struct_size, sizeof(copy));
        std::memcpy(copy, h, n);
        reinterpret_cast<SecantCubinRunHeader*>(copy)->struct_size = (uint32_t)n;
        std::memcpy(copy + sizeof(SecantCubinRunHeader), &pop->set, sizeof(pop->set));
        result = run_unpack(*r->plan, reinterpret_cast<const SecantCubinRunHeader*>(copy), &runs[i]);
        same_bits = same_bits && runs[i].toggle_bits == pop->toggle_bits;
    }
    ProgramRules rules;
    if (result == SECANT_SUCCESS) result = runs_validate(*r->plan, runs.data(), count, &rules, same_bits);
    if (result == SECANT_SUCCESS && !same_bits && rules.toggle_bits < pop->toggle_bits) {
        /* records were encoded for pop->toggle_bits; fewer bits would leave stale patch sites unchecked */
        result = SECANT_ERROR_BAD_PROGRAM;
    }
    if (result == SECANT_SUCCESS) {
        try {
            result = execute_resident(r, pop, runs, &measured);
        } catch (const std::bad_alloc&) {
            result = drain_streams(r) ? SECANT_ERROR_ALLOCATION_FAILED : SECANT_ERROR_COMPLETION_UNKNOWN;
        }
    }
    {
        std::lock_guard<std::mutex> lock(r->mutex);
        r->active = false;
    }
    if (measured.num_modules) measured.total_seconds = now_seconds() - begin;
    if (stats) std::memcpy(stats, &measured, sizeof(measured));
    return result;
}

SecantResult secant_b200_population_run(SecantB200Population pop, const SecantCubinRunHeader* run, SecantRunnerStats* stats) {
    return secant_b200_population_run_batch(pop, &run, 1, stats);
}

uint64_t secant_b200_population_num_ops(SecantB200Population pop) { return pop ? pop->total_ops : 0; }

SecantResult secant_b200_population_destroy(SecantB200Population pop) {
    if (!pop) return SECANT_SUCCESS;
    SecantResult result = SECANT_SUCCESS;
    for (auto& b : pop->batches)
        if (b.device && cudaFree(b.device) != cudaSuccess) result = SECANT_ERROR_DRIVER_FAILED;
    {
        std::lock_guard<std::mutex> lock(pop->runner->mutex);
        if (pop->runner->populations) --pop->runner->populations;
    }
    delete pop;
    return result;
}

SecantResult secant_b200_runner_set_math(SecantCubinRunner r, uint32_t mode) {
    if (!r || mode > SECANT_B200_MATH_FAST) return SECANT_ERROR_INVALID_VALUE;
    std::lock_guard<std::mutex> lock(r->mutex);
    if (r->active) return SECANT_ERROR_INVALID_STATE;
    r->fast_math = mode == SECANT_B200_MATH_FAST ? 1u : 0u;
    return SECANT_SUCCESS;
}

SecantResult secant_b200_runner_set_scratch_limit(SecantCubinRunner r, size_t bytes) {
    if (!r) return SECANT_ERROR_INVALID_VALUE;
    std::lock_guard<std::mutex> lock(r->mutex);
    if (r->active) return SECANT_ERROR_INVALID_STATE;
    r->scratch_limit = bytes ? std::max<size_t>(1, bytes / sizeof(float)) : kDefaultScratchFloats;
    return SECANT_SUCCESS;
}

}  // extern "C"
