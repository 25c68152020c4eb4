/*
 * odezza.cpp - the ODE engine's scoring interface (include/odezza_b200.h) over this library's
 * rollout scorer, grouped top-k and pool kernels.
 *
 * The reference engine specializes a compiled kernel per batch of candidate systems
 * (projects/odezza/core/o_scoring_pipeline.c).  Here a run translates the candidates' right-hand
 * sides into this library's program bytes (the two bytecodes share their shape: postfix tokens,
 * one-byte indices, little-endian literals, toggles over direct leaves), assembles one program per
 * state from the fixed and the per-system right-hand sides, and hands the lot to
 * secant_b200_rk4_score(), whose kernel interprets them.  Validation order and result codes follow
 * the reference so that its own tests pass against this file unchanged.
 */
#include "../../include/odezza_b200.h"
#include "../../include/secant_b200.h"
#include "evaluator.cuh"

#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

namespace {

constexpr size_t kErrorBytes = 1024;
constexpr size_t kRunWorkspaceBytes = 64;   /* validated like the reference's; nothing is kept in it */
constexpr size_t kSystemsPerBatch = 16384;  /* bounds the host memory of one translated batch */
constexpr uint32_t kReferenceThreadsPerBlock = 128; /* projects/odezza/core/o_scoring_pipeline.c:1272 */

double seconds_now() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

bool mul_u64(uint64_t a, uint64_t b, uint64_t* out) {
    if (b && a > UINT64_MAX / b) return false;
    *out = a * b;
    return true;
}

/* a whole byte span of `count` elements at `address`: aligned and not wrapping the address space
 * (projects/odezza/core/o_scoring_pipeline.c:525-529) */
bool span_ok(uint64_t address, uint64_t count, uint64_t element) {
    uint64_t bytes;
    return mul_u64(count, element, &bytes) && (bytes == 0 || (address % element == 0 && bytes - 1 <= UINT64_MAX - address));
}

OdezzaResult from_secant(SecantResult r) {
    switch (r) {
    case SECANT_SUCCESS: return ODEZZA_SUCCESS;
    case SECANT_ERROR_INVALID_VALUE: return ODEZZA_ERROR_INVALID_ARGUMENT;
    case SECANT_ERROR_OVERFLOW: return ODEZZA_ERROR_OVERFLOW;
    case SECANT_ERROR_INSUFFICIENT_BUFFER: return ODEZZA_ERROR_INSUFFICIENT_BUFFER;
    case SECANT_ERROR_ALLOCATION_FAILED: return ODEZZA_ERROR_ALLOCATION;
    case SECANT_ERROR_REGISTER_OVERFLOW: return ODEZZA_ERROR_REGISTER_PRESSURE;
    case SECANT_ERROR_DRIVER_FAILED: return ODEZZA_ERROR_CUDA;
    case SECANT_ERROR_BAD_PROGRAM:
    case SECANT_ERROR_STACK_OVERFLOW:
    case SECANT_ERROR_STACK_UNDERFLOW:
    case SECANT_ERROR_UNSUPPORTED_OP: return ODEZZA_ERROR_AST;
    default: return ODEZZA_ERROR_UNSUPPORTED;
    }
}

/* ---- bytecode ---------------------------------------------------------------------------------- */

struct TokenShape {
    uint8_t payload; /* bytes after the opcode */
    uint8_t pops;    /* operands taken from the stack; 0 for leaves */
    uint8_t secant;  /* the same token in this library's bytecode; 0 = not a token */
};

TokenShape token_shape(uint8_t opcode) {
#define S(name) (uint8_t)SECANT_AST_INSTRUCTION_TYPE_##name
    switch (opcode) {
    case ODEZZA_AST_RETURN_F32: return {0, 0, S(RETURN_F32)};
    case ODEZZA_AST_STATE_F32: return {1, 0, S(COLUMN_F32)};
    case ODEZZA_AST_CONSTANT_F32: return {1, 0, S(BANK_CONSTANT_F32)};
    case ODEZZA_AST_LITERAL_F32: return {4, 0, S(CONSTANT_BITS_F32)};
    case ODEZZA_AST_TOGGLE2_F32: return {1, 2, S(TOGGLE2_F32)};
    case ODEZZA_AST_TOGGLE4_F32: return {2, 4, S(TOGGLE4_F32)};
    case ODEZZA_AST_ADD_F32: return {0, 2, S(ADD_F32)};
    case ODEZZA_AST_SUB_F32: return {0, 2, S(SUB_F32)};
    case ODEZZA_AST_MUL_F32: return {0, 2, S(MUL_F32)};
    case ODEZZA_AST_DIV_F32: return {0, 2, S(DIV_F32)};
    case ODEZZA_AST_MIN_F32: return {0, 2, S(MIN_F32)};
    case ODEZZA_AST_MAX_F32: return {0, 2, S(MAX_F32)};
    case ODEZZA_AST_FMA_F32: return {0, 3, S(FMA_F32)};
    case ODEZZA_AST_NEG_F32: return {0, 1, S(NEG_F32)};
    case ODEZZA_AST_SQRT_F32: return {0, 1, S(SQRT_F32)};
    case ODEZZA_AST_RCP_F32: return {0, 1, S(RCP_F32)};
    case ODEZZA_AST_ABS_F32: return {0, 1, S(ABS_F32)};
    case ODEZZA_AST_SIN_F32: return {0, 1, S(SIN_F32)};
    case ODEZZA_AST_COS_F32: return {0, 1, S(COS_F32)};
    case ODEZZA_AST_EX2_F32: return {0, 1, S(EX2_F32)};
    case ODEZZA_AST_LG2_F32: return {0, 1, S(LG2_F32)};
    case ODEZZA_AST_RSQRT_F32: return {0, 1, S(RSQRT_F32)};
    case ODEZZA_AST_TANH_F32: return {0, 1, S(TANH_F32)};
    case ODEZZA_AST_EXP_F32: return {0, 1, S(EXP_F32)};
    case ODEZZA_AST_LOG_F32: return {0, 1, S(LOG_F32)};
    default: return {0, 0, 0};
    }
#undef S
}

/* Checks one right-hand side by the reference's rules (projects/odezza/core/o_ast.c:81-174: every
 * token inside the byte count, indices in range, finite literals, toggles over direct leaves
 * only, exactly one value left at the single trailing RETURN, at most 2048 tokens and 128 stack
 * entries) and appends the translated program to `out`.  Programs longer than this library's
 * 1024-token limit are a capacity error, as an oversized program is for the reference. */
OdezzaResult translate(const OdezzaAstProgram& program, size_t states, uint32_t constants, uint32_t toggle_bits, bool toggles_allowed,
                       std::vector<uint8_t>& out) {
    if (!program.bytes || !program.byte_count) return ODEZZA_ERROR_INVALID_ARGUMENT;
    bool leaf[SECANT_AST_MAX_STACK_DEPTH];
    size_t depth = 0, tokens = 0, at = 0;
    bool returned = false;
    while (at < program.byte_count) {
        if (tokens == 2048 || returned) return ODEZZA_ERROR_AST;
        const uint8_t opcode = program.bytes[at++];
        const TokenShape shape = token_shape(opcode);
        if (!shape.secant || shape.payload > program.byte_count - at) return ODEZZA_ERROR_AST;
        const uint8_t* payload = program.bytes + at;
        ++tokens;
        if (opcode == ODEZZA_AST_RETURN_F32) {
            if (depth != 1) return ODEZZA_ERROR_AST;
            returned = true;
        } else if (opcode == ODEZZA_AST_TOGGLE2_F32 || opcode == ODEZZA_AST_TOGGLE4_F32) {
            if (!toggles_allowed || depth < shape.pops) return ODEZZA_ERROR_AST;
            for (unsigned b = 0; b < shape.payload; ++b)
                if (payload[b] >= toggle_bits) return ODEZZA_ERROR_AST;
            if (shape.payload == 2 && payload[0] == payload[1]) return ODEZZA_ERROR_AST;
            for (size_t i = depth - shape.pops; i < depth; ++i)
                if (!leaf[i]) return ODEZZA_ERROR_AST;
            depth -= shape.pops - 1u;
            leaf[depth - 1] = false;
        } else if (shape.pops) {
            if (depth < shape.pops) return ODEZZA_ERROR_AST;
            depth -= shape.pops - 1u;
            leaf[depth - 1] = false;
        } else {
            if (opcode == ODEZZA_AST_STATE_F32 && payload[0] >= states) return ODEZZA_ERROR_AST;
            if (opcode == ODEZZA_AST_CONSTANT_F32 && payload[0] >= constants) return ODEZZA_ERROR_AST;
            if (opcode == ODEZZA_AST_LITERAL_F32 && (payload[3] & 0x7f) == 0x7f && (payload[2] & 0x80)) return ODEZZA_ERROR_AST; /* Inf, NaN */
            if (depth == SECANT_AST_MAX_STACK_DEPTH) return ODEZZA_ERROR_AST;
            leaf[depth++] = true;
        }
        out.push_back(shape.secant);
        out.insert(out.end(), payload, payload + shape.payload);
        at += shape.payload;
    }
    if (!returned || depth != 1) return ODEZZA_ERROR_AST;
    return tokens > SECANT_AST_MAX_PROGRAM_INSTRUCTIONS ? ODEZZA_ERROR_SPECIALIZATION_CAPACITY : ODEZZA_SUCCESS;
}

}  // namespace

/* ---- scoring handle ---------------------------------------------------------------------------- */

struct OdezzaScoringPipeline {
    bool complete = false;
    size_t states = 0;
    uint32_t constants = 0, system_capacity = 0;
    std::vector<std::vector<uint8_t>> fixed; /* per state: the translated fixed right-hand side, empty when per-system */
    size_t fixed_count = 0;
    std::mutex mutex;
    bool running = false;
    OdezzaScoringPipelineStats stats{};
    char error[kErrorBytes] = {0};
};

namespace {

void set_error(OdezzaScoringPipeline* p, const char* format, ...) {
    if (!format) { p->error[0] = 0; return; }
    va_list args;
    va_start(args, format);
    std::vsnprintf(p->error, sizeof(p->error), format, args);
    va_end(args);
}

OdezzaResult build_handle(const OdezzaScoringPipelineCreateInfo* info, OdezzaScoringPipeline* p) {
    if (!info || !info->state_count || info->state_capacity < info->state_count || info->state_capacity > 128u ||
        info->constant_capacity < info->constant_count || !info->system_capacity || !info->shared_patch_capacity ||
        !info->system_patch_capacity || !info->worker_count || !info->cubin_slots_per_worker ||
        (uint64_t)info->worker_count * info->cubin_slots_per_worker > UINT32_MAX || (info->fixed_rhs_count && !info->fixed_rhs)) {
        set_error(p, "invalid scoring-pipeline creation description");
        return ODEZZA_ERROR_INVALID_ARGUMENT;
    }
    if (info->sm_version != 100u) {
        set_error(p, "unsupported scoring architecture sm_%u: this library is built for sm_100", info->sm_version);
        return ODEZZA_ERROR_UNSUPPORTED;
    }
    if (info->state_count > 8u || info->constant_count > SECANT_AST_MAX_INPUTS) {
        set_error(p, "the rollout kernel integrates at most 8 states with at most %u constants", SECANT_AST_MAX_INPUTS);
        return ODEZZA_ERROR_UNSUPPORTED;
    }
    if (info->fixed_rhs_count > info->state_count) {
        set_error(p, "more fixed right-hand sides than states");
        return ODEZZA_ERROR_INVALID_ARGUMENT;
    }
    p->states = info->state_count;
    p->constants = info->constant_count;
    p->system_capacity = info->system_capacity;
    p->fixed.assign(p->states, {});
    for (size_t i = 0; i < info->fixed_rhs_count; ++i) {
        const OdezzaScoringRhs& rhs = info->fixed_rhs[i];
        if (rhs.state_index >= p->states || !p->fixed[rhs.state_index].empty()) {
            set_error(p, "fixed right-hand side %zu names a missing or repeated state", i);
            return ODEZZA_ERROR_STATE_LAYOUT;
        }
        const OdezzaResult r = translate(rhs.program, p->states, p->constants, 0, false, p->fixed[rhs.state_index]);
        if (r != ODEZZA_SUCCESS) {
            set_error(p, "fixed right-hand side %zu is not a valid program", i);
            return r;
        }
    }
    p->fixed_count = info->fixed_rhs_count;
    p->complete = true;
    return ODEZZA_SUCCESS;
}

/* projects/odezza/core/o_scoring_pipeline.c:477-523 */
OdezzaResult validate_launch(const OdezzaScoringPipeline* p, const OdezzaScoringLaunch* l, size_t module_systems, uint64_t* configurations,
                             const char** why) {
    if (p->states > UINT32_MAX / l->trajectory_point_count) {
        *why = "runtime reference layout overflows the kernel index ABI";
        return ODEZZA_ERROR_OVERFLOW;
    }
    *configurations = (uint64_t)l->constant_bank_count * (1ull << l->active_toggle_count);
    const uint64_t grid = (*configurations + kReferenceThreadsPerBlock - 1u) / kReferenceThreadsPerBlock;
    if (!grid || grid > INT32_MAX || module_systems > UINT16_MAX) {
        *why = "scoring launch exceeds the supported grid dimensions";
        return ODEZZA_ERROR_UNSUPPORTED;
    }
    /* the reference stages [state + 1][point] values and the offsets in shared memory, sized in 32 bits */
    const uint64_t words = ((uint64_t)p->states + 1u) * l->trajectory_point_count + (uint64_t)l->trajectory_count + 1u;
    if (words * 4u > INT32_MAX) {
        *why = "runtime trajectory shared-memory size overflows the launch ABI";
        return ODEZZA_ERROR_OVERFLOW;
    }
    return ODEZZA_SUCCESS;
}

/* One batch of systems: programs per (system, state) in state order, then one scoring call. */
OdezzaResult score_batch(OdezzaScoringPipeline* p, const OdezzaScoringSystem* systems, size_t count, const OdezzaScoringLaunch& l,
                         std::vector<uint8_t>& bytes, std::vector<size_t>& starts, std::vector<const SecantAstInstruction*>& table,
                         double* encode_seconds) {
    const double t0 = seconds_now();
    const size_t required = p->states - p->fixed_count;
    bytes.clear();
    starts.assign(count * p->states, (size_t)-1);
    for (size_t s = 0; s < count; ++s) {
        const OdezzaScoringSystem& sys = systems[s];
        if (sys.rhs_count != required || (required && !sys.rhs)) return ODEZZA_ERROR_STATE_LAYOUT;
        for (size_t i = 0; i < sys.rhs_count; ++i) {
            const size_t state = sys.rhs[i].state_index;
            if (state >= p->states || !p->fixed[state].empty() || starts[s * p->states + state] != (size_t)-1) return ODEZZA_ERROR_STATE_LAYOUT;
            starts[s * p->states + state] = bytes.size();
            const OdezzaResult r = translate(sys.rhs[i].program, p->states, p->constants, l.active_toggle_count, true, bytes);
            if (r != ODEZZA_SUCCESS) return r;
        }
        for (size_t state = 0; state < p->states; ++state)
            if (p->fixed[state].empty() && starts[s * p->states + state] == (size_t)-1) return ODEZZA_ERROR_STATE_LAYOUT;
    }
    table.resize(count * p->states);
    for (size_t i = 0; i < table.size(); ++i) {
        const size_t state = i % p->states;
        table[i] = p->fixed[state].empty() ? bytes.data() + starts[i] : p->fixed[state].data();
    }
    *encode_seconds = seconds_now() - t0;

    SecantB200Rk4Run run;
    std::memset(&run, 0, sizeof(run));
    run.struct_size = (uint32_t)sizeof(run);
    run.version = SECANT_CUBIN_RUN_VERSION_3;
    run.programs.asts.items = table.data();
    run.programs.asts.count = table.size();
    run.num_systems = count;
    run.num_states = p->states;
    run.num_constants = p->constants;
    run.num_banks = l.constant_bank_count;
    run.toggle_bits = l.active_toggle_count;
    if (p->constants && !l.sampled_parameters_device) {
        run.constants.address = (uintptr_t)l.constant_banks_device;
        run.constants.bank_stride = p->constants;
        run.constants.num_elements = count * (size_t)l.constant_bank_count * p->constants;
    }
    run.reference.address = (uintptr_t)l.reference_data_device;
    run.reference.leading_dimension = l.trajectory_point_count;
    run.reference.num_elements = p->states * (size_t)l.trajectory_point_count;
    run.num_trajectories = l.trajectory_count;
    run.times = (uintptr_t)l.trajectory_times_device;
    run.steps_per_observation = l.steps_per_observation;
    const size_t configurations = (size_t)l.constant_bank_count << l.active_toggle_count;
    run.output.address = (uintptr_t)l.mse_output_device;
    run.output.leading_dimension = configurations;
    run.output.num_elements = count * configurations;
    run.trajectory_offsets = (uintptr_t)l.trajectory_offsets_device;
    run.total_points = l.trajectory_point_count;
    run.allow_missing_observations = l.allow_missing_observations;
    if (p->constants) {
        run.sampled_parameters = (uintptr_t)l.sampled_parameters_device;
        run.uniform_pool = (uintptr_t)l.uniform_pool_device;
        run.normal_pool = (uintptr_t)l.normal_pool_device;
        run.rng_pool_size = l.rng_pool_size;
    }
    return from_secant(secant_b200_rk4_score(&run));
}

}  // namespace

extern "C" {

OdezzaResult odezza_scoring_pipeline_create(const OdezzaScoringPipelineCreateInfo* info, OdezzaScoringPipeline** out) {
    if (!out) return ODEZZA_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    OdezzaScoringPipeline* p = new (std::nothrow) OdezzaScoringPipeline;
    if (!p) return ODEZZA_ERROR_ALLOCATION;
    *out = p; /* kept on failure: the handle then only serves write_error and destroy */
    try {
        return build_handle(info, p);
    } catch (const std::bad_alloc&) {
        set_error(p, "out of host memory");
        return ODEZZA_ERROR_ALLOCATION;
    }
}

OdezzaResult odezza_scoring_pipeline_destroy(OdezzaScoringPipeline* p) {
    if (!p) return ODEZZA_ERROR_INVALID_ARGUMENT;
    {
        std::lock_guard<std::mutex> lock(p->mutex);
        if (p->running) {
            set_error(p, "the scoring handle cannot be destroyed while a run is active");
            return ODEZZA_ERROR_BUSY;
        }
    }
    delete p;
    return ODEZZA_SUCCESS;
}

OdezzaResult odezza_scoring_pipeline_workspace_requirements(const OdezzaScoringPipeline* p, size_t* size, size_t* alignment) {
    if (!p || !size || !alignment) return ODEZZA_ERROR_INVALID_ARGUMENT;
    if (!p->complete) return ODEZZA_ERROR_BUSY;
    *size = kRunWorkspaceBytes;
    *alignment = 8;
    return ODEZZA_SUCCESS;
}

OdezzaResult odezza_scoring_pipeline_write_error(const OdezzaScoringPipeline* p, char* buffer, size_t buffer_size, size_t* bytes_ret) {
    if (!p || !bytes_ret) return ODEZZA_ERROR_INVALID_ARGUMENT;
    const size_t bytes = std::strlen(p->error);
    *bytes_ret = bytes;
    if (buffer) {
        if (buffer_size <= bytes) return ODEZZA_ERROR_INSUFFICIENT_BUFFER;
        std::memcpy(buffer, p->error, bytes + 1);
    }
    return ODEZZA_SUCCESS;
}

OdezzaResult o_scoring_pipeline_stats(const OdezzaScoringPipeline* p, OdezzaScoringPipelineStats* stats) {
    if (!p || !stats) return ODEZZA_ERROR_INVALID_ARGUMENT;
    if (!p->complete) return ODEZZA_ERROR_BUSY;
    std::lock_guard<std::mutex> lock(const_cast<OdezzaScoringPipeline*>(p)->mutex);
    *stats = p->stats;
    return ODEZZA_SUCCESS;
}

/* Order of the checks: projects/odezza/core/o_scoring_pipeline.c:1541-1594. */
OdezzaResult odezza_scoring_pipeline_run(OdezzaScoringPipeline* p, const OdezzaScoringSystem* systems, size_t system_count,
                                         const OdezzaScoringLaunch* l, void* workspace, size_t workspace_size,
                                         OdezzaScoringRunReport* report) {
    if (report) std::memset(report, 0, sizeof(*report));
    if (!p || !p->complete || !systems || !system_count || !l ||
        (p->constants && !l->constant_banks_device && !l->sampled_parameters_device) || !l->constant_bank_count || !l->reference_data_device ||
        !l->trajectory_offsets_device || !l->trajectory_times_device || !l->trajectory_count ||
        l->trajectory_point_count < l->trajectory_count || !l->steps_per_observation || !l->mse_output_device ||
        l->active_toggle_count > ODEZZA_MAX_TOGGLE_BITS || l->allow_missing_observations > 1u || l->profile_timing > 1u) {
        if (p) set_error(p, !p->complete ? "the scoring handle did not complete creation" : "invalid bulk scoring arguments or launch description");
        return ODEZZA_ERROR_INVALID_ARGUMENT;
    }
    uint64_t per_system = 0;
    const char* why = "";
    OdezzaResult result = validate_launch(p, l, system_count < p->system_capacity ? system_count : p->system_capacity, &per_system, &why);
    if (result != ODEZZA_SUCCESS) {
        set_error(p, "%s", why);
        return result;
    }
    if ((uint64_t)system_count > UINT64_MAX / per_system) {
        set_error(p, "bulk scoring configuration count overflows");
        return ODEZZA_ERROR_OVERFLOW;
    }
    const uint64_t total = (uint64_t)system_count * per_system;
    uint64_t bank_values = 0, reference_values = 0;
    if (system_count > SIZE_MAX / sizeof(*systems) || !mul_u64(system_count, l->constant_bank_count, &bank_values) ||
        !mul_u64(bank_values, p->constants, &bank_values) || !mul_u64(p->states, l->trajectory_point_count, &reference_values) ||
        !span_ok(l->constant_banks_device, l->sampled_parameters_device ? 0u : bank_values, sizeof(float)) ||
        !span_ok(l->mse_output_device, total, sizeof(float)) || !span_ok(l->reference_data_device, reference_values, sizeof(float)) ||
        !span_ok(l->trajectory_times_device, l->trajectory_point_count, sizeof(float)) ||
        !span_ok(l->trajectory_offsets_device, (uint64_t)l->trajectory_count + 1u, sizeof(uint32_t))) {
        set_error(p, "bulk scoring buffer span overflows or a device pointer is misaligned");
        return ODEZZA_ERROR_OVERFLOW;
    }
    if (l->sampled_parameters_device) {
        uint64_t descriptors = 0;
        if (!l->rng_pool_size || l->sampled_parameters_device % 8u || (!l->uniform_pool_device && !l->normal_pool_device) ||
            !mul_u64(system_count, p->constants, &descriptors) ||
            !span_ok(l->sampled_parameters_device, descriptors, sizeof(OdezzaSampledParameter)) ||
            (l->uniform_pool_device && !span_ok(l->uniform_pool_device, l->rng_pool_size, sizeof(float))) ||
            (l->normal_pool_device && !span_ok(l->normal_pool_device, l->rng_pool_size, sizeof(float)))) {
            set_error(p, "invalid sampled-constant descriptor or pool span");
            return ODEZZA_ERROR_INVALID_ARGUMENT;
        }
    }
    if (!workspace || ((uintptr_t)workspace & 7u) || workspace_size < kRunWorkspaceBytes) {
        set_error(p, "the supplied scoring workspace is null, undersized, or misaligned");
        return ODEZZA_ERROR_INVALID_ARGUMENT;
    }
    {
        std::lock_guard<std::mutex> lock(p->mutex);
        if (p->running) {
            set_error(p, "the scoring handle is already running");
            return ODEZZA_ERROR_BUSY;
        }
        p->running = true;
    }
    set_error(p, nullptr);
    const double started = seconds_now();
    cudaEvent_t begin = nullptr, end = nullptr;
    OdezzaResult failure = ODEZZA_SUCCESS;
    size_t done = 0, batches = 0;
    double encode_total = 0, score_total = 0;
    float gpu_ms = 0;
    try {
        /* inputs written on another stream are ordered before the scoring kernels (which run on the
         * default stream) through the caller's event */
        if (l->input_ready_event && cudaStreamWaitEvent(nullptr, (cudaEvent_t)l->input_ready_event, 0) != cudaSuccess) {
            set_error(p, "the input-ready event could not be waited on");
            failure = ODEZZA_ERROR_CUDA;
        }
        if (failure == ODEZZA_SUCCESS && l->profile_timing &&
            (cudaEventCreate(&begin) != cudaSuccess || cudaEventCreate(&end) != cudaSuccess || cudaEventRecord(begin, nullptr) != cudaSuccess)) {
            set_error(p, "scoring profiling origin could not be recorded");
            failure = ODEZZA_ERROR_CUDA;
        }
        std::vector<uint8_t> bytes;
        std::vector<size_t> starts;
        std::vector<const SecantAstInstruction*> table;
        while (done < system_count && failure == ODEZZA_SUCCESS) {
            const size_t count = system_count - done < kSystemsPerBatch ? system_count - done : kSystemsPerBatch;
            OdezzaScoringLaunch batch = *l;
            if (l->sampled_parameters_device) batch.sampled_parameters_device += (uint64_t)done * p->constants * sizeof(OdezzaSampledParameter);
            else batch.constant_banks_device += (uint64_t)done * l->constant_bank_count * p->constants * sizeof(float);
            batch.mse_output_device += (uint64_t)done * per_system * sizeof(float);
            double encode_seconds = 0;
            const double t0 = seconds_now();
            failure = score_batch(p, systems + done, count, batch, bytes, starts, table, &encode_seconds);
            const double spent = seconds_now() - t0;
            std::lock_guard<std::mutex> lock(p->mutex);
            if (failure == ODEZZA_SUCCESS) {
                ++batches;
                done += count;
                encode_total += encode_seconds;
                score_total += spent - encode_seconds;
                ++p->stats.submitted_ticket_count;
                ++p->stats.completed_ticket_count;
                if (p->stats.peak_pending_ticket_count < 1) p->stats.peak_pending_ticket_count = 1;
                if (p->stats.peak_inflight_module_count < 1) p->stats.peak_inflight_module_count = 1;
            } else if (failure == ODEZZA_ERROR_CUDA || failure == ODEZZA_ERROR_ALLOCATION) {
                ++p->stats.cuda_failure_count;
                set_error(p, "batch %zu failed on the device with result %d", batches, (int)failure);
            } else {
                ++p->stats.specialization_failure_count;
                set_error(p, "batch %zu failed: a candidate system is not a valid set of right-hand sides (result %d)", batches, (int)failure);
            }
        }
        if (begin && end && failure == ODEZZA_SUCCESS && cudaEventRecord(end, nullptr) == cudaSuccess && cudaEventSynchronize(end) == cudaSuccess)
            cudaEventElapsedTime(&gpu_ms, begin, end);
    } catch (const std::bad_alloc&) {
        set_error(p, "out of host memory");
        failure = ODEZZA_ERROR_ALLOCATION;
    }
    if (begin) cudaEventDestroy(begin);
    if (end) cudaEventDestroy(end);
    {
        std::lock_guard<std::mutex> lock(p->mutex);
        p->stats.specialization_seconds += encode_total;
        p->stats.launch_seconds += score_total;
        p->running = false;
    }
    if (report) {
        report->system_count = done;
        report->module_count = batches;
        report->configuration_count = failure == ODEZZA_SUCCESS ? total : (uint64_t)done * per_system;
        report->specialization_seconds = encode_total;
        report->launch_seconds = score_total;
        report->gpu_sum_seconds = report->gpu_active_seconds = report->gpu_span_seconds = gpu_ms * 1e-3;
        report->profiled_modules = l->profile_timing && failure == ODEZZA_SUCCESS ? batches : 0;
        report->total_seconds = seconds_now() - started;
    }
    return failure;
}

/* ---- random pools ------------------------------------------------------------------------------ */

OdezzaResult odezza_philox4x32(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]) {
    if (!counter || !key || !out) return ODEZZA_ERROR_INVALID_ARGUMENT;
    uint32_t c0 = counter[0], c1 = counter[1], c2 = counter[2], c3 = counter[3], k0 = key[0], k1 = key[1];
    for (int round = 0; round < 10; ++round) {
        const uint64_t p0 = 0xd2511f53ull * c0, p1 = 0xcd9e8d57ull * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        c1 = (uint32_t)p1;
        c3 = (uint32_t)p0;
        c0 = n0;
        c2 = n2;
        k0 += 0x9e3779b9u;
        k1 += 0xbb67ae85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
    return ODEZZA_SUCCESS;
}

OdezzaResult odezza_rng_uniform(uint64_t seed, uint64_t stream, uint64_t sample, float* out) {
    if (!out || stream > (uint64_t)INT64_MAX) return ODEZZA_ERROR_INVALID_ARGUMENT;
    const uint64_t block = sample / 4, domain = stream << 1;
    const uint32_t counter[4] = {(uint32_t)block, (uint32_t)(block >> 32), (uint32_t)domain, (uint32_t)(domain >> 32)};
    const uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
    uint32_t words[4];
    odezza_philox4x32(counter, key, words);
    *out = ((float)(words[sample % 4] >> 9) + 0.5f) * 1.1920928955078125e-7f;
    return ODEZZA_SUCCESS;
}

}  // extern "C"

struct OdezzaRngPool {
    OdezzaRngPoolView view{};
    bool ready = false;
    char error[kErrorBytes] = {0};
};

namespace {

bool pool_info_ok(const OdezzaRngPoolInfo* i) {
    return i && i->size && i->size <= SIZE_MAX / sizeof(float) && i->sample_base <= UINT64_MAX - i->size && i->stream <= (uint64_t)INT64_MAX &&
           i->distributions >= 1u && i->distributions <= 3u;
}

}  // namespace

extern "C" {

OdezzaResult odezza_sampled_parameter_validate(const OdezzaRngPoolInfo* pool, uint32_t banks, const OdezzaSampledParameter* p) {
    if (!pool_info_ok(pool) || !banks || !p || p->distribution > 2 || !std::isfinite(p->scale) || !std::isfinite(p->shift) ||
        !std::isfinite(p->lower) || !std::isfinite(p->upper) || p->lower > p->upper)
        return ODEZZA_ERROR_INVALID_ARGUMENT;
    if (!p->distribution) return p->shift >= p->lower && p->shift <= p->upper ? ODEZZA_SUCCESS : ODEZZA_ERROR_INVALID_ARGUMENT;
    if (!(pool->distributions & p->distribution) || !p->stride || p->offset >= pool->size ||
        (uint64_t)(banks - 1) * p->stride >= pool->size - p->offset)
        return ODEZZA_ERROR_INVALID_ARGUMENT;
    return ODEZZA_SUCCESS;
}

OdezzaResult odezza_rng_pool_create(uint32_t sm, const OdezzaRngPoolInfo* info, OdezzaRngPool** out) {
    if (!out) return ODEZZA_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    if (!pool_info_ok(info) || sm < 70 || sm > 999) return ODEZZA_ERROR_INVALID_ARGUMENT;
    OdezzaRngPool* p = new (std::nothrow) OdezzaRngPool;
    if (!p) return ODEZZA_ERROR_ALLOCATION;
    *out = p;
    p->view.info = *info;
    cudaStream_t stream = nullptr;
    cudaEvent_t begin = nullptr, end = nullptr;
    cudaError_t e = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&begin);
    if (e == cudaSuccess) e = cudaEventCreate(&end);
    for (unsigned plane = ODEZZA_RNG_UNIFORM; plane <= ODEZZA_RNG_NORMAL && e == cudaSuccess; ++plane) {
        if (!(info->distributions & plane)) continue;
        void* memory = nullptr;
        e = cudaMalloc(&memory, (size_t)info->size * sizeof(float));
        if (e != cudaSuccess) break;
        (plane == ODEZZA_RNG_UNIFORM ? p->view.uniform_device : p->view.normal_device) = (CUdeviceptr)(uintptr_t)memory;
        float ms = 0;
        e = cudaEventRecord(begin, stream);
        if (e == cudaSuccess) e = sb::fill_pool((float*)memory, info->size, info->seed, info->stream, info->sample_base, plane == ODEZZA_RNG_NORMAL, stream);
        if (e == cudaSuccess) e = cudaEventRecord(end, stream);
        if (e == cudaSuccess) e = cudaEventSynchronize(end);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, begin, end);
        (plane == ODEZZA_RNG_UNIFORM ? p->view.uniform_seconds : p->view.normal_seconds) = ms * 1e-3;
    }
    if (begin) cudaEventDestroy(begin);
    if (end) cudaEventDestroy(end);
    if (stream) cudaStreamDestroy(stream);
    if (e != cudaSuccess) {
        std::snprintf(p->error, sizeof(p->error), "%s", cudaGetErrorString(e));
        return e == cudaErrorMemoryAllocation ? ODEZZA_ERROR_ALLOCATION : ODEZZA_ERROR_CUDA;
    }
    p->ready = true;
    return ODEZZA_SUCCESS;
}

OdezzaResult odezza_rng_pool_view(const OdezzaRngPool* p, OdezzaRngPoolView* out) {
    if (!p || !p->ready || !out) return ODEZZA_ERROR_INVALID_ARGUMENT;
    *out = p->view;
    return ODEZZA_SUCCESS;
}

OdezzaResult odezza_rng_pool_write_error(const OdezzaRngPool* p, char* out, size_t capacity) {
    if (!p || !out) return ODEZZA_ERROR_INVALID_ARGUMENT;
    if (capacity <= std::strlen(p->error)) return ODEZZA_ERROR_INSUFFICIENT_BUFFER;
    std::strcpy(out, p->error);
    return ODEZZA_SUCCESS;
}

OdezzaResult odezza_rng_pool_destroy(OdezzaRngPool* p) {
    if (!p) return ODEZZA_SUCCESS;
    bool failed = false;
    if (p->view.uniform_device && cudaFree((void*)(uintptr_t)p->view.uniform_device) != cudaSuccess) failed = true;
    if (p->view.normal_device && cudaFree((void*)(uintptr_t)p->view.normal_device) != cudaSuccess) failed = true;
    delete p;
    return failed ? ODEZZA_ERROR_CUDA : ODEZZA_SUCCESS;
}

}  // extern "C"

/* ---- score reduction --------------------------------------------------------------------------- */

struct OdezzaScoreReducer {
    uint32_t k = 1;
    bool ready = false;
    cudaStream_t stream = nullptr;
    cudaEvent_t start = nullptr, stop = nullptr;
    char error[kErrorBytes] = {0};
};

namespace {

OdezzaResult reducer_cuda(OdezzaScoreReducer* r, cudaError_t e) {
    if (e == cudaSuccess) return ODEZZA_SUCCESS;
    std::snprintf(r->error, sizeof(r->error), "%s", cudaGetErrorString(e));
    return ODEZZA_ERROR_CUDA;
}

OdezzaResult grid_layout(const OdezzaScoringLaunch* l, size_t systems, uint64_t* configurations, uint64_t* scores) {
    if (!l || !systems || !l->constant_bank_count || l->active_toggle_count > 32) return ODEZZA_ERROR_INVALID_ARGUMENT;
    *configurations = (uint64_t)l->constant_bank_count << l->active_toggle_count;
    return mul_u64(systems, *configurations, scores) ? ODEZZA_SUCCESS : ODEZZA_ERROR_OVERFLOW;
}

bool range_ok(CUdeviceptr p, size_t bytes, unsigned alignment) { return p && p % alignment == 0 && bytes <= UINT64_MAX - p; }
bool overlaps(CUdeviceptr a, size_t na, CUdeviceptr b, size_t nb) { return a < b + nb && b < a + na; }

}  // namespace

extern "C" {

OdezzaResult odezza_score_reducer_create(uint32_t sm, uint32_t k, OdezzaScoreReducer** out) {
    if (!out) return ODEZZA_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    if (k < 1 || k > 256 || sm < 70 || sm > 999) return ODEZZA_ERROR_INVALID_ARGUMENT;
    OdezzaScoreReducer* r = new (std::nothrow) OdezzaScoreReducer;
    if (!r) return ODEZZA_ERROR_ALLOCATION;
    *out = r;
    r->k = k;
    OdezzaResult result = reducer_cuda(r, cudaStreamCreateWithFlags(&r->stream, cudaStreamNonBlocking));
    if (!result) result = reducer_cuda(r, cudaEventCreate(&r->start));
    if (!result) result = reducer_cuda(r, cudaEventCreate(&r->stop));
    if (result) return result;
    r->ready = true;
    return ODEZZA_SUCCESS;
}

OdezzaResult odezza_score_reducer_set_k(OdezzaScoreReducer* r, uint32_t k) {
    if (!r || !r->ready || k < 1 || k > 256) return ODEZZA_ERROR_INVALID_ARGUMENT;
    r->k = k;
    return ODEZZA_SUCCESS;
}

OdezzaResult odezza_score_reducer_destroy(OdezzaScoreReducer* r) {
    if (!r) return ODEZZA_SUCCESS;
    bool failed = false;
    if (r->stream && cudaStreamSynchronize(r->stream) != cudaSuccess) failed = true;
    if (r->start && cudaEventDestroy(r->start) != cudaSuccess) failed = true;
    if (r->stop && cudaEventDestroy(r->stop) != cudaSuccess) failed = true;
    if (r->stream && cudaStreamDestroy(r->stream) != cudaSuccess) failed = true;
    delete r;
    return failed ? ODEZZA_ERROR_CUDA : ODEZZA_SUCCESS;
}

OdezzaResult odezza_score_reducer_write_error(const OdezzaScoreReducer* r, char* out, size_t capacity) {
    if (!r || !out) return ODEZZA_ERROR_INVALID_ARGUMENT;
    if (capacity <= std::strlen(r->error)) return ODEZZA_ERROR_INSUFFICIENT_BUFFER;
    std::strcpy(out, r->error);
    return ODEZZA_SUCCESS;
}

/* projects/odezza/core/o_score_reduce.c:69-101.  The sizes are the reference's (tiles of 2048
 * scores, two ping-pong levels of partial winners), so that buffers sized for it fit both. */
OdezzaResult odezza_score_reduction_requirements(const OdezzaScoringLaunch* l, size_t systems, OdezzaScoreGrouping grouping, uint32_t k,
                                                 OdezzaScoreReductionSize* out) {
    if (!out || k < 1 || k > 256 || (int)grouping < 0 || grouping > ODEZZA_SCORE_GLOBAL) return ODEZZA_ERROR_INVALID_ARGUMENT;
    std::memset(out, 0, sizeof(*out));
    OdezzaScoreReductionSize s{};
    const OdezzaResult result = grid_layout(l, systems, &s.configuration_count, &s.score_count);
    if (result) return result;
    if (s.score_count > SIZE_MAX / sizeof(float)) return ODEZZA_ERROR_OVERFLOW;
    s.group_count = grouping == ODEZZA_SCORE_GLOBAL ? 1 : systems;
    if (grouping == ODEZZA_SCORE_BY_SYSTEM_PERMUTATION && !mul_u64(systems, 1ull << l->active_toggle_count, &s.group_count))
        return ODEZZA_ERROR_OVERFLOW;
    const uint64_t elements = s.score_count / s.group_count;
    const uint64_t tiles = 1 + (elements - 1) / 2048;
    if (tiles > UINT32_MAX) return ODEZZA_ERROR_OVERFLOW;
    s.tiles_per_group = (uint32_t)tiles;
    uint64_t partials = 0, winner_bytes = 0, count_bytes = 0;
    if (!mul_u64(s.group_count, tiles, &partials) || partials > INT32_MAX) return ODEZZA_ERROR_OVERFLOW;
    if (!mul_u64(partials, k * sizeof(OdezzaScoreWinner), &winner_bytes) || !mul_u64(partials, sizeof(OdezzaScoreCounts), &count_bytes) ||
        count_bytes > SIZE_MAX - winner_bytes || winner_bytes + count_bytes > SIZE_MAX / 2)
        return ODEZZA_ERROR_OVERFLOW;
    s.workspace_bytes = (size_t)(winner_bytes + count_bytes) * (tiles > 1 ? 2 : 1);
    s.winner_bytes = (size_t)(winner_bytes / tiles);
    s.count_bytes = (size_t)(count_bytes / tiles);
    *out = s;
    return ODEZZA_SUCCESS;
}

OdezzaResult odezza_score_decode_index(const OdezzaScoringLaunch* l, size_t systems, uint64_t index, OdezzaScoreIndex* out) {
    if (!out) return ODEZZA_ERROR_INVALID_ARGUMENT;
    std::memset(out, 0, sizeof(*out));
    uint64_t configurations = 0, scores = 0;
    const OdezzaResult result = grid_layout(l, systems, &configurations, &scores);
    if (result) return result;
    if (index >= scores) return ODEZZA_ERROR_INVALID_ARGUMENT;
    out->system_index = index / configurations;
    out->configuration_index = index % configurations;
    out->bank_index = out->configuration_index >> l->active_toggle_count;
    out->permutation = (uint32_t)(out->configuration_index & ((1ull << l->active_toggle_count) - 1));
    return ODEZZA_SUCCESS;
}

OdezzaResult odezza_score_reducer_run(OdezzaScoreReducer* r, const OdezzaScoringLaunch* l, size_t systems, OdezzaScoreGrouping grouping,
                                      CUdeviceptr workspace, size_t workspace_bytes, CUdeviceptr winners, size_t winner_bytes,
                                      CUdeviceptr counts, size_t count_bytes, OdezzaScoreReductionReport* report) {
    if (report) std::memset(report, 0, sizeof(*report));
    if (!r || !r->ready) return ODEZZA_ERROR_INVALID_ARGUMENT;
    OdezzaScoreReductionSize s;
    const OdezzaResult result = odezza_score_reduction_requirements(l, systems, grouping, r->k, &s);
    if (result) return result;
    if (workspace_bytes < s.workspace_bytes || winner_bytes < s.winner_bytes || count_bytes < s.count_bytes) return ODEZZA_ERROR_INSUFFICIENT_BUFFER;
    const CUdeviceptr pointers[4] = {l->mse_output_device, workspace, winners, counts};
    const size_t sizes[4] = {(size_t)s.score_count * 4, s.workspace_bytes, s.winner_bytes, s.count_bytes};
    for (int i = 0; i < 4; ++i) {
        if (!range_ok(pointers[i], sizes[i], i ? 8 : 4)) return ODEZZA_ERROR_INVALID_ARGUMENT;
        for (int j = 0; j < i; ++j)
            if (overlaps(pointers[i], sizes[i], pointers[j], sizes[j])) return ODEZZA_ERROR_INVALID_ARGUMENT;
    }
    if (l->input_ready_event) {
        const OdezzaResult waited = reducer_cuda(r, cudaStreamWaitEvent(r->stream, (cudaEvent_t)l->input_ready_event, 0));
        if (waited) return waited;
    }
    OdezzaResult status = reducer_cuda(r, cudaEventRecord(r->start, r->stream));
    if (status) return status;
    const SecantResult launched = sb::grouped_topk((uintptr_t)l->mse_output_device, systems, l->constant_bank_count, l->active_toggle_count,
                                                   (uint32_t)grouping, r->k, (uintptr_t)winners, (uintptr_t)counts, (uintptr_t)workspace,
                                                   s.workspace_bytes, r->stream);
    if (launched != SECANT_SUCCESS) {
        std::snprintf(r->error, sizeof(r->error), "the reduction could not be launched (result %d)", (int)launched);
        return from_secant(launched);
    }
    float ms = 0;
    status = reducer_cuda(r, cudaEventRecord(r->stop, r->stream));
    if (!status) status = reducer_cuda(r, cudaEventSynchronize(r->stop));
    if (!status) status = reducer_cuda(r, cudaEventElapsedTime(&ms, r->start, r->stop));
    if (status) return status;
    if (report) {
        report->kernel_seconds = ms * 1e-3;
        report->group_count = s.group_count;
        report->score_count = s.score_count;
    }
    return ODEZZA_SUCCESS;
}

/* projects/odezza/core/o_score_reduce.c:228-270 */
OdezzaResult odezza_score_reducer_gather(OdezzaScoreReducer* r, const OdezzaScoringLaunch* l, size_t systems, OdezzaScoreGrouping grouping,
                                         uint32_t constants, CUdeviceptr winners, size_t winner_bytes, CUdeviceptr rows, size_t row_bytes) {
    if (!r || !r->ready) return ODEZZA_ERROR_INVALID_ARGUMENT;
    OdezzaScoreReductionSize s;
    const OdezzaResult result = odezza_score_reduction_requirements(l, systems, grouping, r->k, &s);
    if (result) return result;
    if (!constants) return ODEZZA_SUCCESS;
    const uint64_t entries = s.group_count * r->k;
    uint64_t values = 0, bank_values = 0;
    if (!mul_u64(entries, constants, &values) || !mul_u64(systems, l->constant_bank_count, &bank_values) ||
        !mul_u64(bank_values, constants, &bank_values) || values > SIZE_MAX / 4 || bank_values > SIZE_MAX / 4)
        return ODEZZA_ERROR_OVERFLOW;
    if (winner_bytes < s.winner_bytes || row_bytes < values * 4) return ODEZZA_ERROR_INSUFFICIENT_BUFFER;
    const bool sampled = l->sampled_parameters_device != 0;
    const size_t row_span = (size_t)values * 4, bank_span = (size_t)bank_values * 4;
    if (!range_ok(winners, s.winner_bytes, 8) || !range_ok(rows, row_span, 4) || (!sampled && !range_ok(l->constant_banks_device, bank_span, 4)) ||
        overlaps(winners, s.winner_bytes, rows, row_span) || (!sampled && overlaps(l->constant_banks_device, bank_span, rows, row_span)))
        return ODEZZA_ERROR_INVALID_ARGUMENT;
    if (sampled) {
        uint64_t descriptors = 0;
        if (!mul_u64(systems, constants, &descriptors) || descriptors > SIZE_MAX / sizeof(OdezzaSampledParameter) || !l->rng_pool_size ||
            l->rng_pool_size > SIZE_MAX / 4 || (!l->uniform_pool_device && !l->normal_pool_device))
            return ODEZZA_ERROR_INVALID_ARGUMENT;
        const size_t descriptor_span = (size_t)descriptors * sizeof(OdezzaSampledParameter), pool_span = (size_t)l->rng_pool_size * 4;
        if (!range_ok(l->sampled_parameters_device, descriptor_span, 8) || overlaps(l->sampled_parameters_device, descriptor_span, rows, row_span))
            return ODEZZA_ERROR_INVALID_ARGUMENT;
        if (l->uniform_pool_device && (!range_ok(l->uniform_pool_device, pool_span, 4) || overlaps(l->uniform_pool_device, pool_span, rows, row_span)))
            return ODEZZA_ERROR_INVALID_ARGUMENT;
        if (l->normal_pool_device && (!range_ok(l->normal_pool_device, pool_span, 4) || overlaps(l->normal_pool_device, pool_span, rows, row_span)))
            return ODEZZA_ERROR_INVALID_ARGUMENT;
    }
    sb::GatherProblem g;
    g.winners = reinterpret_cast<const SecantB200Winner*>((uintptr_t)winners);
    g.banks = sampled ? nullptr : reinterpret_cast<const float*>((uintptr_t)l->constant_banks_device);
    g.sampled = reinterpret_cast<const SecantB200SampledParameter*>((uintptr_t)l->sampled_parameters_device);
    g.uniform_pool = reinterpret_cast<const float*>((uintptr_t)l->uniform_pool_device);
    g.normal_pool = reinterpret_cast<const float*>((uintptr_t)l->normal_pool_device);
    g.pool_size = l->rng_pool_size;
    g.entries = entries;
    g.configurations = s.configuration_count;
    g.bank_count = l->constant_bank_count;
    g.score_count = s.score_count;
    g.toggle_bits = l->active_toggle_count;
    g.constants = constants;
    g.rows = reinterpret_cast<float*>((uintptr_t)rows);
    if (l->input_ready_event) {
        const OdezzaResult waited = reducer_cuda(r, cudaStreamWaitEvent(r->stream, (cudaEvent_t)l->input_ready_event, 0));
        if (waited) return waited;
    }
    OdezzaResult status = reducer_cuda(r, sb::gather_constants(g, r->stream));
    if (!status) status = reducer_cuda(r, cudaStreamSynchronize(r->stream));
    return status;
}

}  // extern "C"
