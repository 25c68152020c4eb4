/*
 * rk4.cpp - host side of the RK4 rollout-scoring entry point (secant_b200_rk4_score).
 *
 * The rollout variant scores candidate right-hand sides of an S-state system by integrating
 * them with fixed-step RK4 from the first point of every reference trajectory and returning
 * the mean squared error against the reference, with the reference engine's invalid-data
 * policy (projects/odezza/core/o_generate_scoring_cuda.c:494-588,
 * projects/odezza/core/odezza.h:285-289).  Right-hand sides are ordinary Secant programs:
 * COLUMN s reads state s, BANK_CONSTANT k reads coefficient k of the system's bank.
 * This call is blocking and self-contained: it validates the programs, encodes them in chunks on
 * a few host threads while earlier chunks are already being uploaded and scored on the call's own
 * stream (ordered after whatever the caller queued on the default stream), waits, and releases its
 * temporary device buffers.
 */
#include "evaluator.cuh"
#include "internal.h"

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstddef>
#include <cstring>
#include <exception>
#include <mutex>
#include <system_error>
#include <thread>
#include <vector>

using namespace sb;

extern "C" SecantResult secant_b200_rk4_score(const SecantB200Rk4Run* given) {
    /* the uniform form ends before trajectory_offsets; shorter structs are extended with zeros */
    const size_t uniform_size = offsetof(SecantB200Rk4Run, trajectory_offsets);
    if (!given || given->struct_size < uniform_size) return SECANT_ERROR_INVALID_VALUE;
    SecantB200Rk4Run local;
    std::memset(&local, 0, sizeof(local));
    std::memcpy(&local, given, given->struct_size < sizeof(local) ? given->struct_size : sizeof(local));
    const SecantB200Rk4Run* run = &local;
    const bool ragged = run->trajectory_offsets != 0;
    if (run->reserved3 || run->allow_missing_observations > 1 || run->integrated_intervals % 8) return SECANT_ERROR_INVALID_VALUE;
    if (run->version != SECANT_CUBIN_RUN_VERSION_3) return SECANT_ERROR_UNSUPPORTED_VERSION;
    if (run->flags) return SECANT_ERROR_INVALID_VALUE;
    const size_t S = run->num_states, K = run->num_constants;
    const SecantAstProgramSet& programs = run->programs;
    if (!S || S > 8 || K > SECANT_AST_MAX_INPUTS || !run->num_systems || !programs.asts.items ||
        programs.asts.count != run->num_systems * S || programs.routines.count > SECANT_AST_MAX_ROUTINES ||
        (programs.routines.count && !programs.routines.items) || !run->num_banks || run->toggle_bits > 32 ||
        !run->num_trajectories || (!ragged && run->points_per_trajectory < 2) || !run->steps_per_observation || !run->times ||
        run->num_systems > 0x7fffffffull / S || run->num_trajectories > 0xffffffffull || run->points_per_trajectory > 0xffffffffull ||
        run->steps_per_observation > 0xffffffffull)
        return SECANT_ERROR_INVALID_VALUE;
    if (ragged && (run->trajectory_offsets % 4 || run->total_points < run->num_trajectories || run->total_points > 0xffffffffull))
        return SECANT_ERROR_INVALID_VALUE;
    if (!ragged && run->num_trajectories > 0xffffffffull / run->points_per_trajectory) return SECANT_ERROR_OVERFLOW;
    const size_t total_points = ragged ? run->total_points : run->num_trajectories * run->points_per_trajectory;
    const size_t configs = run->num_banks << run->toggle_bits;
    if (run->reference.leading_dimension < total_points || run->reference.num_elements < (S - 1) * run->reference.leading_dimension + total_points ||
        !run->reference.address || run->reference.address % 4 || run->times % 4)
        return run->reference.address && run->reference.leading_dimension >= total_points ? SECANT_ERROR_INSUFFICIENT_BUFFER : SECANT_ERROR_INVALID_VALUE;
    if (run->output.leading_dimension < configs || !run->output.address || run->output.address % 4) return SECANT_ERROR_INVALID_VALUE;
    if (run->output.num_elements < (run->num_systems - 1) * run->output.leading_dimension + configs) return SECANT_ERROR_INSUFFICIENT_BUFFER;
    const bool sampled = run->sampled_parameters != 0;
    if (sampled && (!K || run->sampled_parameters % 8 || run->uniform_pool % 4 || run->normal_pool % 4 ||
                    (run->rng_pool_size && !run->uniform_pool && !run->normal_pool)))
        return SECANT_ERROR_INVALID_VALUE;
    if (K && !sampled) {
        if (run->constants.bank_stride < K || !run->constants.address || run->constants.address % 4) return SECANT_ERROR_INVALID_VALUE;
        const size_t per_system = run->system_bank_stride ? run->system_bank_stride : run->num_banks * run->constants.bank_stride;
        if (per_system < (run->num_banks - 1) * run->constants.bank_stride + K) return SECANT_ERROR_INVALID_VALUE;
        if (run->constants.num_elements < (run->num_systems - 1) * per_system + (run->num_banks - 1) * run->constants.bank_stride + K)
            return SECANT_ERROR_INSUFFICIENT_BUFFER;
    }

    ProgramRules rules;
    rules.num_columns = S;
    rules.num_constants = K;
    rules.banks_allowed = true;
    rules.toggle_bits = run->toggle_bits;
    rules.columns_are_slots = true;
    rules.reserved_slots = (unsigned)(4 * S); /* stage, next stage, sum, state vectors */
    for (size_t i = 0; i < programs.routines.count; ++i) {
        const SecantResult r = preflight(programs.routines.items[i], rules);
        if (r != SECANT_SUCCESS) return r;
    }
    for (size_t i = 0; i < programs.asts.count; ++i) {
        const SecantResult r = preflight(programs.asts.items[i], rules);
        if (r != SECANT_SUCCESS) return r;
    }
    uint8_t arity[SECANT_AST_MAX_ROUTINES];
    SecantResult result = routine_arities(programs.routines, arity);
    if (result != SECANT_SUCCESS) return result;

    int device = 0, limit = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess)
        return SECANT_ERROR_DRIVER_FAILED;

    /* Systems are encoded in chunks by a few host threads while the calling thread uploads and
     * launches the chunks in order on one stream, so encoding overlaps the kernels of earlier
     * chunks.  A structural error found while encoding a later chunk ends the call with that code;
     * scores of earlier chunks may already have been written. */
    constexpr size_t kChunkSystems = 2048;
    const size_t num_chunks = (run->num_systems + kChunkSystems - 1) / kChunkSystems;
    struct Chunk {
        EncodedBatch enc;
        SecantResult status = SECANT_SUCCESS;
        std::vector<char> host;
        char* device = nullptr;
    };
    std::vector<Chunk> chunks;
    std::mutex mutex;
    std::condition_variable ready;
    std::vector<char> done;
    std::atomic<size_t> next_chunk{0};
    std::atomic<bool> stop{false};
    try {
        chunks.resize(num_chunks);
        done.assign(num_chunks, 0);
    } catch (const std::bad_alloc&) {
        return SECANT_ERROR_ALLOCATION_FAILED;
    }
    auto encode_one = [&](size_t c) {
        Chunk& chunk = chunks[c];
        const size_t first = c * kChunkSystems * S;
        const size_t count = std::min(kChunkSystems, run->num_systems - c * kChunkSystems) * S;
        try {
            chunk.enc.programs.reserve(count);
            for (size_t i = 0; i < count && chunk.status == SECANT_SUCCESS; ++i)
                chunk.status = encode_program(programs.asts.items[first + i], programs.routines, arity, rules, chunk.enc);
        } catch (const std::bad_alloc&) {
            chunk.status = SECANT_ERROR_ALLOCATION_FAILED;
        }
        {
            std::lock_guard<std::mutex> lock(mutex);
            done[c] = 1;
        }
        ready.notify_all();
    };
    auto encode_chunks = [&]() {
        for (;;) {
            const size_t c = next_chunk.fetch_add(1);
            if (c >= num_chunks || stop.load()) return;
            encode_one(c);
        }
    };
    std::vector<std::thread> workers;
    const unsigned hardware = std::thread::hardware_concurrency();
    const size_t want_workers = std::min<size_t>(num_chunks > 1 ? num_chunks - 1 : 0, std::min<unsigned>(hardware ? hardware : 1u, 8u));
    try {
        workers.reserve(want_workers);
        for (size_t w = 0; w < want_workers; ++w) workers.emplace_back(encode_chunks);
    } catch (const std::exception&) {
        /* no memory or no thread to be had: fewer helpers, or none; the calling thread encodes whatever is left */
    }

    /* records travel on their own stream, so an upload never waits for the kernels of earlier chunks;
     * the chunks' kernels go round the compute streams, so a chunk smaller than the GPU shares it
     * with its neighbours */
    constexpr int kComputeStreams = 4;
    cudaStream_t compute[kComputeStreams] = {nullptr, nullptr, nullptr, nullptr}, copies = nullptr;
    cudaEvent_t uploaded = nullptr;
    cudaError_t e = cudaStreamCreateWithFlags(&copies, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&uploaded, cudaEventDisableTiming);
    /* what the caller queued on the default stream before this call (fills, copies, an event wait)
     * comes first, as it did when the kernels themselves ran on that stream */
    if (e == cudaSuccess) e = cudaEventRecord(uploaded, nullptr);
    for (int i = 0; i < kComputeStreams && e == cudaSuccess; ++i) {
        e = cudaStreamCreateWithFlags(&compute[i], cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(compute[i], uploaded, 0);
    }
    auto align256 = [](size_t v) { return (v + 255) / 256 * 256; };
    unsigned launches = 0;
    for (size_t c = 0; c < num_chunks && e == cudaSuccess && result == SECANT_SUCCESS; ++c) {
        for (;;) { /* wait for chunk c; while it is in other hands, encode chunks nobody has taken */
            {
                std::lock_guard<std::mutex> lock(mutex);
                if (done[c]) break;
            }
            const size_t mine = next_chunk.fetch_add(1);
            if (mine < num_chunks) {
                encode_one(mine);
            } else {
                std::unique_lock<std::mutex> lock(mutex);
                ready.wait(lock, [&] { return done[c] != 0; });
            }
        }
        Chunk& chunk = chunks[c];
        if (chunk.status != SECANT_SUCCESS) { result = chunk.status; break; }
        const EncodedBatch& enc = chunk.enc;
        const size_t o_insn = align256(enc.programs.size() * sizeof(SbProgram));
        const size_t o_patch = align256(o_insn + enc.insns.size() * sizeof(SbInsn));
        const size_t o_aff = align256(o_patch + enc.patches.size() * sizeof(SbPatch));
        const size_t o_lit = align256(o_aff + enc.affines.size() * sizeof(SbAffine));
        const size_t o_flag = align256(o_lit + enc.lits.size() * sizeof(float) + 16); /* one word raised by the data validation */
        const size_t total = o_flag + 256;
        try {
            chunk.host.assign(total, 0);
        } catch (const std::bad_alloc&) {
            result = SECANT_ERROR_ALLOCATION_FAILED;
            break;
        }
        char* host = chunk.host.data();
        std::memcpy(host, enc.programs.data(), enc.programs.size() * sizeof(SbProgram));
        std::memcpy(host + o_insn, enc.insns.data(), enc.insns.size() * sizeof(SbInsn));
        if (!enc.patches.empty()) std::memcpy(host + o_patch, enc.patches.data(), enc.patches.size() * sizeof(SbPatch));
        if (!enc.affines.empty()) std::memcpy(host + o_aff, enc.affines.data(), enc.affines.size() * sizeof(SbAffine));
        if (!enc.lits.empty()) std::memcpy(host + o_lit, enc.lits.data(), enc.lits.size() * sizeof(float));
        if (cudaMalloc(&chunk.device, total) != cudaSuccess) { result = SECANT_ERROR_ALLOCATION_FAILED; break; }
        char* d = chunk.device;
        e = cudaMemcpyAsync(d, host, total, cudaMemcpyHostToDevice, copies);
        if (e == cudaSuccess) e = cudaEventRecord(uploaded, copies);
        cudaStream_t stream = compute[c % kComputeStreams];
        if (e == cudaSuccess) e = cudaStreamWaitEvent(stream, uploaded, 0);
        if (e != cudaSuccess) break;
        const size_t first_system = c * kChunkSystems;
        const size_t systems = enc.programs.size() / S;
        DeviceBatch db;
        std::memset(&db, 0, sizeof(db));
        db.programs = reinterpret_cast<const SbProgram*>(d);
        db.insns = reinterpret_cast<const SbInsn*>(d + o_insn);
        db.patches = reinterpret_cast<const SbPatch*>(d + o_patch);
        db.affines = reinterpret_cast<const SbAffine*>(d + o_aff);
        db.lits = reinterpret_cast<const float*>(d + o_lit);
        db.num_programs = (uint32_t)enc.programs.size();
        db.max_insn = enc.max_insn;
        db.max_extra = enc.max_extra;
        db.max_slots = enc.max_slots > rules.reserved_slots ? enc.max_slots : rules.reserved_slots;
        db.max_hoisted = 0;
        Rk4Problem p;
        p.num_systems = (uint32_t)systems; p.num_states = (uint32_t)S; p.num_constants = (uint32_t)K;
        p.num_banks = (uint32_t)run->num_banks; p.toggle_bits = run->toggle_bits;
        p.bank_stride = run->constants.bank_stride;
        p.system_bank_stride = run->system_bank_stride ? run->system_bank_stride : run->num_banks * run->constants.bank_stride;
        p.banks = sampled || !K ? nullptr : reinterpret_cast<const float*>(run->constants.address) + first_system * p.system_bank_stride;
        p.reference = reinterpret_cast<const float*>(run->reference.address);
        p.reference_ld = run->reference.leading_dimension;
        p.num_trajectories = (uint32_t)run->num_trajectories; p.points_per_trajectory = (uint32_t)run->points_per_trajectory;
        p.substeps = (uint32_t)run->steps_per_observation;
        p.times = reinterpret_cast<const float*>(run->times);
        p.offsets = reinterpret_cast<const uint32_t*>(run->trajectory_offsets);
        p.total_points = (uint32_t)total_points;
        p.allow_missing = run->allow_missing_observations;
        p.invalid_flag = reinterpret_cast<int*>(d + o_flag);
        p.queue = reinterpret_cast<unsigned long long*>(d + o_flag + 8); /* uploaded as zeros with the records */
        p.sampled = sampled ? reinterpret_cast<const SecantB200SampledParameter*>(run->sampled_parameters) + first_system * K : nullptr;
        p.uniform_pool = reinterpret_cast<const float*>(run->uniform_pool);
        p.normal_pool = reinterpret_cast<const float*>(run->normal_pool);
        p.pool_size = run->rng_pool_size;
        p.output = reinterpret_cast<float*>(run->output.address) + first_system * run->output.leading_dimension;
        p.output_ld = run->output.leading_dimension;
        p.integrated = reinterpret_cast<unsigned long long*>(run->integrated_intervals);
        e = launch_rk4(db, p, (size_t)limit, stream);
        if (e == cudaErrorInvalidConfiguration) { result = SECANT_ERROR_REGISTER_OVERFLOW; e = cudaSuccess; break; }
        if (e == cudaSuccess) launches += 2;
    }
    stop.store(true);
    for (std::thread& t : workers) t.join();
    cudaStream_t all_streams[kComputeStreams + 1];
    for (int i = 0; i < kComputeStreams; ++i) all_streams[i] = compute[i];
    all_streams[kComputeStreams] = copies;
    for (cudaStream_t q : all_streams) /* also on failure: nothing of this call stays in flight */
        if (q) {
            const cudaError_t f = cudaStreamSynchronize(q);
            if (e == cudaSuccess) e = f;
        }
    for (Chunk& chunk : chunks)
        if (chunk.device) {
            const cudaError_t f = cudaFree(chunk.device);
            if (e == cudaSuccess) e = f;
        }
    if (uploaded) cudaEventDestroy(uploaded);
    for (cudaStream_t q : all_streams)
        if (q) {
            const cudaError_t f = cudaStreamDestroy(q);
            if (e == cudaSuccess) e = f;
        }
    if (launches) note_kernel_launches(launches);
    if (result != SECANT_SUCCESS) return result;
    return e == cudaSuccess ? SECANT_SUCCESS : SECANT_ERROR_DRIVER_FAILED;
}
