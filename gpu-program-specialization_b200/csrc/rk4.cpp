/*
 * rk4.cpp - host side of the RK4 rollout-scoring entry point (secant_b200_rk4_score).
 *
 * The rollout variant scores candidate right-hand sides of an S-state system by integrating
 * them with fixed-step RK4 from the first point of every reference trajectory and returning
 * the mean squared error against the reference, with the reference engine's invalid-data
 * policy (projects/odezza/core/o_generate_scoring_cuda.c:494-588,
 * projects/odezza/core/odezza.h:285-289).  Right-hand sides are ordinary Secant programs:
 * COLUMN s reads state s, BANK_CONSTANT k reads coefficient k of the system's bank.
 * This call is blocking and self-contained: it validates and encodes the programs, uploads
 * the records, launches the kernel, waits, and releases its temporary device buffer.
 */
#include "evaluator.cuh"
#include "internal.h"

#include <cstddef>
#include <cstring>
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
    if (run->reserved3 || run->allow_missing_observations > 1) return SECANT_ERROR_INVALID_VALUE;
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
    EncodedBatch enc;
    try {
        enc.programs.reserve(programs.asts.count);
        for (size_t i = 0; i < programs.asts.count && result == SECANT_SUCCESS; ++i)
            result = encode_program(programs.asts.items[i], programs.routines, arity, rules, enc);
    } catch (const std::bad_alloc&) {
        return SECANT_ERROR_ALLOCATION_FAILED;
    }
    if (result != SECANT_SUCCESS) return result;

    auto align256 = [](size_t v) { return (v + 255) / 256 * 256; };
    const size_t o_insn = align256(enc.programs.size() * sizeof(SbProgram));
    const size_t o_patch = align256(o_insn + enc.insns.size() * sizeof(SbInsn));
    const size_t o_aff = align256(o_patch + enc.patches.size() * sizeof(SbPatch));
    const size_t o_lit = align256(o_aff + enc.affines.size() * sizeof(SbAffine));
    const size_t o_flag = align256(o_lit + enc.lits.size() * sizeof(float) + 16); /* one word raised by the data validation */
    const size_t total = o_flag + 256;
    std::vector<char> host(total, 0);
    std::memcpy(host.data(), enc.programs.data(), enc.programs.size() * sizeof(SbProgram));
    std::memcpy(host.data() + o_insn, enc.insns.data(), enc.insns.size() * sizeof(SbInsn));
    if (!enc.patches.empty()) std::memcpy(host.data() + o_patch, enc.patches.data(), enc.patches.size() * sizeof(SbPatch));
    if (!enc.affines.empty()) std::memcpy(host.data() + o_aff, enc.affines.data(), enc.affines.size() * sizeof(SbAffine));
    if (!enc.lits.empty()) std::memcpy(host.data() + o_lit, enc.lits.data(), enc.lits.size() * sizeof(float));

    int device = 0, limit = 0;
    char* d = nullptr;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess)
        return SECANT_ERROR_DRIVER_FAILED;
    if (cudaMalloc(&d, total) != cudaSuccess) return SECANT_ERROR_ALLOCATION_FAILED;
    cudaError_t e = cudaMemcpy(d, host.data(), total, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) {
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
        p.num_systems = (uint32_t)run->num_systems; p.num_states = (uint32_t)S; p.num_constants = (uint32_t)K;
        p.num_banks = (uint32_t)run->num_banks; p.toggle_bits = run->toggle_bits;
        p.banks = reinterpret_cast<const float*>(run->constants.address);
        p.bank_stride = run->constants.bank_stride;
        p.system_bank_stride = run->system_bank_stride ? run->system_bank_stride : run->num_banks * run->constants.bank_stride;
        p.reference = reinterpret_cast<const float*>(run->reference.address);
        p.reference_ld = run->reference.leading_dimension;
        p.num_trajectories = (uint32_t)run->num_trajectories; p.points_per_trajectory = (uint32_t)run->points_per_trajectory;
        p.substeps = (uint32_t)run->steps_per_observation;
        p.times = reinterpret_cast<const float*>(run->times);
        p.offsets = reinterpret_cast<const uint32_t*>(run->trajectory_offsets);
        p.total_points = (uint32_t)total_points;
        p.allow_missing = run->allow_missing_observations;
        p.invalid_flag = reinterpret_cast<int*>(d + o_flag);
        p.sampled = reinterpret_cast<const SecantB200SampledParameter*>(run->sampled_parameters);
        p.uniform_pool = reinterpret_cast<const float*>(run->uniform_pool);
        p.normal_pool = reinterpret_cast<const float*>(run->normal_pool);
        p.pool_size = run->rng_pool_size;
        if (sampled) p.banks = nullptr;
        p.output = reinterpret_cast<float*>(run->output.address);
        p.output_ld = run->output.leading_dimension;
        e = launch_rk4(db, p, (size_t)limit, nullptr);
        if (e == cudaSuccess) note_kernel_launches(2);
        if (e == cudaErrorInvalidConfiguration) { cudaFree(d); return SECANT_ERROR_REGISTER_OVERFLOW; }
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
    }
    const cudaError_t f = cudaFree(d);
    if (e == cudaSuccess) e = f;
    return e == cudaSuccess ? SECANT_SUCCESS : SECANT_ERROR_DRIVER_FAILED;
}
