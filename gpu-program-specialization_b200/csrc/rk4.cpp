/*
 * rk4.cpp - host side of the RK4 rollout-scoring entry point (secant_b200_rk4_score).
 *
 * The rollout variant scores candidate right-hand sides of an S-state system by integrating
 * them with fixed-step RK4 from the first point of every reference trajectory and returning
 * the mean squared error against the reference, with the reference engine's invalid-data
 * policy (projects/odezza/core/o_generate_scoring_cuda.c:494-588,
 * projects/odezza/core/odezza.h:285-289).  Right-hand sides are ordinary Secant programs:
 * COLUMN s reads state s, BANK_CONSTANT k reads coefficient k of the system's bank.
 * This call is blocking and self-contained: host threads scan the programs and encode them in
 * pieces while the calling thread joins encoded pieces into launches, uploads them and starts their
 * kernels on the call's own streams (ordered after whatever the caller queued on the default
 * stream); it waits for all of them and hands its record buffers back to the library's memory pool.
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

namespace {

/* Record buffers live for one call; the pool keeps their memory between calls. */
constexpr int kMaxPoolDevices = 64;
std::mutex g_pool_mutex;
cudaMemPool_t g_pools[kMaxPoolDevices] = {};

cudaMemPool_t record_pool(int device) {
    if (device < 0 || device >= kMaxPoolDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    if (!g_pools[device]) {
        cudaMemPoolProps props;
        std::memset(&props, 0, sizeof(props));
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = device;
        cudaMemPool_t pool = nullptr;
        if (cudaMemPoolCreate(&pool, &props) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        unsigned long long keep = ~0ull; /* nothing goes back to the driver until it is asked for */
        if (cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep) != cudaSuccess) {
            cudaGetLastError();
            cudaMemPoolDestroy(pool);
            return nullptr;
        }
        g_pools[device] = pool;
    }
    return g_pools[device];
}

}  // namespace

extern "C" SecantResult secant_b200_release_cached_memory(void) {
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    SecantResult result = SECANT_SUCCESS;
    for (cudaMemPool_t pool : g_pools)
        if (pool && cudaMemPoolTrimTo(pool, 0) != cudaSuccess) result = SECANT_ERROR_DRIVER_FAILED;
    return result;
}

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
    rules.split_parts = true;                 /* what depends on the constants only is computed once per candidate, */
    rules.hoist_bank = true;                  /* not once per stage */
    rules.fuse_store_load = true;
    for (size_t i = 0; i < programs.routines.count; ++i) {
        const SecantResult r = preflight(programs.routines.items[i], rules);
        if (r != SECANT_SUCCESS) return r;
    }
    uint8_t arity[SECANT_AST_MAX_ROUTINES];
    SecantResult result = routine_arities(programs.routines, arity);
    if (result != SECANT_SUCCESS) return result;

    /* Host threads work on pieces of 128 systems: first every piece is scanned (nothing is launched
     * before every program has passed the scan, and the first failing program in order decides the
     * result), then the pieces are encoded while the calling thread joins sixteen encoded pieces into
     * one launch, uploads it and starts its kernels, so encoding overlaps the kernels of earlier
     * launches.  A structural error found while encoding a later piece ends the call with that
     * code; scores of earlier launches may already have been written. */
    constexpr size_t kPieceSystems = 128, kPiecesPerLaunch = 16;
    const size_t num_pieces = (run->num_systems + kPieceSystems - 1) / kPieceSystems;
    const size_t num_chunks = (num_pieces + kPiecesPerLaunch - 1) / kPiecesPerLaunch;
    struct Piece {
        EncodedBatch enc;
        std::vector<uint32_t> cost; /* per system: its main parts' instructions, weighted as the rollout machine executes them */
        SecantResult status = SECANT_SUCCESS;
    };
    struct Chunk {
        std::vector<char> host;
        char* device = nullptr;
        bool pooled = false;
    };
    std::vector<Piece> pieces;
    std::vector<Chunk> chunks;
    std::mutex mutex;
    std::condition_variable ready;
    std::vector<char> done;          /* piece encoded */
    size_t scanned = 0;              /* pieces scanned */
    bool encoding_open = false;      /* every piece passed the scan */
    std::atomic<size_t> next_scan{0}, next_piece{0};
    std::atomic<bool> stop{false};
    try {
        pieces.resize(num_pieces);
        chunks.resize(num_chunks);
        done.assign(num_pieces, 0);
    } catch (const std::bad_alloc&) {
        return SECANT_ERROR_ALLOCATION_FAILED;
    }
    auto piece_range = [&](size_t c, size_t* first, size_t* count) {
        *first = c * kPieceSystems * S;
        *count = std::min(kPieceSystems, run->num_systems - c * kPieceSystems) * S;
    };
    auto scan_one = [&](size_t c) {
        size_t first, count;
        piece_range(c, &first, &count);
        SecantResult r = SECANT_SUCCESS;
        for (size_t i = 0; i < count && r == SECANT_SUCCESS; ++i) r = preflight(programs.asts.items[first + i], rules);
        std::lock_guard<std::mutex> lock(mutex);
        pieces[c].status = r;
        ++scanned;
        if (scanned == num_pieces) ready.notify_all();
    };
    auto encode_one = [&](size_t c) {
        Piece& piece = pieces[c];
        size_t first, count;
        piece_range(c, &first, &count);
        try {
            piece.enc.programs.reserve(count);
            for (size_t i = 0; i < count && piece.status == SECANT_SUCCESS; ++i)
                piece.status = encode_program(programs.asts.items[first + i], programs.routines, arity, rules, piece.enc);
            if (piece.status == SECANT_SUCCESS) { /* about 25 issue slots per instruction, 45 more for a function or a division */
                piece.cost.assign(count / S, 0);
                for (size_t i = 0; i < count; ++i) {
                    const SbProgram& pr = piece.enc.programs[i];
                    uint32_t cost = 0;
                    for (uint32_t at = pr.main_off; at < pr.n_insn; ++at) {
                        const unsigned cs = piece.enc.insns[pr.insn_off + at].w0 & 0xffu;
                        const bool division = cs >= SB_CASE_BIN + SB_BIN_DIV * SB_NUM_KINDS && cs < SB_CASE_BIN + (SB_BIN_RDIV + 1) * SB_NUM_KINDS;
                        const bool function = cs >= SB_CASE_UN && cs < SB_CASE_FMA && cs != SB_CASE_UN + SB_UN_NEG && cs != SB_CASE_UN + SB_UN_ABS;
                        cost += division || function ? 70u : 25u;
                    }
                    piece.cost[i / S] += cost;
                }
            }
        } catch (const std::bad_alloc&) {
            piece.status = SECANT_ERROR_ALLOCATION_FAILED;
        }
        {
            std::lock_guard<std::mutex> lock(mutex);
            done[c] = 1;
        }
        ready.notify_all();
    };
    auto scan_pieces = [&]() {
        for (;;) {
            const size_t c = next_scan.fetch_add(1);
            if (c >= num_pieces) return;
            scan_one(c);
        }
    };
    auto worker = [&]() {
        scan_pieces();
        {
            std::unique_lock<std::mutex> lock(mutex);
            ready.wait(lock, [&] { return encoding_open || stop.load(); });
        }
        for (;;) {
            const size_t c = next_piece.fetch_add(1);
            if (c >= num_pieces || stop.load()) return;
            encode_one(c);
        }
    };
    std::vector<std::thread> workers;
    const unsigned hardware = std::thread::hardware_concurrency();
    const size_t want_workers = std::min<size_t>(num_pieces > 1 ? num_pieces - 1 : 0, std::min<unsigned>(hardware ? hardware : 1u, 16u) - 1u);
    try {
        workers.reserve(want_workers);
        for (size_t w = 0; w < want_workers; ++w) workers.emplace_back(worker);
    } catch (const std::exception&) {
        /* no memory or no thread to be had: fewer helpers, or none; the calling thread does whatever is left */
    }
    scan_pieces();
    {
        std::unique_lock<std::mutex> lock(mutex);
        ready.wait(lock, [&] { return scanned == num_pieces; });
        for (size_t c = 0; c < num_pieces && result == SECANT_SUCCESS; ++c) result = pieces[c].status; /* the first failing program in order */
        if (result == SECANT_SUCCESS) encoding_open = true;
        else stop.store(true);
    }
    ready.notify_all();
    /* the device is asked for only now: a request with a malformed program is answered with that
     * program's code whether or not a device can be had */
    int device = 0, limit = 0;
    if (result == SECANT_SUCCESS && (cudaGetDevice(&device) != cudaSuccess ||
                                     cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess)) {
        cudaGetLastError();
        result = SECANT_ERROR_DRIVER_FAILED;
        {
            std::lock_guard<std::mutex> lock(mutex);
            stop.store(true);
        }
        ready.notify_all();
    }
    if (result != SECANT_SUCCESS) {
        for (std::thread& t : workers) t.join();
        return result;
    }
    const cudaMemPool_t pool = record_pool(device); /* null: plain allocations */

    /* records travel on their own stream, so an upload never waits for the kernels of earlier chunks;
     * the chunks' kernels go round the compute streams, so a chunk smaller than the GPU shares it
     * with its neighbours */
    constexpr int kComputeStreams = 8;
    cudaStream_t compute[kComputeStreams] = {}, copies = nullptr;
    const unsigned concurrent = (unsigned)std::min<size_t>(num_chunks, kComputeStreams);
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
        const size_t piece0 = c * kPiecesPerLaunch, piece1 = std::min(num_pieces, piece0 + kPiecesPerLaunch);
        for (size_t q = piece0; q < piece1; ++q)
            for (;;) { /* wait for piece q; while it is in other hands, encode pieces nobody has taken */
                {
                    std::lock_guard<std::mutex> lock(mutex);
                    if (done[q]) break;
                }
                const size_t mine = next_piece.fetch_add(1);
                if (mine < num_pieces) {
                    encode_one(mine);
                } else {
                    std::unique_lock<std::mutex> lock(mutex);
                    ready.wait(lock, [&] { return done[q] != 0; });
                }
            }
        for (size_t q = piece0; q < piece1 && result == SECANT_SUCCESS; ++q) result = pieces[q].status;
        if (result != SECANT_SUCCESS) break;
        /* the pieces' arrays joined section by section; a program's offsets move by what lies before its piece */
        EncodedBatch enc; /* totals and maxima only */
        size_t n_programs = 0, n_insns = 0, n_patches = 0, n_affines = 0, n_lits = 0;
        for (size_t q = piece0; q < piece1; ++q) {
            const EncodedBatch& part = pieces[q].enc;
            n_programs += part.programs.size(); n_insns += part.insns.size(); n_patches += part.patches.size();
            n_affines += part.affines.size(); n_lits += part.lits.size();
            enc.max_insn = std::max(enc.max_insn, part.max_insn); enc.max_extra = std::max(enc.max_extra, part.max_extra);
            enc.max_slots = std::max(enc.max_slots, part.max_slots); enc.max_cst = std::max(enc.max_cst, part.max_cst);
            enc.max_btmp = std::max(enc.max_btmp, part.max_btmp);
        }
        if (n_insns > 0xffffffffull || n_patches > 0xffffffffull || n_affines > 0xffffffffull || n_lits > 0xffffffffull) { result = SECANT_ERROR_OVERFLOW; break; }
        Chunk& chunk = chunks[c];
        const size_t o_insn = align256(n_programs * sizeof(SbProgram));
        const size_t o_patch = align256(o_insn + n_insns * sizeof(SbInsn));
        const size_t o_aff = align256(o_patch + n_patches * sizeof(SbPatch));
        const size_t o_lit = align256(o_aff + n_affines * sizeof(SbAffine));
        const size_t o_flag = align256(o_lit + n_lits * sizeof(float) + 16); /* one word raised by the data validation */
        const size_t o_order = o_flag + 256;
        const size_t total = align256(o_order + n_programs / S * sizeof(uint32_t));
        try {
            chunk.host.assign(total, 0);
        } catch (const std::bad_alloc&) {
            result = SECANT_ERROR_ALLOCATION_FAILED;
            break;
        }
        char* host = chunk.host.data();
        {
            size_t at_program = 0, at_insn = 0, at_patch = 0, at_affine = 0, at_lit = 0;
            for (size_t q = piece0; q < piece1; ++q) {
                EncodedBatch& part = pieces[q].enc;
                SbProgram* out = reinterpret_cast<SbProgram*>(host) + at_program;
                for (size_t i = 0; i < part.programs.size(); ++i) {
                    SbProgram pr = part.programs[i];
                    pr.insn_off += (uint32_t)at_insn; pr.patch_off += (uint32_t)at_patch;
                    pr.affine_off += (uint32_t)at_affine; pr.lit_off += (uint32_t)at_lit;
                    out[i] = pr;
                }
                if (!part.insns.empty()) std::memcpy(host + o_insn + at_insn * sizeof(SbInsn), part.insns.data(), part.insns.size() * sizeof(SbInsn));
                if (!part.patches.empty()) std::memcpy(host + o_patch + at_patch * sizeof(SbPatch), part.patches.data(), part.patches.size() * sizeof(SbPatch));
                if (!part.affines.empty()) std::memcpy(host + o_aff + at_affine * sizeof(SbAffine), part.affines.data(), part.affines.size() * sizeof(SbAffine));
                if (!part.lits.empty()) std::memcpy(host + o_lit + at_lit * sizeof(float), part.lits.data(), part.lits.size() * sizeof(float));
                at_program += part.programs.size(); at_insn += part.insns.size(); at_patch += part.patches.size();
                at_affine += part.affines.size(); at_lit += part.lits.size();
                part = EncodedBatch(); /* the piece's own copy is not needed any more */
            }
            /* Warps take the launch's systems costliest first: a candidate that stays valid runs for its
             * full length, and the long ones should not be the last to start. */
            const size_t n_systems = n_programs / S;
            uint32_t* order = reinterpret_cast<uint32_t*>(host + o_order);
            for (size_t i = 0; i < n_systems; ++i) order[i] = (uint32_t)i;
            try {
                std::vector<uint32_t> cost;
                cost.reserve(n_systems);
                for (size_t q = piece0; q < piece1; ++q) cost.insert(cost.end(), pieces[q].cost.begin(), pieces[q].cost.end());
                if (cost.size() == n_systems)
                    std::stable_sort(order, order + n_systems, [&](uint32_t a, uint32_t b) { return cost[a] > cost[b]; });
            } catch (const std::bad_alloc&) {
                /* no memory for the sort: the systems are taken in their own order */
            }
        }
        if (pool && cudaMallocFromPoolAsync(reinterpret_cast<void**>(&chunk.device), total, pool, copies) == cudaSuccess) {
            chunk.pooled = true;
        } else {
            cudaGetLastError();
            chunk.device = nullptr;
            if (cudaMalloc(&chunk.device, total) != cudaSuccess) { result = SECANT_ERROR_ALLOCATION_FAILED; break; }
        }
        char* d = chunk.device;
        e = cudaMemcpyAsync(d, host, total, cudaMemcpyHostToDevice, copies);
        if (e == cudaSuccess) e = cudaEventRecord(uploaded, copies);
        cudaStream_t stream = compute[c % kComputeStreams];
        if (e == cudaSuccess) e = cudaStreamWaitEvent(stream, uploaded, 0);
        if (e != cudaSuccess) break;
        const size_t first_system = piece0 * kPieceSystems;
        const size_t systems = n_programs / S;
        DeviceBatch db;
        std::memset(&db, 0, sizeof(db));
        db.programs = reinterpret_cast<const SbProgram*>(d);
        db.insns = reinterpret_cast<const SbInsn*>(d + o_insn);
        db.patches = reinterpret_cast<const SbPatch*>(d + o_patch);
        db.affines = reinterpret_cast<const SbAffine*>(d + o_aff);
        db.lits = reinterpret_cast<const float*>(d + o_lit);
        db.num_programs = (uint32_t)n_programs;
        db.max_insn = enc.max_insn;
        db.max_extra = enc.max_extra;
        db.max_slots = enc.max_slots > rules.reserved_slots ? enc.max_slots : rules.reserved_slots;
        db.max_hoisted = 0;
        db.max_cst = enc.max_cst;
        db.max_btmp = enc.max_btmp;
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
        p.order = reinterpret_cast<const uint32_t*>(d + o_order);
        p.sampled = sampled ? reinterpret_cast<const SecantB200SampledParameter*>(run->sampled_parameters) + first_system * K : nullptr;
        p.uniform_pool = reinterpret_cast<const float*>(run->uniform_pool);
        p.normal_pool = reinterpret_cast<const float*>(run->normal_pool);
        p.pool_size = run->rng_pool_size;
        p.output = reinterpret_cast<float*>(run->output.address) + first_system * run->output.leading_dimension;
        p.output_ld = run->output.leading_dimension;
        p.integrated = reinterpret_cast<unsigned long long*>(run->integrated_intervals);
        e = launch_rk4(db, p, (size_t)limit, concurrent, stream);
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
    for (Chunk& chunk : chunks) /* every stream has been waited for: nothing reads the buffers any more */
        if (chunk.device) {
            const cudaError_t f = chunk.pooled ? cudaFreeAsync(chunk.device, copies) : cudaFree(chunk.device);
            if (e == cudaSuccess) e = f;
        }
    if (copies) { /* the pool may hand the memory to the next call once the frees have been reached */
        const cudaError_t f = cudaStreamSynchronize(copies);
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
