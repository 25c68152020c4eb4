/*
 * rollout.cu - RK4 rollout scoring: candidate right-hand sides interpreted inside the integrator.
 *
 * Restates the integration loop of the reference engine's generated scoring kernel
 * (projects/odezza/core/o_generate_scoring_cuda.c:494-588): per observation interval
 * h = interval / substeps; per substep base = stage = state, sum = 0, four stages with
 * sum = fma(w, rhs, sum) (w = 1,2,2,1), stage = fma(h/2 or h, rhs, base), then
 * state = fma(h/6, sum, base); after every interval all states must be finite and
 * sq = fma(err, err, sq).  Score = sq / residuals, or FLT_MAX when anything was not finite.
 *
 * Mapping (different from the reference, which gives a thread one configuration and loops all
 * trajectories inside it): one warp per (system, configuration), lanes = trajectories, RR per
 * lane.  RR is chosen from the trajectory count so that a pass of 32 * RR trajectories keeps all
 * lanes busy: 1 up to 32 trajectories, 2 up to 64, 4 beyond.  The integrator's vectors live in
 * the warp's slots: slot s = stage state s (what COLUMN s of a right-hand side reads), then
 * next-stage, sum and state vectors (the state is not touched during a step, so it doubles as the
 * step's base).  A right-hand side is a flat record (record.h) whose operands are constants of
 * the program (CST) and slots (SLOT); the machine below knows only those two kinds, so its
 * dispatch is an operand fetch followed by a switch over the operation.
 */
#include "evaluator.cuh"
#include "sbmath.cuh"

#include <algorithm>

namespace sb {

namespace {

constexpr int kRolloutMaxWarps = 16;
constexpr float kFltMax = 3.402823466e+38f;

template <int RR>
__device__ __forceinline__ void load_lanes(const float* p, float (&x)[RR]) {
    if constexpr (RR == 4) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    } else if constexpr (RR == 2) {
        const float2 v = *reinterpret_cast<const float2*>(p);
        x[0] = v.x; x[1] = v.y;
    } else {
        x[0] = *p;
    }
}
template <int RR>
__device__ __forceinline__ void store_lanes(float* p, const float (&x)[RR]) {
    if constexpr (RR == 4) *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
    else if constexpr (RR == 2) *reinterpret_cast<float2*>(p) = make_float2(x[0], x[1]);
    else *p = x[0];
}

/* One element through the same pieces as the four-element functions of sbmath.cuh (common-range
 * body, then the general version where the argument asks for it), so a value has the same bits
 * whichever width computed it.  The narrow machines call these instead of padding a four-element
 * call. */
__device__ __noinline__ float unary1(float x, unsigned op) {
    switch (op) {
    case SB_UN_SIN: case SB_UN_COS: {
        const int shift = op == SB_UN_COS ? 1 : 0;
        return fabsf(x) < 4096.0f ? sbm::sincos_small(x, 0.5f * (float)shift) : sbm::sincos_any(x, shift);
    }
    case SB_UN_EXP: {
        float r = sbm::exp_mid(x);
        if (!(fabsf(x) <= 86.0f)) {
            bool hard = false;
            r = sbm::exp_repair(x, r, hard);
            if (hard) r = sbm::exp_any(x);
        }
        return r;
    }
    case SB_UN_LOG: return sbm::log_is_special(x) ? sbm::log_any(x) : sbm::log_normal(x);
    case SB_UN_EX2: return fabsf(x) <= 124.0f ? sbm::exp2_mid(x) : sbm::exp2f_(x);
    case SB_UN_SQRT: return __fsqrt_rn(x);
    case SB_UN_RCP: return __frcp_rn(x);
    case SB_UN_RSQRT: return __frcp_rn(__fsqrt_rn(x));
    case SB_UN_LG2: return log2f(x);
    default: return tanhf(x);
    }
}
__device__ __noinline__ float div1(float a, float b) { return __fdiv_rn(a, b); }

/* The same for two elements behind one call: their dependency chains interleave. */
__device__ __noinline__ float2 unary2(float2 v, unsigned op) {
    float2 o;
    switch (op) {
    case SB_UN_SIN: case SB_UN_COS: {
        const int shift = op == SB_UN_COS ? 1 : 0;
        const float half = 0.5f * (float)shift;
        o.x = sbm::sincos_small(v.x, half); o.y = sbm::sincos_small(v.y, half);
        if (!(fabsf(v.x) < 4096.0f && fabsf(v.y) < 4096.0f)) {
            if (!(fabsf(v.x) < 4096.0f)) o.x = sbm::sincos_any(v.x, shift);
            if (!(fabsf(v.y) < 4096.0f)) o.y = sbm::sincos_any(v.y, shift);
        }
        return o;
    }
    case SB_UN_EXP: {
        o.x = sbm::exp_mid(v.x); o.y = sbm::exp_mid(v.y);
        if (!(fabsf(v.x) <= 86.0f && fabsf(v.y) <= 86.0f)) {
            bool hard = false;
            o.x = sbm::exp_repair(v.x, o.x, hard); o.y = sbm::exp_repair(v.y, o.y, hard);
            if (hard) {
                if (fabsf(v.x) > 86.0f) o.x = sbm::exp_any(v.x);
                if (fabsf(v.y) > 86.0f) o.y = sbm::exp_any(v.y);
            }
        }
        return o;
    }
    case SB_UN_LOG:
        o.x = sbm::log_normal(v.x); o.y = sbm::log_normal(v.y);
        if (sbm::log_is_special(v.x)) o.x = sbm::log_any(v.x);
        if (sbm::log_is_special(v.y)) o.y = sbm::log_any(v.y);
        return o;
    case SB_UN_EX2:
        o.x = fabsf(v.x) <= 124.0f ? sbm::exp2_mid(v.x) : sbm::exp2f_(v.x);
        o.y = fabsf(v.y) <= 124.0f ? sbm::exp2_mid(v.y) : sbm::exp2f_(v.y);
        return o;
    case SB_UN_SQRT: return make_float2(__fsqrt_rn(v.x), __fsqrt_rn(v.y));
    case SB_UN_RCP: return make_float2(__frcp_rn(v.x), __frcp_rn(v.y));
    case SB_UN_RSQRT: return make_float2(__frcp_rn(__fsqrt_rn(v.x)), __frcp_rn(__fsqrt_rn(v.y)));
    case SB_UN_LG2: return make_float2(log2f(v.x), log2f(v.y));
    default: return make_float2(tanhf(v.x), tanhf(v.y));
    }
}
__device__ __noinline__ float2 div2(float2 a, float2 b) { return make_float2(__fdiv_rn(a.x, b.x), __fdiv_rn(a.y, b.y)); }

template <int RR>
struct Rollout {
    float acc[RR];
    float* slots; /* this lane's RR floats of slot 0; slot s lies s * 32 * RR floats further */

    __device__ __forceinline__ void get(uint32_t s, float (&x)[RR]) const { load_lanes<RR>(slots + (size_t)s * (32 * RR), x); }
    __device__ __forceinline__ void put(uint32_t s, const float (&x)[RR]) const { store_lanes<RR>(slots + (size_t)s * (32 * RR), x); }

    __device__ __forceinline__ void apply_unary(unsigned op) {
        if constexpr (RR == 4) {
            const float4 o = sbm::unary4(make_float4(acc[0], acc[1], acc[2], acc[3]), op);
            acc[0] = o.x; acc[1] = o.y; acc[2] = o.z; acc[3] = o.w;
        } else if constexpr (RR == 2) {
            const float2 o = unary2(make_float2(acc[0], acc[1]), op);
            acc[0] = o.x; acc[1] = o.y;
        } else {
            acc[0] = unary1(acc[0], op);
        }
    }
    /* acc = a / b */
    __device__ __forceinline__ void divide(const float (&a)[RR], const float (&b)[RR]) {
        if constexpr (RR == 4) {
            const float4 o = sbm::div4(make_float4(a[0], a[1], a[2], a[3]), make_float4(b[0], b[1], b[2], b[3]));
            acc[0] = o.x; acc[1] = o.y; acc[2] = o.z; acc[3] = o.w;
        } else if constexpr (RR == 2) {
            const float2 o = div2(make_float2(a[0], a[1]), make_float2(b[0], b[1]));
            acc[0] = o.x; acc[1] = o.y;
        } else {
            acc[0] = div1(a[0], b[0]);
        }
    }

    /* acc = value of the record at `exec` with constants `cst` */
    __device__ __forceinline__ void run(const SbInsn* exec, const float* cst) {
        const uint2* ip = reinterpret_cast<const uint2*>(exec);
        uint2 next = *ip++; /* the buffer holds one padding entry after the END */
#pragma unroll 1
        for (;;) {
            const uint2 ins = next;
            next = *ip++;
            const unsigned cs = ins.x & 0xffu;
            const uint32_t idx = ins.x >> 16;
            if (cs == SB_CASE_END) return;
            if (cs == SB_CASE_STORE) { put(idx, acc); continue; }
            if (cs >= SB_CASE_UN) {
                if (cs == SB_CASE_FMA) { fused(ins); continue; }
                const unsigned op = cs - SB_CASE_UN;
                if (op == SB_UN_NEG) {
#pragma unroll
                    for (int q = 0; q < RR; ++q) acc[q] = -acc[q];
                } else if (op == SB_UN_ABS) {
#pragma unroll
                    for (int q = 0; q < RR; ++q) acc[q] = fabsf(acc[q]);
                } else apply_unary(op);
                continue;
            }
            /* a load or a binary operation: fetch the operand, then apply */
            const unsigned rel = cs < SB_CASE_BIN ? cs - SB_CASE_LOAD : (cs - SB_CASE_BIN) % SB_NUM_KINDS;
            float x[RR];
            if (rel == SB_KIND_CST) {
                const float c = cst[idx];
#pragma unroll
                for (int q = 0; q < RR; ++q) x[q] = c;
            } else get(idx, x);
            if (cs < SB_CASE_BIN) {
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = x[q];
                continue;
            }
            switch ((cs - SB_CASE_BIN) / SB_NUM_KINDS) {
            case SB_BIN_ADD:
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = __fadd_rn(acc[q], x[q]);
                break;
            case SB_BIN_SUB:
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = __fsub_rn(acc[q], x[q]);
                break;
            case SB_BIN_RSUB:
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = __fsub_rn(x[q], acc[q]);
                break;
            case SB_BIN_MUL:
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = __fmul_rn(acc[q], x[q]);
                break;
            case SB_BIN_DIV: divide(acc, x); break;
            case SB_BIN_RDIV: divide(x, acc); break;
            case SB_BIN_MIN:
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = fminf(acc[q], x[q]);
                break;
            default:
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = fmaxf(acc[q], x[q]);
                break;
            }
        }
    }

    const float* cst_of_run = nullptr;

    /* FMA_F32 over three operands of any kind (constant, slot, or the accumulator) */
    __device__ __forceinline__ void fused(uint2 ins) {
        const unsigned kinds = (ins.x >> 8) & 0x3fu;
        float v[3][RR];
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const unsigned kind = (kinds >> (2 * i)) & 3u;
            const uint32_t index = (ins.y >> (10 * i)) & 1023u;
            if (kind == SB_KIND_CST) {
                const float c = cst_of_run[index];
#pragma unroll
                for (int q = 0; q < RR; ++q) v[i][q] = c;
            } else if (kind == SB_FMA_ACC) {
#pragma unroll
                for (int q = 0; q < RR; ++q) v[i][q] = acc[q];
            } else get(index, v[i]);
        }
#pragma unroll
        for (int q = 0; q < RR; ++q) acc[q] = __fmaf_rn(v[0][q], v[1][q], v[2][q]);
    }
};

/* projects/odezza/core/o_sampled_constants_source.h:32-44 */
__device__ __forceinline__ float sampled_constant(const Rk4Problem& prob, unsigned long long index, uint32_t bank) {
    const SecantB200SampledParameter p = prob.sampled[index];
    if (!p.distribution) return p.shift;
    const unsigned long long delta = (unsigned long long)bank * p.stride;
    if (p.offset >= prob.pool_size || delta >= prob.pool_size - p.offset) return __int_as_float(0x7fc00000);
    const float* pool = p.distribution == 1 ? prob.uniform_pool : p.distribution == 2 ? prob.normal_pool : nullptr;
    if (!pool) return __int_as_float(0x7fc00000);
    const float value = __fadd_rn(__fmul_rn(pool[p.offset + delta], p.scale), p.shift);
    return fminf(p.upper, fmaxf(p.lower, value));
}

template <int RR>
__global__ void __launch_bounds__(kRolloutMaxWarps * 32, RR == 4 ? 1 : 2)
rk4_kernel(const DeviceBatch batch, const Rk4Problem prob, uint32_t exec_bytes, uint32_t cst_bytes, uint32_t warp_bytes) {
    constexpr uint32_t PASS = 32 * RR; /* trajectories of one pass */
    extern __shared__ __align__(16) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t S = prob.num_states, K = prob.num_constants;
    unsigned char* const warea = smem + (size_t)warp * warp_bytes;
    const unsigned long long configs = (unsigned long long)prob.num_banks << prob.toggle_bits;
    const unsigned long long num_items = configs * prob.num_systems;
    unsigned int integrated = 0; /* (trajectory, observation interval) pairs this lane carried out */
    /* Items are drawn from a device-wide counter: a warp whose candidate went invalid early takes
     * the next one at once, and no warp slot idles behind the longest item of its CTA. */
    for (;;) {
    unsigned long long item = 0;
    if (lane == 0) item = atomicAdd(prob.queue, 1ull);
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= num_items) break;
    const uint32_t sys = (uint32_t)(item / configs);
    const unsigned long long cfg = item % configs;
    const unsigned long long perm = cfg & ((1ull << prob.toggle_bits) - 1ull);
    const uint32_t bank = (uint32_t)(cfg >> prob.toggle_bits);
    const float* bank_ptr = prob.banks ? prob.banks + (size_t)sys * prob.system_bank_stride + (size_t)bank * prob.bank_stride : nullptr;

    for (uint32_t s = 0; s < S; ++s) { /* private copy of every right-hand side, toggles resolved, constants staged */
        const SbProgram pr = batch.programs[sys * S + s];
        SbInsn* exec = reinterpret_cast<SbInsn*>(warea + (size_t)s * exec_bytes);
        float* cst = reinterpret_cast<float*>(warea + (size_t)S * exec_bytes + (size_t)s * cst_bytes);
        for (uint32_t i = lane; i < pr.n_insn; i += 32) exec[i] = batch.insns[pr.insn_off + i];
        if (lane == 0) exec[pr.n_insn] = SbInsn{0u, 0u};
        __syncwarp();
        for (uint32_t i = lane; i < pr.n_patch; i += 32) {
            const SbPatch* p = batch.patches + pr.patch_off + i;
            unsigned choice = (unsigned)(perm >> p->bit0) & 1u;
            if (p->bit1 != 0xffu) choice |= ((unsigned)(perm >> p->bit1) & 1u) << 1;
            exec[p->insn] = p->alt[choice];
        }
        for (uint32_t e = lane; e < K + pr.n_affine + pr.n_lits; e += 32) {
            float v;
            if (e < K) v = prob.sampled ? sampled_constant(prob, (unsigned long long)sys * K + e, bank) : bank_ptr[e];
            else if (e < K + pr.n_affine) {
                const SbAffine a = batch.affines[pr.affine_off + e - K];
                const float slot = prob.sampled ? sampled_constant(prob, (unsigned long long)sys * K + a.slot, bank) : bank_ptr[a.slot];
                v = __fadd_rn(__fmul_rn(slot, a.scale), a.offset);
            } else v = batch.lits[pr.lit_off + e - K - pr.n_affine];
            cst[e] = v;
        }
    }
    __syncwarp();

    const uint32_t STAGE = 0, NEXT = S, SUM = 2 * S, STATE = 3 * S, BASE = STATE;
    const bool ragged = prob.offsets != nullptr;
    Rollout<RR> m;
    m.slots = reinterpret_cast<float*>(warea + (size_t)S * (exec_bytes + cst_bytes)) + lane * RR;
    float sq = 0.0f;
    unsigned long long residuals = 0;
    /* any non-finite time or reference value (NaN excepted where it means "unobserved"), found
     * by the validation kernel, invalidates every score; so do offsets that do not span the data */
    bool ok = *prob.invalid_flag == 0;
    if (ragged) ok = ok && prob.offsets[0] == 0u && prob.offsets[prob.num_trajectories] == prob.total_points;
    /* a candidate that is already invalid scores FLT_MAX whatever follows: the warp stops integrating it */
    bool alive = __all_sync(0xffffffffu, ok);
    for (uint32_t t0 = 0; t0 < prob.num_trajectories && alive; t0 += PASS) {
        uint32_t begin[RR], npts[RR], longest = 0;
#pragma unroll
        for (int q = 0; q < RR; ++q) {
            const uint32_t traj = t0 + lane * RR + q;
            const bool live = traj < prob.num_trajectories;
            begin[q] = 0; npts[q] = 0;
            if (live && ragged) {
                const uint32_t b = prob.offsets[traj], e = prob.offsets[traj + 1];
                const bool sane = e > b && e <= prob.total_points;
                ok = ok && sane;
                if (sane) { begin[q] = b; npts[q] = e - b; }
            } else if (live) {
                begin[q] = traj * prob.points_per_trajectory; npts[q] = prob.points_per_trajectory;
            }
            longest = max(longest, npts[q]);
        }
#pragma unroll
        for (int d = 16; d; d >>= 1) longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, d));
        for (uint32_t s = 0; s < S; ++s) {
            float v[RR];
#pragma unroll
            for (int q = 0; q < RR; ++q) {
                v[q] = npts[q] ? prob.reference[(size_t)s * prob.reference_ld + begin[q]] : 0.0f;
                ok = ok && (fabsf(v[q]) <= kFltMax); /* initial states must be complete and finite */
            }
            m.put(STATE + s, v);
        }
        alive = __all_sync(0xffffffffu, ok);
        for (uint32_t k = 1; k < longest && alive; ++k) {
            /* per trajectory step size; a trajectory that has ended keeps integrating with h = 0
             * and is left out of every check and sum */
            float h[RR], sixth[RR];
            bool act[RR];
#pragma unroll
            for (int q = 0; q < RR; ++q) {
                act[q] = k < npts[q];
                const uint32_t at = ragged ? begin[q] + k : k;
                const float interval = act[q] ? prob.times[at] - prob.times[at - 1] : 0.0f;
                const float step = interval / (float)prob.substeps;
                ok = ok && (!act[q] || ((fabsf(interval) <= kFltMax) && interval > 0.0f && step > 0.0f));
                h[q] = act[q] ? step : 0.0f;
                sixth[q] = h[q] / 6.0f;
            }
            for (uint32_t sub = 0; sub < prob.substeps; ++sub) {
                for (uint32_t s = 0; s < S; ++s) {
                    float v[RR], zero[RR];
                    m.get(STATE + s, v);
                    m.put(STAGE + s, v);
#pragma unroll
                    for (int q = 0; q < RR; ++q) zero[q] = 0.0f;
                    m.put(SUM + s, zero);
                }
#pragma unroll 1
                for (int stage = 0; stage < 4; ++stage) {
                    const float weight = (stage == 0 || stage == 3) ? 1.0f : 2.0f;
                    for (uint32_t s = 0; s < S; ++s) {
                        const SbInsn* exec = reinterpret_cast<const SbInsn*>(warea + (size_t)s * exec_bytes);
                        m.cst_of_run = reinterpret_cast<const float*>(warea + (size_t)S * exec_bytes + (size_t)s * cst_bytes);
                        m.run(exec, m.cst_of_run); /* acc = rhs of state s at the stage values */
                        float v[RR];
                        m.get(SUM + s, v);
#pragma unroll
                        for (int q = 0; q < RR; ++q) v[q] = __fmaf_rn(weight, m.acc[q], v[q]);
                        m.put(SUM + s, v);
                        if (stage != 3) {
                            m.get(BASE + s, v);
#pragma unroll
                            for (int q = 0; q < RR; ++q) v[q] = __fmaf_rn(stage == 2 ? h[q] : __fmul_rn(0.5f, h[q]), m.acc[q], v[q]);
                            m.put(NEXT + s, v);
                        }
                    }
                    if (stage != 3)
                        for (uint32_t s = 0; s < S; ++s) {
                            float v[RR];
                            m.get(NEXT + s, v);
                            m.put(STAGE + s, v);
                        }
                }
                for (uint32_t s = 0; s < S; ++s) {
                    float sum[RR], base[RR];
                    m.get(SUM + s, sum);
                    m.get(BASE + s, base);
#pragma unroll
                    for (int q = 0; q < RR; ++q) base[q] = __fmaf_rn(sixth[q], sum[q], base[q]);
                    m.put(STATE + s, base);
                }
            }
            for (uint32_t s = 0; s < S; ++s) { /* all states must be finite before any residual counts */
                float v[RR];
                m.get(STATE + s, v);
#pragma unroll
                for (int q = 0; q < RR; ++q) ok = ok && (!act[q] || fabsf(v[q]) <= kFltMax);
            }
#pragma unroll
            for (int q = 0; q < RR; ++q) integrated += act[q] ? 1u : 0u;
            alive = __all_sync(0xffffffffu, ok);
            for (uint32_t s = 0; s < S; ++s) {
                float v[RR];
                m.get(STATE + s, v);
#pragma unroll
                for (int q = 0; q < RR; ++q)
                    if (act[q]) {
                        const float ref = prob.reference[(size_t)s * prob.reference_ld + begin[q] + k];
                        if (prob.allow_missing && ref != ref) continue; /* unobserved */
                        const float err = __fsub_rn(v[q], ref);
                        sq = __fmaf_rn(err, err, sq);
                        ++residuals;
                    }
            }
        }
    }
    float total = sq;
#pragma unroll
    for (int d = 16; d; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d);
    uint32_t lo = (uint32_t)residuals, hi = (uint32_t)(residuals >> 32);
#pragma unroll
    for (int d = 16; d; d >>= 1) {
        const unsigned long long other = ((unsigned long long)__shfl_xor_sync(0xffffffffu, hi, d) << 32) | __shfl_xor_sync(0xffffffffu, lo, d);
        residuals += other;
        lo = (uint32_t)residuals; hi = (uint32_t)(residuals >> 32);
    }
    const bool all_ok = __all_sync(0xffffffffu, ok);
    if (lane == 0) {
        const bool finite = fabsf(total) <= kFltMax;
        prob.output[(size_t)sys * prob.output_ld + cfg] = (all_ok && residuals && finite) ? total / (float)residuals : kFltMax;
    }
    __syncwarp(); /* the next item overwrites the warp's program and slot areas */
    }
    if (prob.integrated) {
#pragma unroll
        for (int d = 16; d; d >>= 1) integrated += __shfl_xor_sync(0xffffffffu, integrated, d);
        if (lane == 0) atomicAdd(prob.integrated, (unsigned long long)integrated);
    }
}

/* Raises *flag when a time or a reference value of an active state is not finite; NaN reference
 * values are tolerated when they mean "unobserved" (initial points are checked by the scorer). */
__global__ void rk4_validate_kernel(const Rk4Problem prob) {
    const size_t n = (size_t)prob.total_points * (prob.num_states + 1);
    bool bad = false;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / prob.total_points, col = i % prob.total_points;
        if (row == prob.num_states) {
            if (!prob.offsets && col >= prob.points_per_trajectory) continue; /* uniform form: one shared time axis */
            bad = bad || !(fabsf(prob.times[col]) <= kFltMax);
        } else {
            const float v = prob.reference[row * prob.reference_ld + col];
            bad = bad || !((fabsf(v) <= kFltMax) || (prob.allow_missing && v != v));
        }
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(prob.invalid_flag, 1);
}

uint32_t round16(size_t v) { return (uint32_t)((v + 15) / 16 * 16); }

template <int RR>
cudaError_t launch_width(const DeviceBatch& batch, const Rk4Problem& prob, size_t smem_limit, cudaStream_t stream) {
    const uint32_t exec_bytes = round16(((size_t)batch.max_insn + 1) * sizeof(SbInsn));
    const uint32_t cst_bytes = round16(((size_t)prob.num_constants + batch.max_extra) * 4 + 16);
    /* max_slots already includes the integrator's reserved slots */
    const uint32_t warp_bytes = prob.num_states * (exec_bytes + cst_bytes) + batch.max_slots * (uint32_t)RR * 128u;
    /* warps per CTA: the count that puts most warps on an SM (shared memory per SM is the CTA limit
     * plus 1 KB reserved per resident CTA; the register file bounds the narrow machines at two full
     * CTAs and the wide one at about 24 warps) */
    const int register_warps = RR == 4 ? 24 : 2 * kRolloutMaxWarps;
    int warps = 0, best = 0;
    for (int w = 2; w <= kRolloutMaxWarps; ++w) {
        const size_t cta = (size_t)warp_bytes * w;
        if (cta > smem_limit) break;
        int ctas = (int)((smem_limit + 1024) / (cta + 1024));
        if (ctas * w > register_warps) ctas = register_warps / w;
        if (ctas * w >= best) { best = ctas * w; warps = w; }
    }
    if (!warps) return cudaErrorInvalidConfiguration;
    const size_t smem = (size_t)warp_bytes * warps;
    cudaError_t e = cudaFuncSetAttribute(rk4_kernel<RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_limit);
    if (e != cudaSuccess) return e;
    const unsigned long long items = ((unsigned long long)prob.num_banks << prob.toggle_bits) * prob.num_systems;
    /* warps draw items from the queue until it is empty, so the grid only has to fill the device */
    int device = 0, sms = 0;
    if ((e = cudaGetDevice(&device)) != cudaSuccess || (e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return e;
    const unsigned long long resident = (unsigned long long)sms * (unsigned)std::max(1, best / warps);
    const unsigned long long blocks = std::min<unsigned long long>((items + warps - 1) / warps, resident);
    const size_t values = (size_t)prob.total_points * (prob.num_states + 1);
    rk4_validate_kernel<<<(unsigned)std::min<size_t>(1024, (values + 255) / 256), 256, 0, stream>>>(prob);
    rk4_kernel<RR><<<(unsigned)blocks, warps * 32, smem, stream>>>(batch, prob, exec_bytes, cst_bytes, warp_bytes);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_rk4(const DeviceBatch& batch, const Rk4Problem& prob, size_t smem_limit, cudaStream_t stream) {
    if (prob.num_trajectories <= 32) return launch_width<1>(batch, prob, smem_limit, stream);
    if (prob.num_trajectories <= 64) return launch_width<2>(batch, prob, smem_limit, stream);
    return launch_width<4>(batch, prob, smem_limit, stream);
}

}  // namespace sb
