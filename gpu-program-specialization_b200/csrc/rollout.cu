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

/* ---- shared memory by 32-bit shared-window address ------------------------------------------
 * The interpreter's operands, the integrator's vectors and the instruction stream itself are read
 * through these, so address arithmetic stays 32 bits wide and an operand's address can be stored
 * ready-made in the instruction word. */
__device__ __forceinline__ uint32_t shared_address(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
template <int RR>
__device__ __forceinline__ void lds(uint32_t a, float (&x)[RR]) {
    if constexpr (RR == 4) asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x[0]), "=f"(x[1]), "=f"(x[2]), "=f"(x[3]) : "r"(a));
    else if constexpr (RR == 2) asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(x[0]), "=f"(x[1]) : "r"(a));
    else asm volatile("ld.shared.f32 %0, [%1];" : "=f"(x[0]) : "r"(a));
}
template <int RR>
__device__ __forceinline__ void sts(uint32_t a, const float (&x)[RR]) {
    if constexpr (RR == 4) asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]) : "memory");
    else if constexpr (RR == 2) asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(a), "f"(x[0]), "f"(x[1]) : "memory");
    else asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(x[0]) : "memory");
}
__device__ __forceinline__ void lds_pair(uint32_t a, uint32_t& lo, uint32_t& hi) {
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(a));
}
__device__ __forceinline__ uint32_t lds_word(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}

/* Handlers of the rollout machine.  A warp rewrites the main part of its private copy of a record
 * once per item into this form: word 0 = handler (bits 0..7) and, for H_UNARY, the function (bits
 * 8..15); word 1 = the operand's shared-window address, with bit 31 set when every lane reads its own
 * RR floats of a slot (the lane's offset is added) and clear when all lanes read one table entry.
 * H_STORE_LOAD (slot = acc, then acc = operand) carries the slot's address in bits 8..31 of word 0.
 * H_FMA keeps the record's form (operand kinds in bits 8..13 of word 0, three 10-bit indices in
 * word 1).  One item runs its right-hand sides states x 4 stages x steps times, so the rewrite is free
 * and the dispatch per instruction is an address add, one load and one dense switch. */
enum { H_END = 0, H_STORE, H_LOAD, H_ADD, H_SUB, H_RSUB, H_MUL, H_DIV, H_RDIV, H_MIN, H_MAX, H_NEG, H_ABS, H_UNARY, H_STORE_LOAD, H_FMA };
constexpr uint32_t kPerLane = 0x80000000u;

template <int RR>
struct Rollout {
    float acc[RR];
    uint32_t lane_off; /* byte offset of this lane's RR floats inside a slot */
    uint32_t slot0;    /* shared address of slot 0; slot s lies s * 32 * RR floats further */

    __device__ __forceinline__ uint32_t slot_address(uint32_t s) const { return slot0 + s * (uint32_t)(RR * 128) + lane_off; }
    __device__ __forceinline__ void get(uint32_t s, float (&x)[RR]) const { lds<RR>(slot_address(s), x); }
    __device__ __forceinline__ void put(uint32_t s, const float (&x)[RR]) const { sts<RR>(slot_address(s), x); }

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

    /* acc = value of the rewritten main part: `count` instructions (the closing END not counted)
     * starting at shared address `ip`; `table` is the shared address of the program's constant
     * table (RR copies of every entry) */
    __device__ __forceinline__ void run(uint32_t ip, uint32_t count, uint32_t table) {
        uint32_t n0, n1;
        lds_pair(ip, n0, n1); /* the record ends with END and one padding entry, so reading ahead is safe */
        ip += 8;
#pragma unroll 1
        for (; count; --count) {
            const uint32_t w0 = n0, w1 = n1;
            lds_pair(ip, n0, n1);
            ip += 8;
            const unsigned handler = w0 & 0xffu;
            float x[RR];
            if (handler != H_FMA) lds<RR>((w1 & 0x00ffffffu) + ((uint32_t)((int32_t)w1 >> 31) & lane_off), x);
            if (handler == H_MUL) {
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = __fmul_rn(acc[q], x[q]);
                continue;
            }
            if (handler == H_ADD) {
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = __fadd_rn(acc[q], x[q]);
                continue;
            }
            if (handler == H_LOAD) {
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = x[q];
                continue;
            }
            if (handler == H_STORE_LOAD) {
                sts<RR>((w0 >> 8) + lane_off, acc);
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = x[q];
                continue;
            }
            switch (handler) {
            case H_STORE: sts<RR>((w1 & 0x00ffffffu) + lane_off, acc); break;
            case H_SUB:
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = __fsub_rn(acc[q], x[q]);
                break;
            case H_RSUB:
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = __fsub_rn(x[q], acc[q]);
                break;
            case H_DIV: divide(acc, x); break;
            case H_RDIV: divide(x, acc); break;
            case H_MIN:
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = fminf(acc[q], x[q]);
                break;
            case H_MAX:
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = fmaxf(acc[q], x[q]);
                break;
            case H_NEG:
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = -acc[q];
                break;
            case H_ABS:
#pragma unroll
                for (int q = 0; q < RR; ++q) acc[q] = fabsf(acc[q]);
                break;
            case H_UNARY: apply_unary((w0 >> 8) & 0xffu); break;
            case H_FMA: fused(w0, w1, table); break;
            default: break; /* H_END inside the counted range: unreachable for records produced by the encoder */
            }
        }
    }

    /* FMA_F32 over three operands of any kind (table entry, slot, or the accumulator) */
    __device__ __forceinline__ void fused(uint32_t w0, uint32_t w1, uint32_t table) {
        const unsigned kinds = (w0 >> 8) & 0x3fu;
        float v[3][RR];
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const unsigned kind = (kinds >> (2 * i)) & 3u;
            const uint32_t index = (w1 >> (10 * i)) & 1023u;
            if (kind == SB_FMA_ACC) {
#pragma unroll
                for (int q = 0; q < RR; ++q) v[i][q] = acc[q];
            } else if (kind == SB_KIND_CST) lds<RR>(table + index * (uint32_t)(RR * 4), v[i]);
            else get(index, v[i]);
        }
#pragma unroll
        for (int q = 0; q < RR; ++q) acc[q] = __fmaf_rn(v[0][q], v[1][q], v[2][q]);
    }
};

/* Rewrites instruction `in` of a record's main part for the machine above. */
template <int RR>
__device__ __forceinline__ SbInsn rewritten(SbInsn in, uint32_t table, uint32_t slot0) {
    const unsigned cs = in.w0 & 0xffu;
    const uint32_t idx = in.w0 >> 16;
    unsigned handler = H_END, aux = 0, kind = SB_NUM_KINDS; /* SB_NUM_KINDS: no operand */
    if (cs >= SB_CASE_LOAD && cs < SB_CASE_STORE) { handler = H_LOAD; kind = cs - SB_CASE_LOAD; }
    else if (cs == SB_CASE_STORE && (in.w1 & SB_STORE_THEN_LOAD)) {
        const unsigned loaded = (in.w1 >> 16) & 3u;
        const uint32_t from = in.w1 & 0xffffu;
        if (loaded == SB_KIND_ROW) return SbInsn{H_END, table};
        const uint32_t operand = loaded == SB_KIND_CST ? table + from * (uint32_t)(RR * 4) : ((slot0 + from * (uint32_t)(RR * 128)) | kPerLane);
        return SbInsn{H_STORE_LOAD | ((slot0 + idx * (uint32_t)(RR * 128)) << 8), operand};
    } else if (cs == SB_CASE_STORE) { handler = H_STORE; kind = SB_KIND_SLOT; }
    else if (cs >= SB_CASE_BIN && cs < SB_CASE_UN) { handler = H_ADD + (cs - SB_CASE_BIN) / SB_NUM_KINDS; kind = (cs - SB_CASE_BIN) % SB_NUM_KINDS; }
    else if (cs >= SB_CASE_UN && cs < SB_CASE_FMA) {
        aux = cs - SB_CASE_UN;
        handler = aux == SB_UN_NEG ? H_NEG : aux == SB_UN_ABS ? H_ABS : H_UNARY;
    } else if (cs == SB_CASE_FMA) return SbInsn{(in.w0 & 0xffffff00u) | H_FMA, in.w1};
    if (kind == SB_KIND_ROW) handler = H_END; /* rollout records have no per-row operands */
    uint32_t operand = table; /* instructions without an operand read (and ignore) the table's first entry */
    if (kind == SB_KIND_CST) operand = table + idx * (uint32_t)(RR * 4);
    if (kind == SB_KIND_SLOT) operand = (slot0 + idx * (uint32_t)(RR * 128)) | kPerLane;
    return SbInsn{handler | (aux << 8), operand};
}

/* The bank part of a record (record.h): sub-expressions that depend on the candidate's constants
 * only, computed once per item instead of once per stage.  Every lane runs it on the same values
 * (no divergence, no exchange) and stores the same results: table entry e as RR adjacent copies, so
 * the main part reads a constant with the load it uses for a lane's slot values.  Operand kinds of
 * the bank part: CST = source constant (bank slots, affine entries, literals), ROW = table entry
 * written earlier, SLOT = scalar temporary.  The functions are the scalar pieces the wider
 * machines use, so a value has the bits it would have had in the main part. */
__device__ __noinline__ void rollout_bank_part(const SbInsn* code, const float* source, float* tmp, float* table, int copies) {
    float acc = 0.0f;
    auto operand = [&](unsigned kind, uint32_t idx) -> float {
        return kind == SB_KIND_ROW ? table[idx * copies] : kind == SB_KIND_SLOT ? tmp[idx] : source[idx];
    };
#pragma unroll 1
    for (;; ++code) {
        const SbInsn ins = *code;
        const unsigned cs = ins.w0 & 0xffu;
        const uint32_t idx = ins.w0 >> 16;
        if (cs == SB_CASE_END || cs > SB_CASE_FMA) return;
        if (cs < SB_CASE_STORE) acc = operand(cs - SB_CASE_LOAD, idx);
        else if (cs == SB_CASE_STORE) tmp[idx] = acc;
        else if (cs == SB_CASE_STOREH) {
            for (int q = 0; q < copies; ++q) table[idx * copies + q] = acc;
        } else if (cs < SB_CASE_UN) {
            const float x = operand((cs - SB_CASE_BIN) % SB_NUM_KINDS, idx);
            switch ((cs - SB_CASE_BIN) / SB_NUM_KINDS) {
            case SB_BIN_ADD: acc = __fadd_rn(acc, x); break;
            case SB_BIN_SUB: acc = __fsub_rn(acc, x); break;
            case SB_BIN_RSUB: acc = __fsub_rn(x, acc); break;
            case SB_BIN_MUL: acc = __fmul_rn(acc, x); break;
            case SB_BIN_DIV: acc = div1(acc, x); break;
            case SB_BIN_RDIV: acc = div1(x, acc); break;
            case SB_BIN_MIN: acc = fminf(acc, x); break;
            default: acc = fmaxf(acc, x); break;
            }
        } else if (cs < SB_CASE_FMA) {
            const unsigned op = cs - SB_CASE_UN;
            acc = op == SB_UN_NEG ? -acc : op == SB_UN_ABS ? fabsf(acc) : unary1(acc, op);
        } else {
            const unsigned kinds = (ins.w0 >> 8) & 0x3fu;
            float v[3];
#pragma unroll
            for (int i = 0; i < 3; ++i) {
                const unsigned kind = (kinds >> (2 * i)) & 3u;
                v[i] = kind == SB_FMA_ACC ? acc : operand(kind, (ins.w1 >> (10 * i)) & 1023u);
            }
            acc = __fmaf_rn(v[0], v[1], v[2]);
        }
    }
}

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

/* Shared memory of one warp, in this order: per state the record (exec_bytes) and the constant
 * table (table_bytes); then one area for the source constants of the record being set up and the
 * bank part's temporaries (source_bytes), the main parts' start addresses (16 words), the slots. */
struct RolloutLayout {
    uint32_t exec_bytes, table_bytes, source_bytes, warp_bytes;
};

template <int RR>
__global__ void __launch_bounds__(kRolloutMaxWarps * 32, RR == 4 ? 1 : 2)
rk4_kernel(const DeviceBatch batch, const Rk4Problem prob, const RolloutLayout lay) {
    constexpr uint32_t PASS = 32 * RR; /* trajectories of one pass */
    extern __shared__ __align__(16) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t S = prob.num_states, K = prob.num_constants;
    unsigned char* const warea = smem + (size_t)warp * lay.warp_bytes;
    unsigned char* const tables = warea + (size_t)S * lay.exec_bytes;
    float* const source = reinterpret_cast<float*>(tables + (size_t)S * lay.table_bytes);
    float* const tmp = source + K + batch.max_extra;
    uint32_t* const starts = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(source) + lay.source_bytes);
    float* const slot_area = reinterpret_cast<float*>(starts + 16);
    const uint32_t slot0 = shared_address(slot_area);
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
    const uint32_t turn = (uint32_t)(item / configs);
    const uint32_t sys = prob.order ? prob.order[turn] : turn;
    const unsigned long long cfg = item % configs;
    const unsigned long long perm = cfg & ((1ull << prob.toggle_bits) - 1ull);
    const uint32_t bank = (uint32_t)(cfg >> prob.toggle_bits);
    const float* bank_ptr = prob.banks ? prob.banks + (size_t)sys * prob.system_bank_stride + (size_t)bank * prob.bank_stride : nullptr;

    /* private copy of every right-hand side: toggles resolved, the bank part run once, the main
     * part rewritten for the machine */
    for (uint32_t s = 0; s < S; ++s) {
        const SbProgram pr = batch.programs[sys * S + s];
        SbInsn* exec = reinterpret_cast<SbInsn*>(warea + (size_t)s * lay.exec_bytes);
        float* table = reinterpret_cast<float*>(tables + (size_t)s * lay.table_bytes);
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
            source[e] = v;
        }
        __syncwarp();
        if (pr.main_off) rollout_bank_part(exec, source, tmp, table, RR);
        __syncwarp(); /* the next record's constants overwrite `source` */
        const uint32_t table_address = shared_address(table);
        for (uint32_t i = pr.main_off + lane; i < pr.n_insn; i += 32) exec[i] = rewritten<RR>(exec[i], table_address, slot0);
        /* start address and length of the main part in one word (shared addresses fit 18 bits) */
        if (lane == 0) starts[s] = shared_address(exec + pr.main_off) | ((uint32_t)(pr.n_insn - pr.main_off - 1u) << 18);
    }
    __syncwarp();

    const uint32_t STAGE = 0, NEXT = S, SUM = 2 * S, STATE = 3 * S, BASE = STATE;
    const bool ragged = prob.offsets != nullptr;
    Rollout<RR> m;
    m.slot0 = slot0;
    m.lane_off = (uint32_t)lane * (uint32_t)(RR * 4);
    const uint32_t starts_address = shared_address(starts), tables_address = shared_address(tables);
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
                        const uint32_t start = lds_word(starts_address + 4u * s);
                        m.run(start & 0x3ffffu, start >> 18, tables_address + s * lay.table_bytes); /* acc = rhs of state s at the stage values */
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
cudaError_t launch_width(const DeviceBatch& batch, const Rk4Problem& prob, size_t smem_limit, unsigned concurrent, cudaStream_t stream) {
    RolloutLayout lay;
    lay.exec_bytes = round16(((size_t)batch.max_insn + 1) * sizeof(SbInsn));
    lay.table_bytes = round16(((size_t)batch.max_cst + 1) * RR * 4); /* one entry at least: instructions without an operand read it */
    lay.source_bytes = round16(((size_t)prob.num_constants + batch.max_extra + batch.max_btmp) * 4 + 16);
    /* max_slots already includes the integrator's reserved slots */
    lay.warp_bytes = prob.num_states * (lay.exec_bytes + lay.table_bytes) + lay.source_bytes + 64u + batch.max_slots * (uint32_t)RR * 128u;
    const uint32_t warp_bytes = lay.warp_bytes;
    /* warps per CTA: the count that puts most warps on an SM (shared memory per SM is the CTA limit
     * plus 1 KB reserved per resident CTA; the register file holds 64 K registers, allocated per warp
     * in units of 256) */
    cudaFuncAttributes attributes;
    cudaError_t e = cudaFuncGetAttributes(&attributes, rk4_kernel<RR>);
    if (e != cudaSuccess) return e;
    const int warp_registers = (attributes.numRegs * 32 + 255) / 256 * 256;
    const int register_warps = std::min(64, 65536 / std::max(256, warp_registers));
    int warps = 0, best = 0;
    for (int w = 2; w <= kRolloutMaxWarps; ++w) {
        const size_t cta = (size_t)warp_bytes * w;
        if (cta > smem_limit) break;
        const int ctas = std::min((int)((smem_limit + 1024) / (cta + 1024)), register_warps / w);
        if (ctas && ctas * w >= best) { best = ctas * w; warps = w; }
    }
    /* a main part's length travels in 14 bits; the start words of the states' main parts have 16 places */
    if (!warps || batch.max_insn > 16383u || prob.num_states > 16u) return cudaErrorInvalidConfiguration;
    const size_t smem = (size_t)warp_bytes * warps;
    e = cudaFuncSetAttribute(rk4_kernel<RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_limit);
    if (e != cudaSuccess) return e;
    /* the largest shared-memory carve-out, always: left to itself the driver gave a CTA that fits the
     * 100 KB configuration that one, and only one CTA per SM became resident where two were planned
     * (measured: a call took 169 ms instead of 117 when its CTAs shrank from 101 KB to 98.8 KB) */
    e = cudaFuncSetAttribute(rk4_kernel<RR>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    const unsigned long long items = ((unsigned long long)prob.num_banks << prob.toggle_bits) * prob.num_systems;
    /* warps draw items from the queue until it is empty, so the grid only has to fill the device */
    int device = 0, sms = 0;
    if ((e = cudaGetDevice(&device)) != cudaSuccess || (e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return e;
    /* a launch that shares the device with `concurrent` - 1 others takes its share of the resident
     * CTAs: its warps then work through several items each, and one that drew a short item (an
     * invalid candidate) goes on with the next instead of idling until its CTA's longest item ends */
    const unsigned long long resident = (unsigned long long)sms * (unsigned)std::max(1, best / warps);
    const unsigned long long share = std::max<unsigned long long>(1, (resident + concurrent - 1) / std::max(1u, concurrent));
    const unsigned long long blocks = std::min<unsigned long long>((items + warps - 1) / warps, share);
    const size_t values = (size_t)prob.total_points * (prob.num_states + 1);
    rk4_validate_kernel<<<(unsigned)std::min<size_t>(1024, (values + 255) / 256), 256, 0, stream>>>(prob);
    rk4_kernel<RR><<<(unsigned)blocks, warps * 32, smem, stream>>>(batch, prob, lay);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_rk4(const DeviceBatch& batch, const Rk4Problem& prob, size_t smem_limit, unsigned concurrent, cudaStream_t stream) {
    if (prob.num_trajectories <= 32) return launch_width<1>(batch, prob, smem_limit, concurrent, stream);
    if (prob.num_trajectories <= 64) return launch_width<2>(batch, prob, smem_limit, concurrent, stream);
    return launch_width<4>(batch, prob, smem_limit, concurrent, stream);
}

}  // namespace sb
