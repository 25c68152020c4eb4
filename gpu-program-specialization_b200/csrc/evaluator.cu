/*
 * evaluator.cu - population evaluator for sm_100a.
 *
 * Replaces the reference's generated-and-patched kernels
 * (projects/secant/s_cubin_generate_toggle_sse.c:339-386, s_cubin_generate_sse.c:461-706,
 * s_cubin_generate_materialize.c:475-540) with one resident kernel family that interprets
 * the encoder's records (record.h).
 *
 * Work decomposition
 *   CTA    = one group of programs x one range of rows.  The CTA stages a tile of
 *            (inputs + targets) x tile_rows floats in shared memory once per chunk and all
 *            its warps read operands from that tile.
 *   warp   = one program at a time, taken from the CTA's queue, so long and short
 *            programs balance inside a CTA.  All 32 lanes execute the same instruction
 *            stream (no divergence); toggles are resolved per permutation by patching
 *            the warp's private copy of the program, not by per-thread selects.
 *   thread = a register tile acc[RR rows][RC banks]; one decoded instruction does
 *            RR*RC FP32 operations.  A column operand costs one 128-bit shared load per
 *            four rows and is reused for all RC coefficient banks; a bank constant is one
 *            broadcast load reused for all RR rows.
 * The squared error is accumulated in registers over the passes of a chunk, reduced
 * with warp shuffles, and added to the caller's output once per (program, configuration,
 * chunk): per-row predictions never reach HBM.
 *
 * Numerics follow the reference HOST evaluator (projects/secant/s_cpu.c:329-352): IEEE
 * add/sub/mul/div/sqrt, accurate sin/cos/exp/log, no flush-to-zero, and no contraction of
 * program-level multiplies and adds (only FMA_F32 fuses).
 */
#include "evaluator.cuh"
#include "sbmath.cuh"

#include <math_constants.h>

namespace sb {

namespace {

template <int OP>
__device__ __forceinline__ float binop(float a, float x) {
    if (OP == SB_BIN_ADD) return __fadd_rn(a, x);
    if (OP == SB_BIN_SUB) return __fsub_rn(a, x);
    if (OP == SB_BIN_RSUB) return __fsub_rn(x, a);
    if (OP == SB_BIN_MUL) return __fmul_rn(a, x);
    if (OP == SB_BIN_DIV) return __fdiv_rn(a, x);
    if (OP == SB_BIN_RDIV) return __fdiv_rn(x, a);
    if (OP == SB_BIN_MIN) return fminf(a, x);
    return fmaxf(a, x);
}

template <int OP>
__device__ __forceinline__ float unop(float a) {
    if (OP == SB_UN_NEG) return -a;
    return fabsf(a);
}

/* FMA_F32 takes three arbitrary operands.  It is rare in scoring workloads, so it runs
 * element by element over shared memory (the caller parks the accumulator in the scratch
 * slot first and reloads it afterwards) instead of being unrolled for every combination of
 * operand kinds.  Nothing here touches the register tile, which therefore stays in
 * registers. */
template <int RR, int RC>
__device__ __noinline__ void fma_over_scratch(uint2 ins, const float* rowp, const float* hrowp, uint32_t tile_ld, const float* cst,
                                              float4* slots, uint32_t scratch_slot) {
    constexpr int V = RR * RC;
    const unsigned kinds = (ins.x >> 8) & 0x3fu;
    float* out = reinterpret_cast<float*>(slots + (size_t)scratch_slot * (V / 4) * 32);
#pragma unroll 1
    for (int k = 0; k < V; ++k) {
        float v[3];
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const unsigned kind = (kinds >> (2 * i)) & 3u;
            const uint32_t index = (ins.y >> (10 * i)) & 1023u;
            const int r = k / RC, c = k % RC;
            if (kind == SB_KIND_ROW) {
                const float* q = (index & SB_FMA_ROW_HOISTED) ? hrowp + (size_t)(index & (SB_FMA_ROW_HOISTED - 1u)) * (32 * RR)
                                                              : rowp + (size_t)index * tile_ld;
                v[i] = q[(r / 4) * 128 + (r % 4)];
            } else if (kind == SB_KIND_CST) v[i] = cst[index * RC + c];
            else {
                const uint32_t slot = kind == SB_FMA_ACC ? scratch_slot : index;
                v[i] = reinterpret_cast<const float*>(slots + (size_t)slot * (V / 4) * 32)[(k >> 2) * 128 + (k & 3)];
            }
        }
        out[(k >> 2) * 128 + (k & 3)] = __fmaf_rn(v[0], v[1], v[2]);
    }
}

template <int RR, int RC, bool FAST = false>
struct Machine {
    static constexpr int V = RR * RC;
    static constexpr int PASS = 32 * RR;      /* rows one warp covers per pass */
    static constexpr int GROUPS = RR / 4;     /* float4 row groups per thread */

    float acc[RR][RC];

    /* one float per row, starting at the thread's first row of a column laid out [row of the pass] */
    __device__ __forceinline__ void fetch_column(const float* q, float (&x)[RR]) const {
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
            const float4 v = *reinterpret_cast<const float4*>(q + g * 128);
            x[4 * g + 0] = v.x; x[4 * g + 1] = v.y; x[4 * g + 2] = v.z; x[4 * g + 3] = v.w;
        }
    }
    /* ROW operand: a dataset column of the staged tile, or (SB_ROW_HOISTED) a value the row prelude
     * left in the warp's hoist buffer, which holds PASS floats per value */
    __device__ __forceinline__ void fetch_row(const float* rowp, const float* hrowp, uint32_t tile_ld, uint32_t col,
                                              float (&x)[RR]) const {
        const float* q = (col & SB_ROW_HOISTED) ? hrowp + (size_t)(col & (SB_ROW_HOISTED - 1u)) * PASS : rowp + (size_t)col * tile_ld;
        fetch_column(q, x);
    }
    __device__ __forceinline__ void fetch_cst(const float* cst, uint32_t entry, float (&x)[RC]) const {
        const float* q = cst + entry * RC;
        if (RC == 4) {
            const float4 v = *reinterpret_cast<const float4*>(q);
            x[0] = v.x; x[1 % RC] = v.y; x[2 % RC] = v.z; x[3 % RC] = v.w;
        } else if (RC == 2) {
            const float2 v = *reinterpret_cast<const float2*>(q);
            x[0] = v.x; x[1 % RC] = v.y;
        } else {
            x[0] = q[0];
        }
    }
    /* Slot s of this warp: V/4 float4 vectors per lane, lane-interleaved (conflict free). */
    __device__ __forceinline__ void fetch_slot(const float4* slots, uint32_t s, float (&x)[RR][RC]) const {
        const float4* q = slots + (size_t)s * (V / 4) * 32;
        float* flat = &x[0][0];
#pragma unroll
        for (int j = 0; j < V / 4; ++j) {
            const float4 v = q[j * 32];
            flat[4 * j + 0] = v.x; flat[4 * j + 1] = v.y; flat[4 * j + 2] = v.z; flat[4 * j + 3] = v.w;
        }
    }
    __device__ __forceinline__ void store_slot(float4* slots, uint32_t s) const {
        float4* q = slots + (size_t)s * (V / 4) * 32;
        const float* flat = &acc[0][0];
#pragma unroll
        for (int j = 0; j < V / 4; ++j) q[j * 32] = make_float4(flat[4 * j], flat[4 * j + 1], flat[4 * j + 2], flat[4 * j + 3]);
    }

#define SB_FOR_TILE _Pragma("unroll") for (int r = 0; r < RR; ++r) _Pragma("unroll") for (int c = 0; c < RC; ++c)

#define SB_BIN_CASES(OP)                                                                             \
    case SB_CASE_BIN + OP * SB_NUM_KINDS + SB_KIND_ROW: {                                            \
        float x[RR]; fetch_row(rowp, hrowp, tile_ld, idx, x);                                               \
        SB_FOR_TILE acc[r][c] = binop<OP>(acc[r][c], x[r]);                                          \
        break; }                                                                                     \
    case SB_CASE_BIN + OP * SB_NUM_KINDS + SB_KIND_CST: {                                            \
        float x[RC]; fetch_cst(cst, idx, x);                                                         \
        SB_FOR_TILE acc[r][c] = binop<OP>(acc[r][c], x[c]);                                          \
        break; }                                                                                     \
    case SB_CASE_BIN + OP * SB_NUM_KINDS + SB_KIND_SLOT: {                                           \
        float x[RR][RC]; fetch_slot(slots, idx, x);                                                  \
        SB_FOR_TILE acc[r][c] = binop<OP>(acc[r][c], x[r][c]);                                       \
        break; }

#define SB_UN_CASE(OP) \
    case SB_CASE_UN + OP: { SB_FOR_TILE acc[r][c] = unop<OP>(acc[r][c]); break; }

/* applies an out-of-line four-element function to the whole tile */
#define SB_FOR_QUADS(CALL)                                                                           \
    {                                                                                                \
        float* flat = &acc[0][0];                                                                    \
        _Pragma("unroll") for (int j = 0; j < V / 4; ++j) {                                          \
            const float4 in = make_float4(flat[4 * j], flat[4 * j + 1], flat[4 * j + 2], flat[4 * j + 3]); \
            const float4 o = CALL;                                                                   \
            flat[4 * j] = o.x; flat[4 * j + 1] = o.y; flat[4 * j + 2] = o.z; flat[4 * j + 3] = o.w;  \
        }                                                                                            \
    }

    /* Runs one instruction run of the warp's program over the RR*32 rows starting at rowp. */
    __device__ __forceinline__ void run(const SbInsn* exec, const float* rowp, uint32_t tile_ld, const float* cst,
                                        float4* slots, uint32_t scratch_slot, float* hrowp = nullptr) {
        const uint2* ip = reinterpret_cast<const uint2*>(exec);
        uint2 next = *ip++; /* the buffer holds one padding entry after the last END */
#pragma unroll 1
        for (;;) {
            const uint2 ins = next;
            next = *ip++;
            const uint32_t idx = ins.x >> 16;
            switch (ins.x & 0xffu) {
            case SB_CASE_END:
                return;
            case SB_CASE_LOAD + SB_KIND_ROW: {
                float x[RR]; fetch_row(rowp, hrowp, tile_ld, idx, x);
                SB_FOR_TILE acc[r][c] = x[r];
                break; }
            case SB_CASE_LOAD + SB_KIND_CST: {
                float x[RC]; fetch_cst(cst, idx, x);
                SB_FOR_TILE acc[r][c] = x[c];
                break; }
            case SB_CASE_LOAD + SB_KIND_SLOT:
                fetch_slot(slots, idx, acc);
                break;
            case SB_CASE_STORE:
                store_slot(slots, idx);
                break;
            case SB_CASE_STOREH: { /* bank-independent value: every bank column holds the same number */
                float* q = hrowp + (size_t)idx * PASS;
#pragma unroll
                for (int g = 0; g < GROUPS; ++g)
                    *reinterpret_cast<float4*>(q + g * 128) = make_float4(acc[4 * g][0], acc[4 * g + 1][0], acc[4 * g + 2][0], acc[4 * g + 3][0]);
                break; }
            SB_BIN_CASES(SB_BIN_ADD)
            SB_BIN_CASES(SB_BIN_SUB)
            SB_BIN_CASES(SB_BIN_RSUB)
            SB_BIN_CASES(SB_BIN_MUL)
            /* IEEE division is ~10 instructions per element: the six operand-kind cases
             * only expand the operand, then share one body per direction. */
            case SB_CASE_BIN + SB_BIN_DIV * SB_NUM_KINDS + SB_KIND_ROW:
            case SB_CASE_BIN + SB_BIN_RDIV * SB_NUM_KINDS + SB_KIND_ROW:
            case SB_CASE_BIN + SB_BIN_DIV * SB_NUM_KINDS + SB_KIND_CST:
            case SB_CASE_BIN + SB_BIN_RDIV * SB_NUM_KINDS + SB_KIND_CST:
            case SB_CASE_BIN + SB_BIN_DIV * SB_NUM_KINDS + SB_KIND_SLOT:
            case SB_CASE_BIN + SB_BIN_RDIV * SB_NUM_KINDS + SB_KIND_SLOT: {
                const unsigned rel = (ins.x & 0xffu) - SB_CASE_BIN;
                const unsigned kind = rel % SB_NUM_KINDS;
                float xv[RR][RC];
                if (kind == SB_KIND_ROW) {
                    float x[RR]; fetch_row(rowp, hrowp, tile_ld, idx, x);
                    SB_FOR_TILE xv[r][c] = x[r];
                } else if (kind == SB_KIND_CST) {
                    float x[RC]; fetch_cst(cst, idx, x);
                    SB_FOR_TILE xv[r][c] = x[c];
                } else {
                    fetch_slot(slots, idx, xv);
                }
                if (rel / SB_NUM_KINDS == SB_BIN_RDIV) { /* operand / acc: swap so that one body divides acc by xv */
                    SB_FOR_TILE { const float t = acc[r][c]; acc[r][c] = xv[r][c]; xv[r][c] = t; }
                }
                {
                    float* fa = &acc[0][0];
                    const float* fx = &xv[0][0];
#pragma unroll
                    for (int j = 0; j < V / 4; ++j) {
                        if (FAST) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) fa[4 * j + k] = sbm::fast_div(fa[4 * j + k], fx[4 * j + k]);
                            continue;
                        }
                        const float4 o = sbm::div4(make_float4(fa[4 * j], fa[4 * j + 1], fa[4 * j + 2], fa[4 * j + 3]),
                                                   make_float4(fx[4 * j], fx[4 * j + 1], fx[4 * j + 2], fx[4 * j + 3]));
                        fa[4 * j] = o.x; fa[4 * j + 1] = o.y; fa[4 * j + 2] = o.z; fa[4 * j + 3] = o.w;
                    }
                }
                break; }
            SB_BIN_CASES(SB_BIN_MIN)
            SB_BIN_CASES(SB_BIN_MAX)
            SB_UN_CASE(SB_UN_NEG)
            SB_UN_CASE(SB_UN_ABS)
            case SB_CASE_UN + SB_UN_EX2: case SB_CASE_UN + SB_UN_EXP: case SB_CASE_UN + SB_UN_LOG:
            case SB_CASE_UN + SB_UN_SIN: case SB_CASE_UN + SB_UN_COS: case SB_CASE_UN + SB_UN_SQRT:
            case SB_CASE_UN + SB_UN_RCP: case SB_CASE_UN + SB_UN_LG2: case SB_CASE_UN + SB_UN_RSQRT:
            case SB_CASE_UN + SB_UN_TANH: {
                /* one body for every function: the operation is selected inside the out-of-line call */
                const unsigned op = (ins.x & 0xffu) - SB_CASE_UN;
                if (FAST) {
                    switch (op) { /* a few instructions per element: unrolled in place */
                    case SB_UN_SIN: SB_FOR_TILE acc[r][c] = sbm::fast_unary(SB_UN_SIN, acc[r][c]); break;
                    case SB_UN_COS: SB_FOR_TILE acc[r][c] = sbm::fast_unary(SB_UN_COS, acc[r][c]); break;
                    case SB_UN_EXP: SB_FOR_TILE acc[r][c] = sbm::fast_unary(SB_UN_EXP, acc[r][c]); break;
                    case SB_UN_LOG: SB_FOR_TILE acc[r][c] = sbm::fast_unary(SB_UN_LOG, acc[r][c]); break;
                    case SB_UN_EX2: SB_FOR_TILE acc[r][c] = sbm::fast_unary(SB_UN_EX2, acc[r][c]); break;
                    default: SB_FOR_TILE acc[r][c] = sbm::fast_unary(op, acc[r][c]); break;
                    }
                } else SB_FOR_QUADS(sbm::unary4(in, op))
                break; }
            case SB_CASE_FMA:
                store_slot(slots, scratch_slot);
                fma_over_scratch<RR, RC>(ins, rowp, hrowp, tile_ld, cst, slots, scratch_slot);
                fetch_slot(slots, scratch_slot, acc);
                break;
            default:
                return; /* unreachable for records produced by the encoder */
            }
        }
    }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

/* Sums RC per-lane values over the warp, one total per value, in a fixed order: halves of the warp
 * trade values so that every step adds pairs, and value c ends in lane c * (32 / RC). */
template <int RC>
__device__ __forceinline__ float column_totals(const float (&p)[RC], int lane) {
    float k;
    if (RC == 4) {
        const bool hi = lane & 16, hi8 = lane & 8;
        float k0 = hi ? p[2 % RC] : p[0], k1 = hi ? p[3 % RC] : p[1 % RC];
        const float s0 = hi ? p[0] : p[2 % RC], s1 = hi ? p[1 % RC] : p[3 % RC];
        k0 = __fadd_rn(k0, __shfl_xor_sync(0xffffffffu, s0, 16));
        k1 = __fadd_rn(k1, __shfl_xor_sync(0xffffffffu, s1, 16));
        k = hi8 ? k1 : k0;
        k = __fadd_rn(k, __shfl_xor_sync(0xffffffffu, hi8 ? k0 : k1, 8));
    } else if (RC == 2) {
        const bool hi = lane & 16;
        k = hi ? p[1 % RC] : p[0];
        k = __fadd_rn(k, __shfl_xor_sync(0xffffffffu, hi ? p[0] : p[1 % RC], 16));
        k = __fadd_rn(k, __shfl_xor_sync(0xffffffffu, k, 8));
    } else {
        k = __fadd_rn(p[0], __shfl_xor_sync(0xffffffffu, p[0], 16));
        k = __fadd_rn(k, __shfl_xor_sync(0xffffffffu, k, 8));
    }
    k = __fadd_rn(k, __shfl_xor_sync(0xffffffffu, k, 4));
    k = __fadd_rn(k, __shfl_xor_sync(0xffffffffu, k, 2));
    k = __fadd_rn(k, __shfl_xor_sync(0xffffffffu, k, 1));
    return k;
}

/* ---- the bank part: a scalar machine, one lane per coefficient bank ------------------------- */

struct BankSource {
    const float* banks;      /* this program's table, [bank][slot] */
    size_t bank_stride;
    uint32_t num_banks, K, n_affine;
    const SbAffine* affines; /* of this program */
    const float* lits;       /* of this program */
};

template <bool FAST>
__device__ __forceinline__ float scalar_unary(unsigned op, float a) {
    if (op == SB_UN_NEG) return -a;
    if (op == SB_UN_ABS) return fabsf(a);
    if (FAST) return sbm::fast_unary(op, a);
    return sbm::unary4(make_float4(a, a, a, a), op).x;
}
template <bool FAST>
__device__ __forceinline__ float scalar_binary(unsigned op, float a, float x) {
    switch (op) {
    case SB_BIN_ADD: return __fadd_rn(a, x);
    case SB_BIN_SUB: return __fsub_rn(a, x);
    case SB_BIN_RSUB: return __fsub_rn(x, a);
    case SB_BIN_MUL: return __fmul_rn(a, x);
    case SB_BIN_DIV: return FAST ? sbm::fast_div(a, x) : sbm::div4(make_float4(a, a, a, a), make_float4(x, x, x, x)).x;
    case SB_BIN_RDIV: return FAST ? sbm::fast_div(x, a) : sbm::div4(make_float4(x, x, x, x), make_float4(a, a, a, a)).x;
    case SB_BIN_MIN: return fminf(a, x);
    default: return fmaxf(a, x);
    }
}

/* Runs the bank part of the warp's program for the `count` banks starting at `first_bank` (count is
 * a multiple of RC; banks past the table's end are padding and read zeros) and for `perms`
 * permutations starting at `perm0`.  Lane l handles (permutation, bank) pairs l, l + 32, ...,
 * permutation-major.  Results go to the warp's constant tables laid out [permutation][bank group]
 * [entry][bank of the group], `entries` entries per group; temporaries live in `tmp`, 32 floats
 * apart.  A toggle site of the bank part carries 1 + its index in the second instruction word; every
 * lane takes the alternative of its own permutation from the program's site list, so the state of
 * the warp's patched copy does not matter here.  The same functions as the tile machine are called,
 * so a value computed here has the bits it would have had in the main part. */
template <int RC, bool FAST>
__device__ __noinline__ void run_bank_part(const SbInsn* exec, uint32_t first_bank, uint32_t count, uint32_t perms, uint32_t perm0,
                                           const SbPatch* sites, uint32_t entries, float* table, float* tmp, const BankSource src, int lane) {
    const uint32_t pairs = count * perms;
    for (uint32_t v0 = 0; v0 < pairs; v0 += 32) {
        const uint32_t v = v0 + lane, j = v / count, b = v - j * count, bank = first_bank + b;
        const uint32_t perm = perm0 + j;
        const bool live = v < pairs, real = live && bank < src.num_banks;
        float* const mine = table + ((size_t)(j * (count / RC) + b / RC) * entries) * RC + (b % RC);
        const float* const row = src.banks + (size_t)bank * src.bank_stride;
        auto operand = [&](unsigned kind, uint32_t idx) -> float {
            if (kind == SB_KIND_ROW) return live ? mine[(size_t)idx * RC] : 0.0f;
            if (kind == SB_KIND_SLOT) return tmp[idx * 32 + lane];
            if (idx < src.K) return real ? __ldg(row + idx) : 0.0f;
            if (idx < src.K + src.n_affine) {
                const SbAffine a = src.affines[idx - src.K];
                return real ? __fadd_rn(__fmul_rn(__ldg(row + a.slot), a.scale), a.offset) : 0.0f;
            }
            return __ldg(src.lits + (idx - src.K - src.n_affine));
        };
        const uint2* ip = reinterpret_cast<const uint2*>(exec);
        float acc = 0.0f;
#pragma unroll 1
        for (;;) {
            uint2 ins = *ip++;
            const unsigned cs = ins.x & 0xffu; /* the operation is the same in every alternative of a site */
            if (cs == SB_CASE_END || cs > SB_CASE_FMA) break;
            const bool fma = cs == SB_CASE_FMA, bin = cs >= SB_CASE_BIN && cs < SB_CASE_UN;
            if (!fma && ins.y) { /* a toggle site: this lane's permutation selects the operand */
                const SbPatch* p = sites + (ins.y - 1u);
                unsigned choice = (perm >> p->bit0) & 1u;
                if (p->bit1 != 0xffu) choice |= ((perm >> p->bit1) & 1u) << 1;
                ins.x = p->alt[choice].w0;
            }
            const unsigned mine_cs = ins.x & 0xffu;
            /* operands first, at one site (the fetch is the bulky part): one for loads and binary
             * operations, three for the fused multiply-add, none otherwise */
            float v[3] = {acc, acc, acc};
            const unsigned count = fma ? 3u : (cs < SB_CASE_STORE || bin) ? 1u : 0u;
#pragma unroll 1
            for (unsigned i = 0; i < count; ++i) {
                const unsigned kind = fma ? (ins.x >> (8 + 2 * i)) & 3u : bin ? (mine_cs - SB_CASE_BIN) % SB_NUM_KINDS : mine_cs - SB_CASE_LOAD;
                const uint32_t idx = fma ? (ins.y >> (10 * i)) & 1023u : ins.x >> 16;
                if (kind != SB_FMA_ACC) v[i] = operand(kind, idx);
            }
            const uint32_t idx = ins.x >> 16;
            if (cs < SB_CASE_STORE) acc = v[0];
            else if (cs == SB_CASE_STORE) tmp[idx * 32 + lane] = acc;
            else if (cs == SB_CASE_STOREH) { if (live) mine[(size_t)idx * RC] = acc; }
            else if (bin) acc = scalar_binary<FAST>((cs - SB_CASE_BIN) / SB_NUM_KINDS, acc, v[0]);
            else if (fma) acc = __fmaf_rn(v[0], v[1], v[2]);
            else acc = scalar_unary<FAST>(cs - SB_CASE_UN, acc);
        }
    }
}

/* ---- tile staging ----------------------------------------------------------------------- */

__device__ __forceinline__ void cp_async_16(float* dst, const float* src, uint32_t src_bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_4(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

/* Starts the asynchronous copy of rows [c0, c0 + rows) of every column into a tile buffer laid out
 * [column][tile_ld]; rows up to `padded` are zero-filled.  A column whose first row is 16-byte
 * aligned moves as 16-byte copies, any other as 4-byte copies (callers only promise 4-byte
 * alignment of their matrices).  Completion: cp_async_wait_all() by every thread, then a barrier. */
__device__ __noinline__ void stage_tile(float* tile, uint32_t tile_ld, const EvalProblem& prob, uint32_t ncols, size_t c0,
                                           uint32_t rows, uint32_t padded) {
    for (uint32_t col = 0; col < ncols; ++col) {
        const float* src = (col < prob.num_inputs ? prob.input + (size_t)col * prob.input_ld
                                                  : prob.targets + (size_t)(col - prob.num_inputs) * prob.targets_ld) + c0;
        float* dst = tile + (size_t)col * tile_ld;
        if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
            for (uint32_t i = threadIdx.x * 4; i < padded; i += blockDim.x * 4) {
                if (i < rows) cp_async_16(dst + i, src + i, min(16u, (rows - i) * 4u)); /* short copies zero-fill their tail */
                else *reinterpret_cast<float4*>(dst + i) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        } else {
            for (uint32_t i = threadIdx.x; i < padded; i += blockDim.x) {
                if (i < rows) cp_async_4(dst + i, src + i);
                else dst[i] = 0.0f;
            }
        }
    }
    cp_async_commit();
}

/* 16 values per thread: 20 warps per CTA within 96 registers (32-value tiles were measured
 * slower at the 12 warps their 168 registers allow). */
template <int RR, int RC, bool FAST, bool SPAN>
__global__ void __launch_bounds__(640, 1)
eval_kernel(const DeviceBatch batch, const EvalProblem prob, const Geom geom, float* __restrict__ partial) {
    using M = Machine<RR, RC, FAST>;
    extern __shared__ __align__(16) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* const tiles = reinterpret_cast<float*>(smem);
    unsigned int* const queue = reinterpret_cast<unsigned int*>(smem + (size_t)geom.tile_bytes * geom.tile_buffers);
    unsigned char* const warea = smem + (size_t)geom.tile_bytes * geom.tile_buffers + 16 + (size_t)warp * geom.warp_bytes;
    SbInsn* const exec = reinterpret_cast<SbInsn*>(warea);
    float* const table = reinterpret_cast<float*>(warea + geom.exec_bytes);
    float* const hoist = reinterpret_cast<float*>(warea + geom.exec_bytes + geom.table_bytes);
    float* const slot_base = reinterpret_cast<float*>(warea + geom.exec_bytes + geom.table_bytes + geom.hoist_bytes);
    float4* const slots = reinterpret_cast<float4*>(slot_base) + lane;
    float* const psum = reinterpret_cast<float*>(warea + geom.exec_bytes + geom.table_bytes + geom.hoist_bytes + geom.slot_bytes);

    const uint32_t group = blockIdx.x / geom.row_splits, split = blockIdx.x % geom.row_splits;
    /* this CTA's programs: group, group + num_groups, ... (the batch is sorted by cost) */
    const uint32_t prog_count = (batch.num_programs - group + geom.num_groups - 1) / geom.num_groups;
    const size_t row_begin = (size_t)split * geom.rows_per_split;
    const size_t row_end = min(prob.num_rows, row_begin + (size_t)geom.rows_per_split);
    const bool materialize = prob.mode == EVAL_MATERIALIZE;
    const uint32_t ncols = prob.num_inputs + (materialize ? 0u : prob.num_targets);
    const uint32_t tile_ld = geom.tile_rows;
    const uint32_t T = prob.num_targets;
    const uint32_t nq = prob.mode == EVAL_AFFINE_STATS ? T + 2 : T;
    const uint32_t gpi = geom.groups_per_item;
    const uint32_t ppi = (!SPAN || materialize) ? 1u : geom.perms_per_item; /* SPAN: items may cover several permutations */
    const uint32_t wide = ppi * gpi; /* (permutation, bank group) pairs of an item: the partial sums' middle dimension */
    /* configuration groups of one program: permutation-major, RC banks per group */
    const uint32_t bank_groups = materialize ? 1u : (prob.num_banks + RC - 1) / RC;
    /* items of one program: permutation-major, `chunks` items of gpi bank groups per permutation, or
     * (when one item holds every bank group) one item per block of ppi permutations; the planner keeps
     * items_per_program * prog_count below 2^32 - 256, so item arithmetic is 32-bit */
    const uint32_t chunks = materialize ? 1u : bank_groups / gpi;
    const uint32_t items_per_program = materialize ? 1u : (uint32_t)(((unsigned long long)chunks << prob.toggle_bits) / ppi);
    const unsigned int num_items = items_per_program * prog_count;
    const unsigned long long configs = (unsigned long long)prob.num_banks << prob.toggle_bits;
    const size_t tile_floats = geom.tile_bytes / 4;
    const uint32_t num_tiles = (uint32_t)((row_end - row_begin + geom.tile_rows - 1) / geom.tile_rows);

    /* Tiles: with two buffers tile t + 1 is fetched while tile t is used; with one (a tile so large
     * that only one fits beside the warps' working sets) the fetch follows a barrier after the tile. */
    const bool overlapped = geom.tile_buffers > 1;
    if (threadIdx.x == 0) queue[0] = 0u;
    for (uint32_t t = 0; t < num_tiles; ++t) {
        const size_t c0 = row_begin + (size_t)t * geom.tile_rows;
        const uint32_t chunk_rows = (uint32_t)min((size_t)geom.tile_rows, row_end - c0);
        const uint32_t npass = (chunk_rows + M::PASS - 1) / M::PASS;
        const float* const tile = tiles + (overlapped ? (size_t)(t & 1u) * tile_floats : 0);
        unsigned int* const q = queue + (t & 1u);
        if (t == 0 || !overlapped) {
            if (t) __syncthreads(); /* every warp has left the buffer */
            stage_tile(tiles, tile_ld, prob, ncols, c0, chunk_rows, npass * M::PASS);
        }
        cp_async_wait_all();
        __syncthreads(); /* tile t has landed; every warp has left tile t - 1 */
        if (threadIdx.x == 0) queue[(t + 1) & 1u] = 0u;
        if (overlapped && t + 1 < num_tiles) {
            const size_t n0 = c0 + geom.tile_rows;
            const uint32_t nrows = (uint32_t)min((size_t)geom.tile_rows, row_end - n0);
            stage_tile(tiles + (size_t)((t + 1) & 1u) * tile_floats, tile_ld, prob, ncols, n0, nrows, (nrows + M::PASS - 1) / M::PASS * M::PASS);
        }

        for (;;) {
            unsigned int item = 0;
            if (lane == 0) item = atomicAdd(q, 1u);
            item = __shfl_sync(0xffffffffu, item, 0);
            if (item >= num_items) break;
            const uint32_t pi = item / items_per_program, within = item - pi * items_per_program;
            const uint32_t lp = group + pi * geom.num_groups;                        /* index inside the batch */
            const SbProgram* const hp = batch.programs + lp;
            const uint32_t n_insn = hp->n_insn, pre_off = hp->pre_off, mid_off = hp->mid_off, main_off = hp->main_off, n_cst = hp->n_cst;
            const uint32_t n_patch = hp->n_patch, flags = hp->flags;
            __syncwarp(); /* the previous item's reads of exec, table and psum are done */
            {
                const SbInsn* code = batch.insns + hp->insn_off;
                for (uint32_t i = lane; i < n_insn; i += 32) exec[i] = code[i];
                if (lane == 0) exec[n_insn] = SbInsn{0u, 0u}; /* padding read by the instruction prefetch */
            }
            /* the item's permutations perm0 .. perm0 + ppi - 1 (one, unless the item holds every bank group) */
            const uint32_t block = materialize ? 0u : within / chunks;
            const uint32_t perm0 = materialize ? prob.fixed_permutation : block * ppi;
            const uint32_t first_bg = materialize ? 0u : (within - block * chunks) * gpi;
            const uint32_t ngroups = materialize ? 1u : min(gpi, bank_groups - first_bg);
            const SbPatch* const patches = batch.patches + hp->patch_off;
            /* rewrites the toggle sites of the warp's copy for one permutation */
            auto patch_for = [&](uint32_t perm) {
                __syncwarp(); /* earlier reads and writes of the copy by other lanes are done */
                for (uint32_t i = lane; i < n_patch; i += 32) {
                    const SbPatch* p = patches + i;
                    unsigned choice = (perm >> p->bit0) & 1u;
                    if (p->bit1 != 0xffu) choice |= ((perm >> p->bit1) & 1u) << 1;
                    exec[p->insn] = p->alt[choice];
                }
                __syncwarp();
            };
            for (uint32_t e = lane; e < nq * wide * RC; e += 32) psum[e] = 0.0f;
            const size_t gp = prob.first_program + hp->index; /* position in the run: output row, bank table */
            const uint32_t table_stride = n_cst * RC;
            /* the constant tables of every permutation of the item, all in one run of the bank part; an
             * item of one permutation is then patched for it, the others inside the row passes */
            __syncwarp();
            if (pre_off) {
                BankSource src;
                src.banks = prob.banks ? prob.banks + gp * prob.program_bank_stride : nullptr;
                src.bank_stride = prob.bank_stride;
                src.num_banks = prob.banks ? prob.num_banks : 0u; /* without a table every bank constant reads zero */
                src.K = prob.num_constants;
                src.n_affine = hp->n_affine;
                src.affines = batch.affines + hp->affine_off;
                src.lits = batch.lits + hp->lit_off;
                run_bank_part<RC, FAST>(exec, first_bg * RC, ngroups * RC, ppi, perm0, patches, n_cst, table, slot_base, src, lane);
            }
            if (ppi == 1u && n_patch) patch_for(perm0);
            __syncwarp();
            const bool has_shared = mid_off > pre_off, has_prelude = main_off > mid_off;
            const uint32_t eval_groups = (flags & SB_PROG_BANK_INDEPENDENT) ? 1u : ngroups;

            M m;
#pragma unroll 1
            for (uint32_t pass = 0; pass < npass; ++pass) {
                const float* rowp = tile + pass * M::PASS + lane * 4;
                float* const hrowp = hoist + lane * 4;
                const uint32_t row0 = pass * M::PASS + lane * 4; /* first row of this thread in the tile */
                const bool full = (pass + 1) * M::PASS <= chunk_rows;
                /* One loop over the steps of a pass, so that the interpreter has one call site (a second
                 * inlined copy would not fit the instruction caches).  First (only when the program has
                 * one) the shared row prelude: the row-only sub-expressions no toggle reaches, once for the
                 * pass.  Then, for every permutation of the item: the row-only sub-expressions that depend
                 * on it (only when the program has any), and the main part once per bank group.  Without
                 * SPAN an item has one permutation and the steps are -2 (shared prelude), -1 (prelude),
                 * 0.. (bank groups); with it they are -1 (shared prelude) and then per_perm steps per
                 * permutation. */
                const int per_perm = (has_prelude ? 1 : 0) + (int)eval_groups;
                const int first = SPAN ? (has_shared ? -1 : 0) : (has_shared ? -2 : has_prelude ? -1 : 0);
                const int last = SPAN ? (int)ppi * per_perm : (int)eval_groups;
#pragma unroll 1
                for (int s = first; s < last; ++s) {
                    int j = 0, g = s < 0 ? 0 : s;
                    bool prelude = s < 0;
                    uint32_t start = s == first && has_shared ? pre_off : s < 0 ? mid_off : main_off;
                    if (SPAN) {
                        j = s < 0 ? 0 : s / per_perm;
                        const int w = s - j * per_perm; /* step inside the permutation */
                        prelude = s < 0 || (has_prelude && w == 0);
                        g = prelude ? 0 : w - (has_prelude ? 1 : 0);
                        start = prelude ? (s < 0 ? pre_off : mid_off) : main_off;
                        if (s >= 0 && w == 0 && ppi > 1u && n_patch) patch_for(perm0 + (uint32_t)j);
                    } else if (s == -1 && !has_prelude) continue;
                    const uint32_t gi = (uint32_t)j * ngroups + (uint32_t)g; /* this permutation's table, this group's */
                    m.run(exec + start, rowp, tile_ld, table + gi * table_stride, slots, geom.scratch_slot, hrowp);
                    if (prelude) continue;
                    if (materialize) {
                        float* out = prob.output + gp * prob.out_program_stride + c0;
#pragma unroll
                        for (int r = 0; r < RR; ++r) {
                            const uint32_t row = row0 + (r / 4) * 128 + (r % 4);
                            if (row < chunk_rows) out[row] = m.acc[r][0];
                        }
                    } else if (prob.mode == EVAL_SSE && T == 1) {
                        float tv[RR], part[RC];
                        m.fetch_column(rowp + (size_t)prob.num_inputs * tile_ld, tv);
#pragma unroll
                        for (int c = 0; c < RC; ++c) part[c] = 0.0f;
#pragma unroll
                        for (int r = 0; r < RR; ++r)
                            if (full || row0 + (r / 4) * 128 + (r % 4) < chunk_rows) { /* rows past the data score nothing */
#pragma unroll
                                for (int c = 0; c < RC; ++c) {
                                    const float e = __fsub_rn(m.acc[r][c], tv[r]);
                                    part[c] = __fmaf_rn(e, e, part[c]);
                                }
                            }
                        const float total = column_totals<RC>(part, lane);
                        if ((lane & (32 / RC - 1)) == 0) psum[gi * RC + lane / (32 / RC)] += total;
                    } else {
                        /* several targets, or affine statistics: quantity q of pair gi lives in psum[(q * wide + gi) * RC + c] */
                        for (uint32_t qn = 0; qn < nq; ++qn) {
                            float tv[RR];
                            const bool is_target = prob.mode == EVAL_SSE || qn >= 2;
                            const uint32_t tcol = prob.num_inputs + (prob.mode == EVAL_SSE ? qn : qn - 2);
                            if (is_target) m.fetch_column(rowp + (size_t)tcol * tile_ld, tv);
                            float s[RC];
#pragma unroll
                            for (int c = 0; c < RC; ++c) s[c] = 0.0f;
#pragma unroll
                            for (int r = 0; r < RR; ++r) {
                                const bool ok = full || row0 + (r / 4) * 128 + (r % 4) < chunk_rows;
#pragma unroll
                                for (int c = 0; c < RC; ++c) {
                                    const float p = m.acc[r][c];
                                    float term;
                                    if (prob.mode == EVAL_SSE) { const float e = __fsub_rn(p, tv[r]); term = __fmul_rn(e, e); }
                                    else if (qn == 0) term = p;
                                    else if (qn == 1) term = __fmul_rn(p, p);
                                    else term = __fmul_rn(p, tv[r]);
                                    s[c] = __fadd_rn(s[c], ok ? term : 0.0f);
                                }
                            }
                            const float total = column_totals<RC>(s, lane);
                            if ((lane & (32 / RC - 1)) == 0) psum[(qn * wide + gi) * RC + lane / (32 / RC)] += total;
                        }
                    }
                }
            }
            if (materialize) continue;
            __syncwarp();
            /* this CTA's partial sums of the item: stored on its first tile, added to afterwards (only this
             * CTA touches them, and a barrier separates its tiles) */
            {
                const bool independent = (flags & SB_PROG_BANK_INDEPENDENT) != 0;
                const uint32_t width = ngroups * RC;          /* banks of the item, padding included */
                for (uint32_t j = 0; j < ppi; ++j) {
                    float* mine = partial + ((size_t)split * batch.num_programs + lp) * nq * configs + perm0 + j;
                    const float* sums = psum + j * width;     /* psum is [quantity][permutation][group][bank of the group] */
                    for (uint32_t qn = 0; qn < nq; ++qn, mine += configs, sums += wide * RC)
                        for (uint32_t e = lane; e < width; e += 32) {
                            const uint32_t bank = first_bg * RC + e;
                            if (bank >= prob.num_banks) continue;
                            const float v = independent ? sums[0] : sums[e];
                            float* dst = mine + ((size_t)bank << prob.toggle_bits);
                            *dst = t == 0 ? v : __fadd_rn(*dst, v);
                        }
                }
            }
        }
    }
    cp_async_wait_all();
}

/* Adds the per-split partial sums of every (program, quantity, configuration) in split order and
 * writes the total to the caller's grid (only active bins are written: padding keeps its contents). */
__global__ void combine_kernel(const DeviceBatch batch, const EvalProblem prob, const float* __restrict__ partial, uint32_t splits,
                               uint32_t nq, unsigned long long configs) {
    const unsigned long long per_program = (unsigned long long)nq * configs;
    const unsigned long long total = per_program * batch.num_programs;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (unsigned long long)gridDim.x * blockDim.x) {
        float sum = partial[i];
        for (uint32_t s = 1; s < splits; ++s) sum = __fadd_rn(sum, partial[(unsigned long long)s * total + i]);
        const uint32_t lp = (uint32_t)(i / per_program);
        const unsigned long long rem = i % per_program, qn = rem / configs, cfg = rem % configs;
        const size_t gp = prob.first_program + batch.programs[lp].index;
        prob.output[gp * prob.out_program_stride + (size_t)qn * prob.out_target_stride + cfg] = sum;
    }
}

template <int RR, int RC>
cudaError_t launch_variant(const DeviceBatch& batch, const EvalProblem& prob, const Geom& geom, const LaunchPlan& plan,
                           float* partial, cudaStream_t stream) {
    const bool span = plan.perms_per_item > 1;
    if (prob.fast_math && span)
        eval_kernel<RR, RC, true, true><<<plan.grid_x, plan.warps * 32, plan.smem_bytes, stream>>>(batch, prob, geom, partial);
    else if (prob.fast_math)
        eval_kernel<RR, RC, true, false><<<plan.grid_x, plan.warps * 32, plan.smem_bytes, stream>>>(batch, prob, geom, partial);
    else if (span)
        eval_kernel<RR, RC, false, true><<<plan.grid_x, plan.warps * 32, plan.smem_bytes, stream>>>(batch, prob, geom, partial);
    else
        eval_kernel<RR, RC, false, false><<<plan.grid_x, plan.warps * 32, plan.smem_bytes, stream>>>(batch, prob, geom, partial);
    return cudaGetLastError();
}

uint32_t round16(size_t v) { return (uint32_t)((v + 15) / 16 * 16); }

}  // namespace

#define SB_FOR_VARIANTS(X) X(4, 4) X(8, 2) X(16, 1)

cudaError_t configure_kernels() {
    cudaError_t e;
    int dev = 0, limit = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return e;
#define SB_CONFIGURE(RR, RC) \
    if ((e = cudaFuncSetAttribute(eval_kernel<RR, RC, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, limit)) != cudaSuccess) return e; \
    if ((e = cudaFuncSetAttribute(eval_kernel<RR, RC, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, limit)) != cudaSuccess) return e; \
    if ((e = cudaFuncSetAttribute(eval_kernel<RR, RC, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, limit)) != cudaSuccess) return e; \
    if ((e = cudaFuncSetAttribute(eval_kernel<RR, RC, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, limit)) != cudaSuccess) return e;
    SB_FOR_VARIANTS(SB_CONFIGURE)
#undef SB_CONFIGURE
    return cudaSuccess;
}

cudaError_t launch_eval(const DeviceBatch& batch, const EvalProblem& prob, const LaunchPlan& plan, float* partial,
                        cudaStream_t stream, unsigned* launches) {
    const Geom geom = make_geom(batch, prob, plan);
    cudaError_t e;
    switch (plan.variant) {
    case 0: e = launch_variant<4, 4>(batch, prob, geom, plan, partial, stream); break;
    case 1: e = launch_variant<8, 2>(batch, prob, geom, plan, partial, stream); break;
    default: e = launch_variant<16, 1>(batch, prob, geom, plan, partial, stream); break;
    }
    if (e != cudaSuccess) return e;
    *launches = 1;
    if (prob.mode == EVAL_MATERIALIZE) return cudaSuccess;
    const uint32_t nq = prob.mode == EVAL_AFFINE_STATS ? prob.num_targets + 2u : prob.num_targets;
    const unsigned long long configs = (unsigned long long)prob.num_banks << prob.toggle_bits;
    const unsigned long long total = (unsigned long long)nq * configs * batch.num_programs;
    const unsigned blocks = (unsigned)std::min<unsigned long long>((total + 255) / 256, 148ull * 16ull);
    combine_kernel<<<blocks ? blocks : 1u, 256, 0, stream>>>(batch, prob, partial, plan.row_splits, nq, configs);
    e = cudaGetLastError();
    if (e == cudaSuccess) *launches = 2;
    return e;
}

}  // namespace sb
