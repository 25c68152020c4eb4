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

struct Geom {
    uint32_t tile_rows;      /* floats between consecutive columns of the tile */
    uint32_t programs_per_cta;
    uint32_t row_splits;
    uint32_t exec_bytes;     /* per-warp regions, each a multiple of 16 bytes */
    uint32_t cst_bytes;
    uint32_t tacc_bytes;
    uint32_t hoist_bytes;    /* per-row values left by the prelude: max_hoisted x tile_rows floats */
    uint32_t warp_bytes;
    uint32_t tile_bytes;
    unsigned long long rows_per_split;
    uint32_t groups_per_item; /* configuration groups one queue item covers */
    uint32_t scratch_slot;    /* spill slot reserved for the out-of-line unary functions */
};

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

/* Unary functions that are rare in scoring workloads and bulky when unrolled over the whole
 * register tile.  They run element by element over a copy of the tile in shared memory,
 * so their bodies exist once in the kernel. */
__device__ __noinline__ float rare_unop(unsigned op, float a) {
    switch (op) {
    case SB_UN_SQRT: return __fsqrt_rn(a);
    case SB_UN_RCP: return __frcp_rn(a);
    case SB_UN_RSQRT: return __frcp_rn(__fsqrt_rn(a)); /* host: 1 / sqrtf(x), two roundings */
    case SB_UN_LG2: return log2f(a);
    default: return tanhf(a);
    }
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
            if (kind == SB_KIND_ROW) v[i] = ((index & SB_ROW_HOISTED) ? hrowp : rowp)[(size_t)(index & 0x7fu) * tile_ld + (r / 4) * 128 + (r % 4)];
            else if (kind == SB_KIND_CST) v[i] = cst[index * RC + c];
            else {
                const uint32_t slot = kind == SB_FMA_ACC ? scratch_slot : index;
                v[i] = reinterpret_cast<const float*>(slots + (size_t)slot * (V / 4) * 32)[(k >> 2) * 128 + (k & 3)];
            }
        }
        out[(k >> 2) * 128 + (k & 3)] = __fmaf_rn(v[0], v[1], v[2]);
    }
}

/* Applies a rare unary function to every element of the tile parked in the scratch slot. */
template <int V>
__device__ __noinline__ void rare_over_scratch(unsigned op, float4* slots, uint32_t scratch_slot) {
    float* flat = reinterpret_cast<float*>(slots + (size_t)scratch_slot * (V / 4) * 32);
#pragma unroll 1
    for (int k = 0; k < V; ++k) {
        float* p = flat + (k >> 2) * 128 + (k & 3);
        *p = rare_unop(op, *p);
    }
}

template <int RR, int RC, bool FAST = false>
struct Machine {
    static constexpr int V = RR * RC;
    static constexpr int PASS = 32 * RR;      /* rows one warp covers per pass */
    static constexpr int GROUPS = RR / 4;     /* float4 row groups per thread */

    float acc[RR][RC];

    /* one float per row: a dataset column from the staged tile, or (index bit 7) a value the
     * prelude left in the warp's hoist buffer; both are laid out [column][row of the chunk] */
    __device__ __forceinline__ void fetch_row(const float* rowp, const float* hrowp, uint32_t tile_ld, uint32_t col,
                                              float (&x)[RR]) const {
        const float* q = ((col & SB_ROW_HOISTED) ? hrowp : rowp) + (size_t)(col & 0x7fu) * tile_ld;
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
            const float4 v = *reinterpret_cast<const float4*>(q + g * 128);
            x[4 * g + 0] = v.x; x[4 * g + 1] = v.y; x[4 * g + 2] = v.z; x[4 * g + 3] = v.w;
        }
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

    /* Runs the warp's program once over the RR*32 rows starting at rowp. */
    __device__ __forceinline__ void run(const SbInsn* exec, const float* rowp, uint32_t tile_ld, const float* cst,
                                        float4* slots, uint32_t scratch_slot, float* hrowp = nullptr) {
        const uint2* ip = reinterpret_cast<const uint2*>(exec);
        uint2 next = *ip++; /* the buffer holds one padding entry after END */
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
                float* q = hrowp + (size_t)idx * tile_ld;
#pragma unroll
                for (int g = 0; g < GROUPS; ++g)
                    *reinterpret_cast<float4*>(q + g * 128) = make_float4(acc[4 * g][0], acc[4 * g + 1][0], acc[4 * g + 2][0], acc[4 * g + 3][0]);
                break; }
            SB_BIN_CASES(SB_BIN_ADD)
            SB_BIN_CASES(SB_BIN_SUB)
            SB_BIN_CASES(SB_BIN_RSUB)
            SB_BIN_CASES(SB_BIN_MUL)
            /* IEEE division is ~10 instructions per element: the eight operand-kind cases
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
            case SB_CASE_UN + SB_UN_EX2:
                if (FAST) { SB_FOR_TILE acc[r][c] = sbm::fast_unary(SB_UN_EX2, acc[r][c]); } else SB_FOR_QUADS(sbm::exp2_4(in))
                break;
            case SB_CASE_UN + SB_UN_EXP:
                if (FAST) { SB_FOR_TILE acc[r][c] = sbm::fast_unary(SB_UN_EXP, acc[r][c]); } else SB_FOR_QUADS(sbm::exp4(in))
                break;
            case SB_CASE_UN + SB_UN_LOG:
                if (FAST) { SB_FOR_TILE acc[r][c] = sbm::fast_unary(SB_UN_LOG, acc[r][c]); } else SB_FOR_QUADS(sbm::log4(in))
                break;
            case SB_CASE_UN + SB_UN_SIN:
            case SB_CASE_UN + SB_UN_COS: { /* cos x = sin(x + pi/2): one body, shifted quadrant */
                const int shift = (int)(ins.x & 0xffu) - (SB_CASE_UN + SB_UN_SIN);
                if (FAST) {
                    if (shift) { SB_FOR_TILE acc[r][c] = sbm::fast_unary(SB_UN_COS, acc[r][c]); }
                    else { SB_FOR_TILE acc[r][c] = sbm::fast_unary(SB_UN_SIN, acc[r][c]); }
                } else SB_FOR_QUADS(sbm::sincos4(in, shift))
                break; }
            case SB_CASE_UN + SB_UN_SQRT:
            case SB_CASE_UN + SB_UN_RCP:
            case SB_CASE_UN + SB_UN_LG2:
            case SB_CASE_UN + SB_UN_RSQRT:
            case SB_CASE_UN + SB_UN_TANH:
                if (FAST) {
                    const unsigned op = (ins.x & 0xffu) - SB_CASE_UN;
                    SB_FOR_TILE acc[r][c] = sbm::fast_unary(op, acc[r][c]);
                    break;
                }
                store_slot(slots, scratch_slot);
                rare_over_scratch<V>((ins.x & 0xffu) - SB_CASE_UN, slots, scratch_slot);
                fetch_slot(slots, scratch_slot, acc);
                break;
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

/* 16-value tiles run 16 warps per CTA within 128 registers; 32-value tiles need more
 * registers per thread and run 12 warps. */
template <int RR, int RC, bool FAST>
__global__ void __launch_bounds__(RR * RC > 16 ? 384 : 640, 1)
eval_kernel(const DeviceBatch batch, const EvalProblem prob, const Geom geom) {
    using M = Machine<RR, RC, FAST>;
    extern __shared__ __align__(16) unsigned char smem[];
    float* const tile = reinterpret_cast<float*>(smem);
    unsigned int* const queue = reinterpret_cast<unsigned int*>(smem + geom.tile_bytes);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned char* const warea = smem + geom.tile_bytes + 16 + (size_t)warp * geom.warp_bytes;
    SbInsn* const exec = reinterpret_cast<SbInsn*>(warea);
    float* const cst = reinterpret_cast<float*>(warea + geom.exec_bytes);
    float* const tacc = reinterpret_cast<float*>(warea + geom.exec_bytes + geom.cst_bytes);
    float* const hoist = reinterpret_cast<float*>(warea + geom.exec_bytes + geom.cst_bytes + geom.tacc_bytes);
    float4* const slots = reinterpret_cast<float4*>(warea + geom.exec_bytes + geom.cst_bytes + geom.tacc_bytes + geom.hoist_bytes) + lane;

    const uint32_t group = blockIdx.x / geom.row_splits, split = blockIdx.x % geom.row_splits;
    const uint32_t prog_begin = group * geom.programs_per_cta;
    const uint32_t prog_count = min(geom.programs_per_cta, batch.num_programs - prog_begin);
    const size_t row_begin = (size_t)split * geom.rows_per_split;
    const size_t row_end = min(prob.num_rows, row_begin + (size_t)geom.rows_per_split);
    const bool materialize = prob.mode == EVAL_MATERIALIZE;
    const uint32_t ncols = prob.num_inputs + (materialize ? 0u : prob.num_targets);
    const uint32_t tile_ld = geom.tile_rows;
    const uint32_t K = prob.num_constants;
    const uint32_t T = prob.num_targets;
    /* configuration groups of one program: permutation-major, RC banks per group */
    const uint32_t bank_groups = materialize ? 1u : (prob.num_banks + RC - 1) / RC;
    const unsigned long long cfg_groups = materialize ? 1ull : ((unsigned long long)bank_groups << prob.toggle_bits);
    const unsigned long long items_per_program = (cfg_groups + geom.groups_per_item - 1) / geom.groups_per_item;
    const unsigned long long num_items = items_per_program * prog_count;

    for (size_t c0 = row_begin; c0 < row_end; c0 += geom.tile_rows) {
        const uint32_t chunk_rows = (uint32_t)min((size_t)geom.tile_rows, row_end - c0);
        const uint32_t padded = (chunk_rows + M::PASS - 1) / M::PASS * M::PASS;
        const uint32_t npass = padded / M::PASS;
        __syncthreads();
        for (uint32_t col = 0; col < ncols; ++col) {
            const float* src = col < prob.num_inputs ? prob.input + (size_t)col * prob.input_ld
                                                     : prob.targets + (size_t)(col - prob.num_inputs) * prob.targets_ld;
            float* dst = tile + (size_t)col * tile_ld;
            for (uint32_t i = threadIdx.x; i < padded; i += blockDim.x) dst[i] = i < chunk_rows ? __ldg(src + c0 + i) : 0.0f;
        }
        if (threadIdx.x == 0) *queue = 0u;
        __syncthreads();

        uint32_t loaded = 0xffffffffu; /* program currently held in this warp's exec buffer */
        SbProgram pr;
        for (;;) {
            unsigned int item = 0;
            if (lane == 0) item = atomicAdd(queue, 1u);
            item = __shfl_sync(0xffffffffu, item, 0);
            if (item >= num_items) break;
            const uint32_t pi = (uint32_t)(item / items_per_program);
            const unsigned long long first_group = (item % items_per_program) * geom.groups_per_item;
            const unsigned long long last_group = min(cfg_groups, first_group + geom.groups_per_item);
            const uint32_t lp = prog_begin + pi;           /* index inside the batch */
            __syncwarp();
            if (lp != loaded) {
                pr = batch.programs[lp];
                for (uint32_t i = lane; i < pr.n_insn; i += 32) exec[i] = batch.insns[pr.insn_off + i];
                if (lane == 0) exec[pr.n_insn] = SbInsn{0u, 0u}; /* padding read by the instruction prefetch */
                for (uint32_t i = lane; i < (uint32_t)pr.n_lits * RC; i += 32)
                    cst[(K + pr.n_affine) * RC + i] = batch.lits[pr.lit_off + i / RC];
                loaded = lp;
            }
            const size_t gp = prob.first_program + pr.index; /* position in the run: output row, bank table */
            const float* bank_base = prob.banks ? prob.banks + gp * prob.program_bank_stride : nullptr;
            /* an item never straddles permutations: toggles are patched once per item */
            const unsigned long long perm = materialize ? prob.fixed_permutation : first_group / bank_groups;
            if (pr.n_patch) {
                __syncwarp(); /* the copy above and the patches below touch the same words from different lanes */
                for (uint32_t i = lane; i < pr.n_patch; i += 32) {
                    const SbPatch* p = batch.patches + pr.patch_off + i;
                    unsigned choice = (unsigned)(perm >> p->bit0) & 1u;
                    if (p->bit1 != 0xffu) choice |= ((unsigned)(perm >> p->bit1) & 1u) << 1;
                    exec[p->insn] = p->alt[choice];
                }
            }
            /* iteration -1 (only when the program has a prelude) evaluates the bank-independent
             * sub-expressions once per row; iterations 0.. evaluate the main part per bank group */
            const long long steps = (long long)(last_group - first_group);
            for (long long step = pr.main_off ? -1 : 0; step < steps; ++step) {
                const bool prelude = step < 0;
                const uint32_t bg = prelude ? 0u : (uint32_t)((first_group + (unsigned long long)step) % bank_groups);
                __syncwarp();
                if (!prelude)
                for (uint32_t e = lane; e < (K + pr.n_affine) * RC; e += 32) {
                    const uint32_t entry = e / RC, c = e % RC, bank = bg * RC + c;
                    float v = 0.0f;
                    if (bank < prob.num_banks) {
                        if (entry < K) {
                            v = __ldg(bank_base + (size_t)bank * prob.bank_stride + entry);
                        } else {
                            const SbAffine a = batch.affines[pr.affine_off + entry - K];
                            v = __fadd_rn(__fmul_rn(__ldg(bank_base + (size_t)bank * prob.bank_stride + a.slot), a.scale), a.offset);
                        }
                    }
                    cst[e] = v;
                }
                if (!prelude && (T > 1 || prob.mode == EVAL_AFFINE_STATS))
                    for (uint32_t e = lane; e < (T + 2) * RC; e += 32) tacc[e] = 0.0f;
                __syncwarp();

                M m;
                float part[RC];
#pragma unroll
                for (int c = 0; c < RC; ++c) part[c] = 0.0f;

#pragma unroll 1
                for (uint32_t pass = 0; pass < npass; ++pass) {
                    const float* rowp = tile + pass * M::PASS + lane * 4;
                    m.run(exec + (prelude ? 0u : (uint32_t)pr.main_off), rowp, tile_ld, cst, slots, geom.scratch_slot,
                          hoist + pass * M::PASS + lane * 4);
                    if (prelude) continue;
                    const uint32_t row0 = pass * M::PASS + lane * 4; /* first row of this thread in the chunk */
                    const bool full = (pass + 1) * M::PASS <= chunk_rows;
                    if (materialize) {
                        float* out = prob.output + gp * prob.out_program_stride + c0;
#pragma unroll
                        for (int r = 0; r < RR; ++r) {
                            const uint32_t row = row0 + (r / 4) * 128 + (r % 4);
                            if (row < chunk_rows) out[row] = m.acc[r][0];
                        }
                    } else if (prob.mode == EVAL_SSE && T == 1) {
                        float t[RR];
                        m.fetch_row(rowp, rowp, tile_ld, prob.num_inputs, t);
                        if (full) {
#pragma unroll
                            for (int r = 0; r < RR; ++r)
#pragma unroll
                                for (int c = 0; c < RC; ++c) {
                                    const float e = __fsub_rn(m.acc[r][c], t[r]);
                                    part[c] = __fmaf_rn(e, e, part[c]);
                                }
                        } else {
#pragma unroll
                            for (int r = 0; r < RR; ++r) {
                                const bool ok = row0 + (r / 4) * 128 + (r % 4) < chunk_rows;
#pragma unroll
                                for (int c = 0; c < RC; ++c) {
                                    const float e = ok ? __fsub_rn(m.acc[r][c], t[r]) : 0.0f;
                                    part[c] = __fmaf_rn(e, e, part[c]);
                                }
                            }
                        }
                    } else {
                        /* several targets, or affine statistics: per-pass warp reduction into
                         * the warp's shared accumulators tacc[quantity][bank] */
                        const uint32_t nq = prob.mode == EVAL_AFFINE_STATS ? T + 2 : T;
                        for (uint32_t q = 0; q < nq; ++q) {
                            float t[RR];
                            const bool is_target = prob.mode == EVAL_SSE || q >= 2;
                            const uint32_t tcol = prob.num_inputs + (prob.mode == EVAL_SSE ? q : q - 2);
                            if (is_target) m.fetch_row(rowp, rowp, tile_ld, tcol, t);
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
                                    if (prob.mode == EVAL_SSE) { const float e = __fsub_rn(p, t[r]); term = __fmul_rn(e, e); }
                                    else if (q == 0) term = p;
                                    else if (q == 1) term = __fmul_rn(p, p);
                                    else term = __fmul_rn(p, t[r]);
                                    s[c] = __fadd_rn(s[c], ok ? term : 0.0f);
                                }
                            }
#pragma unroll
                            for (int c = 0; c < RC; ++c) {
                                const float total = warp_sum(s[c]);
                                if (lane == 0) tacc[q * RC + c] += total;
                            }
                        }
                    }
                }

                if (prelude) continue;
                if (prob.mode == EVAL_SSE && T == 1) {
                    float mine = 0.0f;
#pragma unroll
                    for (int c = 0; c < RC; ++c) {
                        const float total = warp_sum(part[c]);
                        if (lane == c) mine = total;
                    }
                    const uint32_t bank = bg * RC + lane;
                    if (lane < RC && bank < prob.num_banks) {
                        float* dst = prob.output + gp * prob.out_program_stride + ((size_t)bank << prob.toggle_bits) + perm;
                        atomicAdd(dst, mine); /* result unused: a reduction that never stalls the warp */
                    }
                } else if (!materialize) {
                    __syncwarp();
                    const uint32_t nq = prob.mode == EVAL_AFFINE_STATS ? T + 2 : T;
                    for (uint32_t e = lane; e < nq * RC; e += 32) {
                        const uint32_t q = e / RC, c = e % RC, bank = bg * RC + c;
                        if (bank < prob.num_banks) {
                            float* dst = prob.output + gp * prob.out_program_stride + (size_t)q * prob.out_target_stride +
                                         ((size_t)bank << prob.toggle_bits) + perm;
                            atomicAdd(dst, tacc[e]);
                        }
                    }
                }
            }
        }
    }
}

/* ---- RK4 rollout scoring ---------------------------------------------------------------
 * Restates the integration loop of the reference's generated scoring kernel
 * (projects/odezza/core/o_generate_scoring_cuda.c:494-588): per observation interval
 * h = interval / substeps; per substep base = stage = state, sum = 0, four stages with
 * sum = fma(w, rhs, sum) (w = 1,2,2,1), stage = fma(h/2 or h, rhs, base), then
 * state = fma(h/6, sum, base); after every interval all states must be finite and
 * sq = fma(err, err, sq).  Score = sq / residuals, or FLT_MAX when anything was not finite.
 *
 * Mapping (different from the reference, which gives a thread one configuration and loops all
 * trajectories inside it): one warp per (system, configuration), lanes = trajectories, four
 * per lane.  The integrator's vectors live in the warp's spill slots: slot s = stage state s
 * (what COLUMN s of a right-hand side reads), then next-stage, sum and state vectors (the state
 * is not touched during a step, so it doubles as the step's base).  Warps per CTA are chosen at
 * launch so that as many warps as possible fit the SM's shared memory. */
constexpr int kRk4MaxWarps = 16;

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

__global__ void __launch_bounds__(kRk4MaxWarps * 32, 1)
rk4_kernel(const DeviceBatch batch, const Rk4Problem prob, uint32_t exec_bytes, uint32_t cst_bytes, uint32_t warp_bytes,
           uint32_t scratch_slot) {
    using M = Machine<4, 1>;
    extern __shared__ __align__(16) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t S = prob.num_states, K = prob.num_constants;
    unsigned char* const warea = smem + (size_t)warp * warp_bytes;
    float4* const slots = reinterpret_cast<float4*>(warea + (size_t)S * (exec_bytes + cst_bytes)) + lane;
    const unsigned long long configs = (unsigned long long)prob.num_banks << prob.toggle_bits;
    const unsigned long long item = (unsigned long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= configs * prob.num_systems) return;
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
    M m;
    float sq = 0.0f;
    unsigned long long residuals = 0;
    /* any non-finite time or reference value (NaN excepted where it means "unobserved"), found
     * by the validation kernel, invalidates every score; so do offsets that do not span the data */
    bool ok = *prob.invalid_flag == 0;
    if (ragged) ok = ok && prob.offsets[0] == 0u && prob.offsets[prob.num_trajectories] == prob.total_points;
    for (uint32_t t0 = 0; t0 < prob.num_trajectories; t0 += 128) {
        uint32_t begin[4], npts[4], longest = 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t traj = t0 + lane * 4 + q;
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
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float v = npts[q] ? prob.reference[(size_t)s * prob.reference_ld + begin[q]] : 0.0f;
                ok = ok && (fabsf(v) <= 3.402823466e+38f); /* initial states must be complete and finite */
                m.acc[q][0] = v;
            }
            m.store_slot(slots, STATE + s);
        }
        for (uint32_t k = 1; k < longest; ++k) {
            /* per trajectory step size; a trajectory that has ended keeps integrating with h = 0
             * and is left out of every check and sum */
            float h[4], sixth[4];
            bool act[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                act[q] = k < npts[q];
                const uint32_t at = ragged ? begin[q] + k : k;
                const float interval = act[q] ? prob.times[at] - prob.times[at - 1] : 0.0f;
                const float step = interval / (float)prob.substeps;
                ok = ok && (!act[q] || ((fabsf(interval) <= 3.402823466e+38f) && interval > 0.0f && step > 0.0f));
                h[q] = act[q] ? step : 0.0f;
                sixth[q] = h[q] / 6.0f;
            }
            for (uint32_t sub = 0; sub < prob.substeps; ++sub) {
                for (uint32_t s = 0; s < S; ++s) {
                    m.fetch_slot(slots, STATE + s, m.acc);
                    m.store_slot(slots, STAGE + s);
#pragma unroll
                    for (int q = 0; q < 4; ++q) m.acc[q][0] = 0.0f;
                    m.store_slot(slots, SUM + s);
                }
#pragma unroll 1
                for (int stage = 0; stage < 4; ++stage) {
                    const float weight = (stage == 0 || stage == 3) ? 1.0f : 2.0f;
                    for (uint32_t s = 0; s < S; ++s) {
                        const SbInsn* exec = reinterpret_cast<const SbInsn*>(warea + (size_t)s * exec_bytes);
                        const float* cst = reinterpret_cast<const float*>(warea + (size_t)S * exec_bytes + (size_t)s * cst_bytes);
                        m.run(exec, nullptr, 0, cst, slots, scratch_slot); /* acc = rhs of state s at the stage values */
                        float rhs[4], v[4][1];
#pragma unroll
                        for (int q = 0; q < 4; ++q) rhs[q] = m.acc[q][0];
                        m.fetch_slot(slots, SUM + s, v);
#pragma unroll
                        for (int q = 0; q < 4; ++q) m.acc[q][0] = __fmaf_rn(weight, rhs[q], v[q][0]);
                        m.store_slot(slots, SUM + s);
                        if (stage != 3) {
                            m.fetch_slot(slots, BASE + s, v);
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                m.acc[q][0] = __fmaf_rn(stage == 2 ? h[q] : __fmul_rn(0.5f, h[q]), rhs[q], v[q][0]);
                            m.store_slot(slots, NEXT + s);
                        }
                    }
                    if (stage != 3)
                        for (uint32_t s = 0; s < S; ++s) {
                            m.fetch_slot(slots, NEXT + s, m.acc);
                            m.store_slot(slots, STAGE + s);
                        }
                }
                for (uint32_t s = 0; s < S; ++s) {
                    float sum[4][1], base[4][1];
                    m.fetch_slot(slots, SUM + s, sum);
                    m.fetch_slot(slots, BASE + s, base);
#pragma unroll
                    for (int q = 0; q < 4; ++q) m.acc[q][0] = __fmaf_rn(sixth[q], sum[q][0], base[q][0]);
                    m.store_slot(slots, STATE + s);
                }
            }
            for (uint32_t s = 0; s < S; ++s) { /* all states must be finite before any residual counts */
                m.fetch_slot(slots, STATE + s, m.acc);
#pragma unroll
                for (int q = 0; q < 4; ++q) ok = ok && (!act[q] || fabsf(m.acc[q][0]) <= 3.402823466e+38f);
            }
            for (uint32_t s = 0; s < S; ++s) {
                m.fetch_slot(slots, STATE + s, m.acc);
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (act[q]) {
                        const float ref = prob.reference[(size_t)s * prob.reference_ld + begin[q] + k];
                        if (prob.allow_missing && ref != ref) continue; /* unobserved */
                        const float err = __fsub_rn(m.acc[q][0], ref);
                        sq = __fmaf_rn(err, err, sq);
                        ++residuals;
                    }
            }
        }
    }
    const float total = warp_sum(sq);
    uint32_t lo = (uint32_t)residuals, hi = (uint32_t)(residuals >> 32);
#pragma unroll
    for (int d = 16; d; d >>= 1) {
        const unsigned long long other = ((unsigned long long)__shfl_xor_sync(0xffffffffu, hi, d) << 32) | __shfl_xor_sync(0xffffffffu, lo, d);
        residuals += other;
        lo = (uint32_t)residuals; hi = (uint32_t)(residuals >> 32);
    }
    const bool all_ok = __all_sync(0xffffffffu, ok);
    if (lane == 0) {
        const bool finite = fabsf(total) <= 3.402823466e+38f;
        prob.output[(size_t)sys * prob.output_ld + cfg] = (all_ok && residuals && finite) ? total / (float)residuals : 3.402823466e+38f;
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
            bad = bad || !(fabsf(prob.times[col]) <= 3.402823466e+38f);
        } else {
            const float v = prob.reference[row * prob.reference_ld + col];
            bad = bad || !((fabsf(v) <= 3.402823466e+38f) || (prob.allow_missing && v != v));
        }
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(prob.invalid_flag, 1);
}

template <int RR, int RC>
cudaError_t launch_variant(const DeviceBatch& batch, const EvalProblem& prob, const Geom& geom, const LaunchPlan& plan,
                           cudaStream_t stream) {
    /* approximate math exists for the 16-value tiles, which are the ones the planner picks */
    if (RR * RC <= 16 && prob.fast_math)
        eval_kernel<RR, RC, (RR * RC <= 16)><<<plan.grid_x, plan.warps * 32, plan.smem_bytes, stream>>>(batch, prob, geom);
    else
    eval_kernel<RR, RC, false><<<plan.grid_x, plan.warps * 32, plan.smem_bytes, stream>>>(batch, prob, geom);
    return cudaGetLastError();
}

/* register-tile variants: rows x banks per thread */
constexpr int kNumVariants = 6;
constexpr int kVariantRows[kNumVariants] = {4, 8, 16, 8, 16, 32};
constexpr int kVariantBanks[kNumVariants] = {4, 2, 1, 4, 2, 1};

uint32_t round16(size_t v) { return (uint32_t)((v + 15) / 16 * 16); }

Geom make_geom(const DeviceBatch& batch, const EvalProblem& prob, const LaunchPlan& plan) {
    const int rr = kVariantRows[plan.variant], rc = kVariantBanks[plan.variant];
    const uint32_t ncols = prob.num_inputs + (prob.mode == EVAL_MATERIALIZE ? 0u : prob.num_targets);
    Geom g;
    g.tile_rows = plan.tile_rows;
    g.programs_per_cta = plan.programs_per_cta;
    g.row_splits = plan.row_splits;
    g.exec_bytes = round16(((size_t)batch.max_insn + 1) * sizeof(SbInsn));
    g.cst_bytes = round16(((size_t)prob.num_constants + batch.max_extra) * rc * 4 + 16);
    g.tacc_bytes = round16(((size_t)prob.num_targets + 2) * rc * 4);
    g.scratch_slot = batch.max_slots; /* one slot beyond what the programs use */
    g.hoist_bytes = round16((size_t)batch.max_hoisted * plan.tile_rows * 4);
    g.warp_bytes = g.exec_bytes + g.cst_bytes + g.tacc_bytes + g.hoist_bytes + ((uint32_t)batch.max_slots + 1u) * rr * rc * 128u;
    g.tile_bytes = round16((size_t)ncols * plan.tile_rows * 4);
    g.rows_per_split = plan.rows_per_split;
    g.groups_per_item = plan.groups_per_item ? plan.groups_per_item : 1u;
    return g;
}

}  // namespace

LaunchPlan plan_launch(const DeviceBatch& batch, const EvalProblem& prob, int sm_count, size_t smem_limit, int forced_variant) {
    LaunchPlan plan;
    plan.ok = false;
    plan.groups_per_item = 1;
    int variant = prob.num_banks >= 4 ? 0 : prob.num_banks >= 2 ? 1 : 2;
    uint32_t forced_warps = 0;
    if (forced_variant >= 0) { forced_warps = (uint32_t)forced_variant >> 8; forced_variant &= 0xff; } /* tuning hook */
    if (forced_variant >= 0 && forced_variant < kNumVariants) variant = forced_variant;
    if (prob.mode == EVAL_MATERIALIZE) variant = 2;
    plan.variant = variant;
    const int rr = kVariantRows[variant], rc = kVariantBanks[variant];
    const uint32_t pass = 32u * rr;
    const uint32_t ncols = prob.num_inputs + (prob.mode == EVAL_MATERIALIZE ? 0u : prob.num_targets);

    /* rows staged per chunk: as many passes as fit in about a third of shared memory,
     * never more than the data has */
    const size_t rows_padded = (prob.num_rows + pass - 1) / pass * pass;
    size_t tile_rows = ncols ? (smem_limit / 3) / ((size_t)ncols * 4) / pass * pass : rows_padded;
    if (tile_rows > 4096) tile_rows = 4096 / pass * pass;
    if (tile_rows < pass) tile_rows = pass;
    if (tile_rows > rows_padded) tile_rows = rows_padded;

    /* Warps per CTA: 20 when that costs no tile rows (register budget 96 at 640 threads; measured
     * +8 % over 16 warps, while 22 and 24 warps lose to spills and smaller tiles), else 16, then
     * whatever still fits.  The 32-value tiles need 168 registers and stop at 12 warps. */
    static const uint32_t kSmallTile[] = {20, 16, 12, 8, 4, 2, 1, 0}, kLargeTile[] = {12, 8, 4, 2, 1, 0};
    if (forced_warps > (rr * rc > 16 ? 12u : 20u)) forced_warps = rr * rc > 16 ? 12u : 20u; /* launch bounds */
    const uint32_t forced_list[] = {forced_warps, 0};
    const uint32_t* candidates = forced_warps ? forced_list : (rr * rc > 16 ? kLargeTile : kSmallTile);
    for (; *candidates; ++candidates) {
        const uint32_t warps = *candidates;
        LaunchPlan trial = plan;
        trial.ok = false;
        trial.warps = warps;
        trial.tile_rows = (uint32_t)tile_rows;
        trial.programs_per_cta = 1;
        trial.row_splits = 1;
        trial.rows_per_split = prob.num_rows;
        Geom g = make_geom(batch, prob, trial);
        size_t need = (size_t)g.tile_bytes + 16 + (size_t)g.warp_bytes * warps;
        while (need > smem_limit && trial.tile_rows > pass) {
            trial.tile_rows = (trial.tile_rows / 2 + pass - 1) / pass * pass;
            g = make_geom(batch, prob, trial);
            need = (size_t)g.tile_bytes + 16 + (size_t)g.warp_bytes * warps;
        }
        if (need > smem_limit) continue;
        trial.smem_bytes = need;
        trial.ok = true;
        if (!plan.ok) {
            plan = trial;
            if (warps != 20 || forced_warps) break;
            continue; /* look at 16 warps too */
        }
        if (trial.tile_rows > plan.tile_rows) plan = trial; /* 16 warps keep a larger tile: prefer them */
        break;
    }
    if (!plan.ok) return plan;

    /* Queue items: an item covers up to sixteen bank groups of one permutation, so the prelude of
     * a program is amortised over them, and never straddles permutations (toggles are patched
     * per item). */
    unsigned long long items_per_program = 1;
    if (prob.mode != EVAL_MATERIALIZE) {
        const unsigned long long bank_groups = (prob.num_banks + rc - 1) / rc;
        const unsigned long long cfg_groups = bank_groups << prob.toggle_bits;
        unsigned long long gpi = bank_groups < 16 ? bank_groups : 16;
        while (bank_groups % gpi) --gpi;
        plan.groups_per_item = (uint32_t)gpi;
        items_per_program = cfg_groups / gpi;
    }
    /* Programs per CTA: enough CTAs to fill the machine several times over, and at least
     * 32 queue items per warp so that the warps of a CTA reach the chunk barrier together
     * (measured on the benchmark mix: 8 items per warp 2.06e11 row-evals/s, 16: 2.13, 32: 2.16, 64: 2.18). */
    const uint32_t P = batch.num_programs;
    const uint32_t target_ctas = (uint32_t)sm_count * 8u;
    uint32_t ppc = (P + target_ctas - 1) / target_ctas;
    unsigned long long min_ppc = ((unsigned long long)plan.warps * 32 + items_per_program - 1) / items_per_program;
    if (min_ppc < 4) min_ppc = 4;
    if (ppc < min_ppc) ppc = (uint32_t)min_ppc;
    if (ppc > P) ppc = P;
    while (items_per_program * ppc > 0xfffffff0ull && ppc > 1) ppc /= 2; /* item ids are 32-bit */
    const uint32_t groups = (P + ppc - 1) / ppc;
    plan.programs_per_cta = ppc;
    /* Split the rows across CTAs as well until the grid is many waves deep: a CTA that walks
     * every row of a large dataset runs for seconds, and the last partial wave of such CTAs
     * leaves most of the GPU idle.  Sums are combined with atomic adds either way.  A split
     * keeps at least eight chunks unless the program groups alone cannot fill the GPU. */
    uint32_t splits = 1;
    const size_t chunks = (prob.num_rows + plan.tile_rows - 1) / plan.tile_rows;
    if (prob.mode != EVAL_MATERIALIZE) {
        const uint32_t want_ctas = (uint32_t)sm_count * 32u;
        size_t most = groups < (uint32_t)sm_count * 2u ? chunks : chunks / 8;
        const size_t fill = ((size_t)sm_count * 2 + groups - 1) / groups; /* splits that fill the GPU twice */
        if (most < fill) most = fill < chunks ? fill : chunks;
        splits = (want_ctas + groups - 1) / groups;
        if (splits > most) splits = (uint32_t)most;
        if (splits < 1) splits = 1;
    }
    const size_t chunks_per_split = (chunks + splits - 1) / splits;
    plan.rows_per_split = chunks_per_split * plan.tile_rows;
    plan.row_splits = (uint32_t)((prob.num_rows + plan.rows_per_split - 1) / plan.rows_per_split);
    plan.grid_x = groups * plan.row_splits;
    return plan;
}

#define SB_FOR_VARIANTS(X) X(4, 4) X(8, 2) X(16, 1) X(8, 4) X(16, 2) X(32, 1)

cudaError_t configure_kernels() {
    cudaError_t e;
    int dev = 0, limit = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return e;
#define SB_CONFIGURE(RR, RC) \
    if ((e = cudaFuncSetAttribute(eval_kernel<RR, RC, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, limit)) != cudaSuccess) return e; \
    if (RR * RC <= 16 && (e = cudaFuncSetAttribute(eval_kernel<RR, RC, (RR * RC <= 16)>, cudaFuncAttributeMaxDynamicSharedMemorySize, limit)) != cudaSuccess) return e;
    SB_FOR_VARIANTS(SB_CONFIGURE)
#undef SB_CONFIGURE
    return cudaSuccess;
}

cudaError_t launch_rk4(const DeviceBatch& batch, const Rk4Problem& prob, size_t smem_limit, cudaStream_t stream) {
    const uint32_t exec_bytes = round16(((size_t)batch.max_insn + 1) * sizeof(SbInsn));
    const uint32_t cst_bytes = round16(((size_t)prob.num_constants + batch.max_extra) * 4 + 16);
    const uint32_t scratch_slot = batch.max_slots; /* max_slots already includes the integrator's reserved slots */
    const uint32_t warp_bytes = prob.num_states * (exec_bytes + cst_bytes) + (batch.max_slots + 1u) * 4u * 128u;
    /* warps per CTA: the count that puts most warps on an SM (shared memory per SM is the CTA
     * limit plus 1 KB reserved per resident CTA; the register file holds about 24 warps) */
    int warps = 0, best = 0;
    for (int w = 2; w <= kRk4MaxWarps; ++w) {
        const size_t cta = (size_t)warp_bytes * w;
        if (cta > smem_limit) break;
        int ctas = (int)((smem_limit + 1024) / (cta + 1024));
        if (ctas * w > 24) ctas = 24 / w; /* registers: about 80 per thread */
        if (ctas * w >= best) { best = ctas * w; warps = w; }
    }
    if (!warps) return cudaErrorInvalidConfiguration;
    const size_t smem = (size_t)warp_bytes * warps;
    cudaError_t e = cudaFuncSetAttribute(rk4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_limit);
    if (e != cudaSuccess) return e;
    const unsigned long long items = ((unsigned long long)prob.num_banks << prob.toggle_bits) * prob.num_systems;
    const unsigned long long blocks = (items + warps - 1) / warps;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidConfiguration;
    const size_t values = (size_t)prob.total_points * (prob.num_states + 1);
    rk4_validate_kernel<<<(unsigned)std::min<size_t>(1024, (values + 255) / 256), 256, 0, stream>>>(prob);
    rk4_kernel<<<(unsigned)blocks, warps * 32, smem, stream>>>(batch, prob, exec_bytes, cst_bytes, warp_bytes, scratch_slot);
    return cudaGetLastError();
}

cudaError_t launch_eval(const DeviceBatch& batch, const EvalProblem& prob, const LaunchPlan& plan, cudaStream_t stream) {
    const Geom geom = make_geom(batch, prob, plan);
    switch (plan.variant) {
    case 0: return launch_variant<4, 4>(batch, prob, geom, plan, stream);
    case 1: return launch_variant<8, 2>(batch, prob, geom, plan, stream);
    case 2: return launch_variant<16, 1>(batch, prob, geom, plan, stream);
    case 3: return launch_variant<8, 4>(batch, prob, geom, plan, stream);
    case 4: return launch_variant<16, 2>(batch, prob, geom, plan, stream);
    default: return launch_variant<32, 1>(batch, prob, geom, plan, stream);
    }
}

}  // namespace sb
