/*
 * validate.cpp - run-request validation with the reference's order and result codes.
 *
 * Everything here happens before an output bin is cleared or a kernel is launched, as the
 * reference contract requires (projects/secant/secant.h:1142-1149).
 */
#include "internal.h"

#include <climits>
#include <cstring>

namespace sb {

namespace {

bool mul_ok(size_t a, size_t b, size_t* out) {
    if (a && b > SIZE_MAX / a) return false;
    *out = a * b;
    return true;
}
/* Elements covered by `count` vectors of `width` elements placed `stride` apart
 * (projects/secant/s_toggle_internal.h:44-51); empty shapes span nothing. */
bool span_ok(size_t count, size_t stride, size_t width, size_t* out) {
    size_t lead;
    if (!count || !width) { *out = 0; return true; }
    if (stride < width || !mul_ok(count - 1, stride, &lead) || width > SIZE_MAX - lead) return false;
    *out = lead + width;
    return true;
}

SecantResult byte_range(uintptr_t address, size_t elements, uintptr_t* end) {
    size_t bytes;
    if (!elements) { *end = address; return SECANT_SUCCESS; }
    if (!address || address % sizeof(float)) return SECANT_ERROR_INVALID_VALUE;
    if (!mul_ok(elements, sizeof(float), &bytes) || bytes > UINTPTR_MAX - address) return SECANT_ERROR_OVERFLOW;
    *end = address + bytes;
    return SECANT_SUCCESS;
}

}  // namespace

SecantResult run_unpack(const SecantCubinPlan& plan, const SecantCubinRunHeader* h, UnpackedRun* out) {
    if (!h || h->struct_size < sizeof(*h) || h->flags) return SECANT_ERROR_INVALID_VALUE;
    if (h->version != SECANT_CUBIN_RUN_VERSION_3) return SECANT_ERROR_UNSUPPORTED_VERSION;
    if (h->shape != plan.shape) return SECANT_ERROR_UNSUPPORTED_SHAPE;
    UnpackedRun r;
    switch (h->shape) {
    case SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32: {
        const auto* v = reinterpret_cast<const SecantCubinMaterializeRun*>(h);
        if (h->struct_size < sizeof(*v)) return SECANT_ERROR_INVALID_VALUE;
        r.programs = v->programs; r.input = v->input; r.output = v->output; r.rows = v->num_rows;
        break;
    }
    case SECANT_KERNEL_SHAPE_STATIC_SSE_F32:
    case SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32:
    case SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32: { /* the three static reductions share one layout */
        const auto* v = reinterpret_cast<const SecantCubinSSERun*>(h);
        if (h->struct_size < sizeof(*v)) return SECANT_ERROR_INVALID_VALUE;
        r.programs = v->programs; r.input = v->input; r.output = v->output; r.rows = v->num_rows;
        r.targets = v->targets; r.num_targets = v->num_targets;
        break;
    }
    case SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32: {
        const auto* v = reinterpret_cast<const SecantCubinToggleSSERun*>(h);
        if (h->struct_size < sizeof(*v)) return SECANT_ERROR_INVALID_VALUE;
        r.programs = v->programs; r.input = v->input; r.output = v->output; r.rows = v->num_rows;
        r.targets = v->targets; r.num_targets = v->num_targets;
        r.banks = v->constants; r.toggle_bits = v->toggle_bits; r.num_banks = v->num_banks;
        if (h->struct_size >= sizeof(SecantB200ToggleSSERun)) {
            const auto* x = reinterpret_cast<const SecantB200ToggleSSERun*>(h);
            r.program_bank_stride = x->program_bank_stride;
            r.first_program_index = x->program_bank_stride ? x->first_program_index : 0;
        }
        /* configuration count and bank extent (s_toggle_internal.h:52-71) */
        if (!r.programs.asts.count || !v->num_banks || v->toggle_bits > 32u || plan.num_constants > SECANT_AST_MAX_INPUTS)
            return SECANT_ERROR_INVALID_VALUE;
        if (!mul_ok(v->num_banks, (size_t)1 << v->toggle_bits, &r.configurations)) return SECANT_ERROR_OVERFLOW;
        if (!plan.num_constants) {
            if (r.banks.bank_stride) return SECANT_ERROR_INVALID_VALUE;
            r.bank_span = 0;
        } else {
            if (r.banks.bank_stride < plan.num_constants) return SECANT_ERROR_INVALID_VALUE;
            if (!span_ok(v->num_banks, r.banks.bank_stride, plan.num_constants, &r.bank_span)) return SECANT_ERROR_OVERFLOW;
            if (r.program_bank_stride) {
                size_t lead, last = r.first_program_index + r.programs.asts.count - 1;
                if (last < r.first_program_index || !mul_ok(last, r.program_bank_stride, &lead) || r.bank_span > SIZE_MAX - lead)
                    return SECANT_ERROR_OVERFLOW;
                r.bank_span += lead;
            }
        }
        if (r.num_targets != plan.num_targets) return SECANT_ERROR_INVALID_VALUE;
        break;
    }
    default:
        return SECANT_ERROR_UNSUPPORTED_SHAPE;
    }
    const bool materialize = plan.shape == SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32;
    size_t count = r.programs.asts.count, width;
    if (!count || !r.programs.asts.items || !r.rows || r.programs.routines.count > SECANT_AST_MAX_ROUTINES ||
        (r.programs.routines.count && !r.programs.routines.items) || r.num_targets > plan.num_targets ||
        (!materialize && !r.num_targets) || (plan.num_inputs && r.input.leading_dimension < r.rows) ||
        (r.num_targets && r.targets.leading_dimension < r.rows))
        return SECANT_ERROR_INVALID_VALUE;
    switch (plan.shape) {
    case SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32: width = r.rows; break;
    case SECANT_KERNEL_SHAPE_STATIC_SSE_F32: width = r.num_targets; break;
    case SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32: width = 2 + r.num_targets; break;
    case SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32:
        width = plan.asts_per_kernel * (1 + plan.asts_per_kernel + r.num_targets);
        count = count / plan.asts_per_kernel + (count % plan.asts_per_kernel != 0);
        break;
    default:
        width = r.configurations;
        if (!mul_ok(count, r.num_targets, &count)) return SECANT_ERROR_OVERFLOW;
        break;
    }
    r.output_count = count;
    r.output_width = width;
    if (r.output.leading_dimension > SIZE_MAX / sizeof(float)) return SECANT_ERROR_OVERFLOW;
    if (r.output.leading_dimension < width) return SECANT_ERROR_INVALID_VALUE;
    if (!span_ok(plan.num_inputs, r.input.leading_dimension, r.rows, &r.input_span) ||
        !span_ok(r.num_targets, r.targets.leading_dimension, r.rows, &r.target_span) ||
        !span_ok(count, r.output.leading_dimension, width, &r.output_span))
        return SECANT_ERROR_OVERFLOW;
    if (r.input.num_elements < r.input_span || r.targets.num_elements < r.target_span ||
        r.banks.num_elements < r.bank_span || r.output.num_elements < r.output_span)
        return SECANT_ERROR_INSUFFICIENT_BUFFER;
    /* the reference bounds its grid by INT_MAX row tiles (s_cubin_runner.c:133-136) */
    const size_t tile = materialize ? 256 : (plan.tile_rows ? plan.tile_rows : 1);
    if ((r.rows - 1) / tile >= (size_t)INT_MAX) return SECANT_ERROR_OVERFLOW;
    *out = r;
    return SECANT_SUCCESS;
}

SecantResult runs_validate(const SecantCubinPlan& plan, const UnpackedRun* runs, size_t count, ProgramRules* rules_ret,
                           bool skip_preflight) {
    unsigned bits = 32;
    const SecantAstProgramSet& programs = runs[0].programs;
    for (size_t i = 0; i < count; ++i) {
        const UnpackedRun& r = runs[i];
        const uintptr_t start[4] = {r.input.address, r.targets.address, r.banks.address, r.output.address};
        const size_t size[4] = {r.input_span, r.target_span, r.bank_span, r.output_span};
        uintptr_t end[4];
        if (r.programs.asts.items != programs.asts.items || r.programs.asts.count != programs.asts.count ||
            r.programs.routines.items != programs.routines.items || r.programs.routines.count != programs.routines.count)
            return SECANT_ERROR_INVALID_VALUE;
        if (r.toggle_bits < bits) bits = r.toggle_bits;
        for (int j = 0; j < 4; ++j) {
            const SecantResult s = byte_range(start[j], size[j], end + j);
            if (s != SECANT_SUCCESS) return s;
            for (int k = 0; k < j; ++k)
                if (size[j] && size[k] && start[j] < end[k] && start[k] < end[j]) return SECANT_ERROR_INVALID_VALUE;
        }
        for (size_t j = 0; j < count; ++j) { /* nobody's output may touch anything this entry reads or writes */
            uintptr_t other_end;
            if (j == i) continue;
            const SecantResult s = byte_range(runs[j].output.address, runs[j].output_span, &other_end);
            if (s != SECANT_SUCCESS) return s;
            for (int k = 0; k < 4; ++k)
                if (size[k] && runs[j].output.address < end[k] && start[k] < other_end) return SECANT_ERROR_INVALID_VALUE;
        }
    }
    ProgramRules rules;
    rules.num_columns = plan.num_inputs;
    rules.num_constants = plan.num_constants;
    rules.banks_allowed = plan.shape == SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32;
    rules.toggle_bits = rules.banks_allowed ? bits : 0;
    /* records in three parts; row-only sub-expressions are worth a prelude as soon as a program
     * is evaluated for more than one group of four banks */
    rules.split_parts = true;
    rules.hoist_bank = true;
    rules.hoist_row = false;
    if (rules.banks_allowed)
        for (size_t i = 0; i < count; ++i) rules.hoist_row = rules.hoist_row || runs[i].num_banks > 4;
    for (size_t i = 0; !skip_preflight && i < programs.routines.count; ++i) {
        const SecantResult s = preflight(programs.routines.items[i], rules);
        if (s != SECANT_SUCCESS) return s;
    }
    for (size_t i = 0; !skip_preflight && i < programs.asts.count; ++i) {
        const SecantResult s = preflight(programs.asts.items[i], rules);
        if (s != SECANT_SUCCESS) return s;
    }
    *rules_ret = rules;
    return SECANT_SUCCESS;
}

}  // namespace sb
