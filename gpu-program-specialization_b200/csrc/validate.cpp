/*
 * validate.cpp - run-request validation with the reference's order and result codes.
 *
 * Everything here happens before an output bin is cleared or a kernel is launched, as the
 * reference contract requires (projects/secant/secant.h:1142-1149).
 */
#include "internal.h"

#include <algorithm>
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

/* A range of device bytes a request reads or writes. */
struct ByteSpan {
    uintptr_t begin = 0, end = 0;
    bool empty() const { return begin == end; }
    bool meets(const ByteSpan& other) const { return !empty() && !other.empty() && begin < other.end && other.begin < end; }
    /* float32 elements at `address`: null or misaligned -> INVALID_VALUE, wrap-around -> OVERFLOW */
    static SecantResult of(uintptr_t address, size_t elements, ByteSpan* out) {
        out->begin = out->end = address;
        if (!elements) return SECANT_SUCCESS;
        if (!address || address % sizeof(float)) return SECANT_ERROR_INVALID_VALUE;
        size_t bytes;
        if (!mul_ok(elements, sizeof(float), &bytes) || bytes > UINTPTR_MAX - address) return SECANT_ERROR_OVERFLOW;
        out->end = address + bytes;
        return SECANT_SUCCESS;
    }
};

/* What each run shape carries beyond programs, input and output. */
struct ShapeFields { bool targets, banks; size_t struct_bytes; };
bool shape_fields(uint32_t shape, ShapeFields* f) {
    switch (shape) {
    case SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32: *f = ShapeFields{false, false, sizeof(SecantCubinMaterializeRun)}; return true;
    case SECANT_KERNEL_SHAPE_STATIC_SSE_F32:
    case SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32:
    case SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32: *f = ShapeFields{true, false, sizeof(SecantCubinSSERun)}; return true;
    case SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32: *f = ShapeFields{true, true, sizeof(SecantCubinToggleSSERun)}; return true;
    default: return false;
    }
}

/* Configuration count and bank extent of a toggle run (projects/secant/s_toggle_internal.h:52-71),
 * with the per-program table of the extension descriptor. */
SecantResult toggle_extent(const SecantCubinPlan& plan, UnpackedRun* r) {
    if (!r->programs.asts.count || !r->num_banks || r->toggle_bits > 32u || plan.num_constants > SECANT_AST_MAX_INPUTS)
        return SECANT_ERROR_INVALID_VALUE;
    if (!mul_ok(r->num_banks, (size_t)1 << r->toggle_bits, &r->configurations)) return SECANT_ERROR_OVERFLOW;
    if (!plan.num_constants) return r->banks.bank_stride ? SECANT_ERROR_INVALID_VALUE : SECANT_SUCCESS;
    if (r->banks.bank_stride < plan.num_constants) return SECANT_ERROR_INVALID_VALUE;
    if (!span_ok(r->num_banks, r->banks.bank_stride, plan.num_constants, &r->bank_span)) return SECANT_ERROR_OVERFLOW;
    if (r->program_bank_stride) { /* tables of consecutive programs, the first one first_program_index tables in */
        const size_t last = r->first_program_index + r->programs.asts.count - 1;
        size_t lead;
        if (last < r->first_program_index || !mul_ok(last, r->program_bank_stride, &lead) || r->bank_span > SIZE_MAX - lead)
            return SECANT_ERROR_OVERFLOW;
        r->bank_span += lead;
    }
    return SECANT_SUCCESS;
}

}  // namespace

/* Order of checks and result codes of s_run_unpack (projects/secant/s_cubin_runner.c:33-137):
 * header, shape, struct size, shape-specific layout, counts and strides, output geometry, extents
 * against the declared buffer sizes, grid bound. */
SecantResult run_unpack(const SecantCubinPlan& plan, const SecantCubinRunHeader* h, UnpackedRun* out) {
    if (!h || h->struct_size < sizeof(*h) || h->flags) return SECANT_ERROR_INVALID_VALUE;
    if (h->version != SECANT_CUBIN_RUN_VERSION_3) return SECANT_ERROR_UNSUPPORTED_VERSION;
    if (h->shape != plan.shape) return SECANT_ERROR_UNSUPPORTED_SHAPE;
    ShapeFields fields;
    if (!shape_fields(h->shape, &fields)) return SECANT_ERROR_UNSUPPORTED_SHAPE;
    if (h->struct_size < fields.struct_bytes) return SECANT_ERROR_INVALID_VALUE;

    UnpackedRun r;
    /* the three descriptors start alike: header, programs, input; then the members differ */
    if (fields.banks) {
        const auto* v = reinterpret_cast<const SecantCubinToggleSSERun*>(h);
        r.programs = v->programs; r.input = v->input; r.targets = v->targets; r.banks = v->constants; r.output = v->output;
        r.rows = v->num_rows; r.num_targets = v->num_targets; r.num_banks = v->num_banks; r.toggle_bits = v->toggle_bits;
        if (h->struct_size >= sizeof(SecantB200ToggleSSERun)) {
            const auto* x = reinterpret_cast<const SecantB200ToggleSSERun*>(h);
            r.program_bank_stride = x->program_bank_stride;
            r.first_program_index = x->program_bank_stride ? x->first_program_index : 0;
        }
        const SecantResult extent = toggle_extent(plan, &r);
        if (extent != SECANT_SUCCESS) return extent;
        if (r.num_targets != plan.num_targets) return SECANT_ERROR_INVALID_VALUE;
    } else if (fields.targets) {
        const auto* v = reinterpret_cast<const SecantCubinSSERun*>(h);
        r.programs = v->programs; r.input = v->input; r.targets = v->targets; r.output = v->output;
        r.rows = v->num_rows; r.num_targets = v->num_targets;
    } else {
        const auto* v = reinterpret_cast<const SecantCubinMaterializeRun*>(h);
        r.programs = v->programs; r.input = v->input; r.output = v->output; r.rows = v->num_rows;
    }

    const SecantAstProgramSet& set = r.programs;
    const bool programs_ok = set.asts.count && set.asts.items && set.routines.count <= SECANT_AST_MAX_ROUTINES &&
                             (!set.routines.count || set.routines.items);
    const bool targets_ok = r.num_targets <= plan.num_targets && (fields.targets ? r.num_targets != 0 : true);
    const bool strides_ok = (!plan.num_inputs || r.input.leading_dimension >= r.rows) &&
                            (!r.num_targets || r.targets.leading_dimension >= r.rows);
    if (!programs_ok || !r.rows || !targets_ok || !strides_ok) return SECANT_ERROR_INVALID_VALUE;

    /* output: `count` vectors of `width` elements */
    size_t count = set.asts.count, width = 0;
    switch (plan.shape) {
    case SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32: width = r.rows; break;
    case SECANT_KERNEL_SHAPE_STATIC_SSE_F32: width = r.num_targets; break;
    case SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32: width = 2 + r.num_targets; break;
    case SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32: /* one block per cohort of asts_per_kernel programs */
        width = plan.asts_per_kernel * (1 + plan.asts_per_kernel + r.num_targets);
        count = (count + plan.asts_per_kernel - 1) / plan.asts_per_kernel;
        break;
    default: /* toggle: one vector per (program, target) */
        width = r.configurations;
        if (!mul_ok(count, r.num_targets, &count)) return SECANT_ERROR_OVERFLOW;
        break;
    }
    r.output_count = count;
    r.output_width = width;
    if (r.output.leading_dimension > SIZE_MAX / sizeof(float)) return SECANT_ERROR_OVERFLOW;
    if (r.output.leading_dimension < width) return SECANT_ERROR_INVALID_VALUE;
    const bool spans_ok = span_ok(plan.num_inputs, r.input.leading_dimension, r.rows, &r.input_span) &&
                          span_ok(r.num_targets, r.targets.leading_dimension, r.rows, &r.target_span) &&
                          span_ok(count, r.output.leading_dimension, width, &r.output_span);
    if (!spans_ok) return SECANT_ERROR_OVERFLOW;
    if (r.input.num_elements < r.input_span || r.targets.num_elements < r.target_span || r.banks.num_elements < r.bank_span ||
        r.output.num_elements < r.output_span)
        return SECANT_ERROR_INSUFFICIENT_BUFFER;
    /* the reference bounds its grid by INT_MAX row tiles (s_cubin_runner.c:133-136) */
    const size_t tile = fields.targets ? std::max<size_t>(1, plan.tile_rows) : 256;
    if ((r.rows - 1) / tile >= (size_t)INT_MAX) return SECANT_ERROR_OVERFLOW;
    *out = r;
    return SECANT_SUCCESS;
}

/* Cross-entry rules of s_runs_validate (projects/secant/s_cubin_runner.c:195-241): every entry names
 * the same program arrays; inside an entry the four device ranges are disjoint; no entry's output
 * touches anything another entry reads or writes; then the program preflight with the smallest
 * toggle_bits of the batch. */
SecantResult runs_validate(const SecantCubinPlan& plan, const UnpackedRun* runs, size_t count, ProgramRules* rules_ret,
                           bool skip_preflight) {
    const SecantAstProgramSet& programs = runs[0].programs;
    unsigned smallest_bits = 32;
    for (size_t i = 0; i < count; ++i) {
        const UnpackedRun& r = runs[i];
        const bool same_programs = r.programs.asts.items == programs.asts.items && r.programs.asts.count == programs.asts.count &&
                                   r.programs.routines.items == programs.routines.items &&
                                   r.programs.routines.count == programs.routines.count;
        if (!same_programs) return SECANT_ERROR_INVALID_VALUE;
        smallest_bits = std::min<unsigned>(smallest_bits, r.toggle_bits);
        const struct { uintptr_t address; size_t elements; } parts[4] = {
            {r.input.address, r.input_span}, {r.targets.address, r.target_span}, {r.banks.address, r.bank_span},
            {r.output.address, r.output_span}};
        ByteSpan mine[4];
        for (int j = 0; j < 4; ++j) {
            const SecantResult s = ByteSpan::of(parts[j].address, parts[j].elements, &mine[j]);
            if (s != SECANT_SUCCESS) return s;
            for (int k = 0; k < j; ++k)
                if (mine[j].meets(mine[k])) return SECANT_ERROR_INVALID_VALUE;
        }
        for (size_t other = 0; other < count; ++other) {
            if (other == i) continue;
            ByteSpan written;
            const SecantResult s = ByteSpan::of(runs[other].output.address, runs[other].output_span, &written);
            if (s != SECANT_SUCCESS) return s;
            for (const ByteSpan& span : mine)
                if (written.meets(span)) return SECANT_ERROR_INVALID_VALUE;
        }
    }
    ProgramRules rules;
    rules.num_columns = plan.num_inputs;
    rules.num_constants = plan.num_constants;
    rules.banks_allowed = plan.shape == SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32;
    rules.toggle_bits = rules.banks_allowed ? smallest_bits : 0;
    /* records in parts; row-only sub-expressions are worth a prelude as soon as a program is
     * evaluated for more than one bank group (more than two banks: three or four are two groups of
     * the 8 x 2 tile, more are groups of four), and those no toggle reaches as soon as there are
     * toggles (an item then covers several permutations and computes them once) */
    rules.split_parts = true;
    rules.hoist_bank = true;
    rules.hoist_toggled = false;
    if (rules.banks_allowed)
        for (size_t i = 0; i < count; ++i) rules.hoist_toggled = rules.hoist_toggled || runs[i].num_banks > 2;
    rules.hoist_row = rules.hoist_toggled || rules.toggle_bits > 0;
    if (!skip_preflight) {
        const SecantAstProgramList* lists[2] = {&programs.routines, &programs.asts};
        for (const SecantAstProgramList* list : lists)
            for (size_t i = 0; i < list->count; ++i) {
                const SecantResult s = preflight(list->items[i], rules);
                if (s != SECANT_SUCCESS) return s;
            }
    }
    *rules_ret = rules;
    return SECANT_SUCCESS;
}

}  // namespace sb
