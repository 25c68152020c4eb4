/*
 * planner.cpp - launch geometry of the population evaluator: register-tile variant, warps per
 * CTA, staged tile size, programs per CTA, row splits, and the shared-memory layout that follows.
 * Host-only arithmetic, so the CPU test-suite can check its bounds without a device.
 *
 * The reference sizes its launches from the recipe (projects/secant/s_runner_pipeline.c:259-283:
 * grid = row tiles x configuration blocks).  Here a CTA owns a set of programs and a range of
 * rows; it walks the range tile by tile and its warps take (program, permutation) items from a
 * queue for every tile.
 */
#include "evaluator.cuh"

#include <algorithm>

namespace sb {

namespace {

uint32_t round16(size_t v) { return (uint32_t)((v + 15) / 16 * 16); }

uint32_t quantities(const EvalProblem& prob) {
    return prob.mode == EVAL_AFFINE_STATS ? prob.num_targets + 2u : prob.num_targets;
}

}  // namespace

Geom make_geom(const DeviceBatch& batch, const EvalProblem& prob, const LaunchPlan& plan) {
    const uint32_t rr = (uint32_t)kVariantRows[plan.variant], rc = (uint32_t)kVariantBanks[plan.variant];
    const uint32_t ncols = prob.num_inputs + (prob.mode == EVAL_MATERIALIZE ? 0u : prob.num_targets);
    const uint32_t gpi = plan.groups_per_item ? plan.groups_per_item : 1u;
    const uint32_t ppi = plan.perms_per_item ? plan.perms_per_item : 1u;
    const uint32_t slots = batch.max_slots + (batch.uses_scratch ? 1u : 0u);
    Geom g;
    g.tile_rows = plan.tile_rows;
    g.tile_buffers = plan.tile_buffers;
    g.tile_bytes = round16((size_t)ncols * plan.tile_rows * 4);
    g.num_groups = plan.num_groups;
    g.row_splits = plan.row_splits;
    g.groups_per_item = gpi;
    g.perms_per_item = ppi;
    g.exec_bytes = round16(((size_t)batch.max_insn + 1) * sizeof(SbInsn));
    g.table_bytes = round16((size_t)std::max<uint32_t>(1u, ppi * gpi * batch.max_cst * rc) * 4);
    g.hoist_bytes = round16((size_t)batch.max_hoisted * 32u * rr * 4);
    g.slot_bytes = round16(std::max<size_t>((size_t)slots * rr * rc * 128u, (size_t)batch.max_btmp * 128u));
    g.psum_bytes = round16((size_t)std::max<uint32_t>(1u, quantities(prob) * ppi * gpi * rc) * 4);
    g.warp_bytes = g.exec_bytes + g.table_bytes + g.hoist_bytes + g.slot_bytes + g.psum_bytes;
    g.scratch_slot = batch.max_slots; /* one slot beyond what the programs use */
    g.rows_per_split = plan.rows_per_split;
    return g;
}

namespace {

LaunchPlan plan_with_tile(const DeviceBatch& batch, const EvalProblem& prob, int sm_count, size_t smem_limit, size_t scratch_limit,
                          int variant) {
    LaunchPlan plan{};
    plan.ok = false;
    plan.overflow = false;
    plan.groups_per_item = 1;
    plan.perms_per_item = 1;
    plan.variant = variant;
    const uint32_t rr = (uint32_t)kVariantRows[variant], rc = (uint32_t)kVariantBanks[variant];
    const uint32_t pass = 32u * rr;
    const uint32_t nq = std::max<uint32_t>(1u, quantities(prob));
    const bool materialize = prob.mode == EVAL_MATERIALIZE;
    const uint32_t P = batch.num_programs;
    if (!P || !prob.num_rows || sm_count <= 0) return plan;

    /* Queue items: an item covers up to sixteen bank groups of one permutation, so the bank part and
     * the row prelude of a program are amortised over them; it never straddles permutations (toggles
     * are patched per item).  Fewer groups per item when the constant table or the partial sums of
     * sixteen groups would crowd out the tile. */
    unsigned long long items_per_program = 1;
    if (!materialize) {
        const unsigned long long bank_groups = (prob.num_banks + rc - 1) / rc;
        unsigned long long gpi = std::min<unsigned long long>(bank_groups, 16);
        for (;; --gpi) {
            if (bank_groups % gpi) continue;
            if (gpi == 1 || (gpi * batch.max_cst * rc * 4 <= 2048 && gpi * nq * rc * 4 <= 2048)) break;
        }
        plan.groups_per_item = (uint32_t)gpi;
        if (prob.toggle_bits > 40 || (bank_groups / gpi) > (~0ull >> prob.toggle_bits)) { plan.overflow = true; return plan; }
        /* An item that holds every bank group of its permutation may go on to the next permutations, up
         * to sixteen (permutation, bank group) pairs within the same table and partial-sum budgets: the
         * program is fetched once for them and its toggle-free row prelude runs once per row pass. */
        unsigned long long ppi = 1;
        if (gpi == bank_groups)
            while (ppi * 2 * gpi <= 16 && ppi * 2 <= (1ull << prob.toggle_bits) && ppi * 2 * gpi * batch.max_cst * rc * 4 <= 2048 &&
                   ppi * 2 * gpi * nq * rc * 4 <= 2048)
                ppi *= 2;
        plan.perms_per_item = (uint32_t)ppi;
        items_per_program = ((bank_groups / gpi) << prob.toggle_bits) / ppi;
    }
    /* item ids are 32-bit and every warp draws one id past the end */
    const unsigned long long kMaxItems = 0xffffff00ull;
    if (items_per_program > kMaxItems) { plan.overflow = true; return plan; }

    /* Warps per CTA and rows per tile.  20 warps run at a 96-register budget; a tile of at least
     * 512 rows keeps the per-item set-up (program copy, toggle patches, bank part) small against
     * the row passes, so fewer warps are preferred over a smaller tile down to 256 rows. */
    static const uint32_t warp_list[] = {20, 16, 12, 8, 4, 2, 1, 0};
    const uint32_t widest_tile = 1024;
    const size_t rows_padded = (prob.num_rows + pass - 1) / pass * pass;
    const uint32_t floors[3] = {512u, 256u, pass};
    for (int attempt = 0; attempt < 3 && !plan.ok; ++attempt) {
        const size_t floor_rows = std::min<size_t>(std::max<uint32_t>(floors[attempt], pass), rows_padded);
        for (const uint32_t* w = warp_list; *w && !plan.ok; ++w) {
            for (uint32_t want = widest_tile; want >= pass; want /= 2) {
                size_t tile_rows = std::min<size_t>(std::max<uint32_t>(want, pass) / pass * pass, rows_padded);
                if (tile_rows < floor_rows) break;
                LaunchPlan trial = plan;
                trial.warps = *w;
                trial.tile_rows = (uint32_t)tile_rows;
                trial.tile_buffers = rows_padded > tile_rows ? 2u : 1u;
                trial.num_groups = 1;
                trial.row_splits = 1;
                trial.rows_per_split = prob.num_rows;
                const Geom g = make_geom(batch, prob, trial);
                const size_t need = (size_t)g.tile_bytes * g.tile_buffers + 16 + (size_t)g.warp_bytes * trial.warps;
                if (need > smem_limit) continue;
                plan = trial;
                plan.smem_bytes = need;
                plan.ok = true;
                break;
            }
        }
    }
    if (!plan.ok) return plan;
    plan.ok = false;

    /* Programs per CTA: at least eight queue items per warp and tile.  Programs arrive sorted by
     * cost and group g takes programs g, g + num_groups, ..., so every CTA's queue runs from its
     * costliest item to its cheapest and the warps reach the end of a tile close together. */
    unsigned long long want_items = 8ull * plan.warps;
    unsigned long long per_cta = (want_items + items_per_program - 1) / items_per_program;
    per_cta = std::max<unsigned long long>(1, std::min<unsigned long long>(per_cta, P));
    unsigned long long groups = std::max<unsigned long long>(1, P / per_cta);
    groups = std::min<unsigned long long>(groups, (unsigned long long)sm_count * 16ull);
    /* keep a CTA's item count inside 32 bits */
    while (((P + groups - 1) / groups) * items_per_program > kMaxItems && groups < P) groups = std::min<unsigned long long>(P, groups * 2);
    if (((P + groups - 1) / groups) * items_per_program > kMaxItems) { plan.overflow = true; return plan; }
    plan.num_groups = (uint32_t)groups;

    /* Rows are split across CTAs until the grid is many waves deep: a CTA that walks every row of
     * a large dataset runs for seconds and the last partial wave of such CTAs leaves most of the GPU
     * idle.  Each split keeps at least four tiles unless the program groups alone cannot fill the GPU. */
    const size_t tiles = (prob.num_rows + plan.tile_rows - 1) / plan.tile_rows;
    size_t want_ctas = (size_t)sm_count * 16;
    size_t most = groups >= (unsigned long long)sm_count * 2ull ? std::max<size_t>(1, tiles / 4) : tiles;
    size_t splits = std::min<size_t>(most, (want_ctas + (size_t)groups - 1) / (size_t)groups);
    splits = std::max<size_t>(1, splits);
    if (groups * splits < (unsigned long long)sm_count) { /* a small run: fewer programs per CTA rather than idle SMs */
        groups = std::min<unsigned long long>(P, ((unsigned long long)sm_count + splits - 1) / splits);
        plan.num_groups = (uint32_t)groups;
    }
    const unsigned long long configs = (unsigned long long)prob.num_banks << prob.toggle_bits;
    if (!materialize && configs) { /* [split][program][quantity][configuration] floats of scratch */
        const unsigned long long per_split = (unsigned long long)P * nq;
        if (per_split > (~0ull >> 3) / configs) { plan.overflow = true; return plan; }
        const unsigned long long fit = std::max<unsigned long long>(1, (unsigned long long)scratch_limit / (per_split * configs));
        splits = (size_t)std::min<unsigned long long>(splits, fit);
    }
    const size_t tiles_per_split = (tiles + splits - 1) / splits;
    plan.rows_per_split = tiles_per_split * plan.tile_rows;
    plan.row_splits = (uint32_t)((prob.num_rows + plan.rows_per_split - 1) / plan.rows_per_split);
    if (tiles_per_split == 1) plan.tile_buffers = 1; /* smem_bytes stays an upper bound */
    const unsigned long long grid = groups * plan.row_splits;
    if (grid > 0x7fffffffull) { plan.overflow = true; return plan; }
    plan.grid_x = (uint32_t)grid;

    plan.partial_elements = 0;
    if (!materialize) {
        const unsigned long long n = (unsigned long long)plan.row_splits * P;
        if (configs && n > (~0ull >> 3) / configs / nq) { plan.overflow = true; return plan; }
        plan.partial_elements = (size_t)(n * nq * configs);
    }
    plan.ok = true;
    return plan;
}

}  // namespace

LaunchPlan plan_launch(const DeviceBatch& batch, const EvalProblem& prob, int sm_count, size_t smem_limit, size_t scratch_limit) {
    /* register tile: 4 rows x 4 banks per thread, or 8 x 2 / 16 x 1 when there are fewer banks.  Up
     * to four banks take the 8 x 2 tile: three or four banks are then two bank groups, so the row
     * prelude serves two runs of the main part and computes each row's value twice instead of four
     * times (measured on 4 banks x 256 permutations: 10 % faster than one 4 x 4 group; with 16 banks
     * and more the 4 x 4 tile is as fast or faster).  A tile with more rows per thread stages more
     * rows per pass; when even one pass of a wide dataset does not fit shared memory, the tiles with
     * fewer rows are tried (their spare bank columns compute padding that is never written). */
    int variant = prob.num_banks > 4 ? 0 : prob.num_banks >= 2 ? 1 : 2;
    if (prob.mode == EVAL_MATERIALIZE) variant = 2;
    LaunchPlan plan{};
    for (; variant >= 0; --variant) {
        plan = plan_with_tile(batch, prob, sm_count, smem_limit, scratch_limit, variant);
        if (plan.ok || plan.overflow) break;
    }
    return plan;
}

}  // namespace sb
