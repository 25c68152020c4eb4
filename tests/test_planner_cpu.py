"""Launch geometry of the evaluator (csrc/planner.cpp) checked without a device, through the
host-only test hooks: shared-memory fit, the 32-bit item index bound, the scratch cap, the
fall-back to narrower register tiles for wide datasets."""
import ctypes as C

import pytest

import support as S

SMEM = 232448          # opt-in shared memory per block of a B200, bytes
FIELDS = "variant warps tile_rows buffers groups gpi splits rows_per_split smem partial grid warp_bytes items ppi".split()
SSE, MATERIALIZE, AFFINE = 0, 1, 2


def plan(programs, rows, banks=64, bits=0, inputs=8, targets=1, mode=SSE, insn=80, slots=2, hoisted=4, table=8, btmp=3,
         sms=148, smem=SMEM, scratch=1 << 28):
    out = (C.c_uint64 * 14)()
    code = S.hooks().sbt_plan(programs, insn, slots, hoisted, table, btmp, mode, inputs, targets, banks, bits, C.c_uint64(rows), sms,
                              C.c_uint64(smem), C.c_uint64(scratch), out)
    return code, dict(zip(FIELDS, list(out)))


def test_headline_shape_fills_the_machine():
    code, p = plan(16384, 1 << 20)
    assert code == 1 and p["variant"] == 0 and p["warps"] == 20 and p["gpi"] == 16
    assert p["smem"] <= SMEM and p["tile_rows"] % 128 == 0 and p["buffers"] == 2
    assert p["grid"] == p["groups"] * p["splits"] >= 148 * 8
    assert p["items"] >= 8 * p["warps"]                        # queue items per CTA and tile
    assert p["partial"] == p["splits"] * 16384 * 64
    assert p["rows_per_split"] % p["tile_rows"] == 0 and p["rows_per_split"] * p["splits"] >= 1 << 20


def test_items_span_permutations_when_one_item_holds_every_bank():
    """Four coefficient sets are two bank groups of the 8 x 2 tile, so an item goes on over eight
    permutations (the program is fetched once for them); with sixteen bank groups per item there
    is no room, and the tables of long programs shrink the span."""
    code, p = plan(16384, 1 << 18, banks=4, bits=8, inputs=6, table=8)
    assert code == 1 and p["variant"] == 1 and p["gpi"] == 2 and p["ppi"] == 8
    assert p["items"] == -(-16384 // p["groups"]) * (256 // 8)
    code, p = plan(16384, 1 << 18, banks=2, bits=8, inputs=6, table=8)          # one group of the 8 x 2 tile
    assert code == 1 and p["variant"] == 1 and p["gpi"] == 1 and p["ppi"] == 16
    assert plan(16384, 1 << 18, banks=64, bits=8)[1]["ppi"] == 1
    assert plan(16384, 1 << 18, banks=8, bits=8)[1]["ppi"] == 8                # two bank groups per permutation
    assert plan(16384, 1 << 18, banks=4, bits=2)[1]["ppi"] == 4                # no more permutations than there are
    assert plan(16384, 1 << 18, banks=4, bits=8, table=24)[1]["ppi"] == 4      # 24 entries x 16 bytes x 4 = 1,536 bytes of tables
    assert plan(16384, 1 << 18, banks=4, bits=0)[1]["ppi"] == 1


def test_scratch_cap_trades_row_splits_for_memory():
    _, free = plan(2048, 1 << 18)
    _, capped = plan(2048, 1 << 18, scratch=3 * 2048 * 64)
    _, one = plan(2048, 1 << 18, scratch=1)
    assert free["splits"] > capped["splits"] == 3 and one["splits"] == 1
    assert capped["partial"] <= 3 * 2048 * 64 and one["partial"] == 2048 * 64


def test_item_index_stays_inside_32_bits():
    """toggle_bits up to 32 is a valid request (projects/secant/s_toggle_internal.h:52-71); the
    queue's item ids are 32-bit, so such runs are refused with OVERFLOW instead of being launched
    (a wrapped counter would never reach the end of the queue).  An item covers up to sixteen
    (permutation, bank group) pairs, so the bound is reached with many banks."""
    assert plan(1, 1000, banks=64, bits=32)[0] == -1           # 2^32 items of sixteen bank groups
    assert plan(1, 1000, banks=128, bits=31)[0] == -1
    code, p = plan(1, 1000, banks=4, bits=32)                  # two bank groups: eight permutations per item
    assert code == 1 and p["ppi"] == 8 and p["items"] == 1 << 29
    code, p = plan(1, 1000, banks=2, bits=32)                  # one bank group: sixteen permutations per item
    assert code == 1 and p["ppi"] == 16 and p["items"] == 1 << 28
    code, p = plan(1, 1000, banks=64, bits=31)
    assert code == 1 and p["ppi"] == 1 and p["items"] == 1 << 31 and p["items"] + 20 < 1 << 32
    code, p = plan(64, 1000, banks=64, bits=28)                # many programs: fewer per CTA, never a wrapped count
    assert code == 1 and p["items"] + 20 < 1 << 32 and p["groups"] >= 4
    code, p = plan(100000, 1000, banks=64, bits=31)
    assert code == 1 and p["groups"] == 100000 and p["items"] == 1 << 31


@pytest.mark.parametrize("mode,targets", [(SSE, 1), (SSE, 2), (MATERIALIZE, 0), (AFFINE, 1)])
def test_widest_datasets_fall_back_to_narrower_tiles(mode, targets):
    """128 columns x one 512-row pass of the 16 x 1 tile is more than shared memory holds; the
    4 x 4 tile (128-row passes) still fits."""
    inputs = 128 - (targets if mode != MATERIALIZE and targets > 1 else 0)
    code, p = plan(20, 300, banks=1, inputs=inputs, targets=targets, mode=mode, hoisted=0, table=4, slots=1)
    assert code == 1 and p["variant"] == 0 and p["smem"] <= SMEM and p["tile_rows"] >= 128
    code, narrow = plan(20, 300, banks=1, inputs=16, targets=targets, mode=mode, hoisted=0, table=4, slots=1)
    assert code == 1 and narrow["variant"] == 2


def test_batches_that_cannot_fit_are_reported_not_launched():
    assert plan(10, 1000, slots=48, hoisted=4, table=200, smem=49152)[0] == 0   # a device without the large opt-in carve-out
    code, p = plan(10, 1000, slots=48, hoisted=4, table=200)   # the encoder's slot limit still runs, on two warps
    assert code == 1 and p["warps"] <= 2 and p["smem"] <= SMEM
    code, p = plan(10, 1000, slots=12, hoisted=4, table=40)     # large working set: fewer warps, still a plan
    assert code == 1 and p["warps"] < 20 and p["smem"] <= SMEM


def test_small_runs_spread_over_the_machine():
    code, p = plan(129, 97, banks=5, bits=8)                    # the reference's random GPU case (toggle_cuda_test.c:535-659)
    assert code == 1 and p["grid"] >= 100 and p["buffers"] == 1 and p["tile_rows"] == 128
