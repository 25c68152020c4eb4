"""The C header and the ctypes mirror must match the reference's struct layouts
(projects/secant/secant.h:245-679) recorded in tests/golden/abi_layout.json."""
import ctypes as C
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from abi_probe import STRUCTS, probe  # noqa: E402

from secant_b200 import abi  # noqa: E402

GOLDEN = json.load(open(os.path.join(HERE, "golden", "abi_layout.json")))


def test_header_layout_matches_reference():
    mine = probe("secant_b200.h", os.path.join(os.path.dirname(HERE), "include"))
    assert mine == GOLDEN


def test_ctypes_mirror_matches_reference():
    mirror = {
        "SecantAstProgramList": abi.ProgramList, "SecantAstProgramSet": abi.ProgramSet,
        "SecantDeviceMatrixF32": abi.DeviceMatrix, "SecantHostMatrixF32": abi.HostMatrix,
        "SecantDeviceConstantBanks": abi.DeviceBanks, "SecantConstHostConstantBanks": abi.HostBanks,
        "SecantCubinRecipeHeader": abi.Header, "SecantCubinMaterializeRecipe": abi.MaterializeRecipe,
        "SecantCubinSSERecipe": abi.TiledRecipe, "SecantCubinToggleSSERecipe": abi.ToggleRecipe,
        "SecantCubinMaterializeRun": abi.MaterializeRun, "SecantCubinSSERun": abi.StaticRun,
        "SecantCubinToggleSSERun": abi.ToggleRun, "SecantCpuMaterializeRun": abi.CpuMaterializeRun,
        "SecantCpuSSERun": abi.CpuStaticRun, "SecantCpuGramStatsRun": abi.CpuGramRun,
        "SecantCpuToggleSSERun": abi.CpuToggleRun, "SecantCubinRunnerOptions": abi.RunnerOptions,
        "SecantCubinPlanInfo": abi.PlanInfo, "SecantRunnerStats": abi.RunnerStats,
    }
    for name, cls in mirror.items():
        want = GOLDEN[name]
        assert C.sizeof(cls) == want["sizeof"], name
        for (field, _), cname in zip(cls._fields_, STRUCTS[name]):
            assert getattr(cls, field).offset == want[cname], (name, field)
