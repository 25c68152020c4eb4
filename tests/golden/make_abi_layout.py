"""Records the struct layouts and key constants of the REFERENCE header
(projects/secant/secant.h) into tests/golden/abi_layout.json.  Needs the reference checkout:

    REF_ROOT=<reference checkout> python tests/golden/make_abi_layout.py
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from abi_probe import probe  # noqa: E402

if "REF_ROOT" not in os.environ:
    sys.exit("set REF_ROOT to the reference checkout")
ref_dir = os.environ["REF_ROOT"] + "/projects/secant"
layout = probe("secant.h", ref_dir)
with open(os.path.join(HERE, "abi_layout.json"), "w") as f:
    json.dump(layout, f, indent=1, sort_keys=True)
print("recorded", len(layout), "entries")
