"""Regenerate tests/golden/boundary_cases.npz from the reference itself.

Runs every dispatch of `test_oracle_pins.golden_case_list()` through the
reference's own CPU backend (oracle/_ref/libthvm_cpu_ref.so, compiled from the
reference checkout by `make -C oracle ref`) and stores the outputs.  Only needed
when the case list changes; needs the reference checkout.

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path[:0] = [str(ROOT), str(ROOT / "tests")]

import checkers  # noqa: E402
from test_oracle_pins import golden_case_list  # noqa: E402

ref = checkers.Reference.try_load()
if ref is None:
    sys.exit("oracle/_ref/libthvm_cpu_ref.so is not built (reference checkout needed)")
out = {key: ref.run(d) for key, d in golden_case_list()}
np.savez_compressed(ROOT / "tests" / "golden" / "boundary_cases.npz", **out)
print(f"wrote {len(out)} outputs")
