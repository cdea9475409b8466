"""Regenerate the committed step traces under tinyhvm_b200/traces/.

Runs the staged LeNet driver of oracle/ref_host.c on the reference's own host runtime
with the dry recording backend (oracle/ref_trace.c: every vtable call is logged, no
dispatch is executed, so a full-size step records in well under a second) for the
per-process batch sizes of the 1/2/4/8-GPU data-parallel runs (global batch 1024).
Needs oracle/_ref/libthvm_host_ref.so, i.e. the reference checkout at build time.

    python tests/golden/make_traces.py
"""
import gzip
import shutil
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path[:0] = [str(ROOT), str(ROOT / "tests")]

import hostref  # noqa: E402
from test_host_dropin import lenet_inputs  # noqa: E402

OUT = ROOT / "tinyhvm_b200" / "traces"
OUT.mkdir(exist_ok=True)
STEPS = 3
_, _, ps = lenet_inputs(8, 1)
for B in (1024, 512, 256, 128):
    x = np.zeros(STEPS * B * 784, np.float32)
    lab = np.zeros(STEPS * B, np.uint8)
    with tempfile.TemporaryDirectory() as td:
        raw = Path(td) / "t.thtr"
        hostref.run("drv_record_lenet", str(raw), 1, B, STEPS, 0.01, x, lab, np.concatenate(ps))
        with open(raw, "rb") as f, gzip.open(OUT / f"lenet_b{B}.thtr.gz", "wb", compresslevel=9) as g:
            shutil.copyfileobj(f, g)
    print(f"lenet_b{B}: {(OUT / f'lenet_b{B}.thtr.gz').stat().st_size} bytes")
