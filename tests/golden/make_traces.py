"""Regenerate the committed step traces under tinyhvm_b200/traces/.

Runs the staged LeNet and VGG-style drivers of oracle/ref_host_cnn.c on the reference's own
host runtime with the dry recording backend (oracle/ref_trace.c: every vtable call is logged,
no dispatch is executed, so a full-size step records in well under a second) for the
per-process batch sizes of the 1/2/4/8-GPU data-parallel runs (global batch 1024 for LeNet,
512 for the VGG-style net).  Needs oracle/_ref/libthvm_host_ref.so, i.e. the reference
checkout at build time.

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
from tinyhvm_b200 import configs  # noqa: E402

OUT = ROOT / "tinyhvm_b200" / "traces"
OUT.mkdir(exist_ok=True)
STEPS = 3


def record(name, driver, head, tail):
    with tempfile.TemporaryDirectory() as td:
        raw = Path(td) / "t.thtr"
        hostref.run(driver, str(raw), 1, *head, STEPS, 0.01, *tail)
        with open(raw, "rb") as f, open(OUT / f"{name}.thtr.gz", "wb") as o, \
                gzip.GzipFile(filename="", fileobj=o, mode="wb", compresslevel=9, mtime=0) as g:     # no timestamp: reruns are byte-identical
            shutil.copyfileobj(f, g)
    print(f"{name}: {(OUT / f'{name}.thtr.gz').stat().st_size} bytes")


ps = np.concatenate(configs.lenet_params())
for B in (1024, 512, 256, 128):
    record(f"lenet_b{B}", "drv_record_lenet", (B,), (np.zeros(STEPS * B * 784, np.float32), np.zeros(STEPS * B, np.uint8), ps))
ps = np.concatenate(configs.vgg_params())
chan = np.array(configs.VGG_CHAN, np.uint32)
for B in (512, 256, 128, 64):
    record(f"vgg_b{B}", "drv_record_vgg", (B, 64, 100, chan),
           (np.zeros(STEPS * B * 3 * 64 * 64, np.float32), np.zeros(STEPS * B, np.uint8), ps))
