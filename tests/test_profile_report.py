"""Backend.profile_report: per kernel family, launches and device time plus the estimated operations and algorithmic
bytes of its dispatches, with the rates they come to — the figures the reference's Metal backend prints per kernel
(src/backend/metal/profile_kernel.m:45-62, estimates at src/backend/metal/codegen.m:1023-1031).  Profiling is
switched on by THVM_PROFILE at init, so the run is a child process."""
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

CHILD = r"""
import sys
sys.path[:0] = [%r, %r]
import numpy as np
import cases, tinyhvm_b200
be = tinyhvm_b200.CudaBackend()
rng = np.random.default_rng(3)
for d in (cases.chain_fwd_case(rng, 2048, 2048), cases.chain_bwd_case(rng, 2048, 2048), cases.mm_case(rng, 512, 256, 384)):
    for _ in range(2):
        be.run(d)
assert be.last_error() == "", be.last_error()
be.lib.thvm_cuda_profile_report()
be.shutdown()
""" % (str(ROOT), str(ROOT / "tests"))


@pytest.mark.gpu
def test_profile_report_carries_operation_and_byte_estimates():
    import os
    r = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, timeout=600, env={**os.environ, "THVM_PROFILE": "1"})
    assert r.returncode == 0, r.stderr[-2000:]
    rows = {}
    for line in r.stderr.splitlines():
        m = re.match(r"thvm_cuda profile: (\S+)\s+(\d+)\s+([\d.]+)\s+([\d.]+)\s+([\d.]+)\s+([\d.]+)\s+([\d.]+)$", line)
        if m:
            rows[m.group(1)] = [float(x) for x in m.groups()[1:]]
    assert rows, r.stderr[-2000:]
    n = 2048 * 2048
    want = {  # family -> (Gop, GB) of two dispatches
        "reduce_rows_cta": (2 * n * 4 * 1e-9, 2 * (3 * n * 4 + 2048 * 4) * 1e-9),       # mul, add, relu, accumulate
        "ew_flat_static": (2 * n * 4 * 1e-9, 2 * (3 * n * 4 + 4 + n * 4) * 1e-9),              # mul, add, cmp, mul; a, b, c, one 0, g
    }
    for fam, (gop, gb) in want.items():
        assert fam in rows, (fam, sorted(rows))
        launches, ms, got_gop, gflops, got_gb, gbs = rows[fam]
        assert launches >= 2 and ms > 0
        assert abs(got_gop - gop) < 2e-3 and abs(got_gb - gb) < 2e-3, (fam, rows[fam], gop, gb)
        assert gbs == pytest.approx(got_gb / (ms * 1e-3), rel=0.15)          # both printed to three decimals
    mm = [v for k, v in rows.items() if k not in want]            # the contraction's launches, whatever kernels it took
    assert mm, sorted(rows)
    assert abs(sum(v[2] for v in mm) - 2 * 2 * 512 * 256 * 384 * 1e-9) < 2e-3       # mul + accumulate per (m, k, n) point
