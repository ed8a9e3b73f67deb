"""GPU: the library built with -DMG_BOUNDS_CHECK (libmoegen_b200_checked.so, selected with the
MOEGEN_B200_LIB environment variable).  compute-sanitizer cannot run on this pool, so this build is the
memory checker: the row-moving kernels compare every row index they read from a table with the rows of
the buffer it points into.  (1) The small exhaustive parity cases run clean under it.  (2) An index
beyond a declared bound is reported in the device status word and the access is skipped: no fault, no
write outside the bound, the context stays usable."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _checked_env():
    from moe_gen_b200 import build
    env = dict(os.environ)
    env["MOEGEN_B200_LIB"] = build.build_library(checked=True)
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    return env


def test_small_parity_cases_run_clean_under_the_checked_build():
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_parity.py"), "-x", "-q",
                        "-k", "exhaustive or permute_plan or combine_matches or edge_token or emulated or layer_against "
                              "or all_tokens_to_one or forward_host"],
                       env=_checked_env(), cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout


VIOLATION = r"""
import torch
import moe_gen_b200.lib as L
from oracle import moe_oracle as O
from tests.util import make_layer
assert L.LIB_PATH.endswith("_checked.so")
DEV = "cuda:0"
spec = O.LayerSpec(256, 128, 8, 2)
x, W = O.make_inputs(spec, 64, 5)
layer = make_layer(spec, W, DEV)
xd = x.to(DEV)
idx, w = layer.gate_route(xd)[:2]
counts, offsets, pad, dst = layer.permute_plan(idx)
rows = layer.padded_rows(64 * 2)
assert int(dst.max()) >= 256                       # the plan does address rows beyond the bound declared below
layer.set_option(L.OPT_ROWS_BOUND, 256)
perm = layer.permute_rows(xd, dst, rows)           # zero-filled buffer of the full size: nothing can fault
torch.cuda.synchronize()
assert layer.device_status() == (L.DEV_BOUNDS, 103), "scatter beyond the declared rows was not reported"
assert int(perm[256:].abs().sum()) == 0, "a row beyond the declared bound was written"
assert int(perm[:256].abs().sum()) > 0
out_rows = torch.ones(rows, 256, dtype=torch.bfloat16, device=DEV)
y = layer.combine(out_rows, dst, idx, w)
torch.cuda.synchronize()
assert layer.device_status() == (L.DEV_BOUNDS, 104), "gather beyond the declared rows was not reported"
layer.set_option(L.OPT_ROWS_BOUND, 0)              # not declared: the full forward sets its own bound
y = layer.forward(xd)
torch.cuda.synchronize()
assert layer.device_status() == (0, 0)
assert O.rel_l2(y.cpu().float(), O.layer_forward(spec, x, W, gold_fp32=True)["y"]) <= 1e-2
print("VIOLATIONS-REPORTED")
"""


def test_checked_build_reports_an_index_beyond_the_declared_rows():
    r = subprocess.run([sys.executable, "-c", VIOLATION], env=_checked_env(), cwd=ROOT, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0 and "VIOLATIONS-REPORTED" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
