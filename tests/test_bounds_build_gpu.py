"""The bounds-checking build of the library (-DKCG_DEBUG_BOUNDS, libkcg_b200_bounds.so): ragged
problems through every kernel variant run clean under it, and its reporting path -- record the
offset, skip the access, finish the kernel -- is exercised by capping the extent the kernels
check against on a buffer that is in fact large enough, so no real out-of-bounds access, fault
or trap is ever produced.  The child process selects the build through KCG_DEBUG_BOUNDS=1."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def report(cuda_device):
    from kernelcodegen_b200 import build

    build.build_bounds()
    env = dict(os.environ, KCG_DEBUG_BOUNDS="1")
    res = subprocess.run([sys.executable, str(ROOT / "tests" / "_bounds_child.py")], env=env, stdout=subprocess.PIPE,
                         stderr=subprocess.PIPE, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    return json.loads(res.stdout.strip().splitlines()[-1])


def test_ragged_cases_run_clean_under_the_bounds_build(report):
    assert report["enabled"] == 1
    assert len(report["cases"]) >= 7
    for case in report["cases"]:
        assert case["status"] == 0, case
        assert case["err"] <= case["tol"], case


def test_a_failed_check_is_reported_and_the_access_skipped(report):
    cap = report["capped"]
    assert cap["status"] == 10                       # DEV_BOUNDS
    assert cap["extent"] == cap["cap"] and cap["offset"] + 16 > cap["cap"]
    assert cap["below_cap_err"] <= 1e-4              # everything inside the extent was written
    assert cap["beyond_cap_untouched"]               # everything outside it was skipped, not stored
    assert report["after"]["status"] == 0 and report["after"]["err"] <= 1e-4


def test_the_normal_build_has_the_checks_compiled_out(native_lib):
    assert native_lib.kcg_debug_bounds_enabled() == 0
