"""The index-checking build of the library (every point index read from a sorted list is range-checked
before it is used for a gather; violations are counted and reported, the access is skipped) must run the
parity tests clean: a stand-in for a memory checker on machines where none can be run."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_parity_tests_pass_with_the_checked_library():
    from inpc_b200 import _build
    if not _build.LIB_CHECKED.exists():
        pytest.skip("libinpc_b200_checked.so has not been built (python -m inpc_b200._build --checked)")
    env = dict(os.environ, INPC_B200_LIB=str(_build.LIB_CHECKED))
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", str(ROOT / "tests" / "test_gpu_raster.py"),
           str(ROOT / "tests" / "test_gpu_rows.py"), str(ROOT / "tests" / "test_gpu_fuzz.py"), "-k",
           "not full_size and not checked"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout
