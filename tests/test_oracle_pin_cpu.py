"""Pins the CPU oracle against the reference's own unit tests: the reference's unmodified Python
layer and unmodified unittests/ run on device="cpu" over the oracle's stand-in for the native
module (oracle/pin_against_reference.py).  Needs the reference tree, which only exists in the
build container; skipped elsewhere.  Set ASH_REFERENCE_ROOT to point at another checkout."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# default: a checkout named "reference" beside this repository
REF = os.environ.get("ASH_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "unittests")), reason="reference tree not available")
def test_reference_unit_tests_pass_on_the_oracle(tmp_path):
    # the reference's tests write their checkpoint files into the working directory
    out = subprocess.run(
        [sys.executable, os.path.join(ROOT, "oracle", "pin_against_reference.py"), "--fast", REF],
        capture_output=True, text=True, timeout=1500, cwd=tmp_path)
    lines = [l for l in out.stdout.splitlines() if l.startswith(("ok", "FAIL", "PIN"))]
    assert out.returncode == 0 and lines and lines[-1] == "PIN PASSED", "\n".join(lines[-40:]) + out.stderr[-2000:]
    assert sum(l.startswith("ok") for l in lines) >= 28
