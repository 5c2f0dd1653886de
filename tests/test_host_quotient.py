"""The division-free quantisation quotient of the device glue, restated for the host and checked against
rintf(x / s) on operands concentrated on ties (tests/host_checks/quotient_rint_check.c)."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_reciprocal_quotient_with_tie_guard_equals_ieee_division(tmp_path):
    exe = str(tmp_path / "quotient_rint_check")
    src = os.path.join(HERE, "host_checks", "quotient_rint_check.c")
    subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-o", exe, src, "-lm"], check=True)
    out = subprocess.run([exe, "3000", "2000"], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout[-2000:]
    fields = out.stdout.split()
    total, bad, slow = int(fields[1]), int(fields[3]), int(fields[5])
    assert total == 6_000_000 and bad == 0
    assert 0 < slow < total  # the guard fires (ties) but most lanes take the multiplication
