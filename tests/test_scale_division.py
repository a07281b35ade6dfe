"""CPU: the quantizer's division-free scale, amax / qmax as a multiplication and a correction
step (csrc/quant_math.cuh), equals the IEEE quotient after the 1e-12 floor. Checked by a small C
program over a strided sweep of all positive floats and over every bf16 and fp16 value; its
stride-1 run (all 2^31 positive floats, under a minute) reports no mismatch either."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("qmax", [448.0, 57344.0])
def test_scale_equals_ieee_quotient(tmp_path, qmax):
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    exe = str(tmp_path / "scale_division_check")
    subprocess.run([gcc, "-O2", "-ffp-contract=off", "-o", exe, os.path.join(HERE, "scale_division_check.c"), "-lm"],
                   check=True)
    r = subprocess.run([exe, str(qmax), "61"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.startswith("mismatches=0 ")
