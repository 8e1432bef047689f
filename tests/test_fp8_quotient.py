"""The E4M3 quantisers divide without a division: reciprocal of the scale + two FMA corrections.  This CPU check
compiles oracle/quotient_check.c (the same arithmetic with libm's fmaf) and compares it with the IEEE quotient over
every bf16 dividend for hundreds of scales, over millions of random fp32 dividends, and - for scales a caller
gives, which may be tiny - over the rule that sends scales outside [1e-12, 3e38] to a real division.  Mode 3 does the same
for the NVFP4 block scale (m / 6 / gs without a division: every bf16 block maximum and random fp32 ones, hundreds of
global scales)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def checker(tmp_path_factory):
    exe = tmp_path_factory.mktemp("quotient") / "quotient_check"
    # -ffp-contract=off: the compiler must not fuse or re-associate the reference expression x / s or the products
    subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-o", str(exe), os.path.join(ROOT, "oracle", "quotient_check.c"), "-lm"],
                   check=True)
    return str(exe)


@pytest.mark.parametrize("scales,mode", [(600, 0), (4000, 1), (2000, 2), (600, 3)])
def test_fma_corrected_quotient_equals_division(checker, scales, mode):
    out = subprocess.run([checker, str(scales), str(mode)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    words = out.stdout.split()
    assert int(words[1]) > 1_000_000 and int(words[3]) == 0
