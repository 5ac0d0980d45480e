"""The quantizer kernel divides by E4M3 scales with a reciprocal + two FMAs; this proves on the CPU,
by enumeration, that the sequence equals IEEE division for every such divisor."""
import os
import shutil
import subprocess
import pytest


@pytest.mark.skipif(shutil.which('gcc') is None, reason='gcc not available')
def test_reciprocal_division_is_exact_for_all_e4m3_divisors(tmp_path):
    src = os.path.join(os.path.dirname(__file__), 'exact_division_check.c')
    exe = tmp_path / 'divcheck'
    subprocess.run(['gcc', '-O2', '-mfma', '-ffp-contract=off', '-o', str(exe), src, '-lm'], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout
    assert 'bad3=0 bad5=0' in out.splitlines()[0], out
