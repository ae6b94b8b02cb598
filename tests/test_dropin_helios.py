"""Drop-in test at the REAL engine's registry boundary: oracle/_ref/hkv_dropin_helios links the
reference's own engine core and kernels (built from the reference checkout by
`make -C oracle dropin`), installs libhkv's ops over them and replays the reference's
known-answer command buffers and its capture-once decode loop (see tests/cpp/hkv_dropin_helios.cpp)."""
import os
import subprocess

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(REPO, "oracle", "_ref", "hkv_dropin_helios")


@pytest.mark.gpu
def test_libhkv_ops_inside_the_real_engine():
    if not os.path.exists(BIN):
        pytest.skip("oracle/_ref/hkv_dropin_helios was not built (reference checkout absent at build time)")
    res = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    print(res.stdout, res.stderr)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.count("PASS:") == 3 and "ALL PASSED" in res.stdout
