"""Host-side failure detection of the multi-GPU decode step (host/hkv_step_watch.hpp), tested
without any GPU: the failures are made on the host. The C++ cases (tests/cpp/hkv_watch_tests.cpp)
use threads and forked processes as ranks: a step that never completes times out, a communicator
error ends the wait, a rank that leaves between steps or never joins is seen before the next launch."""
import os
import subprocess

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(REPO, "tests", "cpp", "hkv_watch_tests")


def test_step_watch_and_roster_cases():
    if not os.path.exists(BIN):
        import importlib
        importlib.import_module("hector-engine_b200.build").build_watch_tests()
    res = subprocess.run([BIN], capture_output=True, text=True, timeout=120)
    print(res.stdout, res.stderr)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.count("PASS:") == 5 and "ALL PASSED" in res.stdout
