"""Runs the C++ test of the sequence-split decoder (tests/cpp/hkv_seqsplit_tests.cpp): one process
per GPU (up to 4), the multi-layer step captured once and replayed, outputs against the oracle on
the full logical cache, owner planes bit-exact — once with the NCCL all-gather on the compute stream
and once with the mailbox exchange (plain peer stores). With two or more GPUs the last rank then
leaves between steps and the others must refuse the next step on the host. With one GPU the same
decoder runs as a world of one (no exchange)."""
import os
import subprocess

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(REPO, "tests", "cpp", "hkv_seqsplit_tests")


def _ensure_built():
    if not os.path.exists(BIN):
        import importlib
        importlib.import_module("hector-engine_b200.build").build_all()
    assert os.path.exists(BIN)


def test_seqsplit_tests_binary_links():
    _ensure_built()
    out = subprocess.run([BIN, "--list"], capture_output=True, text=True, check=True).stdout.split()
    assert out == ["seqsplit_decoder"]


@pytest.mark.gpu
def test_seqsplit_decoder_cpp_on_gpu():
    _ensure_built()
    res = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    print(res.stdout, res.stderr)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "ALL PASSED" in res.stdout and "FAIL" not in res.stdout
