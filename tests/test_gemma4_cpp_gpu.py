"""Runs the C++ tests of the heterogeneous / shared KV cache owner and of the per-layer decode loop
(tests/cpp/hkv_gemma4_tests.cpp): the reference's own layout known answers, the per-layer plan its
graph emission fixes (owners append, shared layers only attend, window and scale per layer), and a
12-layer local(ring)/global decode with shared layers under one captured graph against the oracle."""
import os
import subprocess

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(REPO, "tests", "cpp", "hkv_gemma4_tests")


def _ensure_built():
    if not os.path.exists(BIN):
        import importlib
        importlib.import_module("hector-engine_b200.build").build_all()
    assert os.path.exists(BIN)


def test_gemma4_tests_binary_links_and_lists_cases():
    _ensure_built()
    out = subprocess.run([BIN, "--list"], capture_output=True, text=True, check=True).stdout.split()
    assert out == ["layout_and_aliases", "layer_plan", "decode_local_global_shared"]


@pytest.mark.gpu
def test_gemma4_cache_and_layered_decode_loop_on_gpu():
    _ensure_built()
    res = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    print(res.stdout, res.stderr)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.count("PASS:") == 3 and "ALL PASSED" in res.stdout
