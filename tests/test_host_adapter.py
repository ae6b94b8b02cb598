"""Runs the C++ tests of the registry-boundary adapter (tests/cpp/hkv_host_tests.cpp): the
reference's known answers as command buffers, the CUDA-graph capture-once contract, the fused
five-input op, error behaviour, the C++ cache owner and the batched decode loop (sessions joining and
leaving batch slots under one captured graph)."""
import os
import subprocess

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(REPO, "tests", "cpp", "hkv_host_tests")


def _ensure_built():
    if not os.path.exists(BIN):
        import importlib
        importlib.import_module("hector-engine_b200.build").build_all()
    assert os.path.exists(BIN)


def test_host_tests_binary_links_and_lists_cases():
    _ensure_built()
    out = subprocess.run([BIN, "--list"], capture_output=True, text=True, check=True).stdout.split()
    assert out == ["known_answers", "graph_contract", "graph_contract_fused", "error_behaviour", "qk_norm_rope_op",
                   "cache_owner", "decode_loop"]


@pytest.mark.gpu
def test_host_adapter_cases_on_gpu():
    _ensure_built()
    res = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    print(res.stdout, res.stderr)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.count("PASS:") == 7 and "ALL PASSED" in res.stdout
