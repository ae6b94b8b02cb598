"""Builds the inputs of the reference's known-answer cases (tests/golden/kat_reference_tests.json)."""
import json
import math
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_kats():
    with open(os.path.join(HERE, "golden", "kat_reference_tests.json")) as f:
        return json.load(f)


def build(case):
    H, KVH, HD, S = case["H"], case["KVH"], case["HD"], case["max_seq"]
    nq = case.get("seq_new", 1)
    q = np.zeros((nq, H, HD), dtype=np.float16)
    k = np.zeros((1, S, KVH, HD), dtype=np.float16)
    v = np.zeros((1, S, KVH, HD), dtype=np.float16)
    kind = case["v"]
    if kind == "pos_plus_one":
        for p in range(S):
            v[0, p] = p + 1
    elif kind == "two_except_first_two_rows_1000":
        v[:] = 2.0
        v[0, :2] = 1000.0
    elif kind == "row0_two_row1_six":
        v[0, 0] = 2.0
        v[0, 1] = 6.0
    else:
        raise ValueError(kind)
    scale = 1.0 / math.sqrt(HD) if case["scale"] == "default" else float(case["scale"])
    if "expect_all" in case:
        expect = np.full((nq, H * HD), case["expect_all"], dtype=np.float32)
    else:
        expect = np.asarray(case["expect"], dtype=np.float32)
    return q, k, v, scale, expect
