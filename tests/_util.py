"""Shared helpers for the parity tests: seeded inputs and the path's tolerance rule."""
import numpy as np

ATOL, RTOL = 2e-3, 1e-2  # fp16 attention outputs vs the fp32-accumulated oracle


def normal_f16(rng, *shape):
    return rng.standard_normal(shape, dtype=np.float32).astype(np.float16)


def make_case(seed, B, H, KVH, HD, slots, totals=None, fill="valid"):
    """Seeded q / k_new / v_new / cache planes. Rows >= total are zero (fill='valid'),
    or random garbage (fill='garbage') to prove they are never attended."""
    rng = np.random.default_rng(seed)
    q = normal_f16(rng, B, H, HD)
    k_new = normal_f16(rng, B, 1, KVH, HD)
    v_new = normal_f16(rng, B, 1, KVH, HD)
    kc = normal_f16(rng, B, slots, KVH, HD)
    vc = normal_f16(rng, B, slots, KVH, HD)
    if totals is not None and fill == "valid":
        for b, t in enumerate(totals):
            kc[b, max(t, 0):] = 0
            vc[b, max(t, 0):] = 0
    return q, k_new, v_new, kc, vc


def to_dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def assert_close(oracle, got, ref, what=""):
    ok, err = oracle.within_tolerance(got, ref, ATOL, RTOL)
    assert ok, f"{what}: max abs err {err:.3e} exceeds {ATOL} + {RTOL}*|ref|"
    return err
