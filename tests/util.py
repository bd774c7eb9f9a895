"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch

# tolerance of f32 attention outputs against the reference arithmetic
RTOL, ATOL = 1e-3, 1e-4


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def assert_close(got, want, rtol=RTOL, atol=ATOL, what=""):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    err = np.abs(got - want)
    bound = atol + rtol * np.abs(want)
    bad = err > bound
    assert not bad.any(), (f"{what}: {bad.sum()} of {bad.size} outside |d| <= {atol} + {rtol}|ref|; "
                           f"max abs err {err.max():.3e} at {np.unravel_index(err.argmax(), err.shape)}")


def make_i8_store(k, v, nKV, hd, extra_rows=0):
    """Quantise f32 rows with the oracle quantiser; optionally pad the pool with
    garbage rows (what a slot past the live length holds)."""
    import oracle

    k8, v8, ks, vs = oracle.quant_kv8(k, v, nKV, hd)
    if extra_rows:
        r = np.random.default_rng(5)
        k8 = np.concatenate([k8, r.integers(-128, 128, (extra_rows, nKV, hd), dtype=np.int8)])
        v8 = np.concatenate([v8, r.integers(-128, 128, (extra_rows, nKV, hd), dtype=np.int8)])
        junk = np.full((extra_rows, nKV), np.nan, np.float32)
        ks = np.concatenate([ks, junk])
        vs = np.concatenate([vs, junk])
    return k8, v8, ks, vs
