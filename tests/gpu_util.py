"""Helpers shared by the GPU parity tests: device buffers through torch, calls through the C ABI."""
import numpy as np
import torch

import q4gpu

TOL_ABS, TOL_REL = 2e-3, 1e-3   # attention outputs vs the fp32 oracle (the stated tolerance)


def lib():
    L = q4gpu.init()
    q4gpu.use_torch_stream()
    return L


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def dev_bytes(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.detach().cpu().numpy()


def assert_close(got, ref, what=""):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    err = np.abs(got - ref)
    bound = TOL_ABS + TOL_REL * np.abs(ref)
    assert np.isfinite(got).all(), what
    assert (err <= bound).all(), "%s: max abs err %.3e (bound %.1e + %.0e*|ref|)" % (what, err.max(), TOL_ABS, TOL_REL)
    return float(err.max())


def fill_store(oracle, store, layer, k, v, pos0=0):
    """Append fp32 rows [n][n_kvh*hd] (numpy) into a store; returns the oracle's reference-layout bytes."""
    n = k.shape[0]
    store.append(layer, dev(k), dev(v), pos0, n)
    return oracle.kv_write(k, store.kind), oracle.kv_write(v, store.kind)
