"""The allocation-free decode entry point (q4_gpu_kv_decode_noalloc) through the C ABI.

Some hosts cannot allocate device memory while they run (all of it was planned and handed out at
start-up, or the serving loop must stay out of the allocator), so this entry point keeps its split-KV
scratch in an array that is part of the library image.  The array is shared by all calls and keeps
what the last call left in it, so the check is made on two calls in a row, against the regular entry
point on the same inputs, within the tolerance of the other decode tests.  Collected last on purpose.
"""
import numpy as np
import pytest
import torch

import q4gpu
from gpu_util import assert_close, dev, host, lib

pytestmark = pytest.mark.gpu


def test_noalloc_decode_matches_regular_entry_point_twice(oracle):
    L = lib()
    n_head, n_kvh, hd, ctx, width = 16, 2, 128, 5000, 2051
    kvw = n_kvh * hd
    k = oracle.normal(901, 0, ctx * kvw).reshape(ctx, kvw)
    v = oracle.normal(901, 1, ctx * kvw).reshape(ctx, kvw)
    st = q4gpu.KVStore(2, n_kvh, hd, ctx, q4gpu.KIND_Q8)
    st.append(1, dev(k), dev(v), 0, ctx)
    scale = 1.0 / np.sqrt(hd)
    want = torch.empty(n_head * hd, device="cuda")
    got = torch.empty(n_head * hd, device="cuda")

    def noalloc(*args):
        """the call, with the device's free memory read right before and right after it: the defining
        property of the entry point is that the two readings are equal (cudaMemGetInfo through torch;
        nothing in between goes through an allocator)"""
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        ok = L.q4_gpu_kv_decode_noalloc(*args)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry point changed the free device memory"
        return ok

    for call in range(2):                       # second call starts from the first one's leftovers
        q = oracle.normal(902, call, n_head * hd)
        gate = oracle.normal(903, call, n_head * hd)
        idx = np.stack([oracle.select(904 + call, kh, ctx, width) for kh in range(n_kvh)])
        dq, dg, di = dev(q), dev(gate), dev(idx)
        # sparse
        assert L.q4_gpu_kv_decode(st.h, 1, dq.data_ptr(), 0, dg.data_ptr(), want.data_ptr(), n_head, di.data_ptr(),
                                  width, width, ctx, scale)
        assert noalloc(st.h, 1, dq.data_ptr(), 0, dg.data_ptr(), got.data_ptr(), n_head, di.data_ptr(), width, width, ctx, scale)
        assert_close(host(got), host(want), "noalloc sparse, call %d" % call)
        # dense over all rows (many splits: exercises the clamp to the built-in scratch)
        assert L.q4_gpu_kv_decode(st.h, 1, dq.data_ptr(), 0, None, want.data_ptr(), n_head, None, 0, 0, ctx, scale)
        assert noalloc(st.h, 1, dq.data_ptr(), 0, None, got.data_ptr(), n_head, None, 0, 0, ctx, scale)
        assert_close(host(got), host(want), "noalloc dense, call %d" % call)
        ref = oracle.attn(q, oracle.kv_write(k, 2), oracle.kv_write(v, 2), None, n_head, n_kvh, hd, 1, ctx - 1, ctx,
                          scale, 2)[0]
        assert_close(host(got).reshape(n_head, hd), ref, "noalloc dense vs oracle, call %d" % call)
    assert L.q4_gpu_last_error() == 0
    st.close()


def test_noalloc_rejects_shapes_beyond_its_scratch():
    L = lib()
    st = q4gpu.KVStore(1, 8, 32, 64, q4gpu.KIND_Q8)       # 8 kv heads: more than the built-in scratch covers
    buf = torch.zeros(8 * 32, device="cuda")
    assert not L.q4_gpu_kv_decode_noalloc(st.h, 0, buf.data_ptr(), 0, None, buf.data_ptr(), 8, None, 0, 0, 1, 1.0)
    assert L.q4_gpu_last_error() & 8
    st.close()
