"""GPU parity of the tensor-core (tcgen05) causal prefill attention against the CPU oracle.
Outputs are bf16 by contract, so the comparison allows one bf16 rounding of the result on top of
the stated 2e-3 max-abs / 1e-3 relative tolerance."""
import numpy as np
import pytest
import torch

import q4gpu
from gpu_util import dev, host, lib

pytestmark = pytest.mark.gpu


def check(got, ref, what, out_scale=1.0):
    """2e-3 max-abs (times out_scale, the magnitude of the outputs, for the large-magnitude cases) + 1e-3
    relative, plus one bf16 rounding of the result"""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    assert np.isfinite(got).all(), what
    bound = 2e-3 * out_scale + (1e-3 + 2.0 ** -8) * np.abs(ref)
    err = np.abs(got - ref)
    worst = (err / bound).argmax()
    assert (err <= bound).all(), "%s: max abs err %.3e at ref %.3f; worst err %.3e against bound %.3e at ref %.3f" % (
        what, err.max(), ref.reshape(-1)[err.argmax()], err.reshape(-1)[worst], bound.reshape(-1)[worst], ref.reshape(-1)[worst])
    return err.max()


def run_case(oracle, n_tok, kv_base, n_head, n_kvh, seed, gate=True, rope=False):
    hd = 128
    ctx = kv_base + n_tok
    kvw = n_kvh * hd
    k = oracle.normal(seed, 0, ctx * kvw).reshape(ctx, kvw)
    v = oracle.normal(seed, 1, ctx * kvw).reshape(ctx, kvw)
    q = oracle.normal(seed, 2, n_tok * n_head * hd).reshape(n_tok, n_head, hd)
    if rope:
        k = oracle.rope_rows(k.reshape(ctx, n_kvh, hd), hd, 0, 1e7).reshape(ctx, kvw)
        q = oracle.rope_rows(q, hd, kv_base, 1e7)
    g = oracle.normal(seed, 3, n_tok * n_head * hd) if gate else None
    qb = oracle.f32_to_bf16(q)
    scale = 1.0 / np.sqrt(hd)
    st = q4gpu.KVStore(2, n_kvh, hd, ctx + 3, 2)
    st.append(1, dev(k), dev(v), 0, ctx)
    dq = torch.from_numpy(qb.view(np.int16).reshape(-1)).cuda()
    dout = torch.empty(n_tok * n_head * hd, dtype=torch.bfloat16, device="cuda")
    st.prefill(1, dq, dout, n_head, n_tok, kv_base, scale, gate=dev(g) if gate else None)
    got = host(dout.float()).reshape(n_tok, n_head, hd)
    ref = oracle.attn(oracle.bf16_to_f32(qb), oracle.kv_write(k, 2), oracle.kv_write(v, 2), g, n_head, n_kvh, hd,
                      n_tok, kv_base, ctx + 3, scale, 2, threads=8)
    st.close()
    return check(got, ref, "prefill n_tok %d kv_base %d heads %d/%d" % (n_tok, kv_base, n_head, n_kvh))


@pytest.mark.parametrize("n_tok,kv_base", [(1, 0), (2, 0), (16, 0), (17, 5), (33, 100), (64, 63), (50, 200), (130, 1)])
def test_prefill_small_ragged(oracle, n_tok, kv_base):
    lib()
    run_case(oracle, n_tok, kv_base, 16, 2, 1000 + n_tok)
    assert q4gpu.load().q4_gpu_last_error() == 0


@pytest.mark.parametrize("n_head,n_kvh", [(8, 1), (2, 2), (12, 1), (24, 2), (32, 2), (5, 1)])
def test_prefill_gqa_shapes(oracle, n_head, n_kvh):
    lib()
    run_case(oracle, 40, 77, n_head, n_kvh, 2000 + n_head, gate=(n_head % 2 == 0))


def test_prefill_chunk_over_existing_cache(oracle):
    """the chunked-prefill shape scaled down: 512 new tokens over a 1024-token cache, RoPE'd inputs"""
    lib()
    run_case(oracle, 512, 1024, 16, 2, 20261125 + 3, gate=False, rope=True)


def test_prefill_matches_decode_kernel(oracle):
    """the last query of a prefill chunk == the decode kernel's answer for the same rows"""
    lib()
    n_head, n_kvh, hd, ctx, n_tok = 16, 2, 128, 700, 90
    kvw = n_kvh * hd
    k = oracle.normal(5, 0, ctx * kvw).reshape(ctx, kvw)
    v = oracle.normal(5, 1, ctx * kvw).reshape(ctx, kvw)
    q = oracle.bf16_to_f32(oracle.f32_to_bf16(oracle.normal(5, 2, n_tok * n_head * hd))).reshape(n_tok, n_head, hd)
    st = q4gpu.KVStore(1, n_kvh, hd, ctx, 2)
    st.append(0, dev(k), dev(v), 0, ctx)
    dq = dev(q).to(torch.bfloat16)
    dout = torch.empty(n_tok, n_head, hd, dtype=torch.bfloat16, device="cuda")
    st.prefill(0, dq, dout, n_head, n_tok, ctx - n_tok, 0.0884)
    dd = torch.empty(n_head * hd, device="cuda")
    for t in (0, 45, n_tok - 1):
        st.decode(0, dq[t].contiguous(), dd, n_head, 0.0884, n_kv=ctx - n_tok + t + 1, q_bf16=True)
        check(host(dout[t].float()), host(dd).reshape(n_head, hd), "token %d" % t)
    st.close()


def test_prefill_rejects_unsupported(oracle):
    L = lib()
    st = q4gpu.KVStore(1, 2, 128, 64, 1)      # fp16 store: not the tensor-core path
    buf = torch.zeros(16 * 128, dtype=torch.bfloat16, device="cuda")
    assert not L.q4_gpu_kv_prefill(st.h, 0, buf.data_ptr(), None, buf.data_ptr(), 16, 1, 0, 0.1)
    assert L.q4_gpu_last_error() & 1
    st.close()


@pytest.mark.parametrize("mode", ["sigma8", "head_x50"])
def test_prefill_large_magnitude_queries(oracle, mode):
    """queries ~ N(0, 8^2), or one head of each kv group scaled by 50: scores of several hundred in the
    exponent, softmax close to one-hot.  This checks the running-max rescale, the fp16 weights and the
    accumulators at such magnitudes.  The tensor-core path stages K and V as fp16(code * scale) (the
    reference's own fp16 tile), a rounding that |q| multiplies; to keep it out of this check every 32-value
    block of the rows gets one element of magnitude 127/32, which makes its scale exactly 1/32 and every
    dequantised value exact in fp16 (the rounding itself is covered by the N(0,1) cases at the stated
    tolerance).  The absolute part of the tolerance is relative to the magnitude of the outputs."""
    lib()
    n_tok, kv_base, n_head, n_kvh, hd = 96, 400, 16, 2, 128
    ctx, kvw = kv_base + n_tok, n_kvh * hd

    def rows(stream):
        x = np.clip(oracle.normal(5200, stream, ctx * kvw), -3.9, 3.9).reshape(-1, 32)
        sign = np.where(x[:, 7] < 0, -1.0, 1.0).astype(np.float32)
        x[:, 7] = sign * np.float32(127.0 / 32.0)
        return x.reshape(ctx, kvw)
    k, v = rows(0), rows(1)
    q = oracle.normal(5200, 2, n_tok * n_head * hd).reshape(n_tok, n_head, hd).copy()
    if mode == "sigma8":
        q *= 8.0
    else:
        q[:, 3] *= 50.0
        q[:, 12] *= 50.0
    g = oracle.normal(5200, 3, n_tok * n_head * hd)
    qb = oracle.f32_to_bf16(q)
    scale = 1.0 / np.sqrt(hd)
    kc, vc = oracle.kv_write(k, 2), oracle.kv_write(v, 2)
    assert (kc.reshape(-1, 34)[:, :2].view(np.uint16) == 0x2800).all()      # every block scale is fp16 1/32
    st = q4gpu.KVStore(1, n_kvh, hd, ctx, 2)
    st.append(0, dev(k), dev(v), 0, ctx)
    dq = torch.from_numpy(qb.view(np.int16).reshape(-1)).cuda()
    dout = torch.empty(n_tok * n_head * hd, dtype=torch.bfloat16, device="cuda")
    st.prefill(0, dq, dout, n_head, n_tok, kv_base, scale, gate=dev(g))
    ref = oracle.attn(oracle.bf16_to_f32(qb), kc, vc, g, n_head, n_kvh, hd, n_tok, kv_base, ctx, scale, 2, threads=8)
    check(host(dout.float()).reshape(n_tok, n_head, hd), ref, "prefill, %s" % mode, out_scale=max(1.0, float(np.abs(ref).max())))
    st.close()
