"""numpy front end of the CPU oracle (oracle/q4_oracle.c) and of the reference's own dequantiser
compiled in place (oracle/_ref/libq4ref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline /
reference arm of bench.py -- never by the shipped package.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

u8p = C.POINTER(C.c_uint8)
f32p = C.POINTER(C.c_float)
i32p = C.POINTER(C.c_int32)
u16p = C.POINTER(C.c_uint16)


def build(ref_tree=None):
    """make -C oracle: the restatement always; the reference's own dequantiser and quantiser (oracle/_ref)
    only when a reference tree is given (argument, or the Q4_REF_TREE environment variable) and present."""
    ref_tree = ref_tree or os.environ.get("Q4_REF_TREE", "")
    subprocess.run(["make", "-C", _HERE, "REF=" + ref_tree], check=True,
                   stdout=subprocess.PIPE, stderr=subprocess.STDOUT)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libq4oracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.q4o_u64.restype = C.c_uint64
        L.q4o_u64.argtypes = [C.c_uint64] * 3
        L.q4o_normal_f32.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p]
        L.q4o_select.restype = C.c_uint32
        L.q4o_select.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32,
                                 C.c_uint32, C.c_void_p, C.c_uint32]
        L.q4o_f16_to_f32.restype = C.c_float
        L.q4o_f16_to_f32.argtypes = [C.c_uint16]
        L.q4o_f32_to_f16.restype = C.c_uint16
        L.q4o_f32_to_f16.argtypes = [C.c_float]
        L.q4o_f32_to_f16_n.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        L.q4o_f32_to_bf16.restype = C.c_uint16
        L.q4o_f32_to_bf16.argtypes = [C.c_float]
        L.q4o_quant_q8_0.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        L.q4o_dequant_q8_0.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p]
        L.q4o_kv_token_bytes.restype = C.c_uint64
        L.q4o_kv_token_bytes.argtypes = [C.c_uint32, C.c_uint32, C.c_int]
        L.q4o_kv_write.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_int]
        L.q4o_rope.argtypes = [C.c_void_p, C.c_uint32, C.c_int32, C.c_float]
        L.q4o_rope_table.argtypes = [C.c_uint32, C.c_int32, C.c_uint32, C.c_float, C.c_void_p]
        L.q4o_q_prep.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32,
                                 C.c_uint32, C.c_uint32, C.c_int32, C.c_float, C.c_float,
                                 C.c_uint32]
        L.q4o_k_prep.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                 C.c_int32, C.c_float, C.c_float, C.c_uint32]
        L.q4o_attn.restype = C.c_int
        L.q4o_attn.argtypes = [C.c_void_p] * 5 + [C.c_uint32] * 6 + [C.c_float, C.c_int,
                                                                     C.c_void_p, C.c_uint32,
                                                                     C.c_uint32, C.c_int, C.c_int]
        L.q4o_attn_partial.restype = C.c_int
        L.q4o_attn_partial.argtypes = [C.c_void_p] * 4 + [C.c_uint32] * 3 + [
            C.c_float, C.c_int, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32]
        L.q4o_lse_merge.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p,
                                    C.c_void_p]
        L.q4o_max_threads.restype = C.c_int
        L.q4o_host_procs.restype = C.c_int
        L.q4o_ix_pool.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                  C.c_uint32, C.c_float, C.c_float]
        L.q4o_ix_score.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_uint32] * 7
        L.q4o_ix_topk.argtypes = [C.c_void_p, C.c_void_p] + [C.c_uint32] * 6
        L.q4o_attn_items.restype = C.c_int
        L.q4o_attn_items.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float,
                                     C.c_int, C.c_int]
        _LIB = L
    return _LIB


def ref_lib():
    """The reference's q4_quant.c compiled in place (q4_dequant_row, q4_f16_to_f32); None when it
    was never built (no reference tree and no prebuilt copy)."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libq4ref.so")
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        R.q4_f16_to_f32.restype = C.c_float
        R.q4_f16_to_f32.argtypes = [C.c_uint16]
        R.q4_dequant_row.restype = C.c_bool
        R.q4_dequant_row.argtypes = [C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p]
        _REF = R
    return _REF


_REFQ = None


def ref_quant_lib():
    """The reference's own q8_0 quantiser (the body of f32_to_q8_k, src/q4_rocm.cu:7221-7238, compiled for
    the host); None when it was never built."""
    global _REFQ
    if _REFQ is None:
        path = os.path.join(_HERE, "_ref", "libq4refquant.so")
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        R.q4ref_f32_to_q8.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        _REFQ = R
    return _REFQ


def ref_quant_q8_0(x):
    x = np.ascontiguousarray(x, np.float32)
    assert x.size % 32 == 0
    out = np.empty(x.size // 32 * 34, np.uint8)
    ref_quant_lib().q4ref_f32_to_q8(_p(x), _p(out), x.size // 32)
    return out


Q4_T_Q8_0 = 8  # src/q4.h:26


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def normal(seed, stream, n, offset=0):
    out = np.empty(int(n), np.float32)
    lib().q4o_normal_f32(seed, stream, offset, int(n), _p(out))
    return out


def select(seed, stream, ctx, width=2051, sink=4, recent=1024, nrand=1023):
    out = np.empty(width, np.int32)
    lib().q4o_select(seed, stream, ctx, sink, recent, nrand, _p(out), width)
    return out


def f32_to_f16(x):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().q4o_f32_to_f16_n(_p(x), _p(out), x.size)
    return out


def f32_to_bf16(x):
    """RNE bfloat16 bits of fp32 values (numpy has no bf16)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_to_f32(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def quant_q8_0(x):
    x = np.ascontiguousarray(x, np.float32)
    assert x.size % 32 == 0
    out = np.empty(x.size // 32 * 34, np.uint8)
    lib().q4o_quant_q8_0(_p(x), _p(out), x.size)
    return out


def dequant_q8_0(b, n):
    b = np.ascontiguousarray(b, np.uint8)
    out = np.empty(int(n), np.float32)
    lib().q4o_dequant_q8_0(_p(b), int(n), _p(out))
    return out


def ref_dequant_q8_0(b, n):
    b = np.ascontiguousarray(b, np.uint8)
    out = np.empty(int(n), np.float32)
    assert ref_lib().q4_dequant_row(Q4_T_Q8_0, _p(b), int(n), _p(out))
    return out


def kv_token_bytes(n_kvh, hd, kind):
    return int(lib().q4o_kv_token_bytes(n_kvh, hd, kind))


def kv_write(x, kind):
    """fp32 rows -> cache bytes in the reference layout (q8_0 / f16 / f32 for kind 2 / 1 / 0)."""
    x = np.ascontiguousarray(x, np.float32)
    nbytes = x.size // 32 * 34 if kind == 2 else x.size * (2 if kind == 1 else 4)
    out = np.empty(nbytes, np.uint8)
    lib().q4o_kv_write(_p(out), _p(x), x.size, kind)
    return out


def rope(x, n_rot, pos, base):
    x = np.ascontiguousarray(x, np.float32).copy()
    lib().q4o_rope(_p(x), n_rot, pos, base)
    return x


def rope_rows(x, n_rot, pos0, base):
    """x: [n_tok][n_h][hd]; rotates every head of token t at position pos0+t."""
    x = np.ascontiguousarray(x, np.float32).copy()
    n_tok, n_h, hd = x.shape
    for t in range(n_tok):
        for h in range(n_h):
            lib().q4o_rope(_p(x[t, h]), n_rot, pos0 + t, base)
    return x


def rope_table(n_rot, pos0, n_pos, base):
    cs = np.empty((n_pos, n_rot // 2, 2), np.float32)
    lib().q4o_rope_table(n_rot, pos0, n_pos, base, _p(cs))
    return cs


def q_prep(qg, wn, n_head, hd, n_rot, pos0, base, eps):
    qg = np.ascontiguousarray(qg, np.float32)
    n_tok = qg.size // (n_head * hd * 2)
    q = np.empty((n_tok, n_head, hd), np.float32)
    g = np.empty((n_tok, n_head, hd), np.float32)
    lib().q4o_q_prep(_p(qg), _p(wn), _p(q), _p(g), n_head, hd, n_rot, pos0, base, eps, n_tok)
    return q, g


def k_prep(k, wn, n_kvh, hd, n_rot, pos0, base, eps):
    k = np.ascontiguousarray(k, np.float32).copy()
    n_tok = k.size // (n_kvh * hd)
    lib().q4o_k_prep(_p(k), _p(wn), n_kvh, hd, n_rot, pos0, base, eps, n_tok)
    return k


def attn(q, kc, vc, gate, n_head, n_kvh, hd, n_tok, kv_base, max_kv, scale, kind, idx=None,
         width=0, idx_kvh_stride=0, acc64=False, threads=1):
    q = np.ascontiguousarray(q, np.float32)
    out = np.empty(n_tok * n_head * hd, np.float32)
    if gate is not None:
        gate = np.ascontiguousarray(gate, np.float32)
    if idx is not None:
        idx = np.ascontiguousarray(idx, np.int32)
    rc = lib().q4o_attn(_p(q), _p(kc), _p(vc), _p(gate), _p(out), n_head, n_kvh, hd, n_tok,
                        kv_base, max_kv, scale, kind, _p(idx), width, idx_kvh_stride,
                        int(acc64), threads)
    assert rc == 0
    return out.reshape(n_tok, n_head, hd)


def attn_partial(q, kc, vc, n_head, n_kvh, hd, scale, kind, p0, p1, idx=None, idx_kvh_stride=0):
    q = np.ascontiguousarray(q, np.float32)
    part = np.empty((n_head, hd + 2), np.float32)
    if idx is not None:
        idx = np.ascontiguousarray(idx, np.int32)
    rc = lib().q4o_attn_partial(_p(q), _p(kc), _p(vc), _p(part), n_head, n_kvh, hd, scale, kind,
                                _p(idx), idx_kvh_stride, p0, p1)
    assert rc == 0
    return part


def lse_merge(parts, n_head, hd, gate=None):
    parts = np.ascontiguousarray(parts, np.float32)
    n_parts = parts.size // (n_head * (hd + 2))
    out = np.empty((n_head, hd), np.float32)
    if gate is not None:
        gate = np.ascontiguousarray(gate, np.float32)
    lib().q4o_lse_merge(_p(parts), n_parts, n_head, hd, _p(gate), _p(out))
    return out


def ix_pool(raw_f16, wn, ratio, b0, b1, n_rot, base, eps, pool=None, hd=128):
    """qsa_pool_k: raw fp16 keys [n_tok][hd] (uint16) -> pooled blocks [b0, b1) of pool [n_blocks][hd]"""
    raw_f16 = np.ascontiguousarray(raw_f16, np.uint16)
    if pool is None:
        pool = np.zeros((b1, hd), np.float32)
    wn_c = None if wn is None else np.ascontiguousarray(wn, np.float32)
    lib().q4o_ix_pool(_p(raw_f16), _p(pool), _p(wn_c), hd, ratio, b0, b1, n_rot, base, eps)
    return pool


def ix_score(q, pool, n_tok, n_blocks, stride, n_head, pos0, ratio, hd=128):
    """qsa_score_k: q [n_tok][n_head][hd], pool [.][hd] -> score [n_tok][stride]"""
    q = np.ascontiguousarray(q, np.float32)
    pool = np.ascontiguousarray(pool, np.float32)
    score = np.zeros((n_tok, stride), np.float32)
    lib().q4o_ix_score(_p(q), _p(pool), _p(score), n_tok, n_blocks, stride, n_head, hd, pos0, ratio)
    return score


def ix_topk(score, n_tok, stride, k_blk, ratio, pos0, width):
    """qsa_topk_k + qsa_write_sel: score [n_tok][stride] -> sel [n_tok][width]"""
    score = np.ascontiguousarray(score, np.float32)
    sel = np.zeros((n_tok, width), np.int32)
    lib().q4o_ix_topk(_p(score), _p(sel), n_tok, stride, k_blk, ratio, pos0, width)
    return sel


def max_threads():
    return int(lib().q4o_max_threads())


def host_procs():
    """processors usable by this process, independent of OMP_NUM_THREADS (1 without OpenMP)"""
    return int(lib().q4o_host_procs())


class Item(C.Structure):
    _fields_ = [("q", C.c_void_p), ("kcache", C.c_void_p), ("vcache", C.c_void_p), ("gate", C.c_void_p),
                ("out", C.c_void_p), ("idx", C.c_void_p), ("width", C.c_uint32),
                ("idx_kvh_stride", C.c_uint32), ("kv_base", C.c_uint32), ("max_kv", C.c_uint32)]


def attn_items(items, n_head, n_kvh, hd, scale, kind, threads):
    """items: list of dicts with numpy arrays q, kc, vc, out and optional gate, idx (+ width,
    idx_kvh_stride, kv_base, max_kv); one decode token each; parallel over (item, head)."""
    arr = (Item * len(items))()
    for a, it in zip(arr, items):
        a.q, a.kcache, a.vcache, a.out = _p(it["q"]), _p(it["kc"]), _p(it["vc"]), _p(it["out"])
        a.gate, a.idx = _p(it.get("gate")), _p(it.get("idx"))
        a.width, a.idx_kvh_stride = it.get("width", 0), it.get("idx_kvh_stride", 0)
        a.kv_base, a.max_kv = it.get("kv_base", 0), it.get("max_kv", 0xFFFFFFFF)
    rc = lib().q4o_attn_items(arr, len(items), n_head, n_kvh, hd, scale, kind, threads)
    assert rc == 0
