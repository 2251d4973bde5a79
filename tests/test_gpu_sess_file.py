"""The version-5 session file around a library-owned store (q4_gpu_sess_file_write / _read / _peek_ids)
against a Python restatement of the reference's format (q4_sess_hdr and the section order of q4_sess_save,
src/q4_fwd.c:2256-2377): a file the library writes has exactly the bytes the reference host would write for
the same state, a file laid out by the restatement is accepted and restored, and every refusal of
q4_sess_restore (:2405-2432) is reproduced: other max_kv, other KV kind, other model, ids that differ,
more saved ids than the caller has, a truncated file."""
import ctypes as C
import os
import struct

import numpy as np
import pytest
import torch

import q4gpu
from gpu_util import dev, host, lib

pytestmark = pytest.mark.gpu

HDR = "<IIQ17I4xQ"          # q4_sess_hdr: 96 bytes, user_hash at offset 88
MAGIC, VERSION = 0x53345134, 5
N_LAYERS, N_KVH, HD = 3, 2, 128
KVW = N_KVH * HD
DIMS = dict(bytes_total=0x1234567890, n_layer=48, n_expert=128, n_gdn=2, n_v_h=4, d_v=8, conv_hist=3, conv_ch=20, hc_dim=64)
IDX_DIM = 128


def make_state(oracle, seed, n_kv, kind):
    rng = np.random.default_rng(seed)
    st = dict(
        k=[oracle.normal(seed, 2 * l, n_kv * KVW).reshape(n_kv, KVW) for l in range(N_LAYERS)],
        v=[oracle.normal(seed, 2 * l + 1, n_kv * KVW).reshape(n_kv, KVW) for l in range(N_LAYERS)],
        ids=rng.integers(0, 150000, n_kv).astype(np.int32),
        ple=rng.integers(-5, 5, 8).astype(np.int32),
        a=rng.standard_normal(11 * DIMS["hc_dim"]).astype(np.float32),
        b=rng.standard_normal(DIMS["n_gdn"] * DIMS["n_v_h"] * DIMS["d_v"] ** 2 +
                              DIMS["n_gdn"] * DIMS["conv_hist"] * DIMS["conv_ch"]).astype(np.float32),
        raw=rng.integers(0, 65536, N_LAYERS * n_kv * IDX_DIM).astype(np.uint16),
        pos=n_kv, prompt_n=n_kv - 3, nmsg=5, user_hash=0xDEADBEEFCAFE, kind=kind, n_kv=n_kv)
    return st


def reference_file_bytes(oracle, s, max_kv, with_raw=True):
    """the bytes q4_sess_save writes for this state (section order of src/q4_fwd.c:2336-2372)"""
    tag = {2: 8, 1: 2, 0: 4}[s["kind"]]
    hdr = struct.pack(HDR, MAGIC, VERSION, DIMS["bytes_total"], DIMS["n_layer"], DIMS["n_expert"], max_kv, s["n_kv"], s["pos"],
                      N_LAYERS, KVW, DIMS["n_gdn"], DIMS["n_v_h"], DIMS["d_v"], DIMS["conv_hist"], DIMS["conv_ch"],
                      DIMS["hc_dim"], len(s["ids"]), s["prompt_n"], s["nmsg"], tag, s["user_hash"])
    assert len(hdr) == 96
    out = [hdr, s["ids"].tobytes(), s["ple"].tobytes(), s["a"].tobytes()]
    for l in range(N_LAYERS):
        out.append(oracle.kv_write(s["k"][l], s["kind"]).tobytes())
        out.append(oracle.kv_write(s["v"][l], s["kind"]).tobytes())
    out.append(s["b"].tobytes())
    out.append(struct.pack("<4I", IDX_DIM, N_LAYERS, s["n_kv"], 1 if with_raw else 0))
    if with_raw:
        out.append(s["raw"].tobytes())
    return b"".join(out)


def descriptor(s=None, for_read=None, with_raw=True):
    d = q4gpu.SessDesc()
    for k, v in DIMS.items():
        setattr(d, k, v)
    keep = []
    if s is not None:                               # to write
        d.pos, d.prompt_n, d.nmsg, d.user_hash = s["pos"], s["prompt_n"], s["nmsg"], s["user_hash"]
        d.ids, d.n_ids = s["ids"].ctypes.data, len(s["ids"])
        d.ple_hist = (C.c_int32 * 8)(*[int(x) for x in s["ple"]])
        d.state_a, d.state_a_bytes = s["a"].ctypes.data, s["a"].nbytes
        d.state_b, d.state_b_bytes = s["b"].ctypes.data, s["b"].nbytes
        d.idx_dim = IDX_DIM
        if with_raw:
            d.idx_raw, d.idx_raw_bytes = s["raw"].ctypes.data, s["raw"].nbytes
    else:                                           # to read into fresh buffers
        a = np.zeros(11 * DIMS["hc_dim"], np.float32)
        b = np.zeros(for_read["b"].size, np.float32)
        raw = np.zeros(for_read["raw"].size, np.uint16)
        d.state_a, d.state_a_bytes, d.state_b, d.state_b_bytes = a.ctypes.data, a.nbytes, b.ctypes.data, b.nbytes
        d.idx_dim, d.idx_raw, d.idx_raw_bytes = IDX_DIM, raw.ctypes.data, raw.nbytes
        keep = [a, b, raw]
    return d, keep


def fill(store, s):
    for l in range(N_LAYERS):
        store.append(l, dev(s["k"][l]), dev(s["v"][l]), 0, s["n_kv"])


def exported(store, layer, which, n):
    buf = torch.empty(n * store.token_bytes, dtype=torch.uint8, device="cuda")
    store.export(layer, which, 0, n, buf)
    return host(buf).tobytes()


@pytest.mark.parametrize("kind", [2, 1, 0])
def test_written_file_is_the_reference_format_byte_for_byte(oracle, tmp_path, kind):
    L = lib()
    n_kv, max_kv = 1000, 1500
    s = make_state(oracle, 700 + kind, n_kv, kind)
    store = q4gpu.KVStore(N_LAYERS, N_KVH, HD, max_kv, kind)
    fill(store, s)
    d, _ = descriptor(s)
    path = str(tmp_path / "sess.q4s")
    store.sess_file_write(n_kv, d, path)
    got = open(path, "rb").read()
    want = reference_file_bytes(oracle, s, max_kv)
    assert len(got) == len(want) == L.q4_gpu_sess_file_bytes(store.h, n_kv, C.byref(d))
    assert got[:96] == want[:96], "header"
    assert got == want
    assert not os.path.exists(path + ".tmp")
    # without raw indexer keys the meta block says so and the file ends there
    d2, _ = descriptor(s, with_raw=False)
    store.sess_file_write(n_kv, d2, path)
    assert open(path, "rb").read() == reference_file_bytes(oracle, s, max_kv, with_raw=False)
    # peek: ids and prompt metadata only
    ids = np.zeros(n_kv, np.int32)
    pn, nm, uh = C.c_uint32(), C.c_uint32(), C.c_uint64()
    model, _ = descriptor(s)
    assert L.q4_gpu_sess_file_peek_ids(C.byref(model), os.fsencode(path), ids.ctypes.data, n_kv, C.byref(pn), C.byref(nm),
                                       C.byref(uh)) == n_kv
    assert np.array_equal(ids, s["ids"]) and (pn.value, nm.value, uh.value) == (s["prompt_n"], s["nmsg"], s["user_hash"])
    assert L.q4_gpu_sess_file_peek_ids(C.byref(model), os.fsencode(path), ids.ctypes.data, n_kv - 1, None, None, None) == -1
    # a directory that does not exist: refused, nothing left behind
    assert not L.q4_gpu_sess_file_write(store.h, n_kv, C.byref(d), os.fsencode(str(tmp_path / "nope" / "x.q4s")))
    L.q4_gpu_last_error()
    # state sections of the wrong size are rejected (the format fixes them)
    d.state_a_bytes -= 4
    assert not L.q4_gpu_sess_file_write(store.h, n_kv, C.byref(d), os.fsencode(path))
    assert L.q4_gpu_last_error() & 1
    store.close()


@pytest.mark.parametrize("kind", [2, 1])
def test_reference_format_file_is_restored_and_refusals(oracle, tmp_path, kind):
    L = lib()
    n_kv, max_kv = 777, 900
    s = make_state(oracle, 800 + kind, n_kv, kind)
    path = str(tmp_path / "ref.q4s")
    blob = reference_file_bytes(oracle, s, max_kv)
    open(path, "wb").write(blob)
    longer = np.concatenate([s["ids"], np.array([5, 6, 7], np.int32)])        # the caller's sequence continues

    store = q4gpu.KVStore(N_LAYERS, N_KVH, HD, max_kv, kind)
    d, keep = descriptor(for_read=s)
    assert store.sess_file_read(d, longer, path) == n_kv
    assert (d.pos, d.prompt_n, d.nmsg, d.user_hash, d.n_ids, d.idx_has_raw) == (s["pos"], s["prompt_n"], s["nmsg"],
                                                                               s["user_hash"], n_kv, 1)
    assert list(d.ple_hist) == [int(x) for x in s["ple"]]
    assert np.array_equal(keep[0], s["a"]) and np.array_equal(keep[1], s["b"]) and np.array_equal(keep[2], s["raw"])
    for l in range(N_LAYERS):
        assert exported(store, l, 0, n_kv) == oracle.kv_write(s["k"][l], kind).tobytes()
        assert exported(store, l, 1, n_kv) == oracle.kv_write(s["v"][l], kind).tobytes()
    # written back out it is the same file
    dw, _ = descriptor(s)
    back = str(tmp_path / "back.q4s")
    store.sess_file_write(n_kv, dw, back)
    assert open(back, "rb").read() == blob

    def refused(st, ids, p=path, tweak=None):
        dd, _k = descriptor(for_read=s)
        if tweak:
            tweak(dd)
        return st.sess_file_read(dd, ids, p) == 0

    assert refused(store, longer[:n_kv - 1])                                  # fewer ids than were saved
    bad = longer.copy(); bad[n_kv // 2] ^= 1
    assert refused(store, bad)                                                # prefix differs
    other_cap = q4gpu.KVStore(N_LAYERS, N_KVH, HD, max_kv + 1, kind)
    assert refused(other_cap, longer)                                         # other max_kv
    other_kind = q4gpu.KVStore(N_LAYERS, N_KVH, HD, max_kv, 0)
    assert refused(other_kind, longer)                                        # other KV kind
    assert refused(store, longer, tweak=lambda dd: setattr(dd, "bytes_total", 1))   # other model
    assert refused(store, longer, tweak=lambda dd: setattr(dd, "n_gdn", 3))
    trunc = str(tmp_path / "trunc.q4s")
    open(trunc, "wb").write(blob[:len(blob) // 2])
    marker = exported(store, 1, 0, n_kv)
    assert refused(store, longer, p=trunc)                                    # truncated: refused before anything is applied
    assert exported(store, 1, 0, n_kv) == marker
    for off, val in ((0, 0x12345678), (4, 4)):                                # magic, version
        b2 = bytearray(blob); struct.pack_into("<I", b2, off, val)
        open(trunc, "wb").write(bytes(b2))
        assert refused(store, longer, p=trunc)
    b2 = bytearray(blob); struct.pack_into("<I", b2, 28, n_kv - 1)            # n_kv != n_ids
    open(trunc, "wb").write(bytes(b2))
    assert refused(store, longer, p=trunc)
    assert not os.path.exists(str(tmp_path / "missing.q4s")) and refused(store, longer, p=str(tmp_path / "missing.q4s"))
    L.q4_gpu_last_error()
    for st in (store, other_cap, other_kind):
        st.close()


def test_kv_section_through_descriptors_pipe_and_file(oracle, tmp_path):
    """the KV section alone: a regular file (parallel pwrite / pread) and a pipe (in order) carry the same bytes"""
    lib()
    n_kv = 40000                                     # several 16 MiB chunks per plane
    s = make_state(oracle, 900, 64, 2)
    store = q4gpu.KVStore(2, N_KVH, HD, n_kv, 2)
    torch.manual_seed(9)
    rows = [torch.randn(n_kv, KVW, device="cuda") for _ in range(4)]
    for l in range(2):
        store.append(l, rows[2 * l], rows[2 * l + 1], 0, n_kv)
    want = b"".join(exported(store, l, w, n_kv) for l in range(2) for w in (0, 1))
    path = str(tmp_path / "kv.bin")
    fd = os.open(path, os.O_RDWR | os.O_CREAT)
    os.write(fd, b"HEAD")
    store.write_fd(n_kv, fd)
    assert os.lseek(fd, 0, os.SEEK_CUR) == 4 + len(want)
    os.close(fd)
    assert open(path, "rb").read() == b"HEAD" + want
    other = q4gpu.KVStore(2, N_KVH, HD, n_kv, 2)
    fd = os.open(path, os.O_RDONLY)
    os.lseek(fd, 4, os.SEEK_SET)
    other.read_fd(n_kv, fd)
    os.close(fd)
    assert b"".join(exported(other, l, w, n_kv) for l in range(2) for w in (0, 1)) == want
    # a pipe: sequential path
    import threading
    r, w = os.pipe()
    got = bytearray()

    def drain():
        while True:
            b = os.read(r, 1 << 20)
            if not b:
                break
            got.extend(b)
    t = threading.Thread(target=drain)
    t.start()
    store.write_fd(n_kv, w)
    os.close(w)
    t.join()
    os.close(r)
    assert bytes(got) == want
    store.close()
    other.close()
