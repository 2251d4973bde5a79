"""ctypes binding of libq4gpu (include/q4_gpu.h) plus a thin host-side mirror of the reference
engine's session KV interface (src/q4_fwd.c: kv_write / kv_at / qsa_attend / q4_sess_save).

Device memory, streams and process groups come from PyTorch; every byte of arithmetic on the
path is done by the CUDA library.  There is no fallback: if the shared library is missing or no
CUDA device is present, loading / init raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libq4gpu.so")
HEADER_PATH = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "include", "q4_gpu.h")

KIND_F32, KIND_F16, KIND_Q8 = 0, 1, 2
KIND_NAMES = {"f32": 0, "fp32": 0, "f16": 1, "fp16": 1, "q8": 2, "q8_0": 2}

_b, _v, _u32, _i32, _u64, _f, _sz, _i = (C.c_bool, C.c_void_p, C.c_uint32, C.c_int32, C.c_uint64,
                                        C.c_float, C.c_size_t, C.c_int)

# name -> (restype, argtypes); mirrors include/q4_gpu.h declaration by declaration
SIGNATURES = {
    "q4_hip_init": (_b, []), "q4_hip_shutdown": (None, []), "q4_hip_ok": (_b, []),
    "q4_hip_malloc": (_v, [_sz]), "q4_hip_free": (None, [_v]),
    "q4_hip_h2d": (_b, [_v, _v, _sz]), "q4_hip_d2h": (_b, [_v, _v, _sz]),
    "q4_hip_d2h_async": (_b, [_v, _v, _u64]), "q4_hip_h2d_async": (_b, [_v, _v, _u64]),
    "q4_hip_stream_sync": (_b, []),
    "q4_hip_copy_h2d": (_b, [_v, _v, _sz]), "q4_hip_copy_wait": (None, []), "q4_gpu_copy_stream": (_v, []),
    "q4_gpu_copy_d2h": (_b, [_v, _v, _sz]), "q4_gpu_download_stream": (_v, []),
    "q4_gpu_pipe_create": (_v, []), "q4_gpu_pipe_destroy": (None, [_v]),
    "q4_gpu_pipe_upload": (_b, [_v, _v, _v, _sz]), "q4_gpu_pipe_run": (_b, [_v, _v, _v, _v, _sz]),
    "q4_gpu_pipe_sync": (_b, [_v]),
    "q4_hip_copy": (_b, [_v, _v, _u64]), "q4_hip_fill": (_b, [_v, _f, _u64]),
    "q4_hip_sync": (None, []), "q4_hip_clear": (None, []),
    "q4_hip_pos_push": (None, [_i32]), "q4_hip_capturing": (_i, []), "q4_hip_pos_dev_ok": (_i, []),
    "q4_hip_graph_begin": (_i, []), "q4_hip_graph_end": (_v, []), "q4_hip_graph_nodes": (_u32, [_v]),
    "q4_hip_graph_launch": (_b, [_v]), "q4_hip_graph_free": (None, [_v]),
    "q4_hip_f32_to_f16": (_b, [_v, _v, _u64]), "q4_hip_f32_to_q8": (_b, [_v, _v, _u64]),
    "q4_hip_f32_to_f16_d": (_b, [_v, _u32, _v, _u64]),
    "q4_hip_kv_append_d": (_b, [_v, _v, _v, _v, _u32, _u32, _i]),
    "q4_hip_qsa_q_prep": (_b, [_v, _v, _v, _v, _u32, _u32, _u32, _i32, _f, _f]),
    "q4_hip_qsa_q_prep_n": (_b, [_v, _v, _v, _v, _u32, _u32, _u32, _i32, _f, _f, _u32]),
    "q4_hip_qsa_q_prep_d": (_b, [_v, _v, _v, _v, _u32, _u32, _u32, _f, _f]),
    "q4_hip_qsa_k_prep": (_b, [_v, _v, _u32, _u32, _u32, _i32, _f, _f]),
    "q4_hip_qsa_k_prep_n": (_b, [_v, _v, _u32, _u32, _u32, _i32, _f, _f, _u32]),
    "q4_hip_qsa_k_prep_d": (_b, [_v, _v, _u32, _u32, _u32, _f, _f]),
    "q4_hip_qsa_decode": (_b, [_v, _v, _v, _v, _v, _u32, _u32, _u32, _u32, _u32, _f, _i]),
    "q4_hip_qsa_decode_n": (_b, [_v, _v, _v, _v, _v, _u32, _u32, _u32, _u32, _u32, _u32, _f, _i]),
    "q4_hip_qsa_decode_idx": (_b, [_v, _v, _v, _v, _v, _v, _u32, _u32, _u32, _u32, _u32, _u32, _f, _i]),
    "q4_hip_qsa_topk_alloc": (_b, []),
    "q4_gpu_last_error": (_u32, []), "q4_gpu_stream": (_v, []), "q4_gpu_set_stream": (_b, [_v]),
    "q4_gpu_device": (_i, []), "q4_gpu_pos_word": (_v, []),
    "q4_gpu_kv_bytes": (_u64, [_u32, _u32, _u32, _u32, _i]),
    "q4_gpu_kv_create": (_v, [_u32, _u32, _u32, _u32, _i]), "q4_gpu_kv_destroy": (None, [_v]),
    "q4_gpu_kv_append": (_b, [_v, _u32, _v, _v, _u32, _u32]),
    "q4_gpu_kv_append_d": (_b, [_v, _u32, _v, _v]),
    "q4_gpu_kv_prep_append": (_b, [_v, _u32, _v, _v, _v, _u32, _f, _f, _u32, _u32]),
    "q4_gpu_kv_prep_append_d": (_b, [_v, _u32, _v, _v, _v, _u32, _f, _f]),
    "q4_gpu_kv_export": (_b, [_v, _u32, _i, _u32, _u32, _v]),
    "q4_gpu_kv_import": (_b, [_v, _u32, _i, _u32, _u32, _v]),
    "q4_gpu_kv_snapshot_bytes": (_u64, [_v, _u32]),
    "q4_gpu_kv_save": (_b, [_v, _u32, _v, _i]), "q4_gpu_kv_restore": (_b, [_v, _u32, _v, _i]),
    "q4_gpu_kv_write_fd": (_b, [_v, _u32, _i]), "q4_gpu_kv_read_fd": (_b, [_v, _u32, _i]),
    "q4_gpu_sess_file_bytes": (_u64, [_v, _u32, _v]),
    "q4_gpu_sess_file_write": (_b, [_v, _u32, _v, C.c_char_p]),
    "q4_gpu_sess_file_read": (_i, [_v, _v, _v, _i, C.c_char_p]),
    "q4_gpu_sess_file_peek_ids": (_i, [_v, C.c_char_p, _v, _i, _v, _v, _v]),
    "q4_gpu_kv_decode": (_b, [_v, _u32, _v, _i, _v, _v, _u32, _v, _u32, _u32, _u32, _f]),
    "q4_gpu_kv_decode_noalloc": (_b, [_v, _u32, _v, _i, _v, _v, _u32, _v, _u32, _u32, _u32, _f]),
    "q4_gpu_kv_decode_idx_n": (_b, [_v, _u32, _v, _i, _v, _v, _u32, _v, _u32, _u32, _u32, _u32, _f]),
    "q4_gpu_kv_decode_partial": (_b, [_v, _u32, _v, _i, _v, _u32, _v, _u32, _u32, _u32, _f]),
    "q4_gpu_lse_merge": (_b, [_v, _u32, _u32, _u32, _v, _v]),
    "q4_hip_qsa_pool": (_b, [_v, _v, _v, _u32, _u32, _u32, _u32, _u32, _f, _f]),
    "q4_hip_qsa_pool_d": (_b, [_v, _v, _v, _u32, _u32, _u32, _f, _f]),
    "q4_hip_qsa_score": (_b, [_v, _v, _v, _u32, _u32, _u32, _u32, _u32, _u32, _u32]),
    "q4_hip_qsa_score_d": (_b, [_v, _v, _v, _u32, _u32, _u32, _u32]),
    "q4_hip_qsa_topk": (_b, [_v, _v, _u32, _u32, _u32, _u32, _u32, _u32, _u32]),
    "q4_hip_qsa_topk_d": (_b, [_v, _v, _u32, _u32, _u32, _u32]),
    "q4_gpu_qsa_select_batch": (_b, [_v, _v, _v, _v, _v, _u32, _u32, _u32, _u32, _u32, _u32, _u32]),
    "q4_gpu_xchg_create": (_v, [_u32, _u32, _u32, _u32, _u32]), "q4_gpu_xchg_destroy": (None, [_v]),
    "q4_gpu_xchg_handle": (_b, [_v, _v]), "q4_gpu_xchg_window": (_v, [_v]),
    "q4_gpu_xchg_attach": (_b, [_v, _u32, _v]), "q4_gpu_xchg_attach_ptr": (_b, [_v, _u32, _v]),
    "q4_gpu_xchg_set_timeout_ms": (_b, [_v, _u32]),
    "q4_gpu_kv_decode_xchg": (_b, [_v, _v, _u32, _v, _i, _v, _v, _u32, _f, _i]),
    "q4_gpu_comm_unique_id": (_b, [_v]), "q4_gpu_comm_create": (_v, [_v, _u32, _u32]),
    "q4_gpu_comm_destroy": (None, [_v]), "q4_gpu_comm_allgather_merge": (_b, [_v, _v, _v, _u32, _u32, _v, _v]),
    "q4_gpu_kv_prefill": (_b, [_v, _u32, _v, _v, _v, _u32, _u32, _u32, _f]),
    "q4_gpu_batch_create": (_v, [_u32]), "q4_gpu_batch_destroy": (None, [_v]),
    "q4_gpu_batch_bind": (_b, [_v, _u32, _v]), "q4_gpu_batch_set_pos": (_b, [_v, _v, _u32]),
    "q4_gpu_batch_advance": (_b, [_v, _i32]),
    "q4_gpu_batch_append": (_b, [_v, _u32, _v, _v]),
    "q4_gpu_batch_decode": (_b, [_v, _u32, _v, _i, _v, _v, _v, _u32, _u32, _u32, _u32, _f]),
    "q4_gpu_batch_append_decode": (_b, [_v, _u32, _v, _v, _v, _i, _v, _v, _v, _u32, _u32, _u32, _u32, _f]),
    "q4_gpu_kv_append_decode_d": (_b, [_v, _u32, _v, _v, _v, _i, _v, _v, _u32, _v, _u32, _u32, _f]),
}

class SessDesc(C.Structure):
    """q4_gpu_sess_desc of include/q4_gpu.h: the host's part of a version-5 session file"""
    _fields_ = [("bytes_total", C.c_uint64), ("n_layer", C.c_uint32), ("n_expert", C.c_uint32), ("pos", C.c_uint32),
                ("n_gdn", C.c_uint32), ("n_v_h", C.c_uint32), ("d_v", C.c_uint32), ("conv_hist", C.c_uint32),
                ("conv_ch", C.c_uint32), ("hc_dim", C.c_uint32), ("prompt_n", C.c_uint32), ("nmsg", C.c_uint32),
                ("user_hash", C.c_uint64), ("ids", C.c_void_p), ("n_ids", C.c_uint32), ("ple_hist", C.c_int32 * 8),
                ("state_a", C.c_void_p), ("state_a_bytes", C.c_uint64), ("state_b", C.c_void_p),
                ("state_b_bytes", C.c_uint64), ("idx_dim", C.c_uint32), ("idx_has_raw", C.c_uint32),
                ("idx_raw", C.c_void_p), ("idx_raw_bytes", C.c_uint64)]


_lib = None


def load():
    """dlopen libq4gpu.so and type every entry point.  Raises if the library was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("libq4gpu.so is not built (%s): run __graft_entry__.build() or "
                               "`make -C suzuqu-engine-4exp_b200/csrc`; there is no fallback path" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def init():
    """q4_hip_init(); raises when no sm_100 device is usable."""
    L = load()
    if not L.q4_hip_init():
        raise RuntimeError("q4_hip_init failed: no usable CUDA device (libq4gpu has no CPU path)")
    return L


def _ptr(t):
    """Device (or host) address of a torch tensor / numpy array / int / None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


def check(ok, what):
    if not ok:
        raise RuntimeError("%s failed (status %#x)" % (what, load().q4_gpu_last_error()))


def use_torch_stream():
    """Run the library on torch's current CUDA stream so torch ops and library calls are ordered."""
    import torch
    # torch's default stream has handle 0; its explicit CUDA name is cudaStreamLegacy (0x1)
    check(load().q4_gpu_set_stream(torch.cuda.current_stream().cuda_stream or 1), "q4_gpu_set_stream")


class KVStore:
    """One session's KV cache in the library's planar layout -- the role of q4_sess's
    d_qsa_k / d_qsa_v / kv_kind / kv_bpt / max_kv fields (src/q4_fwd.c:26-57,1944-1950)."""

    def __init__(self, n_layers, n_kvh, hd, max_kv, kind=KIND_Q8):
        self.L = init()
        self.n_layers, self.n_kvh, self.hd, self.max_kv, self.kind = n_layers, n_kvh, hd, max_kv, kind
        self.h = self.L.q4_gpu_kv_create(n_layers, n_kvh, hd, max_kv, kind)
        if not self.h:
            raise RuntimeError("q4_gpu_kv_create failed (status %#x)" % self.L.q4_gpu_last_error())
        self.n_kv = 0

    def close(self):
        if self.h:
            self.L.q4_gpu_kv_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def token_bytes(self):
        """kv_token_bytes (src/q4_fwd.c:644-650): bytes per token per cache in the reference layout."""
        kvw = self.n_kvh * self.hd
        return kvw // 32 * 34 if self.kind == KIND_Q8 else kvw * (2 if self.kind == KIND_F16 else 4)

    def bytes(self):
        return self.L.q4_gpu_kv_bytes(self.n_layers, self.n_kvh, self.hd, self.max_kv, self.kind)

    def append(self, layer, k, v, pos0, n_tok):
        check(self.L.q4_gpu_kv_append(self.h, layer, _ptr(k), _ptr(v), pos0, n_tok), "q4_gpu_kv_append")

    def append_d(self, layer, k, v):
        check(self.L.q4_gpu_kv_append_d(self.h, layer, _ptr(k), _ptr(v)), "q4_gpu_kv_append_d")

    def export(self, layer, which, tok0, n_tok, dst):
        check(self.L.q4_gpu_kv_export(self.h, layer, which, tok0, n_tok, _ptr(dst)), "q4_gpu_kv_export")

    def import_(self, layer, which, tok0, n_tok, src):
        check(self.L.q4_gpu_kv_import(self.h, layer, which, tok0, n_tok, _ptr(src)), "q4_gpu_kv_import")

    def snapshot_bytes(self, n_kv):
        return self.L.q4_gpu_kv_snapshot_bytes(self.h, n_kv)

    def save(self, n_kv, buf, host=False):
        check(self.L.q4_gpu_kv_save(self.h, n_kv, _ptr(buf), int(host)), "q4_gpu_kv_save")

    def restore(self, n_kv, buf, host=False):
        check(self.L.q4_gpu_kv_restore(self.h, n_kv, _ptr(buf), int(host)), "q4_gpu_kv_restore")

    def write_fd(self, n_kv, fd):
        check(self.L.q4_gpu_kv_write_fd(self.h, n_kv, fd), "q4_gpu_kv_write_fd")

    def read_fd(self, n_kv, fd):
        check(self.L.q4_gpu_kv_read_fd(self.h, n_kv, fd), "q4_gpu_kv_read_fd")

    def sess_file_write(self, n_kv, desc, path):
        """the whole version-5 session file (q4_sess_save); desc: SessDesc"""
        check(self.L.q4_gpu_sess_file_write(self.h, n_kv, C.byref(desc), os.fsencode(path)), "q4_gpu_sess_file_write")

    def sess_file_read(self, desc, ids, path):
        """q4_sess_restore: the saved prefix length, or 0 when the file is refused; ids: int32 numpy array"""
        return self.L.q4_gpu_sess_file_read(self.h, C.byref(desc), ids.ctypes.data, len(ids), os.fsencode(path))

    def decode(self, layer, q, out, n_head, scale, gate=None, idx=None, width=0, idx_kvh_stride=0,
               n_kv=0, q_bf16=False):
        check(self.L.q4_gpu_kv_decode(self.h, layer, _ptr(q), int(q_bf16), _ptr(gate), _ptr(out), n_head,
                                      _ptr(idx), width, idx_kvh_stride, n_kv, scale), "q4_gpu_kv_decode")

    def prefill(self, layer, q_bf16, out_bf16, n_head, n_tok, kv_base, scale, gate=None):
        """causal attention of n_tok queries (bf16) over rows [0, kv_base + t + 1); bf16 output"""
        check(self.L.q4_gpu_kv_prefill(self.h, layer, _ptr(q_bf16), _ptr(gate), _ptr(out_bf16), n_head, n_tok,
                                       kv_base, scale), "q4_gpu_kv_prefill")

    def append_decode_d(self, layer, k, v, q, out, n_head, scale, gate=None, idx=None, width=0, idx_kvh_stride=0,
                        q_bf16=False):
        """append at the device position word + decode over rows [0, position] in one call"""
        check(self.L.q4_gpu_kv_append_decode_d(self.h, layer, _ptr(k), _ptr(v), _ptr(q), int(q_bf16), _ptr(gate),
                                               _ptr(out), n_head, _ptr(idx), width, idx_kvh_stride, scale),
              "q4_gpu_kv_append_decode_d")

    def decode_idx_n(self, layer, q, out, n_head, scale, idx, width, n_tok, idx_tok_stride, idx_kvh_stride=0,
                     gate=None, q_bf16=False):
        """sparse prefill: n_tok queries, each over the rows of its own list (one launch)"""
        check(self.L.q4_gpu_kv_decode_idx_n(self.h, layer, _ptr(q), int(q_bf16), _ptr(gate), _ptr(out), n_head,
                                            _ptr(idx), width, idx_kvh_stride, idx_tok_stride, n_tok, scale),
              "q4_gpu_kv_decode_idx_n")

    def decode_partial(self, layer, q, part, n_head, scale, idx=None, width=0, idx_kvh_stride=0, n_kv=0,
                       q_bf16=False):
        check(self.L.q4_gpu_kv_decode_partial(self.h, layer, _ptr(q), int(q_bf16), _ptr(part), n_head,
                                              _ptr(idx), width, idx_kvh_stride, n_kv, scale),
              "q4_gpu_kv_decode_partial")


class Exchange:
    """Exchange window of one rank of a sequence-sharded decode (q4_gpu_xchg_*): the decode kernel
    pushes its record into the peers' windows and merges theirs, one launch per layer."""
    FUSED, PUSH, MERGE = 0, 1, 2

    def __init__(self, rank, world, n_head, n_kvh, hd):
        self.L = init()
        self.rank, self.world = rank, world
        self.h = self.L.q4_gpu_xchg_create(rank, world, n_head, n_kvh, hd)
        if not self.h:
            raise RuntimeError("q4_gpu_xchg_create failed (status %#x)" % self.L.q4_gpu_last_error())

    def handle(self):
        """the 64-byte IPC handle of the local window"""
        buf = C.create_string_buffer(64)
        check(self.L.q4_gpu_xchg_handle(self.h, C.cast(buf, C.c_void_p)), "q4_gpu_xchg_handle")
        return bytes(buf.raw)

    def window(self):
        return self.L.q4_gpu_xchg_window(self.h)

    def attach(self, peer_rank, handle):
        buf = C.create_string_buffer(bytes(handle), 64)
        check(self.L.q4_gpu_xchg_attach(self.h, peer_rank, C.cast(buf, C.c_void_p)), "q4_gpu_xchg_attach")

    def attach_ptr(self, peer_rank, window):
        check(self.L.q4_gpu_xchg_attach_ptr(self.h, peer_rank, window), "q4_gpu_xchg_attach_ptr")

    def attach_all(self, dist):
        """exchange the handles over a torch.distributed process group (host side, once) and open them"""
        handles = [None] * self.world
        dist.all_gather_object(handles, self.handle())
        for r, hd_ in enumerate(handles):
            if r != self.rank:
                self.attach(r, hd_)
        dist.barrier()

    def set_timeout_ms(self, ms):
        check(self.L.q4_gpu_xchg_set_timeout_ms(self.h, ms), "q4_gpu_xchg_set_timeout_ms")

    def decode(self, store, layer, q, out, scale, n_kv, gate=None, q_bf16=False, phase=0):
        check(self.L.q4_gpu_kv_decode_xchg(store.h if store is not None else None, self.h, layer, _ptr(q),
                                           int(q_bf16), _ptr(gate), _ptr(out), n_kv, scale, phase),
              "q4_gpu_kv_decode_xchg")

    def close(self):
        if self.h:
            self.L.q4_gpu_xchg_destroy(self.h)
            self.h = None


class Comm:
    """NCCL communicator of the library (q4_gpu_comm_*), built from a unique id that the host distributes --
    here over a torch.distributed process group, by broadcast from rank 0."""

    def __init__(self, rank, world, dist=None):
        self.L = init()
        buf = C.create_string_buffer(128)
        if rank == 0:
            check(self.L.q4_gpu_comm_unique_id(C.cast(buf, C.c_void_p)), "q4_gpu_comm_unique_id")
        box = [bytes(buf.raw)]
        if world > 1:
            dist.broadcast_object_list(box, src=0)
        idbuf = C.create_string_buffer(box[0], 128)
        self.h = self.L.q4_gpu_comm_create(C.cast(idbuf, C.c_void_p), rank, world)
        if not self.h:
            raise RuntimeError("q4_gpu_comm_create failed (status %#x)" % self.L.q4_gpu_last_error())
        self.world = world

    def allgather_merge(self, part, parts_all, n_head, hd, out, gate=None):
        check(self.L.q4_gpu_comm_allgather_merge(self.h, _ptr(part), _ptr(parts_all), n_head, hd, _ptr(gate), _ptr(out)),
              "q4_gpu_comm_allgather_merge")

    def close(self):
        if self.h:
            self.L.q4_gpu_comm_destroy(self.h)
            self.h = None


class Batch:
    """Concurrent sessions decoded with one launch per layer."""

    def __init__(self, stores):
        self.L = init()
        self.stores = list(stores)
        self.h = self.L.q4_gpu_batch_create(len(self.stores))
        if not self.h:
            raise RuntimeError("q4_gpu_batch_create failed")
        for i, s in enumerate(self.stores):
            check(self.L.q4_gpu_batch_bind(self.h, i, s.h), "q4_gpu_batch_bind")

    def close(self):
        if self.h:
            self.L.q4_gpu_batch_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_pos(self, pos):
        arr = (C.c_int32 * len(pos))(*[int(p) for p in pos])
        check(self.L.q4_gpu_batch_set_pos(self.h, arr, len(pos)), "q4_gpu_batch_set_pos")

    def advance(self, delta=1):
        """pos[s] += delta on the device (capturable)"""
        check(self.L.q4_gpu_batch_advance(self.h, delta), "q4_gpu_batch_advance")

    def append(self, layer, k, v):
        check(self.L.q4_gpu_batch_append(self.h, layer, _ptr(k), _ptr(v)), "q4_gpu_batch_append")

    def decode(self, layer, q, out, n_head, scale, gate=None, idx=None, width=0, idx_kvh_stride=0,
               idx_sess_stride=0, q_bf16=False):
        check(self.L.q4_gpu_batch_decode(self.h, layer, _ptr(q), int(q_bf16), _ptr(gate), _ptr(out), _ptr(idx),
                                         width, idx_kvh_stride, idx_sess_stride, n_head, scale),
              "q4_gpu_batch_decode")

    def append_decode(self, layer, k, v, q, out, n_head, scale, gate=None, idx=None, width=0, idx_kvh_stride=0,
                      idx_sess_stride=0, q_bf16=False):
        """append + decode in one call (one launch per layer on a q8_0 store at hd 128)"""
        check(self.L.q4_gpu_batch_append_decode(self.h, layer, _ptr(k), _ptr(v), _ptr(q), int(q_bf16), _ptr(gate),
                                                _ptr(out), _ptr(idx), width, idx_kvh_stride, idx_sess_stride,
                                                n_head, scale), "q4_gpu_batch_append_decode")
