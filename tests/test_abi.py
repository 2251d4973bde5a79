"""The C-ABI boundary without a GPU: the library loads, exports every symbol the header declares,
the Python signature table covers exactly those, and without a device every call fails cleanly
instead of falling back to anything."""
import ctypes
import os
import re

import pytest

import q4gpu


def header_functions():
    src = open(q4gpu.HEADER_PATH).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    names = re.findall(r"\b(q4_(?:hip|gpu)_\w+)\s*\(", src)
    return sorted(set(names))


def test_header_declares_the_reference_entry_points():
    names = header_functions()
    for must in ("q4_hip_init", "q4_hip_malloc", "q4_hip_f32_to_q8", "q4_hip_kv_append_d",
                 "q4_hip_qsa_decode_n", "q4_hip_qsa_decode_idx", "q4_hip_qsa_q_prep_d",
                 "q4_hip_pos_push", "q4_hip_graph_begin", "q4_gpu_kv_create", "q4_gpu_kv_append",
                 "q4_gpu_kv_decode", "q4_gpu_batch_decode", "q4_gpu_kv_save", "q4_gpu_lse_merge"):
        assert must in names


def test_library_exports_every_declared_symbol():
    assert os.path.exists(q4gpu.LIB_PATH), "libq4gpu.so not built"
    lib = ctypes.CDLL(q4gpu.LIB_PATH)
    for name in header_functions():
        assert hasattr(lib, name), name


def test_signature_table_matches_header():
    assert sorted(q4gpu.SIGNATURES) == header_functions()
    src = re.sub(r"/\*.*?\*/", "", open(q4gpu.HEADER_PATH).read(), flags=re.S)
    for name, (_, args) in q4gpu.SIGNATURES.items():
        m = re.search(r"\b%s\s*\(([^)]*)\)" % name, src)
        params = m.group(1).strip()
        n = 0 if params in ("void", "") else params.count(",") + 1
        assert n == len(args), name


def test_no_device_means_failure_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = q4gpu.load()
    assert L.q4_hip_init() is False
    assert L.q4_hip_ok() is False
    assert not L.q4_hip_malloc(64)
    buf = (ctypes.c_float * 64)()
    out = (ctypes.c_uint8 * 68)()
    assert L.q4_hip_f32_to_q8(out, buf, 64) is False
    assert L.q4_hip_qsa_decode_n(buf, buf, buf, buf, buf, 2, 1, 32, 1, 0, 1, 1.0, 2) is False
    assert not L.q4_gpu_kv_create(1, 2, 128, 16, 2)
    with pytest.raises(RuntimeError):
        q4gpu.init()
    with pytest.raises(RuntimeError):
        q4gpu.KVStore(1, 2, 128, 16)


def test_product_never_imports_the_oracle():
    root = os.path.dirname(os.path.dirname(q4gpu.HEADER_PATH))
    pkg = os.path.join(root, "suzuqu-engine-4exp_b200")
    for dp, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".h", ".cc", ".cpp")):
                txt = open(os.path.join(dp, f)).read()
                assert "q4_oracle" not in txt and "q4o_" not in txt and "oracle/" not in txt, f
