"""The C-ABI library loads without a GPU and exports every declared symbol."""
import ctypes
import os
import re

from megaqwen_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(mq_\w+)\s*\(", text))
    return names


def test_library_loads_and_exports_all(built_lib):
    lib = ctypes.CDLL(built_lib)
    decl = declared_symbols()
    assert len(decl) >= 8
    for name in decl:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    # the ctypes signature table covers exactly the declared entry points
    assert set(_lib.SIGNATURES) == decl


def test_pure_host_entry_points(built_lib):
    lib = _lib.load_library(built_lib)
    assert lib.mq_abi_version() >= 1
    assert lib.mq_decode_launch_count(28) == 5 * 28 + 1
    for max_seq in (64, 128, 2048, 2304, 4096, 8192):
        ns = lib.mq_decode_attn_nsplit(max_seq)
        assert 1 <= ns <= 64
        assert lib.mq_decode_partials_bytes(max_seq) == 16 * ns * 130 * 4


def test_argument_validation_without_gpu(built_lib):
    lib = _lib.load_library(built_lib)
    # null model / buffers are rejected before any CUDA call
    assert lib.mq_launch_decode(None, None, None, None, None, None, 0, None) == -1
    assert lib.mq_launch_fill_iota(None, 0, 4, None) == -1
    assert lib.mq_launch_find_first_eos(None, 4, None, 0, None, None) == -1


def test_struct_layout_matches_header():
    # 11 pointers, in the reference's LDGLayerWeights order
    assert ctypes.sizeof(_lib.MqLayerWeights) == 11 * 8
    assert [n for n, _ in _lib.MqLayerWeights._fields_][:4] == ["input_layernorm", "q_proj", "k_proj", "v_proj"]
    assert ctypes.sizeof(_lib.MqModel) == 6 * 8 + 3 * 4 + 4
    assert ctypes.sizeof(_lib.MqDecodeBuffers) == 10 * 8 + 8
