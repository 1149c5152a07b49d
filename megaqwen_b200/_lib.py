"""ctypes binding of libmegaqwen_b200.so (the C ABI in include/megaqwen_b200.h).

There is no fallback: if the shared library is missing this module raises at
import time, and the decoder refuses to run without CUDA.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MQ_LIB_PATH") or os.path.join(_HERE, "libmegaqwen_b200.so")

MQ_OK = 0
MQ_ERR = {-1: "bad argument", -2: "sequence too long for the cache or scratch", -3: "unsupported device or geometry",
          -4: "pointer not 16-byte aligned"}
MQ_STATUS_WAIT_TIMEOUT = 1
MQ_STATUS_BAD_POSITION = 2
MQ_STATUS_BAD_TOKEN = 4
MQ_FLAG_CHAINED = 1
MQ_FLAG_NO_PDL = 2


class MqLayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "input_layernorm", "q_proj", "k_proj", "v_proj", "q_norm", "k_norm", "o_proj",
        "post_attn_layernorm", "gate_proj", "up_proj", "down_proj")]


class MqModel(C.Structure):
    _fields_ = [("embed", C.c_void_p), ("layers", C.POINTER(MqLayerWeights)), ("final_norm", C.c_void_p),
                ("lm_head", C.c_void_p), ("cos_table", C.c_void_p), ("sin_table", C.c_void_p),
                ("num_layers", C.c_int), ("vocab_size", C.c_int), ("max_seq_len", C.c_int)]


class MqDecodeBuffers(C.Structure):
    _fields_ = [("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("hidden", C.c_void_p), ("qkv", C.c_void_p),
                ("attn_out", C.c_void_p), ("mlp_act", C.c_void_p), ("attn_partials", C.c_void_p),
                ("counters", C.c_void_p), ("argmax_slot", C.c_void_p), ("status", C.c_void_p),
                ("attn_nsplit", C.c_int)]


class MqPrefillBuffers(C.Structure):
    _fields_ = [("h", C.c_void_p), ("x", C.c_void_p), ("qkv", C.c_void_p), ("attn", C.c_void_p), ("act", C.c_void_p),
                ("max_tokens", C.c_int)]


class MqBatchBuffers(C.Structure):
    _fields_ = [("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("positions", C.c_void_p), ("logits", C.c_void_p),
                ("act", MqPrefillBuffers), ("status", C.c_void_p), ("batch", C.c_int), ("partials", C.c_void_p),
                ("partials_bytes", C.c_size_t), ("attn_parts", C.c_void_p), ("attn_parts_bytes", C.c_size_t),
                ("attn_tickets", C.c_void_p)]


class MqKvFp8(C.Structure):
    _fields_ = [("k_fp8", C.c_void_p), ("v_fp8", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p)]


# name -> (restype, argtypes); every symbol include/megaqwen_b200.h declares.
SIGNATURES = {
    "mq_abi_version": (C.c_int, []),
    "mq_init_device": (C.c_int, []),
    "mq_device_info": (C.c_int, [C.POINTER(C.c_int)] * 3),
    "mq_decode_attn_nsplit": (C.c_int, [C.c_int]),
    "mq_decode_partials_bytes": (C.c_size_t, [C.c_int]),
    "mq_decode_launch_count": (C.c_int, [C.c_int]),
    "mq_launch_decode": (C.c_int, [C.POINTER(MqModel), C.POINTER(MqDecodeBuffers), C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "mq_launch_decode_noalloc": (C.c_int, [C.POINTER(MqModel), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                           C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "mq_stream_packed_bytes": (C.c_size_t, [C.POINTER(MqModel)]),
    "mq_stream_pack": (C.c_int, [C.POINTER(MqModel), C.c_void_p, C.c_size_t, C.c_void_p]),
    "mq_stream_scratch_bytes": (C.c_size_t, []),
    "mq_stream_max_context": (C.c_int, []),
    "mq_stream_grid": (C.c_int, []),
    "mq_stream_stage_count": (C.c_int, []),
    "mq_launch_decode_stream": (C.c_int, [C.POINTER(MqModel), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int,
                                          C.c_void_p, C.c_void_p]),
    "mq_launch_prefill": (C.c_int, [C.POINTER(MqModel), C.POINTER(MqDecodeBuffers), C.POINTER(MqPrefillBuffers), C.c_void_p,
                                    C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "mq_launch_prefill_asr": (C.c_int, [C.POINTER(MqModel), C.POINTER(MqDecodeBuffers), C.POINTER(MqPrefillBuffers), C.c_void_p,
                                        C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "mq_launch_decode_batch": (C.c_int, [C.POINTER(MqModel), C.POINTER(MqBatchBuffers), C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_void_p]),
    "mq_launch_prefill_packed": (C.c_int, [C.POINTER(MqModel), C.POINTER(MqBatchBuffers)] + [C.c_void_p] * 7 +
                                 [C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "mq_decode_batch_launch_count": (C.c_int, [C.c_int]),
    "mq_launch_kv_quantize_fp8": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(MqKvFp8), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "mq_launch_decode_kv8": (C.c_int, [C.POINTER(MqModel), C.POINTER(MqDecodeBuffers), C.POINTER(MqKvFp8), C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "mq_launch_decode_batch_kv8": (C.c_int, [C.POINTER(MqModel), C.POINTER(MqBatchBuffers), C.POINTER(MqKvFp8), C.c_void_p, C.c_void_p,
                                             C.c_void_p, C.c_void_p]),
    "mq_prefill_launch_count": (C.c_int, [C.c_int]),
    "mq_launch_gemm_bf16": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                      C.c_int, C.c_void_p, C.c_void_p]),
    "mq_debug_gemm_drop_load": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_void_p, C.c_void_p, C.c_int]),
    "mq_launch_rms_norm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p]),
    "mq_launch_silu_mul": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p]),
    "mq_launch_rope": (C.c_int, [C.c_void_p] * 6 + [C.c_int] * 4 + [C.c_void_p]),
    "mq_launch_rope_single": (C.c_int, [C.c_void_p] * 4 + [C.c_int] * 3 + [C.c_void_p]),
    "mq_launch_attention_decode": (C.c_int, [C.c_void_p] * 4 + [C.c_int] * 6 + [C.c_float, C.c_void_p]),
    "mq_launch_fill_iota": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "mq_launch_find_first_eos": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
}


def load_library(path: str = LIB_PATH) -> C.CDLL:
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m megaqwen_b200.csrc.build` "
            "(there is no CPU or PyTorch fallback)")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = load_library()
    return _lib


def check(rc: int, what: str) -> None:
    if rc == MQ_OK:
        return
    if rc < 0:
        raise RuntimeError(f"{what}: {MQ_ERR.get(rc, 'error')} (code {rc})")
    raise RuntimeError(f"{what}: CUDA error {rc}")
