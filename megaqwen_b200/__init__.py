"""megaqwen_b200 — sm_100a Qwen3-0.6B greedy prefill + decode engine.

Drop-in for the hot path of the reference's ``megaqwen`` package: the decoder
object (``MegakernelDecoder`` / ``MegakernelPrefillDecoder``), the generators
and the weight-dict layout keep the reference's names and semantics; all
arithmetic runs in hand-written CUDA behind the C ABI of
``libmegaqwen_b200.so`` (see include/megaqwen_b200.h).  No Triton, no
multi-backend dispatch, no CPU fallback.
"""
from .spec import ModelSpec, QWEN3_0_6B, QWEN3_TINY  # noqa: F401


def __getattr__(name):
    # The decoder needs the shared library; import it lazily so that the pure
    # Python helpers (spec, synthetic weights) stay importable without it.
    if name in ("MegakernelDecoder", "MegakernelPrefillDecoder", "MegakernelFusedPrefillDecoder"):
        from . import decoder
        return getattr(decoder, name)
    if name in ("MegakernelGenerator", "MegakernelPrefillGenerator", "MegakernelFusedPrefillGenerator"):
        from . import generators
        return getattr(generators, name)
    if name == "load_qwen3_weights":
        from .weights import load_qwen3_weights
        return load_qwen3_weights
    raise AttributeError(name)
