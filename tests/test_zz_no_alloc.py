"""The allocation-free decode entry point against the regular one.

`mq_launch_decode_noalloc` exists for hosts that may not allocate device memory
after start-up (fixed-arena plug-ins, loops that cannot tolerate cudaMalloc's
device-wide synchronisation): it keeps the step's scratch in a static device
array inside the library.  This test calls it through the C ABI on buffers the
test owns, twice in a row, and requires the same token, logits and KV rows as
`mq_launch_decode` with caller-provided scratch (same kernels, so equality is
exact).  It is collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from megaqwen_b200.spec import QWEN3_TINY
from megaqwen_b200.synthetic import random_prompt, random_weights

pytestmark = pytest.mark.gpu

MAX_SEQ = 512


def test_noalloc_matches_regular_entry_point_twice():
    from megaqwen_b200 import _lib
    from megaqwen_b200.decoder import MegakernelDecoder

    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    w = random_weights(QWEN3_TINY, MAX_SEQ)
    embed = w["embed_weight"].to(dev)
    dec = MegakernelDecoder(embed, [t.to(dev) for t in w["layer_weights"]], w["final_norm_weight"].to(dev), embed,
                            w["cos_table"].to(dev), w["sin_table"].to(dev), QWEN3_TINY.num_layers, MAX_SEQ, MAX_SEQ)
    # a 200-token context, so that the attention runs several KV splits and the
    # shared partial / ticket scratch is really used
    prompt = random_prompt(QWEN3_TINY, 200, 11, 0)
    dec.reset()
    first = dec.prefill_step(prompt)

    # buffers of the allocation-free path: all created before the calls
    k2, v2 = dec.get_k_cache().clone(), dec.get_v_cache().clone()
    tok_in = torch.zeros(1, dtype=torch.int32, device=dev)
    tok_out = torch.zeros(1, dtype=torch.int32, device=dev)
    pos = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    logits = torch.zeros(QWEN3_TINY.vocab_size, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    cur = first
    for call in range(2):
        p = dec.position()
        ref_tok, ref_logits = dec.decode_step_logits(cur)
        tok_in.fill_(cur)
        pos.fill_(p)
        before = torch.cuda.memory_allocated(dev)
        rc = lib.mq_launch_decode_noalloc(C.byref(dec._model), k2.data_ptr(), v2.data_ptr(), tok_in.data_ptr(),
                                          tok_out.data_ptr(), pos.data_ptr(), logits.data_ptr(), status.data_ptr(),
                                          0, stream)
        assert rc == 0, rc
        torch.cuda.synchronize(dev)
        assert torch.cuda.memory_allocated(dev) == before
        assert int(status.item()) == 0
        assert int(tok_out.item()) == ref_tok, call
        assert torch.equal(logits, ref_logits), call
        assert torch.equal(k2[:, :, p], dec.get_k_cache()[:, :, p]) and torch.equal(v2[:, :, p], dec.get_v_cache()[:, :, p])
        cur = ref_tok


def test_noalloc_rejects_oversized_cache():
    from megaqwen_b200 import _lib

    lib = _lib.lib()
    model = _lib.MqModel()
    model.max_seq_len = 8192 + 1
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    p = dummy.data_ptr()
    rc = lib.mq_launch_decode_noalloc(C.byref(model), p, p, p, p, p, None, p, 0, None)
    assert rc == -2
