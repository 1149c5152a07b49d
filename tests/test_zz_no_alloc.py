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



def run_case(max_seq, prompt_len, start_pos=None):
    """Two steps in a row through both entry points on a max_seq-position cache.  With
    start_pos the steps run at that position over a cache of random values instead of after
    a prompt, so that a long context costs no long prefill."""
    from megaqwen_b200 import _lib
    from megaqwen_b200.decoder import MegakernelDecoder

    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    w = random_weights(QWEN3_TINY, max_seq)
    embed = w["embed_weight"].to(dev)
    dec = MegakernelDecoder(embed, [t.to(dev) for t in w["layer_weights"]], w["final_norm_weight"].to(dev), embed,
                            w["cos_table"].to(dev), w["sin_table"].to(dev), QWEN3_TINY.num_layers, max_seq, max_seq)
    dec.reset()
    if start_pos is None:
        first = dec.prefill_step(random_prompt(QWEN3_TINY, prompt_len, 11, 0))
    else:
        g = torch.Generator(device="cpu").manual_seed(3)
        dec.get_k_cache().copy_(torch.randn(dec.get_k_cache().shape, generator=g).to(torch.bfloat16))
        dec.get_v_cache().copy_(torch.randn(dec.get_v_cache().shape, generator=g).to(torch.bfloat16))
        dec.position_, first = start_pos, 17

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
        torch.cuda.synchronize(dev)
        # free bytes as the driver reports them (cudaMemGetInfo): this also sees an allocation made
        # by the library itself, which torch's allocator statistics would not.  The first call on a
        # device may load the kernels' code; the second call must leave the figure unchanged.
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc = lib.mq_launch_decode_noalloc(C.byref(dec._model), k2.data_ptr(), v2.data_ptr(), tok_in.data_ptr(),
                                          tok_out.data_ptr(), pos.data_ptr(), logits.data_ptr(), status.data_ptr(),
                                          0, stream)
        assert rc == 0, rc
        torch.cuda.synchronize(dev)
        if call == 1:
            assert torch.cuda.mem_get_info(dev)[0] == free_before
        assert int(status.item()) == 0
        assert int(tok_out.item()) == ref_tok, call
        assert torch.equal(logits, ref_logits), call
        assert torch.equal(k2[:, :, p], dec.get_k_cache()[:, :, p]) and torch.equal(v2[:, :, p], dec.get_v_cache()[:, :, p])
        cur = ref_tok


def test_noalloc_matches_regular_entry_point_twice():
    # a 200-token context in a 512-position cache: several KV splits, so the shared partial /
    # ticket scratch is really used
    run_case(512, 200)


def test_noalloc_at_its_maximum_cache_length():
    # the largest cache the static array is sized for: 64 KV splits, every one of them active
    # (context above 63 * 128 positions), partials filling the array up to the ticket words
    run_case(8192, 0, start_pos=8150)


def test_noalloc_rejects_oversized_cache():
    from megaqwen_b200 import _lib

    lib = _lib.lib()
    model = _lib.MqModel()
    model.max_seq_len = 8192 + 1
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    p = dummy.data_ptr()
    rc = lib.mq_launch_decode_noalloc(C.byref(model), p, p, p, p, p, None, p, 0, None)
    assert rc == -2
