"""GPU parity of the speech hook: prefill with a span of the embedded prompt replaced by external
embeddings (reference: prefill_asr, csrc/megakernel/bindings_prefill.cpp:835-955)."""
import pytest
import torch

from helpers import logit_report
from megaqwen_b200.spec import QWEN3_TINY
from megaqwen_b200.synthetic import random_prompt, random_weights
from test_decode_parity import make_decoder

pytestmark = pytest.mark.gpu


def test_prefill_asr_matches_restatement_and_checks_arguments():
    from oracle.qwen3_restatement import RestatedQwen3
    dec, w = make_decoder(QWEN3_TINY, 512)
    prompt = random_prompt(QWEN3_TINY, 150, 13, 0)
    g = torch.Generator().manual_seed(5)
    audio = (torch.randn((97, 1024), generator=g) * 0.02).to(torch.bfloat16)
    start = 20
    ref = RestatedQwen3(QWEN3_TINY, w, 512)
    ref_lg = ref.forward(prompt, patch=(start, audio))
    dec.reset()
    tok = dec.prefill_asr(prompt, audio.cuda(), start)
    assert dec.position() == 150
    top = ref_lg.topk(2).values
    assert tok == int(ref_lg.argmax()) or float(top[0] - top[1]) <= 6.25e-2
    # the cache holds the patched sequence: the next step's logits agree with the restatement's
    nxt = int(ref_lg.argmax())
    _, lg = dec.decode_step_logits(nxt)
    r = logit_report(lg.cpu(), ref.forward([nxt]))
    assert r["max"] <= 6e-2 and r["mean"] <= 8e-3, r
    kd, kr = dec.get_k_cache()[:, :, :150].float().cpu(), ref.k_cache[:, :, :150].float()
    assert (kd[0] - kr[0]).abs().max() <= 2 ** -5 and (kd - kr).abs().mean() <= 4e-3
    # without the patch the result differs (the span really was replaced)
    dec.reset()
    dec.prefill_step(prompt)
    assert not torch.equal(dec.get_k_cache()[0, :, start:start + 97].cpu(), kd[0, :, start:start + 97].to(torch.bfloat16))
    # argument checks, with the reference's texts
    a = audio.cuda()
    with pytest.raises(RuntimeError, match="audio_embeds must be a CUDA bfloat16 2D tensor"):
        dec.prefill_asr(prompt, audio, start)
    with pytest.raises(RuntimeError, match="hidden_size mismatch"):
        dec.prefill_asr(prompt, a[:, :512].contiguous(), start)
    with pytest.raises(RuntimeError, match="Invalid audio_start_idx/audio_len"):
        dec.prefill_asr(prompt, a, 100)
    with pytest.raises(RuntimeError, match="audio_embeds must have audio_len > 0"):
        dec.prefill_asr(prompt, a[:0], 0)
    with pytest.raises(RuntimeError, match="Empty input sequence"):
        dec.prefill_asr(torch.zeros(0, dtype=torch.int32), a, 0)
    dec.check_status()
