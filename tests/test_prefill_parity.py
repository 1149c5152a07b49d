"""GPU parity of the prefill path: the tcgen05 GEMM against a torch fp32
reference of the same op, and the full-sequence forward against the CPU
restatement and the HF golden vectors."""
import ctypes as C

import pytest
import torch

from helpers import assert_logits_close, assert_tokens_match, load_golden, logit_report
from megaqwen_b200.spec import QWEN3_0_6B, QWEN3_TINY
from megaqwen_b200.synthetic import random_prompt, random_weights
from test_decode_parity import make_decoder

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,resid", [(128, 128, 64, False), (1024, 2048, 1024, False), (100, 1024, 2048, True),
                                         (1, 1024, 3072, True), (333, 3072, 1024, False)])
def test_tcgen05_gemm_matches_torch(M, N, K, resid):
    from megaqwen_b200 import _lib
    lib = _lib.lib()
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N + K)
    a = (torch.randn((M, K), generator=g) * 0.5).to(torch.bfloat16).cuda()
    b = (torch.randn((N, K), generator=g) * 0.05).to(torch.bfloat16).cuda()
    r = (torch.randn((M, N), generator=g)).to(torch.bfloat16).cuda() if resid else None
    c = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.mq_launch_gemm_bf16(a.data_ptr(), K, b.data_ptr(), c.data_ptr(), r.data_ptr() if resid else None, M, N, K, N,
                                 status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = (a.float() @ b.float().t()).to(torch.bfloat16)
    if resid:
        ref = (r.float() + ref.float()).to(torch.bfloat16)
    d = (c.float() - ref.float()).abs()
    # fp32 accumulation in a different order: isolated one-ulp bf16 flips only
    assert float((d > 0).float().mean()) < 2e-2, float((d > 0).float().mean())
    assert float(d.max()) <= 2 ** -5 * max(1.0, float(ref.float().abs().max()))


def test_gemm_operand_written_by_the_preceding_launch():
    """The library's own chains request weight tiles before the dependency wait; the public GEMM must not: its
    B operand may be what the launch just before it on the stream has written.  Twenty back-to-back pairs
    C1 = A1 B1^T, C2 = A2 C1^T with C1 overwritten by a different product each time."""
    from megaqwen_b200 import _lib
    lib = _lib.lib()
    g = torch.Generator(device="cpu").manual_seed(11)
    M1, K1, N2 = 256, 512, 384                      # C1 [M1, 1024] is GEMM 2's B: N = M1, K = 1024
    a2 = (torch.randn((N2, 1024), generator=g) * 0.1).to(torch.bfloat16).cuda()
    c1 = torch.zeros((M1, 1024), dtype=torch.bfloat16, device="cuda")
    c2 = torch.zeros((N2, M1), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for it in range(20):
        a1 = (torch.randn((M1, K1), generator=g) * 0.5).to(torch.bfloat16).cuda()
        b1 = (torch.randn((1024, K1), generator=g) * 0.05).to(torch.bfloat16).cuda()
        torch.cuda.synchronize()
        assert lib.mq_launch_gemm_bf16(a1.data_ptr(), K1, b1.data_ptr(), c1.data_ptr(), None, M1, 1024, K1, 1024, status.data_ptr(), stream) == 0
        assert lib.mq_launch_gemm_bf16(a2.data_ptr(), 1024, c1.data_ptr(), c2.data_ptr(), None, N2, M1, 1024, M1, status.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        ref1 = (a1.float() @ b1.float().t()).to(torch.bfloat16)
        assert float((c1.float() - ref1.float()).abs().max()) <= 2 ** -5 * max(1.0, float(ref1.float().abs().max()))
        ref2 = (a2.float() @ c1.float().t()).to(torch.bfloat16)          # against the C1 actually produced
        d = (c2.float() - ref2.float()).abs()
        assert float(d.max()) <= 2 ** -5 * max(1.0, float(ref2.float().abs().max())), (it, float(d.max()))
    assert int(status.item()) == 0


@pytest.mark.parametrize("drop_kb", [0, 9])
def test_expired_wait_sets_status_and_leaves_the_device_usable(drop_kb):
    """The error path every bounded device wait shares, made to run out on the host's terms: the GEMM's
    TMA producer is told never to request one k-block (a wait for something nothing will ever deliver).
    The kernel must come back by itself (about 0.2 s), report MQ_STATUS_WAIT_TIMEOUT, store nothing, and
    the same GEMM must be correct right afterwards once the sticky word is cleared."""
    import time
    from megaqwen_b200 import _lib
    lib = _lib.lib()
    M, N, K = 300, 512, 1024                      # 3 x 4 tiles, 16 k-blocks: drop_kb 9 lies beyond the 6-stage ring's first lap
    g = torch.Generator(device="cpu").manual_seed(5)
    a = (torch.randn((M, K), generator=g) * 0.5).to(torch.bfloat16).cuda()
    b = (torch.randn((N, K), generator=g) * 0.05).to(torch.bfloat16).cuda()
    c = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rc = lib.mq_debug_gemm_drop_load(a.data_ptr(), K, b.data_ptr(), c.data_ptr(), M, N, K, N, status.data_ptr(), stream, drop_kb)
    assert rc == 0
    torch.cuda.synchronize()                      # the kernel returned: no hang, no fault
    assert time.perf_counter() - t0 < 5.0
    assert int(status.item()) & _lib.MQ_STATUS_WAIT_TIMEOUT
    assert bool((c == 7.0).all())                 # nothing was stored from half-finished accumulators
    # bad arguments are refused on the host
    assert lib.mq_debug_gemm_drop_load(a.data_ptr(), K, b.data_ptr(), c.data_ptr(), M, N, K, N, status.data_ptr(), stream, K // 64) != 0
    # a second launch while the sticky bit is still set returns as well, and the bit stays until the host clears it
    # (waits that are satisfied anyway no longer look at it, so this launch may even compute its result)
    rc = lib.mq_launch_gemm_bf16(a.data_ptr(), K, b.data_ptr(), c.data_ptr(), None, M, N, K, N, status.data_ptr(), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) & _lib.MQ_STATUS_WAIT_TIMEOUT
    c.fill_(7.0)
    # cleared: the device, the tensor memory and the barriers are as good as new
    status.zero_()
    rc = lib.mq_launch_gemm_bf16(a.data_ptr(), K, b.data_ptr(), c.data_ptr(), None, M, N, K, N, status.data_ptr(), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = (a.float() @ b.float().t()).to(torch.bfloat16)
    d = (c.float() - ref.float()).abs()
    assert float((d > 0).float().mean()) < 2e-2 and float(d.max()) <= 2 ** -5 * max(1.0, float(ref.float().abs().max()))


@pytest.fixture(scope="module")
def tiny():
    return make_decoder(QWEN3_TINY, 2304)


@pytest.mark.parametrize("plen", [1, 17, 64, 300, 1000])
def test_tiny_prefill_matches_restatement(tiny, plen):
    from oracle.qwen3_restatement import RestatedQwen3
    dec, w = tiny
    prompt = random_prompt(QWEN3_TINY, plen, 12, plen)
    ref = RestatedQwen3(QWEN3_TINY, w, 2304)
    ref_lg = ref.forward(prompt)
    dec.reset()
    tok, lg = dec.prefill_step_logits(prompt)
    r = logit_report(lg.cpu(), ref_lg)
    assert r["max"] <= 6e-2 and r["mean"] <= 8e-3, (plen, r)
    assert dec.position() == plen
    kd, kr = dec.get_k_cache()[:, :, :plen].float().cpu(), ref.k_cache[:, :, :plen].float()
    vd, vr = dec.get_v_cache()[:, :, :plen].float().cpu(), ref.v_cache[:, :, :plen].float()
    assert (kd[0] - kr[0]).abs().max() <= 2 ** -5 and ((kd[0] != kr[0]).float().mean() < 2e-2)
    assert (vd[0] - vr[0]).abs().max() <= 2 ** -5 and ((vd[0] != vr[0]).float().mean() < 2e-2)
    assert (kd - kr).abs().mean() <= 4e-3 and (vd - vr).abs().mean() <= 4e-3
    assert float(dec.get_k_cache()[:, :, plen:].abs().max()) == 0.0
    # decode continues from the prefilled cache
    nxt, lg2 = dec.decode_step_logits(int(ref_lg.argmax()))
    ref_lg2 = ref.forward([int(ref_lg.argmax())])
    r2 = logit_report(lg2.cpu(), ref_lg2)
    assert r2["max"] <= 6e-2 and r2["mean"] <= 8e-3, (plen, r2)


@pytest.mark.parametrize("plen", [300, 1000])
def test_prefill_ignores_cache_rows_beyond_the_prompt(tiny, plen):
    """The attention's last key tile reaches past the prompt; what the cache holds there (here: NaN in K and
    V) belongs to nobody and must not reach the result: same logits, bit for bit, as over a zeroed cache."""
    dec, _ = tiny
    prompt = random_prompt(QWEN3_TINY, plen, 12, plen)
    dec.reset()
    _, clean = dec.prefill_step_logits(prompt)
    clean = clean.clone()
    dec.reset()
    dec.get_k_cache()[:, :, plen:] = float("nan")
    dec.get_v_cache()[:, :, plen:] = float("nan")
    _, lg = dec.prefill_step_logits(prompt)
    assert not bool(torch.isnan(lg).any())
    assert torch.equal(lg, clean)
    dec.reset()


def test_tiny_prefill_matches_hf_golden_and_decode_only_path(tiny):
    dec, _ = tiny
    g = load_golden("tiny_p300_n24")
    dec.reset()
    tok, lg = dec.prefill_step_logits(g["prompt"])
    assert_logits_close(lg.cpu()[None], g["logits"][:1], "tiny prefill vs HF")
    rows = [lg.cpu()]
    for t in g["tokens"][:-1]:
        _, l2 = dec.decode_step_logits(int(t))
        rows.append(l2.cpu())
    lgs = torch.stack(rows)
    assert_logits_close(lgs, g["logits"], "tiny prefill+decode vs HF")
    m = (g["top_vals"][:, 0] - g["top_vals"][:, 1]).tolist()
    assert_tokens_match(lgs.argmax(-1).tolist(), g["tokens"], m, "tiny prefill+decode")
    # chunked prefill (two calls) equals one call up to rounding
    dec.reset()
    dec.prefill_step(g["prompt"][:128])
    tok2, lgc = dec.prefill_step_logits(g["prompt"][128:], append=True)
    assert dec.position() == int(g["prompt"].numel())
    r = logit_report(lgc.cpu(), lg.cpu())
    assert r["max"] <= 6e-2 and r["mean"] <= 8e-3, r


@pytest.fixture(scope="module")
def full():
    return make_decoder(QWEN3_0_6B, 2304)


@pytest.mark.parametrize("name", ["full_cfg3_p1024_n32", "full_cfg2_p2048_n256"])
def test_full_prefill_then_decode_matches_hf_golden(full, name):
    dec, _ = full
    g = load_golden(name)
    n = len(g["tokens"])          # every recorded step: 32 for config 3, all 256 for config 2
    dec.reset()
    tok, lg = dec.prefill_step_logits(g["prompt"])
    rows = [lg.cpu()]
    for t in g["tokens"][:n - 1]:
        _, l2 = dec.decode_step_logits(int(t))
        rows.append(l2.cpu())
    lgs = torch.stack(rows)
    r1 = assert_logits_close(lgs[:, ::64], g["strided"][:n], name + " strided")
    r2 = assert_logits_close(torch.gather(lgs, 1, g["top_idx"][:n]), g["top_vals"][:n], name + " top-8")
    m = (g["top_vals"][:n, 0] - g["top_vals"][:n, 1]).tolist()
    same = assert_tokens_match(lgs.argmax(-1).tolist(), g["tokens"][:n], m, name)
    print(name, r1, r2, "tokens identical", same, "of", n)
