"""Standalone ops (C ABI) against the CPU restatement of the same stages."""
import pytest
import torch

from megaqwen_b200.synthetic import rope_tables
from oracle import qwen3_restatement as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def k():
    from megaqwen_b200.kernels import get_kernels
    return get_kernels()


def rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16)


def close(a, b, frac=2e-2, ulps=2 ** -6):
    d = (a.float().cpu() - b.float()).abs()
    assert float((d > 0).float().mean()) <= frac, float((d > 0).float().mean())
    assert float(d.max()) <= ulps * max(1.0, float(b.float().abs().max()))


@pytest.mark.parametrize("rows,cols", [(1, 1024), (37, 1024), (5, 128), (0, 1024), (3, 3072)])
def test_rms_norm(k, rows, cols):
    x, w = rand(rows, cols, seed=1), rand(cols, seed=2, scale=0.5) + 1
    out = k.rms_norm(x.cuda(), w.cuda(), 1e-6)
    assert out.shape == x.shape
    if rows:
        close(out, R.rms_norm(x, w, 1e-6), frac=5e-3)


@pytest.mark.parametrize("n", [1, 3072, 5 * 3072 + 7])
def test_silu_mul(k, n):
    g, u = rand(n, seed=3, scale=2.0), rand(n, seed=4)
    out = k.silu_mul(g.cuda(), u.cuda())
    close(out, R.silu_mul(g, u), frac=5e-3)


def test_rope_and_rope_single(k):
    cos, sin = rope_tables(64, 1e6, 128)
    q, kk = rand(2, 16, 9, 128, seed=5), rand(2, 8, 9, 128, seed=6)
    qo, ko = k.rope(q.cuda(), kk.cuda(), cos[:9].cuda(), sin[:9].cuda())
    c, s = cos[:9].view(1, 1, 9, 128), sin[:9].view(1, 1, 9, 128)
    assert torch.equal(qo.cpu(), R.rope(q, c, s)) and torch.equal(ko.cpu(), R.rope(kk, c, s))
    x = rand(16, 128, seed=7)
    out = k.rope_single(x.cuda(), cos.cuda(), sin.cuda(), 41)
    assert torch.equal(out.cpu(), R.rope(x, cos[41].view(1, 128), sin[41].view(1, 128)))
    with pytest.raises(RuntimeError, match="outside the RoPE table"):
        k.rope_single(x.cuda(), cos.cuda(), sin.cuda(), 64)


@pytest.mark.parametrize("cache_len", [1, 7, 200, 1500])
def test_attention_decode(k, cache_len):
    max_seq = 2048
    q = rand(2, 16, 1, 128, seed=8)
    kc, vc = rand(2, 8, max_seq, 128, seed=9), rand(2, 8, max_seq, 128, seed=10)
    out = k.attention_decode(q.cuda(), kc.cuda(), vc.cuda(), cache_len)
    for b in range(2):
        ref = R.attention_rows(q[b, :, 0].unsqueeze(0), kc[b, :, :cache_len], vc[b, :, :cache_len], cache_len - 1, 128 ** -0.5)
        close(out[b].reshape(1, -1), ref, frac=5e-2)
    with pytest.raises(RuntimeError):
        k.attention_decode(q.cuda(), kc.cuda(), vc.cuda(), max_seq + 1)


def test_dtype_checks(k):
    with pytest.raises(RuntimeError, match="must be bfloat16"):
        k.rms_norm(torch.zeros(2, 8, device="cuda"), torch.ones(8, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        k.silu_mul(torch.zeros(4, dtype=torch.bfloat16), torch.zeros(4, dtype=torch.bfloat16))
