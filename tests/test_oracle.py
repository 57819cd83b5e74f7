"""CPU: pin the oracle against golden vectors produced by the reference's own attention_ref + autograd
(tests/golden/make_golden.py) and check its internal consistency."""
import os

import numpy as np
import pytest
import torch

from oracle import attention_oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
D = 512


def _inputs(meta):
    B, sq, sk, hq, hkv, causal, seed, bf16_inputs = (int(x) for x in meta)
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, sq, hq, D, generator=gen)
    k = torch.randn(B, sk, hkv, D, generator=gen)
    v = torch.randn(B, sk, hkv, D, generator=gen)
    do = torch.randn(B, sq, hq, D, generator=gen)
    if bf16_inputs:
        q, k, v, do = (t.to(torch.bfloat16).float() for t in (q, k, v, do))
    return q, k, v, do, bool(causal)


@pytest.mark.parametrize("name", ["cfg1", "gqa_causal", "mha_tail", "cfg1_bf16", "gqa_causal_bf16"])
def test_oracle_matches_reference_golden(name):
    g = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    q, k, v, do, causal = _inputs(g["meta"])
    out, lse = O.attention_fwd(q, k, v, causal, D**-0.5)
    dq, dk, dv = O.attention_bwd(q, k, v, do, causal, D**-0.5)
    sub = lambda t: t[..., ::16].numpy()
    np.testing.assert_allclose(sub(out), g["out"], rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(lse.numpy(), g["lse"], rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(sub(dq), g["dq"], rtol=2e-4, atol=5e-5)
    np.testing.assert_allclose(sub(dk), g["dk"], rtol=2e-4, atol=5e-5)
    np.testing.assert_allclose(sub(dv), g["dv"], rtol=2e-4, atol=5e-5)


def test_oracle_bwd_matches_autograd_with_dlse():
    torch.manual_seed(3)
    q = torch.randn(1, 40, 4, D, dtype=torch.float64, requires_grad=True)
    k = torch.randn(1, 56, 2, D, dtype=torch.float64, requires_grad=True)
    v = torch.randn(1, 56, 2, D, dtype=torch.float64, requires_grad=True)
    do = torch.randn(1, 40, 4, D, dtype=torch.float64)
    dl = torch.randn(1, 4, 40, dtype=torch.float64)
    scale = 0.05
    kt = k.transpose(1, 2).repeat_interleave(2, dim=1)
    vt = v.transpose(1, 2).repeat_interleave(2, dim=1)
    s = torch.matmul(q.transpose(1, 2) * scale, kt.transpose(-2, -1))
    mask = torch.triu(torch.ones(40, 56, dtype=torch.bool), diagonal=56 - 40 + 1)
    s = s.masked_fill(mask, float("-inf"))
    out = torch.matmul(torch.softmax(s, -1), vt).transpose(1, 2)
    lse = torch.logsumexp(s, -1)
    gq, gk, gv = torch.autograd.grad((out, lse), (q, k, v), (do, dl))
    dq, dk, dv = O.attention_bwd(q.detach(), k.detach(), v.detach(), do, True, scale, dlse=dl, compute_dtype=torch.float64)
    for a, b in ((dq, gq), (dk, gk), (dv, gv)):
        assert (a - b).abs().max().item() < 1e-9


def test_oracle_fully_masked_rows():
    # causal with Sq > Sk: the first Sq-Sk rows see no key -> out 0, lse -inf (softmax.py:106-135)
    q = torch.randn(1, 8, 1, D)
    k = torch.randn(1, 4, 1, D)
    v = torch.randn(1, 4, 1, D)
    out, lse = O.attention_fwd(q, k, v, True)
    assert torch.all(out[0, :4] == 0) and torch.all(torch.isinf(lse[0, 0, :4]))
    assert torch.isfinite(lse[0, 0, 4:]).all()


def test_oracle_varlen_equals_per_sequence():
    torch.manual_seed(1)
    cu = [0, 5, 5, 18]
    q = torch.randn(18, 2, D)
    k = torch.randn(18, 1, D)
    v = torch.randn(18, 1, D)
    out, lse = O.attention_fwd_varlen(q, k, v, cu, cu, True)
    o0, l0 = O.attention_fwd(q[None, 5:18], k[None, 5:18], v[None, 5:18], True)
    assert torch.equal(out[5:18], o0[0]) and torch.equal(lse[:, 5:18], l0[0])


def test_flops_formula():
    # src/bench_utils.py:16-46: 4*B*H*Sq*Sk*D, causal halves when Sq == Sk
    assert O.attention_flops(16, 32, 1024, 1024, 512, False) == pytest.approx(1.0995e12, rel=1e-3)
    assert O.attention_flops(1, 32, 16384, 16384, 512, True) == pytest.approx(8.796e12, rel=1e-3)
