"""GPU parity of the packed (varlen) layout, forward and backward, with ARBITRARY sequence lengths
(the reference rounds lengths to multiples of 64 in its varlen backward test,
tests/test_flash_fwd_splitd_sdpa.py:995-1002; the packed training-step configuration draws unrounded lengths)."""
import pytest
import torch

from gpu_utils import D, ERR_FACTOR, ATOL, assert_status_ok, max_err

from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


def _packed(lens, hq, hkv, seed, grad=False):
    T = sum(lens)
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda h: torch.randn(T, h, D, device="cuda", generator=g).to(torch.bfloat16)
    q, k, v, do = mk(hq), mk(hkv), mk(hkv), mk(hq)
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    if grad:
        q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    return q, k, v, do, cu


def _yard_fwd(q, k, v, cul, causal):
    errs = []
    for b in range(len(cul) - 1):
        s, e = cul[b], cul[b + 1]
        if e == s:
            continue
        ref, _ = O.attention_fwd(q[None, s:e], k[None, s:e], v[None, s:e], causal)
        errs.append(max_err(O.attention_math_lowp(q[None, s:e], k[None, s:e], v[None, s:e], causal), ref))
    return max(errs)


def _seeded_lengths(total, lo, hi, seed):
    g = torch.Generator().manual_seed(seed)
    lens, acc = [], 0
    while acc < total:
        n = int(torch.randint(lo, hi + 1, (1,), generator=g))
        n = min(n, total - acc)
        lens.append(n)
        acc += n
    return lens


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize(
    "lens,hq,hkv",
    [([128, 300, 77, 512], 8, 1), ([200, 1000, 333], 32, 4), ([64, 64], 4, 4), ([1, 15, 257], 6, 1), ([5, 0, 130], 8, 2)],
)
def test_varlen_fwd_bwd(lens, hq, hkv, causal):
    from splitd_flash_attn import split_flash_attn_varlen_func

    q, k, v, do, cu = _packed(lens, hq, hkv, seed=42, grad=True)
    out, lse = split_flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=causal, return_lse=True)
    assert out.shape == q.shape and lse.shape == (hq, sum(lens)) and lse.dtype == torch.float32
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    cul = cu.tolist()
    qd, kd, vd = q.detach(), k.detach(), v.detach()
    ro, rl = O.attention_fwd_varlen(qd, kd, vd, cul, cul, causal)
    rq, rk, rv = O.attention_bwd_varlen(qd, kd, vd, do, cul, cul, causal)
    yard = _yard_fwd(qd, kd, vd, cul, causal)
    assert max_err(out, ro) <= ERR_FACTOR * yard + ATOL
    assert (lse - rl).abs().max().item() <= 1e-3
    # gradients: same absolute bound the reference uses for its varlen backward (0.05-0.06)
    for name, got, ref in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        assert not torch.isnan(got).any()
        assert max_err(got, ref) <= 0.06, name
    assert_status_ok()


def test_varlen_different_q_and_k_lengths():
    from splitd_flash_attn import split_flash_attn_varlen_func

    ql, kl = [100, 37, 260], [300, 64, 260]
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn(sum(ql), 8, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(sum(kl), 2, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(sum(kl), 2, D, device="cuda", generator=g).to(torch.bfloat16)
    cq = torch.tensor([0, 100, 137, 397], dtype=torch.int32, device="cuda")
    ck = torch.tensor([0, 300, 364, 624], dtype=torch.int32, device="cuda")
    out, lse = split_flash_attn_varlen_func(q, k, v, cq, ck, 260, 300, causal=True, return_lse=True)
    ro, rl = O.attention_fwd_varlen(q, k, v, cq.tolist(), ck.tolist(), True)
    assert max_err(out, ro) <= 2e-2 and (lse - rl).abs().max().item() <= 1e-3


def test_varlen_config4_shape_reduced():
    """The packed training-step configuration's packing rule (uniform-integer lengths from a seed until the total is reached,
    last sequence truncated) at a reduced total so the oracle finishes in seconds."""
    from splitd_flash_attn import split_flash_attn_varlen_func

    lens = _seeded_lengths(4096, 128, 1500, seed=0)
    q, k, v, do, cu = _packed(lens, 32, 4, seed=1, grad=True)
    out = split_flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    cul = cu.tolist()
    ro, _ = O.attention_fwd_varlen(q.detach(), k.detach(), v.detach(), cul, cul, True)
    rq, rk, rv = O.attention_bwd_varlen(q.detach(), k.detach(), v.detach(), do, cul, cul, True)
    assert max_err(out, ro) <= 3e-2
    for got, ref in ((dq, rq), (dk, rk), (dv, rv)):
        assert max_err(got, ref) <= 0.06
    assert_status_ok()


def test_varlen_matches_batched_when_lengths_equal():
    from splitd_flash_attn import split_flash_attn_func, split_flash_attn_varlen_func

    B, S = 3, 192
    q, k, v, do, cu = _packed([S] * B, 8, 2, seed=8)
    a = split_flash_attn_varlen_func(q, k, v, cu, cu, S, S, causal=True)
    b = split_flash_attn_func(q.view(B, S, 8, D), k.view(B, S, 2, D), v.view(B, S, 2, D), causal=True)
    assert torch.equal(a.view(B, S, 8, D), b)
