"""Helpers shared by the GPU parity tests: seeded inputs, error yardstick, acceptance rule.

Acceptance (stricter than the reference's own tests, which allow 2x-4x the 16-bit PyTorch error plus
an absolute slack, tests/test_flash_fwd_splitd_sdpa.py:300-331,790-809): the max-abs error of the CUDA
result against the fp32 oracle must be <= 2x the max-abs error of a 16-bit PyTorch math attention on the
same inputs (the "yardstick"), and |LSE - oracle LSE| <= 1e-3.
"""
import torch

from oracle import attention_oracle as O

D = 512
LSE_TOL = 1e-3
ERR_FACTOR = 2.0
ATOL = 1e-5


def make_qkv(B, sq, sk, hq, hkv, dtype, seed, requires_grad=False, with_do=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, sq, hq, D, device="cuda", dtype=torch.float32, generator=g).to(dtype)
    k = torch.randn(B, sk, hkv, D, device="cuda", dtype=torch.float32, generator=g).to(dtype)
    v = torch.randn(B, sk, hkv, D, device="cuda", dtype=torch.float32, generator=g).to(dtype)
    do = torch.randn(B, sq, hq, D, device="cuda", dtype=torch.float32, generator=g).to(dtype) if with_do else None
    if requires_grad:
        q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    return q, k, v, do


def max_err(a, b):
    return (a.float() - b.float()).abs().max().item()


def check_fwd(out, lse, q, k, v, causal, scale=None):
    ref, lref = O.attention_fwd(q.detach(), k.detach(), v.detach(), causal, scale)
    yard = max_err(O.attention_math_lowp(q.detach(), k.detach(), v.detach(), causal, scale), ref)
    err = max_err(out, ref)
    assert not torch.isnan(out).any()
    assert err <= ERR_FACTOR * yard + ATOL, f"out err {err:.3e} > {ERR_FACTOR} x yardstick {yard:.3e}"
    if lse is not None:
        finite = torch.isfinite(lref)
        assert torch.equal(torch.isfinite(lse), finite), "LSE -inf pattern differs"
        if finite.any():
            lerr = (lse - lref)[finite].abs().max().item()
            assert lerr <= LSE_TOL, f"lse err {lerr:.3e}"
    return err, yard


def yardstick_grads(q, k, v, do, causal, scale=None):
    q2, k2, v2 = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    o2 = O.attention_math_lowp(q2, k2, v2, causal, scale)
    return torch.autograd.grad(o2, (q2, k2, v2), do)


def check_bwd(dq, dk, dv, q, k, v, do, causal, scale=None):
    rq, rk, rv = O.attention_bwd(q.detach(), k.detach(), v.detach(), do, causal, scale)
    yq, yk, yv = yardstick_grads(q, k, v, do, causal, scale)
    for name, got, ref, y in (("dq", dq, rq, yq), ("dk", dk, rk, yk), ("dv", dv, rv, yv)):
        assert not torch.isnan(got).any(), name
        err, yard = max_err(got, ref), max_err(y, ref)
        assert err <= ERR_FACTOR * yard + ATOL, f"{name} err {err:.3e} > {ERR_FACTOR} x yardstick {yard:.3e}"


def assert_status_ok():
    from splitd_flash_attn.interface import kernel_status

    assert kernel_status() == 0, "a kernel gave up a bounded wait"
