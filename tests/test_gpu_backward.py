"""GPU parity of the backward kernels (preprocess, dQ, dK/dV with GQA reduction) through autograd;
parametrisation follows test_splitd_bwd_correctness / test_splitd_bwd_gqa
(tests/test_flash_fwd_splitd_sdpa.py:731-809,882-944)."""
import pytest
import torch

from gpu_utils import assert_status_ok, check_bwd, check_fwd, make_qkv, max_err

pytestmark = pytest.mark.gpu

SHAPES = [(64, 128), (128, 128), (256, 256), (113, 203), (512, 256), (1024, 1024)]


def _run(B, sq, sk, hq, hkv, causal, seed, scale=None):
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, do = make_qkv(B, sq, sk, hq, hkv, torch.bfloat16, seed, requires_grad=True, with_do=True)
    out = split_flash_attn_func(q, k, v, softmax_scale=scale, causal=causal)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    assert dq.dtype == torch.bfloat16 and dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
    check_fwd(out, None, q, k, v, causal, scale)
    check_bwd(dq, dk, dv, q, k, v, do, causal, scale)
    assert_status_ok()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sq,sk", SHAPES)
def test_bwd_mha(sq, sk, causal):
    _run(2 if sq >= 1024 else 4, sq, sk, 4, 4, causal, seed=42)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sq,sk", [(128, 128), (256, 256), (113, 203), (600, 600)])
def test_bwd_gqa_32_4(sq, sk, causal):
    """Pins the reduction of dK/dV over the 8 query heads of each KV head."""
    _run(2, sq, sk, 32, 4, causal, seed=42)


@pytest.mark.parametrize("heads", [(6, 3), (6, 1), (12, 4)])
def test_bwd_other_group_sizes(heads):
    """6:1 (group 6 does not divide 64) exercises the non-folded path that loops query heads."""
    _run(2, 200, 264, heads[0], heads[1], True, seed=7, scale=0.05)


def test_bwd_with_lse_gradient():
    """lse is differentiable when returned (interface.py:1152-1158 of the reference)."""
    from splitd_flash_attn import split_flash_attn_func

    from oracle import attention_oracle as O

    q, k, v, do = make_qkv(2, 160, 160, 8, 2, torch.bfloat16, 13, requires_grad=True, with_do=True)
    out, lse = split_flash_attn_func(q, k, v, causal=True, return_lse=True)
    dl = torch.randn_like(lse)
    dq, dk, dv = torch.autograd.grad((out, lse), (q, k, v), (do, dl))
    rq, rk, rv = O.attention_bwd(q.detach(), k.detach(), v.detach(), do, True, None, dlse=dl)
    for got, ref in ((dq, rq), (dk, rk), (dv, rv)):
        assert max_err(got, ref) <= 0.06


def test_bwd_dout_none_gives_zero_grads():
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, _ = make_qkv(1, 128, 128, 4, 4, torch.bfloat16, 1, requires_grad=True)
    out, lse = split_flash_attn_func(q, k, v, return_lse=True)
    (dq,) = torch.autograd.grad(lse.sum(), (q,), allow_unused=True)
    assert dq is not None and torch.isfinite(dq).all()


def test_bwd_deterministic():
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, do = make_qkv(2, 384, 384, 16, 2, torch.bfloat16, 17, requires_grad=True, with_do=True)
    out = split_flash_attn_func(q, k, v, causal=True)
    a = torch.autograd.grad(out, (q, k, v), do, retain_graph=True)
    b = torch.autograd.grad(out, (q, k, v), do)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_config1_against_reference_golden():
    """The CPU plumbing configuration of the reference plan (B=1,S=256,Hq=8,Hkv=1, seed 0): CUDA result on the bf16-rounded inputs vs the
    fp32 golden vectors of the reference's attention_ref + autograd (tests/golden/cfg1.npz)."""
    import os

    import numpy as np

    from splitd_flash_attn import split_flash_attn_func

    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "cfg1.npz"))
    gen = torch.Generator().manual_seed(0)
    q = torch.randn(1, 256, 8, 512, generator=gen)
    k = torch.randn(1, 256, 1, 512, generator=gen)
    v = torch.randn(1, 256, 1, 512, generator=gen)
    do = torch.randn(1, 256, 8, 512, generator=gen)
    qc, kc, vc = (t.cuda().to(torch.bfloat16).requires_grad_(True) for t in (q, k, v))
    out, lse = split_flash_attn_func(qc, kc, vc, return_lse=True)
    dq, dk, dv = torch.autograd.grad(out, (qc, kc, vc), do.cuda().to(torch.bfloat16))
    sub = lambda t: t.detach().float().cpu()[..., ::16].numpy()
    # input rounding to bf16 (2^-9 relative) dominates these differences
    assert np.abs(sub(out) - g["out"]).max() < 2e-2
    assert np.abs(lse.detach().cpu().numpy() - g["lse"]).max() < 2e-2
    assert np.abs(sub(dq) - g["dq"]).max() < 5e-2
    assert np.abs(sub(dk) - g["dk"]).max() < 1e-1
    assert np.abs(sub(dv) - g["dv"]).max() < 1e-1


def test_one_pass_tile_kernel_agrees_with_default():
    """SPLITD_PDS_ONE_PASS=1 (read once per process, hence the child process) selects the single-launch P/dS
    kernel; its gradients must agree with the default two-pass path to bf16 rounding."""
    import os
    import subprocess
    import sys
    import tempfile

    code = r'''
import sys, torch
sys.path.insert(0, sys.argv[1])
from splitd_flash_attn import interface as I
torch.manual_seed(11)
B, S, HQ, HKV, D = 2, 640, 8, 2, 512
q = torch.randn(B, S, HQ, D, device="cuda", dtype=torch.bfloat16)
k = torch.randn(B, S, HKV, D, device="cuda", dtype=torch.bfloat16)
v = torch.randn(B, S, HKV, D, device="cuda", dtype=torch.bfloat16)
do = torch.randn(B, S, HQ, D, device="cuda", dtype=torch.bfloat16)
out, lse = I._flash_attn_fwd(q, k, v, causal=True, return_lse=True)
g = I._flash_attn_bwd(q, k, v, out, do, lse, causal=True)
torch.cuda.synchronize()
assert I.kernel_status() == 0
torch.save([t.float().cpu() for t in g], sys.argv[2])
'''
    pkg = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gemm4-attention-kernels_b200")
    res = []
    with tempfile.TemporaryDirectory() as tmp:
        for one_pass in ("0", "1"):
            path = os.path.join(tmp, f"g{one_pass}.pt")
            env = dict(os.environ, SPLITD_PDS_ONE_PASS=one_pass)
            subprocess.run([sys.executable, "-c", code, pkg, path], check=True, env=env, timeout=300)
            res.append(torch.load(path))
    for a, b in zip(*res):
        scale = a.abs().max().item()
        assert (a - b).abs().max().item() <= 2e-2 * scale  # both are bf16 results of the same fp32 quantities
