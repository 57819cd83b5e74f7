"""Randomised shapes against the oracle under the 2 x SDPA-MATH rule: group sizes from 1 to 64 (with and without
head folding), odd lengths, Sq != Sk, packed batches with empty and one-token sequences, and workspace limits
from the minimum upwards (chunked backward). Seeds are fixed, so the cases are the same in every run."""
import random

import pytest
import torch

from gpu_utils import assert_status_ok, check_bwd, check_fwd, check_varlen, make_qkv

pytestmark = pytest.mark.gpu

GROUPS = [(1, 1), (2, 1), (4, 4), (8, 1), (8, 2), (6, 3), (12, 4), (16, 1), (32, 1), (64, 1), (32, 4), (3, 1), (128, 2), (5, 5)]


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_shapes(seed):
    from splitd_flash_attn import split_flash_attn_func, split_flash_attn_varlen_func
    from splitd_flash_attn.interface import set_backward_workspace_limit

    rng = random.Random(seed)
    old = set_backward_workspace_limit(None)
    try:
        for it in range(16):
            hq, hkv = rng.choice(GROUPS)
            packed = rng.random() < 0.4
            causal = rng.random() < 0.6
            set_backward_workspace_limit(rng.choice([None, None, 0, 1 << 20, 64 << 20]))
            if not packed:
                B = rng.choice([1, 1, 2, 3])
                sq = rng.choice([1, 2, 17, 64, 100, 128, 129, 255, 300, 513])
                sk = rng.choice([3, 64, 100, 128, 200, 256, 257, 400, 700])  # one key: see the test below
                if hq * sq * sk * B > 40e6:
                    sq = min(sq, 128)
                print(f"  batched B={B} Sq={sq} Sk={sk} Hq={hq} Hkv={hkv} causal={causal}")
                q, k, v, do = make_qkv(B, sq, sk, hq, hkv, torch.bfloat16, seed=100 * seed + it, requires_grad=True, with_do=True)
                out, lse = split_flash_attn_func(q, k, v, causal=causal, return_lse=True)
                dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
                check_fwd(out, lse, q, k, v, causal)
                check_bwd(dq, dk, dv, q, k, v, do, causal)
            else:
                nseq = rng.choice([1, 2, 5, 9, 33])
                lens_q = [rng.choice([0, 2, 5, 40, 64, 65, 130, 260]) for _ in range(nseq)]
                lens_k = lens_q if rng.random() < 0.7 else [rng.choice([0, 2, 7, 64, 100, 300]) for _ in range(nseq)]
                lens_q, lens_k = list(lens_q), list(lens_k)
                if sum(lens_q) == 0:
                    lens_q[0] = 5
                if sum(lens_k) == 0:
                    lens_k[0] = 6
                print(f"  packed q={lens_q} k={lens_k} Hq={hq} Hkv={hkv} causal={causal}")
                g = torch.Generator(device="cuda").manual_seed(100 * seed + it)
                mk = lambda t, h: torch.randn(t, h, 512, device="cuda", generator=g).to(torch.bfloat16)
                q, k, v, do = mk(sum(lens_q), hq), mk(sum(lens_k), hkv), mk(sum(lens_k), hkv), mk(sum(lens_q), hq)
                q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
                cq = torch.tensor([0] + torch.tensor(lens_q).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
                ck = torch.tensor([0] + torch.tensor(lens_k).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
                out, lse = split_flash_attn_varlen_func(q, k, v, cq, ck, max(lens_q), max(lens_k), causal=causal, return_lse=True)
                grads = torch.autograd.grad(out, (q, k, v), do)
                check_varlen(out, lse, grads, q, k, v, do, cq.tolist(), ck.tolist(), causal)
            assert_status_ok()
    finally:
        set_backward_workspace_limit(old)


@pytest.mark.parametrize("hq,hkv", [(8, 1), (128, 2), (4, 4)])
def test_single_key_gives_zero_dq_and_dk_up_to_accumulation_noise(hq, hkv):
    """With one key every probability is 1, dS = P (dP - rowsum(dO * O)) is exactly 0 and so are dq and dk. Here dP
    comes from the tensor cores and the row sum from a warp reduction, two fp32 sums of the same 512 products in
    different orders, so what is left is their rounding noise (~2^-19 of |dP| ~ 22): a few 1e-6 where the exact answer
    is 0. A math-backend SDPA and the fp32 oracle leave noise of the same kind (1e-6 to 1e-5); the ratio of two
    noise levels says nothing, hence an absolute bound here. dv (= the sum of dO over rows and heads) follows the rule."""
    from gpu_utils import sdpa_math
    from oracle import attention_oracle as O
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, do = make_qkv(2, 130, 1, hq, hkv, torch.bfloat16, seed=9, requires_grad=True, with_do=True)
    out = split_flash_attn_func(q, k, v)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    assert torch.equal(out, v.detach().repeat_interleave(hq // hkv, dim=2).expand_as(out))
    # dk adds that noise up over the 130 rows and the heads of the group
    assert dq.float().abs().max().item() <= 3e-5 and dk.float().abs().max().item() <= 3e-4
    rq, rk, rv = O.attention_bwd(q.detach(), k.detach(), v.detach(), do, False)
    assert rq.abs().max().item() <= 3e-5 and rk.abs().max().item() <= 3e-4
    _, _, _, yv = sdpa_math(q.detach(), k.detach(), v.detach(), False, do=do)
    assert (dv.float() - rv).abs().max().item() <= 2 * (yv.float() - rv).abs().max().item() + 1e-6
    assert_status_ok()
