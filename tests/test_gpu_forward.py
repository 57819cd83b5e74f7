"""GPU parity of the forward kernel through the public API; parametrisation follows the reference's
test_splitd_fwd_correctness / test_splitd_lse (tests/test_flash_fwd_splitd_sdpa.py:264-331,534-582)."""
import math

import pytest
import torch

from gpu_utils import D, assert_status_ok, check_fwd, make_qkv

pytestmark = pytest.mark.gpu

SHAPES = [(64, 128), (128, 128), (256, 256), (113, 203), (512, 256), (1024, 1024)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("heads", [(6, 6), (6, 3), (6, 1)], ids=["mha", "gqa", "mqa"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sq,sk", SHAPES)
def test_fwd_correctness(dtype, heads, causal, sq, sk):
    from splitd_flash_attn import split_flash_attn_func

    hq, hkv = heads
    B = 2 if sq >= 1024 else 4
    q, k, v, _ = make_qkv(B, sq, sk, hq, hkv, dtype, seed=42)
    for pack in (None, True, False):
        out, lse = split_flash_attn_func(q, k, v, causal=causal, pack_gqa=pack, return_lse=True)
        assert out.shape == (B, sq, hq, D) and out.dtype == dtype
        assert lse.shape == (B, hq, sq) and lse.dtype == torch.float32
        check_fwd(out, lse, q, k, v, causal)
    assert_status_ok()


@pytest.mark.parametrize("sq,sk", [(128, 128), (1024, 1024), (2048, 2048), (113, 203)])
@pytest.mark.parametrize("causal", [False, True])
def test_lse_against_logsumexp(sq, sk, causal):
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, _ = make_qkv(4 if sq < 2048 else 1, sq, sk, 4, 4, torch.bfloat16, seed=0)
    _, lse = split_flash_attn_func(q, k, v, causal=causal, return_lse=True)
    scale = 1.0 / math.sqrt(D)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float() * scale, k.float())
    if causal:
        m = torch.triu(torch.ones(sq, sk, dtype=torch.bool, device="cuda"), diagonal=sk - sq + 1)
        s.masked_fill_(m, float("-inf"))
    ref = torch.logsumexp(s, dim=-1)
    assert (lse - ref).abs().max().item() <= 1e-3


def test_gqa_32_4_and_custom_scale():
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, _ = make_qkv(2, 333, 517, 32, 4, torch.bfloat16, seed=5)
    for scale in (None, 0.03):
        out, lse = split_flash_attn_func(q, k, v, softmax_scale=scale, causal=True, return_lse=True)
        check_fwd(out, lse, q, k, v, True, scale)
    assert_status_ok()


def test_causal_sq_greater_than_sk_has_empty_rows():
    """Bottom-right aligned mask with Sq > Sk: the first Sq-Sk rows see no key -> out 0, lse -inf."""
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, _ = make_qkv(2, 300, 172, 8, 2, torch.bfloat16, seed=9)
    out, lse = split_flash_attn_func(q, k, v, causal=True, return_lse=True)
    assert torch.all(out[:, : 300 - 172] == 0)
    assert torch.isinf(lse[:, :, : 300 - 172]).all() and (lse[:, :, : 300 - 172] < 0).all()
    check_fwd(out, lse, q, k, v, True)


def test_strided_head_slice_inputs_need_no_copy():
    """A (batch, kv-head group) shard of a larger tensor is a strided view; results must match."""
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, _ = make_qkv(2, 256, 256, 16, 2, torch.bfloat16, seed=11)
    full = split_flash_attn_func(q, k, v, causal=True)
    part = split_flash_attn_func(q[1:, :, 8:16], k[1:, :, 1:2], v[1:, :, 1:2], causal=True)
    assert torch.equal(part, full[1:, :, 8:16])


def test_deterministic():
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, _ = make_qkv(2, 700, 700, 8, 2, torch.bfloat16, seed=3)
    a = split_flash_attn_func(q, k, v, causal=True)
    b = split_flash_attn_func(q, k, v, causal=True)
    assert torch.equal(a, b)


def test_large_scores_trigger_accumulator_rescale():
    """Row maxima that keep growing along the keys force the in-TMEM rescale of O."""
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, _ = make_qkv(1, 128, 1024, 8, 1, torch.bfloat16, seed=21)
    ramp = torch.linspace(0.2, 3.0, 1024, device="cuda").view(1, 1024, 1, 1)
    k = (k * ramp).to(torch.bfloat16)
    out, lse = split_flash_attn_func(q, k, v, softmax_scale=0.2, return_lse=True)
    check_fwd(out, lse, q, k, v, False, 0.2)
