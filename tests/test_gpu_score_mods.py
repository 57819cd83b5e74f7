"""GPU: forward-only score modifiers -- softcap (tested by the reference in test_splitd_fwd_correctness,
tests/test_flash_fwd_splitd_sdpa.py:266,292-293,328) and sliding windows (interface.py:297-318; the reference
has no test for them, so these cases pin the semantics of src/testing.py:237-266)."""
import pytest
import torch

from gpu_utils import D, ATOL, ERR_FACTOR, assert_status_ok, check_fwd, make_qkv, max_err, rounding_yardstick

from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("heads", [(6, 6), (6, 3), (32, 4)])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sq,sk", [(128, 128), (113, 203), (512, 256), (1024, 1024)])
def test_softcap_forward(dtype, heads, causal, sq, sk):
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, _ = make_qkv(2, sq, sk, heads[0], heads[1], dtype, seed=42)
    out, lse = split_flash_attn_func(q, k, v, causal=causal, softcap=15.0, return_lse=True)
    ref, lref = O.attention_fwd(q, k, v, causal, softcap=15.0)
    # SDPA has no softcap: the yardstick is the exact result rounded once to the input dtype, which is what the
    # math backend's error amounts to (gpu_utils.rounding_yardstick). The reference allows 3x a looser figure here.
    yard = rounding_yardstick(ref, dtype)
    err = max_err(out, ref)
    assert err <= ERR_FACTOR * yard + ATOL, f"{err:.3e} vs yardstick {yard:.3e}"
    fin = torch.isfinite(lref)
    assert (lse - lref)[fin].abs().max().item() <= 1e-3
    assert_status_ok()


@pytest.mark.parametrize("window", [(64, 0), (100, 100), (0, 0), (300, None), (None, 37), (-1, 64), (1000, 1000)])
@pytest.mark.parametrize("sq,sk,heads", [(512, 512, (8, 2)), (300, 700, (32, 4)), (700, 300, (4, 4)), (1100, 1100, (6, 1))])
def test_sliding_window_forward(window, sq, sk, heads):
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, _ = make_qkv(2, sq, sk, heads[0], heads[1], torch.bfloat16, seed=7)
    out, lse = split_flash_attn_func(q, k, v, window_size=window, return_lse=True)
    w = tuple(None if (x is None or x < 0) else x for x in window)
    check_fwd(out, lse, q, k, v, False, window=w)
    assert_status_ok()


def test_window_varlen_and_softcap_together():
    from splitd_flash_attn import split_flash_attn_varlen_func

    lens = [200, 77, 513]
    g = torch.Generator(device="cuda").manual_seed(5)
    T = sum(lens)
    q = torch.randn(T, 8, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(T, 2, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(T, 2, D, device="cuda", generator=g).to(torch.bfloat16)
    cu = torch.tensor([0, 200, 277, 790], dtype=torch.int32, device="cuda")
    out = split_flash_attn_varlen_func(q, k, v, cu, cu, 513, 513, window_size=(128, 0), softcap=20.0)
    for b in range(3):
        s, e = int(cu[b]), int(cu[b + 1])
        ref, _ = O.attention_fwd(q[None, s:e], k[None, s:e], v[None, s:e], False, softcap=20.0, window=(128, 0))
        assert max_err(out[s:e], ref[0]) <= ERR_FACTOR * rounding_yardstick(ref[0], torch.bfloat16) + ATOL


def test_training_with_softcap_or_window_is_rejected():
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, _ = make_qkv(1, 128, 128, 4, 4, torch.bfloat16, seed=1, requires_grad=True)
    with pytest.raises(NotImplementedError, match="softcap"):
        split_flash_attn_func(q, k, v, softcap=15.0)
    with pytest.raises(NotImplementedError, match="window"):
        split_flash_attn_func(q, k, v, window_size=(16, 16))
