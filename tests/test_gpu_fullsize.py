"""GPU parity at the full sizes of the reference plan's configurations.

The fp32 oracle on a whole B*S = 16384 problem would need hours on a CPU, so these tests (a) run the oracle
ON THE GPU (it is device agnostic) for one sampled (batch, KV-head group) shard -- shards are independent, so
a shard of the full-size result can be checked exactly like a small problem -- and (b) check size-independent
properties on the full result: rows of softmax sum to one (V = ones gives out = 1), out is linear in V,
dV summed over keys equals the column sums of dO (because sum_j P_ij = 1), and LSE matches logsumexp.
"""
import pytest
import torch

from gpu_utils import D, assert_status_ok, max_err

from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu
HQ, HKV = 32, 4


def _inputs(B, S, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda h: torch.randn(B, S, h, D, device="cuda", generator=g).to(torch.bfloat16)
    return mk(HQ), mk(HKV), mk(HKV), mk(HQ)


@pytest.mark.parametrize("B,S", [(16, 1024), (4, 4096), (1, 16384)])
@pytest.mark.parametrize("causal", [False, True])
def test_sweep_shapes_forward_backward_shard_parity(B, S, causal):
    """The forward / backward sweep shapes: one (batch, kv-group) shard vs the oracle."""
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, do = _inputs(B, S, seed=S + causal)
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    out, lse = split_flash_attn_func(q, k, v, causal=causal, return_lse=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    assert_status_ok()
    b, g = B - 1, 2  # sampled shard
    sl = slice(g * 8, g * 8 + 8)
    qs, ks, vs, dos = q.detach()[b : b + 1, :, sl], k.detach()[b : b + 1, :, g : g + 1], v.detach()[b : b + 1, :, g : g + 1], do[b : b + 1, :, sl]
    ro, rl = O.attention_fwd(qs, ks, vs, causal)
    assert max_err(out[b : b + 1, :, sl], ro) <= 2e-2
    assert (lse[b : b + 1, sl] - rl).abs().max().item() <= 1e-3
    rq, rk, rv = O.attention_bwd(qs, ks, vs, dos, causal)
    assert max_err(dq[b : b + 1, :, sl], rq) <= 6e-2
    assert max_err(dk[b : b + 1, :, g : g + 1], rk) <= 6e-2
    assert max_err(dv[b : b + 1, :, g : g + 1], rv) <= 6e-2
    # property: sum over keys of dV[j, :] == sum over (rows, heads of the group) of dO[i, :]  (rows of P sum to 1)
    lhs = dv.float().sum(dim=1)  # (B, Hkv, D)
    rhs = do.float().view(B, S, HKV, 8, D).sum(dim=(1, 3))
    assert (lhs - rhs).abs().max().item() <= 2e-2 * rhs.abs().max().item() + 0.5
    for t in (out, dq, dk, dv):
        assert torch.isfinite(t).all()


@pytest.mark.parametrize("B,S,causal", [(2, 8192, True), (8, 2048, False)])
def test_softmax_rows_sum_to_one_and_linearity(B, S, causal):
    from splitd_flash_attn import split_flash_attn_func

    q, k, v, _ = _inputs(B, S, seed=3)
    ones = torch.ones_like(v)
    o1 = split_flash_attn_func(q, k, ones, causal=causal)
    assert (o1.float() - 1.0).abs().max().item() <= 8e-3  # bf16 rounding of P and of the output
    v2 = torch.randn_like(v)
    a = split_flash_attn_func(q, k, v, causal=causal).float()
    b = split_flash_attn_func(q, k, v2, causal=causal).float()
    c = split_flash_attn_func(q, k, (v.float() + v2.float()).to(torch.bfloat16), causal=causal).float()
    assert (a + b - c).abs().max().item() <= 5e-2
    assert_status_ok()


def test_config4_varlen_training_step_full_size():
    """The packed training-step configuration: packed causal fwd+bwd, lengths uniform-integer in [128, 8192] from a seed until the
    total reaches 32768 tokens (last sequence truncated), Hq=32, Hkv=4. Two sampled sequences are checked
    against the oracle per (sequence, kv group); everything must be finite."""
    from splitd_flash_attn import split_flash_attn_varlen_func

    gen = torch.Generator().manual_seed(0)
    lens, acc = [], 0
    while acc < 32768:
        n = min(int(torch.randint(128, 8193, (1,), generator=gen)), 32768 - acc)
        lens.append(n)
        acc += n
    T = 32768
    g = torch.Generator(device="cuda").manual_seed(4)
    mk = lambda h: torch.randn(T, h, D, device="cuda", generator=g).to(torch.bfloat16)
    q, k, v, do = mk(HQ), mk(HKV), mk(HKV), mk(HQ)
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    out, lse = split_flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True, return_lse=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    assert_status_ok()
    for t in (out, lse, dq, dk, dv):
        assert torch.isfinite(t).all()
    order = sorted(range(len(lens)), key=lambda i: lens[i])
    for i in (order[0], order[len(order) // 2]):  # shortest and a median-length sequence
        s, e = int(cu[i]), int(cu[i + 1])
        gq = 1
        sl = slice(gq * 8, gq * 8 + 8)
        qs, ks, vs = q.detach()[None, s:e, sl], k.detach()[None, s:e, gq : gq + 1], v.detach()[None, s:e, gq : gq + 1]
        ro, rl = O.attention_fwd(qs, ks, vs, True)
        rq, rk, rv = O.attention_bwd(qs, ks, vs, do[None, s:e, sl], True)
        assert max_err(out[s:e, sl], ro[0]) <= 3e-2
        assert (lse[sl, s:e] - rl[0]).abs().max().item() <= 1e-3
        assert max_err(dq[s:e, sl], rq[0]) <= 6e-2
        assert max_err(dk[s:e, gq : gq + 1], rk[0]) <= 6e-2
        assert max_err(dv[s:e, gq : gq + 1], rv[0]) <= 6e-2


def test_config5_layer_shards_equal_full_layer():
    """The 8-GPU layer configuration's sharding rule at a reduced sequence length: the 8 (batch, kv-group) shards of a
    B=2, Hq=32, Hkv=4 causal layer, run as independent calls on strided views, reproduce the unsharded
    result bit for bit (forward and backward)."""
    from splitd_flash_attn import sharding, split_flash_attn_func

    B, S = 2, 2048
    q, k, v, do = _inputs(B, S, seed=5)
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    out = split_flash_attn_func(q, k, v, causal=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    for (b, g) in sharding.layer_shards(B, HKV):
        qs, ks, vs = sharding.shard_views(q.detach(), k.detach(), v.detach(), (b, g), HQ, HKV)
        qs, ks, vs = qs.requires_grad_(True), ks.requires_grad_(True), vs.requires_grad_(True)
        os_ = split_flash_attn_func(qs, ks, vs, causal=True)
        gq, gk, gv = torch.autograd.grad(os_, (qs, ks, vs), do[b : b + 1, :, g * 8 : g * 8 + 8])
        assert torch.equal(os_, out[b : b + 1, :, g * 8 : g * 8 + 8])
        assert torch.equal(gq, dq[b : b + 1, :, g * 8 : g * 8 + 8])
        assert torch.equal(gk, dk[b : b + 1, :, g : g + 1]) and torch.equal(gv, dv[b : b + 1, :, g : g + 1])
    assert_status_ok()
