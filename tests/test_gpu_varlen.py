"""GPU parity of the packed (varlen) layout, forward and backward, with ARBITRARY sequence lengths
(the reference rounds lengths to multiples of 64 in its varlen backward test,
tests/test_flash_fwd_splitd_sdpa.py:995-1002; the packed training-step configuration draws unrounded lengths)."""
import pytest
import torch

from gpu_utils import D, ERR_FACTOR, ATOL, assert_status_ok, check_varlen, max_err, sdpa_math

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
    check_varlen(out, lse, (dq, dk, dv), q, k, v, do, cul, cul, causal)
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
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    do = torch.randn(sum(ql), 8, D, device="cuda", generator=g).to(torch.bfloat16)
    out, lse = split_flash_attn_varlen_func(q, k, v, cq, ck, 260, 300, causal=True, return_lse=True)
    grads = torch.autograd.grad(out, (q, k, v), do)
    check_varlen(out, lse, grads, q, k, v, do, cq.tolist(), ck.tolist(), True)
    assert_status_ok()


def test_varlen_config4_shape_reduced():
    """The packed training-step configuration's packing rule (uniform-integer lengths from a seed until the total is reached,
    last sequence truncated) at a reduced total so the oracle finishes in seconds."""
    from splitd_flash_attn import split_flash_attn_varlen_func

    lens = _seeded_lengths(4096, 128, 1500, seed=0)
    q, k, v, do, cu = _packed(lens, 32, 4, seed=1, grad=True)
    out, lse = split_flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True, return_lse=True)
    grads = torch.autograd.grad(out, (q, k, v), do)
    cul = cu.tolist()
    check_varlen(out, lse, grads, q, k, v, do, cul, cul, True)
    assert_status_ok()


def test_varlen_matches_batched_when_lengths_equal():
    from splitd_flash_attn import split_flash_attn_func, split_flash_attn_varlen_func

    B, S = 3, 192
    q, k, v, do, cu = _packed([S] * B, 8, 2, seed=8)
    a = split_flash_attn_varlen_func(q, k, v, cu, cu, S, S, causal=True)
    b = split_flash_attn_func(q.view(B, S, 8, D), k.view(B, S, 2, D), v.view(B, S, 2, D), causal=True)
    assert torch.equal(a.view(B, S, 8, D), b)


def test_varlen_without_host_synchronisation():
    """With the value checks of cu_seqlens switched off the packed forward + backward contains no blocking call:
    torch's sync debug mode turns any device->host synchronisation into an error. Results are unchanged."""
    from splitd_flash_attn import split_flash_attn_varlen_func
    from splitd_flash_attn.interface import cu_seqlens_validation

    lens = [200, 1000, 333]
    q, k, v, do, cu = _packed(lens, 8, 2, seed=4, grad=True)
    ref = split_flash_attn_varlen_func(q, k, v, cu, cu, 1000, 1000, causal=True)
    rg = torch.autograd.grad(ref, (q, k, v), do)
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        with cu_seqlens_validation(False):
            out = split_flash_attn_varlen_func(q, k, v, cu, cu, 1000, 1000, causal=True)
            grads = torch.autograd.grad(out, (q, k, v), do)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    assert torch.equal(out, ref)
    for a, b in zip(grads, rg):
        assert torch.equal(a, b)
    assert_status_ok()


def test_c_abi_reports_a_sequence_longer_than_max_seqlen_k():
    """A C-ABI caller that understates max_seqlen_k gets rows that are too short for its longest sequence. The
    kernels must not write past them: they skip that sequence and store code 106 in the status word."""
    import ctypes

    from splitd_flash_attn import _capi
    from splitd_flash_attn import interface as I

    lens = [100, 700]
    q, k, v, do, cu = _packed(lens, 8, 2, seed=6)
    out, lse = I._flash_attn_fwd(q, k, v, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=700, max_seqlen_k=700,
                                 causal=True, return_lse=True)
    p = I._fill_params(q, k, v, out, lse, cu, cu, 700, 256, D**-0.5, True)  # 256 < 700
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    p.status_flag = ctypes.c_void_p(status.data_ptr())
    grads = [torch.zeros_like(t) for t in (q, k, v)]
    p.dout = ctypes.c_void_p(do.data_ptr())
    p.dq, p.dk, p.dv = (ctypes.c_void_p(t.data_ptr()) for t in grads)
    for name, t in (("do_strides", do), ("dq_strides", grads[0]), ("dk_strides", grads[1]), ("dv_strides", grads[2])):
        getattr(p, name)[:] = I._strides3(t, True)
    lib = _capi.load_library()
    stat = torch.empty(2 * lib.splitd_bwd_rowstat_elems(ctypes.byref(p)), device="cuda")
    n_ws = lib.splitd_bwd_workspace_bytes(ctypes.byref(p))
    ws = torch.full((n_ws + 4096,), 0x5A, dtype=torch.uint8, device="cuda")  # guard band behind the workspace
    p.dpsum = ctypes.c_void_p(stat.data_ptr())
    p.lse_log2 = ctypes.c_void_p(stat.data_ptr() + stat.numel() * 2)
    p.workspace, p.workspace_bytes = ctypes.c_void_p(ws.data_ptr()), n_ws
    assert lib.splitd_bwd(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 106
    assert torch.all(ws[n_ws:] == 0x5A)
    # the sequence that fits was processed
    ro = O.attention_bwd(q[None, :100], k[None, :100], v[None, :100], do[None, :100], True)
    assert max_err(grads[0][:100], ro[0][0]) <= 0.05
