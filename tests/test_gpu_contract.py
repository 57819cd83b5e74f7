"""API contract of the two public functions on a GPU; restates the reference's contract tests
(tests/test_flash_fwd_splitd_sdpa.py:339-526): return shapes/dtypes, exception types and messages."""
import pytest
import torch

pytestmark = pytest.mark.gpu
D = 512


def _t(*shape, dtype=torch.bfloat16):
    return torch.randn(*shape, device="cuda", dtype=dtype)


def test_return_shapes_batched():
    from splitd_flash_attn import split_flash_attn_func

    q, k, v = _t(2, 128, 4, D), _t(2, 128, 2, D), _t(2, 128, 2, D)
    out = split_flash_attn_func(q, k, v)
    assert isinstance(out, torch.Tensor) and out.shape == (2, 128, 4, D)
    out, lse = split_flash_attn_func(q, k, v, return_lse=True)
    assert lse.shape == (2, 4, 128) and lse.dtype == torch.float32


def test_return_shapes_varlen():
    from splitd_flash_attn import split_flash_attn_varlen_func

    cu = torch.tensor([0, 100, 256], dtype=torch.int32, device="cuda")
    q, k, v = _t(256, 4, D), _t(256, 2, D), _t(256, 2, D)
    out = split_flash_attn_varlen_func(q, k, v, cu, cu, 156, 156)
    assert out.shape == (256, 4, D)
    out, lse = split_flash_attn_varlen_func(q, k, v, cu, cu, 156, 156, return_lse=True)
    assert lse.shape == (4, 256) and lse.dtype == torch.float32


@pytest.mark.parametrize("dq,dv", [(384, 384), (512, 384)])
def test_rejects_other_head_dims(dq, dv):
    from splitd_flash_attn import split_flash_attn_func

    with pytest.raises(ValueError, match="head_dim == 512"):
        split_flash_attn_func(_t(1, 64, 2, dq), _t(1, 64, 2, dq), _t(1, 64, 2, dv))


def test_rejects_int64_cu_seqlens():
    from splitd_flash_attn import split_flash_attn_varlen_func

    cu = torch.tensor([0, 64], dtype=torch.int64, device="cuda")
    with pytest.raises(TypeError, match="int32"):
        split_flash_attn_varlen_func(_t(64, 2, D), _t(64, 2, D), _t(64, 2, D), cu, cu, 64, 64)


def test_fp16_training_is_rejected():
    from splitd_flash_attn import split_flash_attn_func

    q = _t(1, 64, 2, D, dtype=torch.float16).requires_grad_(True)
    with pytest.raises(NotImplementedError, match="bfloat16 only"):
        split_flash_attn_func(q, _t(1, 64, 2, D, dtype=torch.float16), _t(1, 64, 2, D, dtype=torch.float16))


def test_missing_max_seqlen():
    from splitd_flash_attn import split_flash_attn_varlen_func

    cu = torch.tensor([0, 64], dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="max_seqlen_q"):
        split_flash_attn_varlen_func(_t(64, 2, D), _t(64, 2, D), _t(64, 2, D), cu, cu, None, 64)


@pytest.mark.parametrize(
    "vals,msg", [([1, 64], r"\[0\] must be 0"), ([0, 63], "total tokens"), ([0, 40, 30, 64], "non-decreasing")]
)
def test_bad_cu_seqlens_values(vals, msg):
    from splitd_flash_attn import split_flash_attn_varlen_func

    cu = torch.tensor(vals, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match=msg):
        split_flash_attn_varlen_func(_t(64, 2, D), _t(64, 2, D), _t(64, 2, D), cu, cu, 64, 64)


def test_too_small_max_seqlen():
    from splitd_flash_attn import split_flash_attn_varlen_func

    cu = torch.tensor([0, 50, 64], dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="max_seqlen_q"):
        split_flash_attn_varlen_func(_t(64, 2, D), _t(64, 2, D), _t(64, 2, D), cu, cu, 20, 64)


def test_window_resolution_on_device():
    from splitd_flash_attn import split_flash_attn_func

    q, k, v = _t(1, 64, 2, D), _t(1, 64, 2, D), _t(1, 64, 2, D)
    with pytest.raises(ValueError, match="mutually exclusive"):
        split_flash_attn_func(q, k, v, causal=True, window_size=(16, 0))
    # (-1, 0) is the causal window, (-1, -1) the full one (interface.py:297-318 of the reference)
    a = split_flash_attn_func(q, k, v, window_size=(-1, 0))
    b = split_flash_attn_func(q, k, v, causal=True)
    assert torch.equal(a, b)


def test_heads_must_divide():
    from splitd_flash_attn import split_flash_attn_func

    with pytest.raises(ValueError, match="divisible"):
        split_flash_attn_func(_t(1, 64, 6, D), _t(1, 64, 4, D), _t(1, 64, 4, D))


def test_c_abi_rejects_missing_workspace():
    """The C-ABI itself reports a too-small backward workspace instead of launching."""
    import ctypes

    from splitd_flash_attn import _capi
    from splitd_flash_attn import interface as I

    q, k, v = _t(1, 128, 2, D), _t(1, 128, 2, D), _t(1, 128, 2, D)
    out, lse = I._flash_attn_fwd(q, k, v, return_lse=True)
    p = I._fill_params(q, k, v, out, lse, None, None, None, None, 0.05, False)
    g = torch.empty_like(q)
    stat = torch.empty(2 * 128, device="cuda")
    p.dout = p.dq = ctypes.c_void_p(g.data_ptr())
    p.dk = p.dv = ctypes.c_void_p(g.data_ptr())
    p.dpsum = p.lse_log2 = ctypes.c_void_p(stat.data_ptr())
    p.do_strides[:] = p.dq_strides[:] = p.dk_strides[:] = p.dv_strides[:] = I._strides3(g, False)
    lib = _capi.load_library()
    tiles = 2 * 2 * 128 * (256 + 64) * 2  # 2 head units x (P, dS) x 128 rows x (256 keys + 64 of padding) x fp16
    copies = 2 * q.numel() * 2 + k.numel() * 2  # fp16 dO, Q, K
    full = lib.splitd_bwd_workspace_bytes_limit(ctypes.byref(p), ctypes.c_size_t(-1).value)
    assert tiles + copies < full <= tiles + copies + 4096  # + work counters and per-group maxima
    assert lib.splitd_bwd_workspace_bytes(ctypes.byref(p)) == full  # small problem: everything at once
    assert lib.splitd_bwd_workspace_bytes_limit(ctypes.byref(p), 0) > copies
    assert lib.splitd_bwd_dq(ctypes.byref(p), None) == -5
    assert lib.splitd_bwd(ctypes.byref(p), None) == -5
    ws = torch.empty(full, dtype=torch.uint8, device="cuda")
    p.workspace, p.workspace_bytes = ctypes.c_void_p(ws.data_ptr()), full - 4096
    assert lib.splitd_bwd_dq(ctypes.byref(p), None) == -5  # the two-call form needs the whole problem at once
    assert b"splitd_bwd_chunk" in lib.splitd_last_error()


def test_a_wait_that_runs_out_ends_the_kernel_and_leaves_the_gpu_usable():
    """Every wait in the kernels is bounded. This runs that code to its limit on purpose, in the harmless form the
    library exports for it: one small CTA waits 2 ms on a barrier nobody arrives on, then reports code 104 through
    the status word and ends normally. Afterwards a real forward + backward on the same device still passes."""
    import ctypes

    from splitd_flash_attn import _capi, split_flash_attn_func

    lib = _capi.load_library()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.splitd_wait_probe(ctypes.c_void_p(status.data_ptr()), 2000, ctypes.c_void_p(waited.data_ptr()), stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 104
    assert 2_000_000 <= int(waited.item()) < 200_000_000  # gave up after the limit, not much later
    assert lib.splitd_wait_probe(ctypes.c_void_p(status.data_ptr()), 0, None, stream) == -1  # limit out of range
    q, k, v = (_t(1, 256, 8, D).requires_grad_(True), _t(1, 256, 2, D).requires_grad_(True),
               _t(1, 256, 2, D).requires_grad_(True))
    out = split_flash_attn_func(q, k, v, causal=True)
    torch.autograd.grad(out, (q, k, v), torch.ones_like(out))
    torch.cuda.synchronize()
    from splitd_flash_attn.interface import kernel_status

    assert kernel_status() == 0 and torch.isfinite(out).all()


def test_same_tensor_as_k_and_v():
    """k and v may be the same storage (the reference has a shared-tile fast path for that, src/interface.py:439)."""
    from gpu_utils import check_bwd, check_fwd, make_qkv

    from splitd_flash_attn import split_flash_attn_func

    q, k, _, do = make_qkv(2, 300, 300, 8, 2, torch.bfloat16, seed=12, with_do=True)
    q.requires_grad_(True), k.requires_grad_(True)
    out, lse = split_flash_attn_func(q, k, k, causal=True, return_lse=True)
    (dq, dkv) = torch.autograd.grad(out, (q, k), do)
    # autograd sums the gradients of the two uses of k: compare with dk + dv of the oracle and the yardstick
    k2 = k.detach().clone()
    check_fwd(out, lse, q, k2, k2, True)
    from gpu_utils import ATOL, ERR_FACTOR, max_err, sdpa_math

    from oracle import attention_oracle as O

    rq, rk, rv = O.attention_bwd(q.detach(), k2, k2, do, True)
    _, yq, yk, yv = sdpa_math(q.detach(), k2, k2, True, do=do)
    assert max_err(dq, rq) <= ERR_FACTOR * max_err(yq, rq) + ATOL
    ref = rk + rv
    assert max_err(dkv, ref) <= ERR_FACTOR * max_err(yk.float() + yv.float(), ref) + 2 ** -8 * ref.abs().max().item()


def test_two_streams_side_by_side():
    """Calls on different streams share nothing but the library: each backward has its own workspace (and with
    it its own work counter), so overlapping launches must give the same bits as running alone."""
    from splitd_flash_attn import split_flash_attn_func

    torch.manual_seed(6)
    cases = []
    for S in (512, 768):
        q, k, v = (_t(2, S, 8, D).requires_grad_(True), _t(2, S, 2, D).requires_grad_(True),
                   _t(2, S, 2, D).requires_grad_(True))
        cases.append((q, k, v, _t(2, S, 8, D)))

    def run(q, k, v, do):
        out = split_flash_attn_func(q, k, v, causal=True)
        return (out.detach(),) + torch.autograd.grad(out, (q, k, v), do)

    alone = [run(*c) for c in cases]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream() for _ in cases]
    together = []
    for _ in range(3):  # a few rounds so that the launches really interleave
        together = []
        for c, st in zip(cases, streams):
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                together.append(run(*c))
    for st in streams:
        torch.cuda.current_stream().wait_stream(st)
    torch.cuda.synchronize()
    for a, b in zip(alone, together):
        for x, y in zip(a, b):
            assert torch.equal(x, y)


def test_public_functions_run_under_torch_compile_fullgraph():
    """Both layouts are custom ops with fake kernels and registered autograd, so `torch.compile(fullgraph=True)`
    traces through them without a graph break; the compiled forward + backward give the gradients of the eager run
    bit for bit (the ops are opaque to the compiler; only the arithmetic around them is fused)."""
    from splitd_flash_attn import split_flash_attn_func, split_flash_attn_varlen_func
    from splitd_flash_attn.interface import cu_seqlens_validation

    g = torch.Generator(device="cuda").manual_seed(0)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16).requires_grad_(True)

    def batched(q, k, v):
        return split_flash_attn_func(q * 1.0, k, v, causal=True).float().square().sum()

    q, k, v = mk(2, 256, 8, 512), mk(2, 256, 2, 512), mk(2, 256, 2, 512)
    eager = torch.autograd.grad(batched(q, k, v), (q, k, v))
    compiled = torch.autograd.grad(torch.compile(batched, fullgraph=True)(q, k, v), (q, k, v))
    assert all(torch.equal(a, b) for a, b in zip(eager, compiled))

    cu = torch.tensor([0, 100, 256, 300], dtype=torch.int32, device="cuda")

    def packed(q, k, v):
        return split_flash_attn_varlen_func(q * 1.0, k, v, cu, cu, 156, 156, causal=True).float().square().sum()

    q, k, v = mk(300, 8, 512), mk(300, 2, 512), mk(300, 2, 512)
    with cu_seqlens_validation(False):  # value checks of cu_seqlens need the host; a traced graph has none
        eager = torch.autograd.grad(packed(q, k, v), (q, k, v))
        compiled = torch.autograd.grad(torch.compile(packed, fullgraph=True)(q, k, v), (q, k, v))
    assert all(torch.equal(a, b) for a, b in zip(eager, compiled))
    from splitd_flash_attn.interface import kernel_status

    assert kernel_status() == 0


def test_forward_and_backward_can_be_captured_in_a_cuda_graph():
    """Nothing in the batched path synchronises, allocates outside torch's allocator or reads device values on the
    host, so a forward + backward can be captured once and replayed on new data in the same buffers."""
    from splitd_flash_attn import split_flash_attn_func
    from splitd_flash_attn.interface import kernel_status

    g = torch.Generator(device="cuda").manual_seed(0)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    q, k, v, do = mk(2, 512, 8, 512), mk(2, 512, 2, 512), mk(2, 512, 2, 512), mk(2, 512, 8, 512)
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture (first calls look up function attributes)
        out = split_flash_attn_func(q, k, v, causal=True)
        torch.autograd.grad(out, (q, k, v), do)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_g = split_flash_attn_func(q, k, v, causal=True)
        grads_g = torch.autograd.grad(out_g, (q, k, v), do)
    with torch.no_grad():
        q.add_(0.5)
        do.mul_(2.0)
    graph.replay()
    torch.cuda.synchronize()
    out_e = split_flash_attn_func(q, k, v, causal=True)
    grads_e = torch.autograd.grad(out_e, (q, k, v), do)
    assert torch.equal(out_g, out_e) and all(torch.equal(a, b) for a, b in zip(grads_g, grads_e))
    assert kernel_status() == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensors_on_a_device_that_is_not_the_current_one():
    """The launches follow the tensors' device, not torch's current device (the reference's kernels are launched on
    the current stream of the tensors' device as well): same bits on cuda:1 as on cuda:0, current device unchanged."""
    from splitd_flash_attn import split_flash_attn_func
    from splitd_flash_attn.interface import kernel_status

    res = {}
    for dev in ("cuda:0", "cuda:1"):
        g = torch.Generator(device=dev).manual_seed(0)
        mk = lambda *s: torch.randn(*s, device=dev, generator=g).to(torch.bfloat16)
        q, k, v, do = mk(2, 300, 8, 512), mk(2, 300, 2, 512), mk(2, 300, 2, 512), mk(2, 300, 8, 512)
        q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        out, lse = split_flash_attn_func(q, k, v, causal=True, return_lse=True)
        grads = torch.autograd.grad(out, (q, k, v), do)
        torch.cuda.synchronize(dev)
        res[dev] = [t.cpu() for t in (out.detach(), lse) + tuple(grads)]
    assert torch.cuda.current_device() == 0
    assert all(torch.equal(a, b) for a, b in zip(res["cuda:0"], res["cuda:1"]))
    assert kernel_status(torch.device("cuda:0")) == 0 and kernel_status(torch.device("cuda:1")) == 0
