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
    assert lib.splitd_bwd_workspace_bytes(ctypes.byref(p)) == 2 * 2 * 128 * (256 + 64) * 2 + 256  # tiles + work counters
    assert lib.splitd_bwd_dq(ctypes.byref(p), None) == -5


def test_debug_counters_stay_inside_64_floats():
    """The optional `debug` buffer of the C-ABI is documented as 64 floats (include/splitd_attn.h): the
    kernels' cycle counters must land there and nowhere behind it, and results must not change."""
    from splitd_flash_attn import interface as I

    torch.manual_seed(5)
    q, k, v, do = _t(1, 1024, 8, D), _t(1, 1024, 1, D), _t(1, 1024, 1, D), _t(1, 1024, 8, D)
    out0, lse0 = I._flash_attn_fwd(q, k, v, causal=True, return_lse=True)
    g0 = I._flash_attn_bwd(q, k, v, out0, do, lse0, causal=True)
    buf = torch.zeros(256, device="cuda")
    out1, lse1 = I._flash_attn_fwd(q, k, v, causal=True, return_lse=True, debug=buf)
    g1 = I._flash_attn_bwd(q, k, v, out1, do, lse1, causal=True, debug=buf)
    torch.cuda.synchronize()
    assert I.kernel_status() == 0
    assert torch.count_nonzero(buf[64:]) == 0
    assert torch.count_nonzero(buf[32:52]) > 0 and torch.count_nonzero(buf[:16]) > 0
    assert torch.equal(out0, out1) and torch.equal(lse0, lse1)
    for a, b in zip(g0, g1):
        assert torch.equal(a, b)


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
