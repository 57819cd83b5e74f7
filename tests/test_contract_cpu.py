"""CPU: the parts of the public API contract that must fail before any CUDA work is attempted."""
import pytest
import torch

D = 512


def test_cpu_tensors_are_rejected_with_a_cuda_message():
    # tests/test_flash_fwd_splitd_sdpa.py:400-406 of the reference
    from splitd_flash_attn import split_flash_attn_func

    q = torch.randn(1, 16, 2, D, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        split_flash_attn_func(q, q, q)


def test_rank_and_dtype_errors():
    from splitd_flash_attn import split_flash_attn_func, split_flash_attn_varlen_func

    q = torch.randn(16, 2, D, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="rank 4"):
        split_flash_attn_func(q, q, q)
    q4 = torch.randn(1, 16, 2, D, dtype=torch.float32)
    with pytest.raises(TypeError):
        split_flash_attn_func(q4, q4, q4)
    with pytest.raises(ValueError, match="cu_seqlens"):
        split_flash_attn_varlen_func(q, q, q)
    cu = torch.tensor([0, 16], dtype=torch.int32)
    with pytest.raises(ValueError, match="max_seqlen_q"):
        split_flash_attn_varlen_func(q, q, q, cu, cu, None, 16)
    with pytest.raises(NotImplementedError):
        split_flash_attn_varlen_func(q, q, q, cu, cu, 16, 16, score_mod=lambda *a: 0)
    with pytest.raises(TypeError, match="tuple"):
        split_flash_attn_varlen_func(q, q, q, cu, cu, 16, 16, window_size=[None, None])


def test_window_resolution_table():
    from splitd_flash_attn.interface import _resolve_causal_local_window as r

    assert r(False, None, None) == (False, False)
    assert r(True, None, None) == (True, False)
    assert r(False, -1, -1) == (False, False)
    assert r(False, -1, 0) == (True, False)
    assert r(False, 16, 0) == (False, True)
    assert r(False, 16, None) == (False, True)
    with pytest.raises(ValueError):
        r(True, 16, 0)


def test_library_is_mandatory(monkeypatch):
    """No CPU / PyTorch fallback: without the shared object the package refuses to run."""
    from splitd_flash_attn import _capi

    monkeypatch.setattr(_capi, "_lib", None)
    monkeypatch.setattr(_capi, "LIB_PATH", "/nonexistent/libsplitd_attn.so")
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _capi.load_library()


def test_varlen_custom_op_traces_under_fake_tensors():
    """The packed path is a torch.library custom op pair with fake kernels (like the reference's
    splitd_flash_attn::varlen_fwd / varlen_bwd, interface.py:909-1061): shapes propagate without a GPU."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    from splitd_flash_attn import split_flash_attn_varlen_func

    with FakeTensorMode():
        q = torch.empty(96, 8, D, dtype=torch.bfloat16, device="cuda", requires_grad=True)
        kv = torch.empty(96, 2, D, dtype=torch.bfloat16, device="cuda", requires_grad=True)
        cu = torch.empty(4, dtype=torch.int32, device="cuda")
        out, lse = split_flash_attn_varlen_func(q, kv, kv, cu, cu, 40, 40, causal=True, return_lse=True)
        assert out.shape == (96, 8, D) and out.dtype == torch.bfloat16
        assert lse.shape == (8, 96) and lse.dtype == torch.float32
        # the fake backward kernel (the autograd engine itself needs a real CUDA device, so call the op)
        gq, gk, gv = torch.ops.splitd_flash_attn.varlen_bwd(
            q.detach(), kv.detach(), kv.detach(), out.detach(), out.detach(), lse, cu, cu, 40, 40, 0.05, True,
            -(2**31), -(2**31), 0.0, None,
        )
        assert gq.shape == q.shape and gk.shape == kv.shape and gv.shape == kv.shape
    assert hasattr(torch.ops.splitd_flash_attn, "varlen_fwd") and hasattr(torch.ops.splitd_flash_attn, "varlen_bwd")


def test_batched_custom_op_traces_under_fake_tensors():
    """The batched layout goes through a custom op pair of its own (splitd_flash_attn::fwd / ::bwd) with fake
    kernels, so it is traceable without a GPU like the packed one."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    from splitd_flash_attn import split_flash_attn_func

    with FakeTensorMode():
        q = torch.empty(2, 96, 8, D, dtype=torch.bfloat16, device="cuda", requires_grad=True)
        kv = torch.empty(2, 80, 2, D, dtype=torch.bfloat16, device="cuda", requires_grad=True)
        out, lse = split_flash_attn_func(q, kv, kv, causal=True, return_lse=True)
        assert out.shape == (2, 96, 8, D) and out.dtype == torch.bfloat16
        assert lse.shape == (2, 8, 96) and lse.dtype == torch.float32
        gq, gk, gv = torch.ops.splitd_flash_attn.bwd(
            q.detach(), kv.detach(), kv.detach(), out.detach(), out.detach(), lse, 0.05, True, -(2**31), -(2**31), 0.0, None
        )
        assert gq.shape == q.shape and gk.shape == kv.shape and gv.shape == kv.shape
        q16 = torch.empty(2, 96, 8, D, dtype=torch.float16, device="cuda", requires_grad=True)
        with pytest.raises(NotImplementedError, match="bfloat16 only"):
            split_flash_attn_func(q16, q16, q16)
    assert hasattr(torch.ops.splitd_flash_attn, "fwd") and hasattr(torch.ops.splitd_flash_attn, "bwd")


def test_training_forward_ops_return_the_low_word_of_the_output():
    """A forward that can be differentiated goes through ``fwd_resid`` / ``varlen_fwd_resid``: the two-result
    ops plus a third result, an opaque uint8 scratch (a flag byte per output row, padded to 256, then a 16-bit
    remainder row per output row), which the backward ops take as a trailing optional argument. All of it traces without a GPU; a no-grad call stays on the two-result ops."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    from splitd_flash_attn import interface as I

    ops = torch.ops.splitd_flash_attn
    none = -(2**31)
    with FakeTensorMode():
        q = torch.empty(2, 96, 8, D, dtype=torch.bfloat16, device="cuda")
        kv = torch.empty(2, 80, 2, D, dtype=torch.bfloat16, device="cuda")
        out, lse, resid = ops.fwd_resid(q, kv, kv, 0.05, True, none, none, 0.0, True)
        assert out.shape == q.shape and resid.dtype == torch.uint8
        assert resid.shape == (2 * 96 * 8 + 2 * 96 * 8 * D * 2,)  # 1536 flag bytes are a multiple of 256 already
        gq, gk, gv = ops.bwd(q, kv, kv, out, out, lse, 0.05, True, none, none, 0.0, None, resid)
        assert gq.shape == q.shape and gk.shape == kv.shape and gv.shape == kv.shape
        qp = torch.empty(96, 8, D, dtype=torch.bfloat16, device="cuda")
        kp = torch.empty(96, 2, D, dtype=torch.bfloat16, device="cuda")
        cu = torch.empty(4, dtype=torch.int32, device="cuda")
        out, lse, resid = ops.varlen_fwd_resid(qp, kp, kp, cu, cu, 40, 40, 0.05, True, none, none, 0.0, True)
        assert out.shape == qp.shape and lse.shape == (8, 96) and resid.shape == (96 * 8 + 96 * 8 * D * 2,)
        gq, gk, gv = ops.varlen_bwd(qp, kp, kp, out, out, lse, cu, cu, 40, 40, 0.05, True, none, none, 0.0, None, resid)
        assert gq.shape == qp.shape and gk.shape == kp.shape
        assert not I._wants_residual(q, kv, kv)
        assert I._wants_residual(q.requires_grad_(True), kv, kv)
        with torch.no_grad():
            assert not I._wants_residual(q, kv, kv)
        old = I.set_output_residual(False)
        try:
            assert not I._wants_residual(q, kv, kv)
        finally:
            I.set_output_residual(old)
        assert I.set_output_residual("all") is True and I._wants_residual(q, kv, kv)
        assert I.set_output_residual(True) == "all"


def test_backward_workspace_is_bounded_for_the_full_layer():
    """Sizing needs no GPU. The B=2, S=32768, Hq=32, Hkv=4 layer would need 275 GB for all of its P / dS tiles;
    the default workspace caps the tiles at 9 GiB and the smallest accepted one is the operand copies plus a
    few tiles. Whatever lies between is accepted, and more memory never means more chunks."""
    import ctypes

    from splitd_flash_attn import _capi

    lib = _capi.load_library()
    p = _capi.SplitdParams()
    p.batch, p.seqlen_q, p.seqlen_k, p.heads_q, p.heads_kv, p.head_dim = 2, 32768, 32768, 32, 4, 512
    everything = lib.splitd_bwd_workspace_bytes_limit(ctypes.byref(p), ctypes.c_size_t(-1).value)
    default = lib.splitd_bwd_workspace_bytes(ctypes.byref(p))
    smallest = lib.splitd_bwd_workspace_bytes_limit(ctypes.byref(p), 0)
    copies = (2 * 2 * 32768 * 32 + 2 * 32768 * 4) * 512 * 2
    assert everything > 270e9
    assert copies < smallest < copies + (1 << 30)
    assert smallest < default < copies + (11 << 30)
    # the sweep's shapes fit the default without row splitting: whole KV heads or everything at once
    p.batch, p.seqlen_q, p.seqlen_k = 16, 1024, 1024
    assert lib.splitd_bwd_workspace_bytes(ctypes.byref(p)) == lib.splitd_bwd_workspace_bytes_limit(
        ctypes.byref(p), ctypes.c_size_t(-1).value
    )
