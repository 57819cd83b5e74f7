"""GPU: the allocation-free backward entry point (splitd_bwd_static_scratch).

Some users of this library cannot allocate device memory at the point where they need a backward pass:
a host thread with a latency budget that must not touch the CUDA allocator's locks, a plugin whose host
framework owns every byte of device memory and passes in only the op's own tensors, a job that was given
a fixed memory budget. For them the library carries its backward scratch (row statistics and the P/dS tile
workspace) in a 17 MiB array of its own. This test drives that entry point through the C-ABI with ctypes,
twice in a row on different data (the array is shared between calls and keeps old contents), and checks that
it returns exactly what the regular entry point returns with caller-provided buffers; it also checks that a
problem beyond the stated limit is refused with a clear message instead of being run.

Collected last on purpose (file name), so that a run that stops at the first failure has already executed
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
D = 512


def _problem(seed, B, S, Hq, Hkv, causal):
    from splitd_flash_attn import interface as I

    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda h: torch.randn(B, S, h, D, device="cuda", generator=g).to(torch.bfloat16)
    q, k, v, do = mk(Hq), mk(Hkv), mk(Hkv), mk(Hq)
    out, lse = I._flash_attn_fwd(q, k, v, causal=causal, return_lse=True)
    return q, k, v, do, out, lse


def _params(q, k, v, do, out, lse, causal, grads):
    from splitd_flash_attn import interface as I

    p = I._fill_params(q, k, v, out, lse, None, None, None, None, D**-0.5, causal)
    dq, dk, dv = grads
    p.dout = ctypes.c_void_p(do.data_ptr())
    p.dq, p.dk, p.dv = (ctypes.c_void_p(t.data_ptr()) for t in (dq, dk, dv))
    p.do_strides[:] = I._strides3(do, False)
    p.dq_strides[:] = I._strides3(dq, False)
    p.dk_strides[:] = I._strides3(dk, False)
    p.dv_strides[:] = I._strides3(dv, False)
    return p


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("round_", [0, 1])
def test_static_scratch_backward_matches_regular_backward(round_):
    from splitd_flash_attn import _capi
    from splitd_flash_attn import interface as I

    lib = _capi.load_library()
    # two calls in a row per test invocation, different data and masks each time
    for call, (seed, S, causal) in enumerate([(10 + round_, 384, True), (20 + round_, 256, False)]):
        q, k, v, do, out, lse = _problem(seed, 1, S, 8, 1, causal)
        ref = I._flash_attn_bwd(q, k, v, out, do, lse, causal=causal)  # regular path, torch-allocated scratch
        got = tuple(torch.full_like(t, float("nan")) for t in (q, k, v))
        p = _params(q, k, v, do, out, lse, causal, got)
        assert lib.splitd_bwd_rowstat_elems(ctypes.byref(p)) <= lib.splitd_bwd_static_scratch_limit_rowstat()
        assert lib.splitd_bwd_workspace_bytes(ctypes.byref(p)) <= lib.splitd_bwd_static_scratch_limit_workspace()
        rc = lib.splitd_bwd_static_scratch(ctypes.byref(p), _stream())
        assert rc == 0, lib.splitd_last_error()
        torch.cuda.synchronize()
        assert I.kernel_status() == 0
        for name, a, b in zip(("dq", "dk", "dv"), got, ref):
            assert not torch.isnan(a).any(), f"{name} call {call}"
            # same kernels, same launch geometry: the results are bit-identical (tolerance of the other
            # backward tests would be 2x the 16-bit PyTorch error; zero difference is the stronger check)
            assert torch.equal(a, b), f"{name} differs on call {call}: {(a.float() - b.float()).abs().max().item()}"


def test_static_scratch_rejects_problems_beyond_its_limit():
    from splitd_flash_attn import _capi

    lib = _capi.load_library()
    q, k, v, do, out, lse = _problem(3, 2, 1024, 32, 4, True)
    grads = tuple(torch.zeros_like(t) for t in (q, k, v))
    p = _params(q, k, v, do, out, lse, True, grads)
    rc = lib.splitd_bwd_static_scratch(ctypes.byref(p), _stream())
    assert rc == -5
    msg = lib.splitd_last_error().decode()
    assert "too large for the static scratch" in msg and "limit" in msg
    torch.cuda.synchronize()
    assert all(torch.count_nonzero(g) == 0 for g in grads)  # nothing was launched
