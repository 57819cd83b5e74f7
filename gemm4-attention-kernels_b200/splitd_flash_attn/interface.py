"""Public API of the B200 SplitD FlashAttention (head_dim == 512).

Drop-in for ``splitd-flash-attn/src/interface.py`` of cmriat/gemm4-attention-kernels: the two public
functions keep the reference's signatures (interface.py:1226-1236, 1255-1271), argument meaning,
return values, validation order and exception types; the kernels behind them are hand-written
sm_100a CUDA reached through the C-ABI in ``include/splitd_attn.h``.

Layouts: batched (B, S, H, 512); packed (T, H, 512) with int32 ``cu_seqlens`` of B+1 entries.
LSE is fp32, (B, Hq, S) batched and (Hq, T) packed, natural log, -inf for rows without keys.
Forward accepts bf16 and fp16; training (any input requiring grad) is bf16 only.
"""

from __future__ import annotations

import contextlib
import ctypes
import math
import os
from typing import Callable, Optional, Tuple

import torch

from . import _capi

SUPPORTED_HEAD_DIM = 512

__all__ = [
    "split_flash_attn_func",
    "split_flash_attn_varlen_func",
    "kernel_status",
    "cu_seqlens_validation",
    "set_backward_workspace_limit",
    "set_output_residual",
]

# Value checks of cu_seqlens (first entry 0, last entry = token count, non-decreasing, max_seqlen large enough)
# need the values on the host: one blocking device->host copy per tensor per call, in forward and again in
# backward (the reference does the same with .item(), src/interface.py:164-172,187-188). A training loop that
# builds its cu_seqlens correctly can switch them off; shape, dtype and device checks stay on.
_VALIDATE_CU_SEQLENS = os.environ.get("SPLITD_VALIDATE_CU_SEQLENS", "1") != "0"


@contextlib.contextmanager
def cu_seqlens_validation(enabled: bool):
    """``with cu_seqlens_validation(False): ...`` runs the packed API without any host synchronisation.

    The caller then guarantees what the checks would have verified: cu_seqlens start at 0, end at the token
    count, never decrease, and no sequence is longer than max_seqlen_q / max_seqlen_k. (A sequence with more
    keys than max_seqlen_k is skipped by the backward kernels and reported through ``kernel_status()``.)
    """
    global _VALIDATE_CU_SEQLENS
    old = _VALIDATE_CU_SEQLENS
    _VALIDATE_CU_SEQLENS = bool(enabled)
    try:
        yield
    finally:
        _VALIDATE_CU_SEQLENS = old


# Cap on the bytes of P / dS tiles the backward keeps in memory at once (None: the library's default, 9 GiB).
# Larger problems are processed in chunks that reuse the same memory; results do not depend on it.
_env_limit = os.environ.get("SPLITD_BWD_WORKSPACE_LIMIT_BYTES")
_WORKSPACE_LIMIT: Optional[int] = int(_env_limit) if _env_limit else None


# A training forward keeps, for the output rows whose probability mass sits on few keys, the 16-bit remainder
# (exact output - out). The backward's rowsum(dout * out) then sees those rows to ~16 significant bits instead
# of 8. With the 16-bit output alone the rounding of `out` is the largest error in dq / dk for such rows (the
# first rows of a causal sequence): 2.2x the error of a math-backend SDPA was measured there, against <= 1.3x
# with the remainder. Costs a scratch tensor of the size of `out` kept until the backward has run (only the
# flagged rows of it are ever written or read). SPLITD_OUTPUT_RESIDUAL=0 (or the setter) turns it off: the
# backward is then the reference's, which reads the 16-bit output (src/interface.py:732-741).
#
# The default keeps it for concentrated rows only, which is where N(0,1)-like data needs it. Data whose v (or k)
# has a common component that is large against its spread (v = 8 + N(0,1): |out| ~ 8 in every row) needs it in
# every row: dq 11.6x the SDPA-MATH error with the default, 1.2x with "all" (measured). "all" costs the forward one
# more output-sized write (about 6 % at the B*S = 16384 sizes).
def _parse_residual_mode(v):
    if isinstance(v, str):
        v = v.strip().lower()
        return "all" if v == "all" else (v not in ("0", "", "false", "off"))
    return bool(v)


_KEEP_RESIDUAL = _parse_residual_mode(os.environ.get("SPLITD_OUTPUT_RESIDUAL", "1"))


def set_output_residual(mode):
    """Keep the low word of the output between forward and backward: ``True`` (default: for the rows that are
    concentrated on few keys), ``"all"`` (every row) or ``False`` (the reference's backward). Returns the old
    setting."""
    global _KEEP_RESIDUAL
    old = _KEEP_RESIDUAL
    _KEEP_RESIDUAL = _parse_residual_mode(mode)
    return old


def set_backward_workspace_limit(nbytes: Optional[int]) -> Optional[int]:
    """Set the cap on the backward's tile memory (bytes; None = library default). Returns the old value."""
    global _WORKSPACE_LIMIT
    old = _WORKSPACE_LIMIT
    _WORKSPACE_LIMIT = None if nbytes is None else int(nbytes)
    return old


# ---------------------------------------------------------------------------
# validation (mirrors interface.py:79-261 of the reference)
# ---------------------------------------------------------------------------


def _validate_head_dims(head_dim: int, head_dim_v: int) -> None:
    if head_dim != SUPPORTED_HEAD_DIM or head_dim_v != SUPPORTED_HEAD_DIM:
        raise ValueError(
            f"(head_dim, head_dim_v)=({head_dim}, {head_dim_v}) is not supported. "
            f"This SplitD interface requires q/k head_dim == {SUPPORTED_HEAD_DIM} and "
            f"v head_dim_v == {SUPPORTED_HEAD_DIM}."
        )


def _validate_tensor(tensor, name, expected_shape, expected_dtype, expected_device) -> None:
    if tensor is None:
        raise ValueError(f"{name} must not be None")
    if tuple(tensor.shape) != tuple(expected_shape):
        raise ValueError(f"{name} has shape {tuple(tensor.shape)}, expected {tuple(expected_shape)}")
    if tensor.dtype != expected_dtype:
        raise TypeError(f"{name} has dtype {tensor.dtype}, expected {expected_dtype}")
    if tensor.device != expected_device:
        raise RuntimeError(f"{name} is on {tensor.device}, expected {expected_device}")


def _validate_device_arch(device: torch.device) -> None:
    """Replaces ``_validate_sm90_arch`` (interface.py:123-130): this build needs sm_100."""
    lib = _capi.load_library()
    index = device.index if device.index is not None else torch.cuda.current_device()
    ok = lib.splitd_device_supported(index)
    if ok != 1:
        major, minor = torch.cuda.get_device_capability(index)
        raise RuntimeError(
            f"This SplitD interface requires Blackwell B200 (SM 10.x), got compute capability {major}.{minor}."
        )


def _validate_training_dtype(q, requires_grad: bool) -> None:
    if requires_grad and q.dtype != torch.bfloat16:
        raise NotImplementedError(
            "SplitD training currently supports torch.bfloat16 only. "
            f"Got q/k/v dtype {q.dtype}; use bfloat16 inputs or a different attention backend."
        )


def _validate_cu_seqlens(tensor, name, batch_size=None, total_tokens=None) -> None:
    if tensor is None:
        return
    if tensor.ndim != 1:
        raise ValueError(f"{name} must be a 1D tensor, got rank {tensor.ndim}")
    if tensor.numel() == 0:
        raise ValueError(f"{name} must have at least one element")
    if batch_size is not None and tuple(tensor.shape) != (batch_size + 1,):
        raise ValueError(f"{name} must have shape ({batch_size + 1},), got {tuple(tensor.shape)}")
    if tensor.dtype != torch.int32:
        raise TypeError(f"{name} must have dtype torch.int32, got {tensor.dtype}")
    if tensor.stride(0) != 1:
        raise ValueError(f"{name} must be contiguous")
    if not tensor.is_cuda:
        raise RuntimeError(f"{name} must be on a CUDA device, got {tensor.device}")
    if not _VALIDATE_CU_SEQLENS:
        return None
    # one device->host copy for all value checks (the reference does three .item() syncs here)
    host = tensor.detach().cpu()
    _raise_if_a_kernel_gave_up(tensor.device)  # the copy synchronised anyway: look at the status word too
    first = int(host[0])
    if first != 0:
        raise ValueError(f"{name}[0] must be 0, got {first}")
    if total_tokens is not None:
        last = int(host[-1])
        if last != total_tokens:
            raise ValueError(f"{name}[-1] must equal total tokens ({total_tokens}), got {last}")
    if host.numel() > 1 and bool(torch.any(host[1:] < host[:-1])):
        raise ValueError(f"{name} must be monotonically non-decreasing")
    return host


def _validate_max_seqlen(cu, host_cu, name, max_seqlen, max_name) -> None:
    """`cu` is the device tensor (None = batched layout), `host_cu` its host copy (None = value checks are off)."""
    if cu is None:
        return
    if max_seqlen is None:
        raise ValueError(f"{max_name} must be provided when {name} is provided")
    if isinstance(max_seqlen, bool) or not isinstance(max_seqlen, int):
        raise TypeError(f"{max_name} must be an int, got {type(max_seqlen).__name__}")
    if max_seqlen < 0:
        raise ValueError(f"{max_name} must be non-negative, got {max_seqlen}")
    if host_cu is None:
        return
    lengths = host_cu[1:] - host_cu[:-1]
    actual_max = int(lengths.max()) if lengths.numel() > 0 else 0
    if max_seqlen < actual_max:
        raise ValueError(f"{max_name} ({max_seqlen}) must be >= max sequence length from {name} ({actual_max})")


def _validate_qkv_common(q, k, v, cu_seqlens_q=None, cu_seqlens_k=None):
    q_rank = 3 if cu_seqlens_q is not None else 4
    kv_rank = 3 if cu_seqlens_k is not None else 4
    if q.ndim != q_rank:
        raise ValueError(f"q must have rank {q_rank}, got rank {q.ndim}")
    if k.ndim != kv_rank:
        raise ValueError(f"k must have rank {kv_rank}, got rank {k.ndim}")
    if v.ndim != kv_rank:
        raise ValueError(f"v must have rank {kv_rank}, got rank {v.ndim}")

    num_head, head_dim = q.shape[-2:]
    seqlen_k = k.shape[-3]
    num_head_kv = k.shape[-2]
    head_dim_v = v.shape[-1]
    host_cu_q = host_cu_k = None

    if cu_seqlens_q is None:
        batch_size, seqlen_q = q.shape[:2]
        total_q = batch_size * seqlen_q
    else:
        batch_size = cu_seqlens_q.numel() - 1
        seqlen_q = None
        total_q = q.shape[0]
        host_cu_q = _validate_cu_seqlens(cu_seqlens_q, "cu_seqlens_q", batch_size, total_tokens=total_q)

    if k.shape[-1] != head_dim:
        raise ValueError(f"k head_dim is {k.shape[-1]}, expected {head_dim}")
    if v.shape[-3] != seqlen_k or v.shape[-2] != num_head_kv:
        raise ValueError(
            f"v has shape {tuple(v.shape)}, expected matching seqlen/head dims (*, {seqlen_k}, {num_head_kv}, {head_dim_v})"
        )
    if cu_seqlens_k is None:
        expected_k_shape = (batch_size, seqlen_k, num_head_kv, head_dim)
        expected_v_shape = (batch_size, seqlen_k, num_head_kv, head_dim_v)
    else:
        host_cu_k = _validate_cu_seqlens(cu_seqlens_k, "cu_seqlens_k", batch_size, total_tokens=seqlen_k)
        expected_k_shape = (seqlen_k, num_head_kv, head_dim)
        expected_v_shape = (seqlen_k, num_head_kv, head_dim_v)
    if tuple(k.shape) != expected_k_shape:
        raise ValueError(f"k has shape {tuple(k.shape)}, expected {expected_k_shape}")
    if tuple(v.shape) != expected_v_shape:
        raise ValueError(f"v has shape {tuple(v.shape)}, expected {expected_v_shape}")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("SplitD inputs must be torch.float16 or torch.bfloat16")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise TypeError(f"q, k, and v must have the same dtype, got {q.dtype}, {k.dtype}, {v.dtype}")
    for name, t in (("q", q), ("k", k), ("v", v), ("cu_seqlens_q", cu_seqlens_q), ("cu_seqlens_k", cu_seqlens_k)):
        if t is not None and not t.is_cuda:
            raise RuntimeError(f"{name} must be on a CUDA device, got {t.device}")
    if num_head % num_head_kv != 0:
        raise ValueError(f"num_head ({num_head}) must be divisible by num_head_kv ({num_head_kv})")
    _validate_head_dims(head_dim, head_dim_v)
    return batch_size, seqlen_q, total_q, seqlen_k, num_head, num_head_kv, host_cu_q, host_cu_k


def _resolve_causal_local_window(causal, window_size_left, window_size_right):
    """Same decision table as interface.py:297-318 (window (-1,-1) = full, (-1,0) = causal)."""
    local = False
    if window_size_left is not None or window_size_right is not None:
        if causal:
            raise ValueError("causal and window_size are mutually exclusive")
        if window_size_left is not None and window_size_right is not None:
            if window_size_left < 0 and window_size_right < 0:
                causal, local = False, False
            elif window_size_right == 0 and window_size_left < 0:
                causal, local = True, False
            else:
                causal, local = False, True
        else:
            causal, local = False, True
    return causal, local


def _unsupported_features(requires_grad, softcap, local, score_mod=None, aux_tensors=None) -> None:
    """softcap and sliding windows are forward-only, as in the reference
    (``_unsupported_training_features``, interface.py:264-286)."""
    if not requires_grad:
        return
    unsupported = []
    if softcap is not None and softcap != 0.0:
        unsupported.append("softcap")
    if local:
        unsupported.append("local/window attention")
    if score_mod is not None:
        unsupported.append("score_mod")
    if aux_tensors is not None:
        unsupported.append("aux_tensors")
    if unsupported:
        raise NotImplementedError("SplitD backward does not support training with " + ", ".join(unsupported) + ".")


# ---------------------------------------------------------------------------
# C-ABI plumbing
# ---------------------------------------------------------------------------

_status_flags: dict = {}


def _status_flag(device: torch.device) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    flag = _status_flags.get(key)
    if flag is None:
        flag = torch.zeros(1, dtype=torch.int32, device=device)
        _status_flags[key] = flag
    return flag


def kernel_status(device: Optional[torch.device] = None) -> int:
    """Synchronise and return the device's status word: 0 = every kernel of this library ran to its end.

    The kernels never spin forever: a wait that exceeds 4 s is given up, the kernel ends early and stores a
    code here (101 loads, 102 tensor-core issue, 103 softmax/epilogue, 104 peer CTA, 105 shared-memory
    alignment, 106 a packed sequence longer than max_seqlen_k). Outputs of such a call are incomplete. The calls
    of this module are asynchronous, so nothing can raise at the call itself: check this after a step (it costs
    one 4-byte copy), e.g. where the loss is read. The packed API looks at it whenever it validates cu_seqlens.
    ``reset_kernel_status()`` re-arms it.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    return int(_status_flag(device).item())


def reset_kernel_status(device: Optional[torch.device] = None) -> None:
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    _status_flag(device).zero_()


def _raise_if_a_kernel_gave_up(device: torch.device) -> None:
    key = device.index if device.index is not None else torch.cuda.current_device()
    flag = _status_flags.get(key)
    if flag is not None:
        code = int(flag.item())
        if code != 0:
            raise RuntimeError(
                f"an earlier SplitD attention kernel on {device} ended early with status {code} "
                "(see kernel_status); its outputs are incomplete"
            )


def _strides3(t: torch.Tensor, packed: bool):
    if t.stride(-1) != 1:
        raise ValueError("innermost (head_dim) stride must be 1")
    if packed:
        return (0, t.stride(0), t.stride(1))
    return (t.stride(0), t.stride(1), t.stride(2))


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _needs_copy(t: torch.Tensor) -> bool:
    """TMA needs unit stride on D and 16-byte aligned outer strides; anything else is copied."""
    if t.stride(-1) != 1 or t.data_ptr() % 16 != 0:
        return True
    return any(s % 8 != 0 for s in t.stride()[:-1])


def _prep(t: Optional[torch.Tensor]):
    if t is None:
        return None
    return t.contiguous() if _needs_copy(t) else t


def _fill_params(q, k, v, out, lse, cu_q, cu_k, max_q, max_k, scale, causal, debug=None) -> _capi.SplitdParams:
    packed = cu_q is not None
    p = _capi.SplitdParams()
    p.q, p.k, p.v, p.o, p.lse = _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse)
    p.cu_seqlens_q, p.cu_seqlens_k = _ptr(cu_q), _ptr(cu_k)
    if packed:
        p.batch = cu_q.numel() - 1
        p.total_q, p.total_k = q.shape[0], k.shape[0]
        p.max_seqlen_q, p.max_seqlen_k = int(max_q), int(max_k)
    else:
        p.batch, p.seqlen_q, p.seqlen_k = q.shape[0], q.shape[1], k.shape[1]
    p.heads_q, p.heads_kv, p.head_dim = q.shape[-2], k.shape[-2], q.shape[-1]
    p.q_strides[:] = _strides3(q, packed)
    p.k_strides[:] = _strides3(k, packed)
    p.v_strides[:] = _strides3(v, packed)
    p.o_strides[:] = _strides3(out, packed)
    p.softmax_scale = float(scale)
    p.causal = 1 if causal else 0
    p.dtype = _capi.SPLITD_DTYPE_FP16 if q.dtype == torch.float16 else _capi.SPLITD_DTYPE_BF16
    p.status_flag = _ptr(_status_flag(q.device))
    p.debug = _ptr(debug)
    p.softcap = 0.0
    p.local = 0
    return p


def _stream_ptr(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


# ---------------------------------------------------------------------------
# host wrappers (replace _flash_attn_fwd_sm90 / _flash_attn_bwd_sm90)
# ---------------------------------------------------------------------------


def _flash_attn_fwd(
    q,
    k,
    v,
    cu_seqlens_q=None,
    cu_seqlens_k=None,
    max_seqlen_q=None,
    max_seqlen_k=None,
    softmax_scale=None,
    causal=False,
    softcap=None,
    window_size_left=None,
    window_size_right=None,
    pack_gqa=None,
    return_lse=False,
    out=None,
    lse=None,
    debug=None,
    keep_resid=False,
):
    """Forward host wrapper; same contract as ``_flash_attn_fwd_sm90`` (interface.py:362-554).

    ``pack_gqa`` is accepted for compatibility: heads are always folded into rows when the group
    size allows it, which gives identical results. With ``keep_resid=True`` a third value is returned: an
    opaque uint8 tensor holding, for the output rows that are concentrated on few keys, the part of the exact
    output that rounding ``out`` to 16 bits dropped; ``_flash_attn_bwd(out_resid=...)`` uses it for a
    ``rowsum(dout * out)`` that is free of that rounding.
    """
    (batch_size, seqlen_q, total_q, seqlen_k, num_head, num_head_kv, host_cu_q, host_cu_k) = _validate_qkv_common(
        q, k, v, cu_seqlens_q, cu_seqlens_k
    )
    requires_grad = q.requires_grad or k.requires_grad or v.requires_grad
    _validate_training_dtype(q, requires_grad)
    _validate_max_seqlen(cu_seqlens_q, host_cu_q, "cu_seqlens_q", max_seqlen_q, "max_seqlen_q")
    _validate_max_seqlen(cu_seqlens_k, host_cu_k, "cu_seqlens_k", max_seqlen_k, "max_seqlen_k")
    if (cu_seqlens_q is None) != (cu_seqlens_k is None):
        raise ValueError("cu_seqlens_q and cu_seqlens_k must be given together")
    _validate_device_arch(q.device)
    head_dim = q.shape[-1]
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(head_dim)
    if softcap == 0.0:
        softcap = None
    causal, local = _resolve_causal_local_window(causal, window_size_left, window_size_right)
    _unsupported_features(requires_grad, softcap, local)

    q, k, v = (_prep(t.detach()) for t in (q, k, v))
    device = q.device
    q_lead = (batch_size, seqlen_q) if cu_seqlens_q is None else (total_q,)
    lse_shape = (batch_size, num_head, seqlen_q) if cu_seqlens_q is None else (num_head, total_q)
    if out is None:
        out = torch.empty(*q_lead, num_head, head_dim, dtype=q.dtype, device=device)
    else:
        _validate_tensor(out, "out", (*q_lead, num_head, head_dim), q.dtype, device)
    if lse is None:
        lse = torch.empty(lse_shape, dtype=torch.float32, device=device) if (requires_grad or return_lse) else None
    else:
        _validate_tensor(lse, "lse", lse_shape, torch.float32, device)

    if total_q == 0 or k.shape[-3] == 0:
        out.zero_()
        if lse is not None:
            lse.fill_(float("-inf"))
        # no row has a low word: all flags zero
        return (out, lse, torch.zeros(_resid_bytes(out), dtype=torch.uint8, device=device)) if keep_resid else (out, lse)

    params = _fill_params(
        q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal, debug
    )
    if softcap is not None:
        params.softcap = float(softcap)
    if local:  # negative or missing side = unbounded on that side
        params.local = 1
        params.window_left = -1 if window_size_left is None or window_size_left < 0 else int(window_size_left)
        params.window_right = -1 if window_size_right is None or window_size_right < 0 else int(window_size_right)
    lib = _capi.load_library()
    out_resid = None
    if keep_resid:
        out_resid = torch.empty(lib.splitd_out_resid_bytes(ctypes.byref(params)), dtype=torch.uint8, device=device)
        params.o_resid = _ptr(out_resid)
        params.o_resid_all = 1 if _KEEP_RESIDUAL == "all" else 0
    n_ws = lib.splitd_fwd_workspace_bytes(ctypes.byref(params))  # fp16 copy of v (bf16 inputs only)
    if n_ws:
        workspace = torch.empty(n_ws, dtype=torch.uint8, device=device)
        params.workspace, params.workspace_bytes = _ptr(workspace), n_ws
    with torch.cuda.device(device):
        _capi.check(lib.splitd_fwd(ctypes.byref(params), _stream_ptr(device)))
    return (out, lse, out_resid) if keep_resid else (out, lse)


def _flash_attn_bwd(
    q,
    k,
    v,
    out,
    dout,
    lse,
    softmax_scale=None,
    causal=False,
    softcap=0.0,
    window_size_left=None,
    window_size_right=None,
    cu_seqlens_q=None,
    cu_seqlens_k=None,
    max_seqlen_q=None,
    max_seqlen_k=None,
    dlse=None,
    stage_events=None,
    debug=None,
    out_resid=None,
):
    """Backward host wrapper; same contract as ``_flash_attn_bwd_sm90`` (interface.py:652-888):
    preprocess, dQ and dK/dV launches on the current stream, dq/dk/dv in the input dtype with
    dk/dv already reduced over the query heads of each KV head. ``out_resid``: the low word of ``out``
    that the forward kept (optional, see ``_flash_attn_fwd``)."""
    _validate_device_arch(q.device)
    if softcap != 0.0:
        raise NotImplementedError("SplitD backward does not support softcap yet")
    causal, local = _resolve_causal_local_window(causal, window_size_left, window_size_right)
    if local:
        raise NotImplementedError("SplitD backward does not support local/window attention yet")
    (batch_size, seqlen_q, total_q, seqlen_k, num_head, num_head_kv, host_cu_q, host_cu_k) = _validate_qkv_common(
        q, k, v, cu_seqlens_q, cu_seqlens_k
    )
    _validate_max_seqlen(cu_seqlens_q, host_cu_q, "cu_seqlens_q", max_seqlen_q, "max_seqlen_q")
    _validate_max_seqlen(cu_seqlens_k, host_cu_k, "cu_seqlens_k", max_seqlen_k, "max_seqlen_k")
    if q.dtype == torch.float16:
        raise NotImplementedError("SplitD backward currently supports bfloat16 only.")
    device = q.device
    head_dim = q.shape[-1]
    if cu_seqlens_q is not None:
        out_shape, lse_shape = (total_q, num_head, head_dim), (num_head, total_q)
    else:
        out_shape, lse_shape = (batch_size, seqlen_q, num_head, head_dim), (batch_size, num_head, seqlen_q)
    _validate_tensor(out, "out", out_shape, q.dtype, device)
    _validate_tensor(dout, "dout", out_shape, q.dtype, device)
    _validate_tensor(lse, "lse", lse_shape, torch.float32, device)
    if dlse is not None:
        _validate_tensor(dlse, "dlse", lse_shape, torch.float32, device)
        dlse = dlse.contiguous()
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(head_dim)

    q, k, v, out, dout = (_prep(t.detach()) for t in (q, k, v, out, dout))
    lse = lse.contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if total_q == 0 or k.shape[-3] == 0:
        return dq.zero_(), dk.zero_(), dv.zero_()

    packed = cu_seqlens_q is not None
    params = _fill_params(
        q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal
    )
    params.dout, params.dlse = _ptr(dout), _ptr(dlse)
    params.debug = _ptr(debug)
    params.dq, params.dk, params.dv = _ptr(dq), _ptr(dk), _ptr(dv)
    params.do_strides[:] = _strides3(dout, packed)
    params.dq_strides[:] = _strides3(dq, packed)
    params.dk_strides[:] = _strides3(dk, packed)
    params.dv_strides[:] = _strides3(dv, packed)
    lib = _capi.load_library()
    if out_resid is not None and out_resid.numel():
        if out_resid.dtype != torch.uint8 or out_resid.device != device or not out_resid.is_contiguous():
            raise TypeError("out_resid must be the uint8 tensor a forward with keep_resid=True returned")
        if out_resid.numel() != lib.splitd_out_resid_bytes(ctypes.byref(params)):
            raise ValueError("out_resid does not belong to a forward of this shape")
        params.o_resid = _ptr(out_resid)
    n_stat = lib.splitd_bwd_rowstat_elems(ctypes.byref(params))
    if _WORKSPACE_LIMIT is None:
        n_ws = lib.splitd_bwd_workspace_bytes(ctypes.byref(params))
    else:
        n_ws = lib.splitd_bwd_workspace_bytes_limit(ctypes.byref(params), _WORKSPACE_LIMIT)
    dpsum = torch.empty(n_stat, dtype=torch.float32, device=device)
    lse_log2 = torch.empty(n_stat, dtype=torch.float32, device=device)
    workspace = torch.empty(n_ws, dtype=torch.uint8, device=device)
    params.dpsum, params.lse_log2 = _ptr(dpsum), _ptr(lse_log2)
    params.workspace, params.workspace_bytes = _ptr(workspace), n_ws
    with torch.cuda.device(device):
        if stage_events is None:
            _capi.check(lib.splitd_bwd(ctypes.byref(params), _stream_ptr(device)))
        else:
            # the launches splitd_bwd makes (preprocess; per chunk: P/dS tiles, gradient GEMMs), with a CUDA event
            # in front of each and one after the last: (label, event) pairs for per-kernel timing
            def mark(label):
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                stage_events.append((label, ev))

            mark("bwd_preprocess")
            _capi.check(lib.splitd_bwd_preprocess(ctypes.byref(params), _stream_ptr(device)))
            n_chunks = lib.splitd_bwd_num_chunks(ctypes.byref(params))
            if n_chunks < 0:
                _capi.check(n_chunks)
            for c in range(n_chunks):
                mark("bwd_tiles")
                _capi.check(lib.splitd_bwd_chunk(ctypes.byref(params), c, 1, _stream_ptr(device)))
                mark("bwd_grads")
                _capi.check(lib.splitd_bwd_chunk(ctypes.byref(params), c, 2, _stream_ptr(device)))
            mark("end")
    return dq, dk, dv


# ---------------------------------------------------------------------------
# autograd (FlashAttnFunc, interface.py:1117-1173; varlen op pair, interface.py:909-1109)
# ---------------------------------------------------------------------------


class FlashAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, window_size, softcap, pack_gqa, return_lse):
        keep = bool(_KEEP_RESIDUAL) and any(ctx.needs_input_grad[:3])
        out, lse, *rest = _flash_attn_fwd(
            q,
            k,
            v,
            softmax_scale=softmax_scale,
            causal=causal,
            window_size_left=window_size[0],
            window_size_right=window_size[1],
            softcap=softcap,
            pack_gqa=pack_gqa,
            return_lse=return_lse,
            keep_resid=keep,
        )
        ctx.has_resid = keep
        ctx.save_for_backward(q, k, v, out, lse, *rest)
        ctx.softmax_scale = softmax_scale
        ctx.causal = causal
        ctx.window_size = window_size
        ctx.softcap = softcap
        ctx.return_lse = return_lse
        ctx.set_materialize_grads(False)
        return out, lse

    @staticmethod
    def backward(ctx, dout, dlse):
        q, k, v, out, lse = ctx.saved_tensors[:5]
        resid = ctx.saved_tensors[5] if ctx.has_resid else None
        if not ctx.return_lse:
            dlse = None
        if dout is None:
            dout = torch.zeros_like(out)
        dq, dk, dv = _flash_attn_bwd(
            q,
            k,
            v,
            out,
            dout,
            lse,
            ctx.softmax_scale,
            ctx.causal,
            ctx.softcap,
            window_size_left=ctx.window_size[0],
            window_size_right=ctx.window_size[1],
            dlse=dlse,
            out_resid=resid,
        )
        return dq, dk, dv, None, None, None, None, None, None


# ---------------------------------------------------------------------------
# PyTorch custom ops for the packed layout (same op names, schemas and fake kernels as the reference's
# ``splitd_flash_attn::varlen_fwd`` / ``varlen_bwd``, interface.py:909-1109), so the packed path can be
# traced by FakeTensor / torch.compile. Optional window ints are encoded as -2**31 for "None".
# ---------------------------------------------------------------------------
_NONE_INT = -(2**31)


def _enc(v: Optional[int]) -> int:
    return _NONE_INT if v is None else int(v)


def _dec(v: int) -> Optional[int]:
    return None if v == _NONE_INT else v


@torch.library.custom_op("splitd_flash_attn::varlen_fwd", mutates_args=())
def _varlen_fwd_custom(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    softmax_scale: float,
    causal: bool,
    window_size_left: int,
    window_size_right: int,
    softcap: float,
    pack_gqa: bool,
) -> tuple[torch.Tensor, torch.Tensor]:
    return _flash_attn_fwd(
        q,
        k,
        v,
        cu_seqlens_q=cu_seqlens_q,
        cu_seqlens_k=cu_seqlens_k,
        max_seqlen_q=max_seqlen_q,
        max_seqlen_k=max_seqlen_k,
        softmax_scale=softmax_scale,
        causal=causal,
        window_size_left=_dec(window_size_left),
        window_size_right=_dec(window_size_right),
        softcap=softcap,
        pack_gqa=pack_gqa,
        return_lse=True,
    )


def _fake_shapes(q, k, v, cu_seqlens_q, cu_seqlens_k):
    """Shape / dtype checks that need no device values (what a fake kernel may look at)."""
    if q.ndim != 3 or k.ndim != 3 or v.ndim != 3:
        raise ValueError("q, k and v must be rank-3 packed tensors")
    if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_k.dtype != torch.int32:
        raise TypeError("cu_seqlens must have dtype torch.int32")
    _validate_head_dims(q.shape[-1], v.shape[-1])
    if q.shape[-2] % k.shape[-2] != 0:
        raise ValueError(f"num_head ({q.shape[-2]}) must be divisible by num_head_kv ({k.shape[-2]})")


@torch.library.register_fake("splitd_flash_attn::varlen_fwd")
def _varlen_fwd_fake(
    q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal, window_size_left,
    window_size_right, softcap, pack_gqa,
):
    _fake_shapes(q, k, v, cu_seqlens_q, cu_seqlens_k)
    _validate_training_dtype(q, q.requires_grad or k.requires_grad or v.requires_grad)
    out = q.new_empty((q.shape[0], q.shape[1], v.shape[-1]))
    lse = q.new_empty((q.shape[1], q.shape[0]), dtype=torch.float32)
    return out, lse


@torch.library.custom_op("splitd_flash_attn::varlen_bwd", mutates_args=())
def _varlen_bwd_custom(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    dout: torch.Tensor,
    lse: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    softmax_scale: float,
    causal: bool,
    window_size_left: int,
    window_size_right: int,
    softcap: float,
    dlse: Optional[torch.Tensor],
    out_resid: Optional[torch.Tensor] = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _flash_attn_bwd(
        q,
        k,
        v,
        out,
        dout,
        lse,
        softmax_scale=softmax_scale,
        causal=causal,
        softcap=softcap,
        window_size_left=_dec(window_size_left),
        window_size_right=_dec(window_size_right),
        cu_seqlens_q=cu_seqlens_q,
        cu_seqlens_k=cu_seqlens_k,
        max_seqlen_q=max_seqlen_q,
        max_seqlen_k=max_seqlen_k,
        dlse=dlse,
        out_resid=out_resid,
    )


@torch.library.register_fake("splitd_flash_attn::varlen_bwd")
def _varlen_bwd_fake(
    q, k, v, out, dout, lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal,
    window_size_left, window_size_right, softcap, dlse, out_resid=None,
):
    _fake_shapes(q, k, v, cu_seqlens_q, cu_seqlens_k)
    if q.dtype == torch.float16:
        raise NotImplementedError("SplitD backward currently supports bfloat16 only.")
    if softcap != 0.0:
        raise NotImplementedError("SplitD backward does not support softcap yet")
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _varlen_setup_context(ctx, inputs, output) -> None:
    q, k, v, cu_seqlens_q, cu_seqlens_k = inputs[:5]
    ctx.max_seqlen_q, ctx.max_seqlen_k, ctx.softmax_scale, ctx.causal = inputs[5:9]
    ctx.window_size_left, ctx.window_size_right, ctx.softcap = inputs[9:12]
    out, lse = output
    ctx.save_for_backward(q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k)
    ctx.set_materialize_grads(False)


def _varlen_backward(ctx, dout, dlse):
    q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
    if dout is None:
        dout = torch.zeros_like(out)
    dq, dk, dv = torch.ops.splitd_flash_attn.varlen_bwd(
        q, k, v, out, dout, lse, cu_q, cu_k, ctx.max_seqlen_q, ctx.max_seqlen_k, ctx.softmax_scale, ctx.causal,
        ctx.window_size_left, ctx.window_size_right, ctx.softcap, dlse,
    )
    return dq, dk, dv, *((None,) * 10)


torch.library.register_autograd("splitd_flash_attn::varlen_fwd", _varlen_backward, setup_context=_varlen_setup_context)


# ---------------------------------------------------------------------------
# PyTorch custom ops for the batched layout: ``splitd_flash_attn::fwd`` / ``::bwd``. The reference registers
# ops for the packed layout only and runs the batched one through ``FlashAttnFunc`` (interface.py:1117-1173);
# with an op pair of its own the batched call is traceable by FakeTensor / torch.compile too. Same encoding of
# the optional window ints as above.
# ---------------------------------------------------------------------------


@torch.library.custom_op("splitd_flash_attn::fwd", mutates_args=())
def _fwd_custom(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: float,
    causal: bool,
    window_size_left: int,
    window_size_right: int,
    softcap: float,
    pack_gqa: bool,
) -> tuple[torch.Tensor, torch.Tensor]:
    return _flash_attn_fwd(
        q,
        k,
        v,
        softmax_scale=softmax_scale,
        causal=causal,
        window_size_left=_dec(window_size_left),
        window_size_right=_dec(window_size_right),
        softcap=softcap,
        pack_gqa=pack_gqa,
        return_lse=True,
    )


def _fake_shapes_batched(q, k, v):
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("q, k and v must be rank-4 (batch, seqlen, heads, head_dim) tensors")
    _validate_head_dims(q.shape[-1], v.shape[-1])
    if q.shape[-2] % k.shape[-2] != 0:
        raise ValueError(f"num_head ({q.shape[-2]}) must be divisible by num_head_kv ({k.shape[-2]})")


@torch.library.register_fake("splitd_flash_attn::fwd")
def _fwd_fake(q, k, v, softmax_scale, causal, window_size_left, window_size_right, softcap, pack_gqa):
    _fake_shapes_batched(q, k, v)
    _validate_training_dtype(q, q.requires_grad or k.requires_grad or v.requires_grad)
    out = q.new_empty((q.shape[0], q.shape[1], q.shape[2], v.shape[-1]))
    lse = q.new_empty((q.shape[0], q.shape[2], q.shape[1]), dtype=torch.float32)
    return out, lse


@torch.library.custom_op("splitd_flash_attn::bwd", mutates_args=())
def _bwd_custom(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    dout: torch.Tensor,
    lse: torch.Tensor,
    softmax_scale: float,
    causal: bool,
    window_size_left: int,
    window_size_right: int,
    softcap: float,
    dlse: Optional[torch.Tensor],
    out_resid: Optional[torch.Tensor] = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _flash_attn_bwd(
        q,
        k,
        v,
        out,
        dout,
        lse,
        softmax_scale=softmax_scale,
        causal=causal,
        softcap=softcap,
        window_size_left=_dec(window_size_left),
        window_size_right=_dec(window_size_right),
        dlse=dlse,
        out_resid=out_resid,
    )


@torch.library.register_fake("splitd_flash_attn::bwd")
def _bwd_fake(
    q, k, v, out, dout, lse, softmax_scale, causal, window_size_left, window_size_right, softcap, dlse, out_resid=None
):
    _fake_shapes_batched(q, k, v)
    if q.dtype == torch.float16:
        raise NotImplementedError("SplitD backward currently supports bfloat16 only.")
    if softcap != 0.0:
        raise NotImplementedError("SplitD backward does not support softcap yet")
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _batched_setup_context(ctx, inputs, output) -> None:
    q, k, v = inputs[:3]
    ctx.softmax_scale, ctx.causal, ctx.window_size_left, ctx.window_size_right, ctx.softcap = inputs[3:8]
    out, lse = output
    ctx.save_for_backward(q, k, v, out, lse)
    ctx.set_materialize_grads(False)


def _batched_backward(ctx, dout, dlse):
    q, k, v, out, lse = ctx.saved_tensors
    if dout is None:
        dout = torch.zeros_like(out)
    dq, dk, dv = torch.ops.splitd_flash_attn.bwd(
        q, k, v, out, dout, lse, ctx.softmax_scale, ctx.causal, ctx.window_size_left, ctx.window_size_right,
        ctx.softcap, dlse,
    )
    return dq, dk, dv, *((None,) * 6)


torch.library.register_autograd("splitd_flash_attn::fwd", _batched_backward, setup_context=_batched_setup_context)


# ---------------------------------------------------------------------------
# Training forwards that also return the low word of the output (see _KEEP_RESIDUAL): ``fwd_resid`` and
# ``varlen_fwd_resid`` are ``fwd`` / ``varlen_fwd`` with a third result, and their backward hands it to the
# ``bwd`` / ``varlen_bwd`` ops above. The two-result ops keep the reference's schemas (and its backward, which
# reads the 16-bit output).
# ---------------------------------------------------------------------------


def _resid_bytes(out: torch.Tensor) -> int:
    """Size of the low-word scratch of an output (what splitd_out_resid_bytes returns): a flag byte per row of
    512, padded to 256 bytes, then a 16-bit row of 512 per row."""
    rows = out.numel() // out.shape[-1]
    return (rows + 255) // 256 * 256 + rows * out.shape[-1] * 2


@torch.library.custom_op("splitd_flash_attn::fwd_resid", mutates_args=())
def _fwd_resid_custom(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: float,
    causal: bool,
    window_size_left: int,
    window_size_right: int,
    softcap: float,
    pack_gqa: bool,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _flash_attn_fwd(
        q,
        k,
        v,
        softmax_scale=softmax_scale,
        causal=causal,
        window_size_left=_dec(window_size_left),
        window_size_right=_dec(window_size_right),
        softcap=softcap,
        pack_gqa=pack_gqa,
        return_lse=True,
        keep_resid=True,
    )


@torch.library.register_fake("splitd_flash_attn::fwd_resid")
def _fwd_resid_fake(q, k, v, softmax_scale, causal, window_size_left, window_size_right, softcap, pack_gqa):
    out, lse = _fwd_fake(q, k, v, softmax_scale, causal, window_size_left, window_size_right, softcap, pack_gqa)
    return out, lse, out.new_empty((_resid_bytes(out),), dtype=torch.uint8)


def _batched_resid_setup_context(ctx, inputs, output) -> None:
    q, k, v = inputs[:3]
    ctx.softmax_scale, ctx.causal, ctx.window_size_left, ctx.window_size_right, ctx.softcap = inputs[3:8]
    out, lse, resid = output
    ctx.save_for_backward(q, k, v, out, lse, resid)
    ctx.set_materialize_grads(False)


def _batched_resid_backward(ctx, dout, dlse, _dresid):
    q, k, v, out, lse, resid = ctx.saved_tensors
    if dout is None:
        dout = torch.zeros_like(out)
    dq, dk, dv = torch.ops.splitd_flash_attn.bwd(
        q, k, v, out, dout, lse, ctx.softmax_scale, ctx.causal, ctx.window_size_left, ctx.window_size_right,
        ctx.softcap, dlse, resid,
    )
    return dq, dk, dv, *((None,) * 6)


torch.library.register_autograd(
    "splitd_flash_attn::fwd_resid", _batched_resid_backward, setup_context=_batched_resid_setup_context
)


@torch.library.custom_op("splitd_flash_attn::varlen_fwd_resid", mutates_args=())
def _varlen_fwd_resid_custom(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    softmax_scale: float,
    causal: bool,
    window_size_left: int,
    window_size_right: int,
    softcap: float,
    pack_gqa: bool,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _flash_attn_fwd(
        q,
        k,
        v,
        cu_seqlens_q=cu_seqlens_q,
        cu_seqlens_k=cu_seqlens_k,
        max_seqlen_q=max_seqlen_q,
        max_seqlen_k=max_seqlen_k,
        softmax_scale=softmax_scale,
        causal=causal,
        window_size_left=_dec(window_size_left),
        window_size_right=_dec(window_size_right),
        softcap=softcap,
        pack_gqa=pack_gqa,
        return_lse=True,
        keep_resid=True,
    )


@torch.library.register_fake("splitd_flash_attn::varlen_fwd_resid")
def _varlen_fwd_resid_fake(
    q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal, window_size_left,
    window_size_right, softcap, pack_gqa,
):
    out, lse = _varlen_fwd_fake(
        q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal, window_size_left,
        window_size_right, softcap, pack_gqa,
    )
    return out, lse, out.new_empty((_resid_bytes(out),), dtype=torch.uint8)


def _varlen_resid_setup_context(ctx, inputs, output) -> None:
    q, k, v, cu_seqlens_q, cu_seqlens_k = inputs[:5]
    ctx.max_seqlen_q, ctx.max_seqlen_k, ctx.softmax_scale, ctx.causal = inputs[5:9]
    ctx.window_size_left, ctx.window_size_right, ctx.softcap = inputs[9:12]
    out, lse, resid = output
    ctx.save_for_backward(q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, resid)
    ctx.set_materialize_grads(False)


def _varlen_resid_backward(ctx, dout, dlse, _dresid):
    q, k, v, out, lse, cu_q, cu_k, resid = ctx.saved_tensors
    if dout is None:
        dout = torch.zeros_like(out)
    dq, dk, dv = torch.ops.splitd_flash_attn.varlen_bwd(
        q, k, v, out, dout, lse, cu_q, cu_k, ctx.max_seqlen_q, ctx.max_seqlen_k, ctx.softmax_scale, ctx.causal,
        ctx.window_size_left, ctx.window_size_right, ctx.softcap, dlse, resid,
    )
    return dq, dk, dv, *((None,) * 10)


torch.library.register_autograd(
    "splitd_flash_attn::varlen_fwd_resid", _varlen_resid_backward, setup_context=_varlen_resid_setup_context
)


# ---------------------------------------------------------------------------
# public API
# ---------------------------------------------------------------------------


def _wants_residual(q, k, v) -> bool:
    """A forward whose result can be differentiated keeps the low word of the output (if that is switched on)."""
    return bool(_KEEP_RESIDUAL) and torch.is_grad_enabled() and any(
        isinstance(t, torch.Tensor) and t.requires_grad for t in (q, k, v)
    )


def _reject_unsupported_training(q, k, v, softcap, window_size) -> None:
    """Inside a custom op the tensors no longer say whether they require grad, so what training does not
    support (fp16, softcap, sliding windows; interface.py:133-138,264-286 of the reference) is refused here."""
    tensors = [t for t in (q, k, v) if isinstance(t, torch.Tensor)]
    if not (torch.is_grad_enabled() and any(t.requires_grad for t in tensors)):
        return
    _validate_training_dtype(q, True)
    if isinstance(window_size, tuple) and len(window_size) == 2:
        try:
            _, local = _resolve_causal_local_window(False, window_size[0], window_size[1])
        except ValueError:
            local = False
        _unsupported_features(True, softcap, local)


def split_flash_attn_func(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    window_size: Tuple[Optional[int], Optional[int]] = (None, None),
    softcap: float = 0.0,
    pack_gqa: Optional[bool] = None,
    return_lse: bool = False,
):
    """Batched SplitD FlashAttention for D=512 (interface.py:1226-1252 of the reference).

    q (B, Sq, Hq, 512), k/v (B, Sk, Hkv, 512) with Hq % Hkv == 0. Returns ``out`` or ``(out, lse)``.
    Training requires bf16 q/k/v; fp16 is accepted only for no-grad forward. Runs through the
    ``splitd_flash_attn::fwd`` / ``::bwd`` custom ops (``FlashAttnFunc`` is the same thing as a plain
    autograd.Function, as in the reference).
    """
    if not isinstance(window_size, tuple) or len(window_size) != 2:
        raise TypeError("window_size must be a tuple of (left, right)")
    _reject_unsupported_training(q, k, v, softcap, window_size)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    if pack_gqa is None:
        pack_gqa = q.ndim == 4 and k.ndim == 4 and q.shape[-2] > k.shape[-2]
    op = torch.ops.splitd_flash_attn.fwd_resid if _wants_residual(q, k, v) else torch.ops.splitd_flash_attn.fwd
    out, lse = op(
        q,
        k,
        v,
        float(softmax_scale),
        bool(causal),
        _enc(window_size[0]),
        _enc(window_size[1]),
        float(softcap),
        bool(pack_gqa),
    )[:2]
    return (out, lse) if return_lse else out


def split_flash_attn_varlen_func(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens_q: Optional[torch.Tensor] = None,
    cu_seqlens_k: Optional[torch.Tensor] = None,
    max_seqlen_q: Optional[int] = None,
    max_seqlen_k: Optional[int] = None,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    window_size: Tuple[Optional[int], Optional[int]] = (None, None),
    softcap: float = 0.0,
    pack_gqa: Optional[bool] = None,
    score_mod: Optional[Callable] = None,
    aux_tensors: Optional[list] = None,
    return_lse: bool = False,
):
    """Packed (varlen) SplitD FlashAttention for D=512 (interface.py:1255-1316 of the reference).

    q (Tq, Hq, 512), k/v (Tk, Hkv, 512); ``cu_seqlens_q/k`` int32 CUDA tensors of B+1 entries and
    ``max_seqlen_q/k`` are mandatory. Returns ``out`` or ``(out, lse)`` with lse (Hq, Tq).
    """
    if cu_seqlens_q is None or cu_seqlens_k is None:
        raise ValueError("split_flash_attn_varlen_func requires cu_seqlens_q and cu_seqlens_k")
    if max_seqlen_q is None:
        raise ValueError("max_seqlen_q must be provided when cu_seqlens_q is provided")
    if max_seqlen_k is None:
        raise ValueError("max_seqlen_k must be provided when cu_seqlens_k is provided")
    if score_mod is not None:
        raise NotImplementedError("score_mod is not supported by the SplitD varlen path")
    if aux_tensors is not None:
        raise NotImplementedError("aux_tensors is not supported by the SplitD varlen path")
    if not isinstance(window_size, tuple) or len(window_size) != 2:
        raise TypeError("window_size must be a tuple of (left, right)")
    _reject_unsupported_training(q, k, v, softcap, window_size)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    if pack_gqa is None:
        pack_gqa = q.shape[-2] > k.shape[-2]
    op = torch.ops.splitd_flash_attn.varlen_fwd_resid if _wants_residual(q, k, v) else torch.ops.splitd_flash_attn.varlen_fwd
    out, lse = op(
        q,
        k,
        v,
        cu_seqlens_q,
        cu_seqlens_k,
        max_seqlen_q,
        max_seqlen_k,
        float(softmax_scale),
        bool(causal),
        _enc(window_size[0]),
        _enc(window_size[1]),
        float(softcap),
        bool(pack_gqa),
    )[:2]
    return (out, lse) if return_lse else out
