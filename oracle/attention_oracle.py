"""CPU oracle for the D=512 attention path -- TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import this
file. The product (gemm4-attention-kernels_b200/) never does and has no CPU fallback.

It restates, in plain fp32 PyTorch tensor algebra, the reference's own definition of the path:

* ``attention_fwd``  follows ``attention_ref`` in the reference's test-suite
  (splitd-flash-attn/tests/test_flash_fwd_splitd_sdpa.py:132-157): GQA by repeating each KV head
  over its query heads, scores = (q * scale) k^T, bottom-right aligned causal mask
  ``triu(diagonal = Sk - Sq + 1)`` (:151-155), softmax, probabilities times v.
* ``lse``            follows the reference's LSE check (:562-571): logsumexp of the masked scaled scores.
* ``attention_bwd``  is the closed form of what the reference obtains with ``torch.autograd.grad`` on
  ``attention_ref`` (:758-760) and what its kernels compute (src/flash_bwd_preprocess.py:289-315,
  src/fmha_dkdv_sm90_d512.py:971-1170, src/fmha_dq_sm90_d512.py:942-1112):
      P = exp(S - lse), dV = P^T dO, dP = dO V^T, delta = rowsum(dO * O) - dlse,
      dS = P * (dP - delta) * scale, dQ = dS K, dK = dS^T Q, with dK/dV summed over the query heads
      of each KV head.
* ``attention_math_lowp`` is the error yardstick: the same algebra with 16-bit matmuls and an fp32
  softmax (``attention_ref_pt``, :160-185).

Parity pin: tests/golden/ holds outputs of the reference's own ``attention_ref`` + autograd, generated
in a container where the reference is importable (tests/golden/make_golden.py); tests/test_oracle.py
checks this file against them.

Everything is chunked over (batch, KV head, query-row block) so full benchmark shapes fit in memory;
it runs on any torch device (CPU for the baseline, and the GPU box's device when a test needs a
full-size check in reasonable time).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

ROW_BLOCK = 2048


def _causal_mask(rows: torch.Tensor, sk: int, sq: int, device) -> torch.Tensor:
    """True where key j is hidden from query i: j > i + sk - sq (bottom-right aligned)."""
    cols = torch.arange(sk, device=device)
    return cols[None, :] > (rows[:, None] + (sk - sq))


def _window_mask(rows: torch.Tensor, sk: int, sq: int, window, device) -> torch.Tensor:
    """Sliding window (left, right), None / negative = unbounded: key j is hidden from query i when
    j > i + sk - sq + right or j < i + sk - sq - left (src/testing.py:237-266 of the reference)."""
    cols = torch.arange(sk, device=device)[None, :]
    diag = rows[:, None] + (sk - sq)
    m = torch.zeros(rows.numel(), sk, dtype=torch.bool, device=device)
    left, right = window
    if right is not None and right >= 0:
        m |= cols > diag + right
    if left is not None and left >= 0:
        m |= cols < diag - left
    return m


def attention_fwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    causal: bool = False,
    softmax_scale: Optional[float] = None,
    compute_dtype: torch.dtype = torch.float32,
    softcap: float = 0.0,
    window: Tuple[Optional[int], Optional[int]] = (None, None),
) -> Tuple[torch.Tensor, torch.Tensor]:
    """q (B,Sq,Hq,D), k/v (B,Sk,Hkv,D) -> out (B,Sq,Hq,D) fp32, lse (B,Hq,Sq) fp32.
    softcap > 0: scores = softcap * tanh(scores / softcap) before masking
    (tests/test_flash_fwd_splitd_sdpa.py:111-113); window: see _window_mask."""
    B, sq, hq, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    g = hq // hkv
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else float(softmax_scale)
    dev = q.device
    out = torch.empty(B, sq, hq, v.shape[-1], dtype=compute_dtype, device=dev)
    lse = torch.empty(B, hq, sq, dtype=compute_dtype, device=dev)
    for b in range(B):
        for h in range(hkv):
            kh = k[b, :, h].to(compute_dtype)  # (Sk, D)
            vh = v[b, :, h].to(compute_dtype)
            for r0 in range(0, sq, ROW_BLOCK):
                r1 = min(sq, r0 + ROW_BLOCK)
                qh = q[b, r0:r1, h * g : (h + 1) * g].to(compute_dtype)  # (R, G, D)
                s = torch.einsum("rgd,kd->grk", qh * scale, kh)  # (G, R, Sk)
                if softcap > 0:
                    s = softcap * torch.tanh(s / softcap)
                rows = torch.arange(r0, r1, device=dev)
                if causal:
                    s = s.masked_fill(_causal_mask(rows, sk, sq, dev)[None], float("-inf"))
                if window[0] is not None or window[1] is not None:
                    s = s.masked_fill(_window_mask(rows, sk, sq, window, dev)[None], float("-inf"))
                l = torch.logsumexp(s, dim=-1)  # (G, R)
                p = torch.exp(s - torch.where(torch.isinf(l), torch.zeros_like(l), l)[..., None])
                p = torch.where(torch.isinf(l)[..., None], torch.zeros_like(p), p)
                out[b, r0:r1, h * g : (h + 1) * g] = torch.einsum("grk,kd->rgd", p, vh)
                lse[b, h * g : (h + 1) * g, r0:r1] = l
    return out, lse


def attention_bwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    dout: torch.Tensor,
    causal: bool = False,
    softmax_scale: Optional[float] = None,
    dlse: Optional[torch.Tensor] = None,
    compute_dtype: torch.dtype = torch.float32,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of attention_fwd w.r.t. q, k, v for upstream dout (and optionally dlse)."""
    B, sq, hq, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    g = hq // hkv
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else float(softmax_scale)
    dev = q.device
    dq = torch.zeros(B, sq, hq, d, dtype=compute_dtype, device=dev)
    dk = torch.zeros(B, sk, hkv, d, dtype=compute_dtype, device=dev)
    dv = torch.zeros(B, sk, hkv, v.shape[-1], dtype=compute_dtype, device=dev)
    for b in range(B):
        for h in range(hkv):
            kh = k[b, :, h].to(compute_dtype)
            vh = v[b, :, h].to(compute_dtype)
            for r0 in range(0, sq, ROW_BLOCK):
                r1 = min(sq, r0 + ROW_BLOCK)
                qh = q[b, r0:r1, h * g : (h + 1) * g].to(compute_dtype)  # (R,G,D)
                doh = dout[b, r0:r1, h * g : (h + 1) * g].to(compute_dtype)
                s = torch.einsum("rgd,kd->grk", qh * scale, kh)
                if causal:
                    m = _causal_mask(torch.arange(r0, r1, device=dev), sk, sq, dev)
                    s = s.masked_fill(m[None], float("-inf"))
                l = torch.logsumexp(s, dim=-1)
                dead = torch.isinf(l)
                p = torch.exp(s - torch.where(dead, torch.zeros_like(l), l)[..., None])
                p = torch.where(dead[..., None], torch.zeros_like(p), p)  # (G,R,Sk)
                o = torch.einsum("grk,kd->grd", p, vh)
                delta = (o * doh.permute(1, 0, 2)).sum(-1)  # (G,R)
                if dlse is not None:
                    delta = delta - dlse[b, h * g : (h + 1) * g, r0:r1].to(compute_dtype)
                dp = torch.einsum("rgd,kd->grk", doh, vh)
                ds = p * (dp - delta[..., None]) * scale
                dv[b, :, h] += torch.einsum("grk,rgd->kd", p, doh)
                dk[b, :, h] += torch.einsum("grk,rgd->kd", ds, qh)
                dq[b, r0:r1, h * g : (h + 1) * g] = torch.einsum("grk,kd->rgd", ds, kh)
    return dq, dk, dv


def attention_math_lowp(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False, softmax_scale: Optional[float] = None,
    softcap: float = 0.0, window: Tuple[Optional[int], Optional[int]] = (None, None),
) -> torch.Tensor:
    """Error yardstick: matmuls in the input's 16-bit dtype, softmax in fp32, probabilities cast back
    (tests/test_flash_fwd_splitd_sdpa.py:160-185). Returns (B,Sq,Hq,D) in the input dtype."""
    B, sq, hq, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    g = hq // hkv
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else float(softmax_scale)
    qt = q.transpose(1, 2)
    kt = k.transpose(1, 2).repeat_interleave(g, dim=1)
    vt = v.transpose(1, 2).repeat_interleave(g, dim=1)
    s = torch.matmul(qt * scale, kt.transpose(-2, -1))
    if softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    rows = torch.arange(sq, device=q.device)
    if causal:
        s = s.masked_fill(_causal_mask(rows, sk, sq, q.device), float("-inf"))
    if window[0] is not None or window[1] is not None:
        s = s.masked_fill(_window_mask(rows, sk, sq, window, q.device), float("-inf"))
    attn = torch.softmax(s, dim=-1, dtype=torch.float32)
    attn = torch.nan_to_num(attn, nan=0.0).to(q.dtype)
    return torch.matmul(attn, vt).transpose(1, 2)


def attention_fwd_varlen(q, k, v, cu_q, cu_k, causal=False, softmax_scale=None, compute_dtype=torch.float32):
    """Packed layout: q (Tq,Hq,D), k/v (Tk,Hkv,D), cu_* python lists / int tensors of B+1 offsets.
    Per-sequence application of attention_fwd (the reference's varlen tests do the same,
    tests/test_flash_fwd_splitd_sdpa.py:655-690). Returns out (Tq,Hq,D), lse (Hq,Tq)."""
    cu_q = [int(x) for x in cu_q]
    cu_k = [int(x) for x in cu_k]
    out = torch.empty(q.shape[0], q.shape[1], v.shape[-1], dtype=compute_dtype, device=q.device)
    lse = torch.empty(q.shape[1], q.shape[0], dtype=compute_dtype, device=q.device)
    for b in range(len(cu_q) - 1):
        qs, qe, ks, ke = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
        if qe == qs:
            continue
        o, l = attention_fwd(q[None, qs:qe], k[None, ks:ke], v[None, ks:ke], causal, softmax_scale, compute_dtype)
        out[qs:qe] = o[0]
        lse[:, qs:qe] = l[0]
    return out, lse


def attention_bwd_varlen(q, k, v, dout, cu_q, cu_k, causal=False, softmax_scale=None, compute_dtype=torch.float32):
    cu_q = [int(x) for x in cu_q]
    cu_k = [int(x) for x in cu_k]
    dq = torch.zeros(q.shape, dtype=compute_dtype, device=q.device)
    dk = torch.zeros(k.shape, dtype=compute_dtype, device=q.device)
    dv = torch.zeros(v.shape, dtype=compute_dtype, device=q.device)
    for b in range(len(cu_q) - 1):
        qs, qe, ks, ke = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
        if qe == qs or ke == ks:
            continue
        a, bb, c = attention_bwd(
            q[None, qs:qe], k[None, ks:ke], v[None, ks:ke], dout[None, qs:qe], causal, softmax_scale, None, compute_dtype
        )
        dq[qs:qe], dk[ks:ke], dv[ks:ke] = a[0], bb[0], c[0]
    return dq, dk, dv


def attention_flops(batch, heads_q, sq, sk, d, causal) -> float:
    """4*B*Hq*Sq*Sk_avg*D with the causal average key count (src/bench_utils.py:16-46)."""
    sk_avg = (max(0, sk - sq) + sk) / 2 if causal else sk
    return 4.0 * batch * heads_q * sq * sk_avg * d
