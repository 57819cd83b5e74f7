"""Helpers shared by the GPU parity tests: seeded inputs, the error yardstick, the acceptance rule.

Acceptance: the max-abs error of the CUDA result (out, dq, dk, dv) against the fp32 oracle must be
<= 2x the max-abs error of PyTorch's math scaled-dot-product attention run in the inputs' 16-bit dtype
on the same inputs (`F.scaled_dot_product_attention` under `SDPBackend.MATH`, GQA by `repeat_interleave`,
bottom-right aligned causal mask, gradients from autograd), and |LSE - oracle LSE| <= 1e-3. This is
stricter than the reference's own tests, which allow 2x-4x the error of a 16-bit matmul restatement plus
an absolute slack (tests/test_flash_fwd_splitd_sdpa.py:300-331,790-809); that looser figure
(`attention_math_lowp`) is still computed and printed beside the ratio.
"""
import torch
import torch.nn.functional as F
from torch.nn.attention import SDPBackend, sdpa_kernel

from oracle import attention_oracle as O

D = 512
LSE_TOL = 1e-3
ERR_FACTOR = 2.0
ATOL = 1e-6
SDPA_ROW_BLOCK = 2048


def make_qkv(B, sq, sk, hq, hkv, dtype, seed, requires_grad=False, with_do=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, sq, hq, D, device="cuda", dtype=torch.float32, generator=g).to(dtype)
    k = torch.randn(B, sk, hkv, D, device="cuda", dtype=torch.float32, generator=g).to(dtype)
    v = torch.randn(B, sk, hkv, D, device="cuda", dtype=torch.float32, generator=g).to(dtype)
    do = torch.randn(B, sq, hq, D, device="cuda", dtype=torch.float32, generator=g).to(dtype) if with_do else None
    if requires_grad:
        q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    return q, k, v, do


def max_err(a, b):
    return (a.float() - b.float()).abs().max().item()


def _visible(rows, sk, sq, causal, window, device):
    """Boolean (R, Sk) mask, True where the key is visible (what SDPA's attn_mask wants)."""
    hidden = torch.zeros(rows.numel(), sk, dtype=torch.bool, device=device)
    if causal:
        hidden |= O._causal_mask(rows, sk, sq, device)
    if window[0] is not None or window[1] is not None:
        hidden |= O._window_mask(rows, sk, sq, window, device)
    return ~hidden


def sdpa_math(q, k, v, causal=False, scale=None, window=(None, None), do=None):
    """The yardstick: math-backend SDPA in the dtype of q (no softcap: SDPA has none).

    q (B,Sq,Hq,D), k/v (B,Sk,Hkv,D). Returns out, or (out, dq, dk, dv) when `do` is given. One call per
    (batch, KV head): shards are independent, so this is the same computation as one call on the whole
    tensor, in pieces that fit in memory. Up to SDPA_ROW_BLOCK query rows the call is literally
    `F.scaled_dot_product_attention` on the 16-bit tensors (GQA by `repeat_interleave`, whose backward sums
    the query heads' dk/dv in 16 bit). Beyond that, the (heads, rows, keys) score tensors of a whole sequence
    no longer fit, so the rows go through in blocks. For 16-bit inputs the math backend computes in fp32 and
    rounds its results once; the blocked form does the same thing explicitly: fp32 SDPA on the upcast inputs
    per row block, out and dq rounded to the input dtype per block (rows are independent), dk and dv
    accumulated over the blocks in fp32 and rounded once. That is never looser than a single call.
    """
    B, sq, hq, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    g = hq // hkv
    dev = q.device
    out = torch.empty(B, sq, hq, v.shape[-1], dtype=q.dtype, device=dev)
    want_grad = do is not None
    if want_grad:
        dq = torch.empty_like(q)
        dk = torch.empty_like(k)
        dv = torch.empty_like(v)
    blocked = sq > SDPA_ROW_BLOCK
    cdt = torch.float32 if blocked else q.dtype
    masked = causal or window[0] is not None or window[1] is not None
    for b in range(B):
        for h in range(hkv):
            kin = k[b, :, h].detach().to(cdt).clone().requires_grad_(want_grad)
            vin = v[b, :, h].detach().to(cdt).clone().requires_grad_(want_grad)
            kacc = vacc = None
            for r0 in range(0, sq, SDPA_ROW_BLOCK):
                r1 = min(sq, r0 + SDPA_ROW_BLOCK)
                rows = torch.arange(r0, r1, device=dev)
                mask = _visible(rows, sk, sq, causal, window, dev) if masked else None
                qb = q[b, r0:r1, h * g : (h + 1) * g].detach().to(cdt).transpose(0, 1).unsqueeze(0).clone()  # (1,G,R,D)
                qb.requires_grad_(want_grad)
                # GQA by repeat_interleave, like the reference's sdpa_ref (tests/test_flash_fwd_splitd_sdpa.py:107-110)
                kr = kin.unsqueeze(0).repeat_interleave(g, dim=0).unsqueeze(0)  # (1,G,Sk,D)
                vr = vin.unsqueeze(0).repeat_interleave(g, dim=0).unsqueeze(0)
                with sdpa_kernel(SDPBackend.MATH):
                    ob = F.scaled_dot_product_attention(qb, kr, vr, attn_mask=mask, scale=scale)
                if mask is not None:  # rows without a visible key: the reference defines out = 0 there
                    dead = ~mask.any(dim=-1)
                    if dead.any():
                        ob = torch.where(dead[None, None, :, None], torch.zeros_like(ob), ob)
                out[b, r0:r1, h * g : (h + 1) * g] = ob.detach()[0].transpose(0, 1).to(q.dtype)
                if want_grad:
                    dob = do[b, r0:r1, h * g : (h + 1) * g].to(cdt).transpose(0, 1).unsqueeze(0)
                    gq, gk, gv = torch.autograd.grad(ob, (qb, kin, vin), dob)
                    dq[b, r0:r1, h * g : (h + 1) * g] = gq[0].transpose(0, 1).to(q.dtype)
                    kacc = gk if kacc is None else kacc + gk
                    vacc = gv if vacc is None else vacc + gv
            if want_grad:
                dk[b, :, h], dv[b, :, h] = kacc.to(q.dtype), vacc.to(q.dtype)
    return (out, dq, dk, dv) if want_grad else out


def rounding_yardstick(ref, dtype):
    """Error of the exact result rounded once to `dtype`. For 16-bit inputs the math backend computes in fp32
    and rounds its results once, so this IS its error (measured: identical for out and dq, and for dk/dv of
    MHA); used where SDPA cannot express the case (softcap, a gradient flowing into lse)."""
    return max_err(ref.to(dtype), ref)


def _report(name, err, yard, loose=None):
    extra = "" if loose is None else f", 16-bit-matmul restatement {loose:.3e}"
    print(f"    {name}: err {err:.3e} = {err / max(yard, 1e-30):.2f} x SDPA-MATH yardstick {yard:.3e}{extra}")


def check_fwd(out, lse, q, k, v, causal, scale=None, window=(None, None)):
    qd, kd, vd = q.detach(), k.detach(), v.detach()
    ref, lref = O.attention_fwd(qd, kd, vd, causal, scale, window=window)
    yard = max_err(sdpa_math(qd, kd, vd, causal, scale, window), ref)
    err = max_err(out, ref)
    _report("out", err, yard)
    assert not torch.isnan(out).any()
    assert err <= ERR_FACTOR * yard + ATOL, f"out err {err:.3e} > {ERR_FACTOR} x yardstick {yard:.3e}"
    if lse is not None:
        check_lse(lse, lref)
    return err, yard


def check_lse(lse, lref):
    finite = torch.isfinite(lref)
    assert torch.equal(torch.isfinite(lse), finite), "LSE -inf pattern differs"
    if finite.any():
        lerr = (lse - lref)[finite].abs().max().item()
        assert lerr <= LSE_TOL, f"lse err {lerr:.3e}"


def check_bwd(dq, dk, dv, q, k, v, do, causal, scale=None):
    qd, kd, vd = q.detach(), k.detach(), v.detach()
    rq, rk, rv = O.attention_bwd(qd, kd, vd, do, causal, scale)
    _, yq, yk, yv = sdpa_math(qd, kd, vd, causal, scale, do=do)
    ratios = {}
    for name, got, ref, y in (("dq", dq, rq, yq), ("dk", dk, rk, yk), ("dv", dv, rv, yv)):
        assert not torch.isnan(got).any(), name
        err, yard = max_err(got, ref), max_err(y, ref)
        _report(name, err, yard)
        assert err <= ERR_FACTOR * yard + ATOL, f"{name} err {err:.3e} > {ERR_FACTOR} x yardstick {yard:.3e}"
        ratios[name] = err / max(yard, 1e-30)
    return ratios


def check_all(out, lse, dq, dk, dv, q, k, v, do, causal, scale=None):
    """Forward + backward acceptance on one (B, S, H, D) problem small enough for the oracle."""
    check_fwd(out, lse, q, k, v, causal, scale)
    return check_bwd(dq, dk, dv, q, k, v, do, causal, scale)


def check_varlen(out, lse, grads, q, k, v, do, cu_q, cu_k, causal, scale=None, heads=None):
    """Packed layout: oracle and yardstick per sequence (that is what the packed call computes), errors and
    yardsticks taken over the whole packed tensors. `heads` = (query-head slice, kv-head slice) restricts the
    check to some heads of a large problem. `grads` = (dq, dk, dv) or None."""
    hs_q, hs_k = heads if heads is not None else (slice(None), slice(None))
    names = ("out", "dq", "dk", "dv") if grads is not None else ("out",)
    errs = dict.fromkeys(names, 0.0)
    yards = dict.fromkeys(names, 0.0)
    for b in range(len(cu_q) - 1):
        qs, qe, ks, ke = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
        if qe == qs:
            continue
        qb, kb, vb = q.detach()[None, qs:qe, hs_q], k.detach()[None, ks:ke, hs_k], v.detach()[None, ks:ke, hs_k]
        ro, rl = O.attention_fwd(qb, kb, vb, causal, scale)
        check_lse(lse[hs_q, qs:qe][None], rl)
        got = {"out": out[None, qs:qe, hs_q]}
        ref = {"out": ro}
        if grads is not None and ke > ks:
            dob = do[None, qs:qe, hs_q]
            ref["dq"], ref["dk"], ref["dv"] = O.attention_bwd(qb, kb, vb, dob, causal, scale)
            yo, yq, yk, yv = sdpa_math(qb, kb, vb, causal, scale, do=dob)
            yd = {"out": yo, "dq": yq, "dk": yk, "dv": yv}
            got["dq"], got["dk"], got["dv"] = grads[0][None, qs:qe, hs_q], grads[1][None, ks:ke, hs_k], grads[2][None, ks:ke, hs_k]
        else:
            yd = {"out": sdpa_math(qb, kb, vb, causal, scale)}
        for n in got:
            assert not torch.isnan(got[n]).any(), n
            errs[n] = max(errs[n], max_err(got[n], ref[n]))
            yards[n] = max(yards[n], max_err(yd[n], ref[n]))
    for n in names:
        _report(n, errs[n], yards[n])
        assert errs[n] <= ERR_FACTOR * yards[n] + ATOL, f"{n} err {errs[n]:.3e} > {ERR_FACTOR} x yardstick {yards[n]:.3e}"


def assert_status_ok():
    from splitd_flash_attn.interface import kernel_status

    assert kernel_status() == 0, "a kernel gave up a bounded wait"
