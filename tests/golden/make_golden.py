"""Generate golden vectors from the REFERENCE's own pure-PyTorch attention.

Run in a container where the reference checkout is importable:

    python tests/golden/make_golden.py <path to the reference checkout>

It imports ``attention_ref`` (fp32 attention with autograd) and ``attention_ref_pt`` (16-bit yardstick)
from the reference's test module splitd-flash-attn/tests/test_flash_fwd_splitd_sdpa.py:132-185, runs
them on seeded inputs and stores inputs as seeds only + outputs as fp16-compressed-free fp32 arrays.
The fixtures are small (head_dim is fixed at 512 by the path, so sequence lengths are kept short).

Cases
  cfg1      : the CPU plumbing configuration -- B=1, S=256, Hq=8, Hkv=1, fp32 N(0,1) inputs, seed 0, non-causal
  gqa_causal: B=2, Sq=113, Sk=203, Hq=4, Hkv=2, causal (bottom-right aligned), seed 42
  mha_tail  : B=1, Sq=64,  Sk=128, Hq=2, Hkv=2, causal, seed 7
  cfg1_bf16, gqa_causal_bf16: the same two cases with q, k, v and dO rounded to bfloat16 first (still computed in
              fp32 by the reference): the inputs a 16-bit kernel can be given exactly, so its outputs can be
              compared with these vectors under the 2 x yardstick rule
Outputs: out, lse (logsumexp of masked scaled scores, test :562-571), dq, dk, dv from autograd.
Only a strided subsample of each output is stored to keep the files a few hundred KB.
"""

import os
import sys

import numpy as np
import torch

CASES = {
    "cfg1": dict(B=1, sq=256, sk=256, hq=8, hkv=1, causal=False, seed=0),
    "gqa_causal": dict(B=2, sq=113, sk=203, hq=4, hkv=2, causal=True, seed=42),
    "mha_tail": dict(B=1, sq=64, sk=128, hq=2, hkv=2, causal=True, seed=7),
    "cfg1_bf16": dict(B=1, sq=256, sk=256, hq=8, hkv=1, causal=False, seed=0, bf16_inputs=True),
    "gqa_causal_bf16": dict(B=2, sq=113, sk=203, hq=4, hkv=2, causal=True, seed=42, bf16_inputs=True),
}
D = 512


def make_inputs(c):
    gen = torch.Generator().manual_seed(c["seed"])
    q = torch.randn(c["B"], c["sq"], c["hq"], D, generator=gen)
    k = torch.randn(c["B"], c["sk"], c["hkv"], D, generator=gen)
    v = torch.randn(c["B"], c["sk"], c["hkv"], D, generator=gen)
    do = torch.randn(c["B"], c["sq"], c["hq"], D, generator=gen)
    if c.get("bf16_inputs"):
        q, k, v, do = (t.to(torch.bfloat16).float() for t in (q, k, v, do))
    return q, k, v, do


def subsample(t):
    """Every 16th element along D, all rows: keeps enough signal to catch any indexing error."""
    return t[..., ::16].contiguous().numpy().astype(np.float32)


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "splitd-flash-attn"))
    from tests.test_flash_fwd_splitd_sdpa import attention_ref  # the reference's own oracle

    here = os.path.dirname(os.path.abspath(__file__))
    for name, c in CASES.items():
        q, k, v, do = make_inputs(c)
        q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        scale = D ** -0.5
        out = attention_ref(q, k, v, causal=c["causal"], softmax_scale=scale)
        dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
        # LSE exactly as the reference's test computes it (:562-571)
        qt = q.detach().transpose(1, 2)
        kt = k.detach().transpose(1, 2).repeat_interleave(c["hq"] // c["hkv"], dim=1)
        scores = torch.matmul(qt * scale, kt.transpose(-2, -1))
        if c["causal"]:
            mask = torch.triu(torch.ones(c["sq"], c["sk"], dtype=torch.bool), diagonal=c["sk"] - c["sq"] + 1)
            scores.masked_fill_(mask, float("-inf"))
        lse = torch.logsumexp(scores, dim=-1)
        np.savez_compressed(
            os.path.join(here, f"{name}.npz"),
            out=subsample(out.detach()),
            lse=lse.numpy().astype(np.float32),
            dq=subsample(dq),
            dk=subsample(dk),
            dv=subsample(dv),
            meta=np.array([c["B"], c["sq"], c["sk"], c["hq"], c["hkv"], int(c["causal"]), c["seed"],
                           int(c.get("bf16_inputs", False))], dtype=np.int64),
        )
        print(name, "written")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
