"""Run one shape of the attention path a few times and print CUDA-event timings per kernel.

    python gemm4-attention-kernels_b200/profile_case.py --batch 1 --seqlen 4096 [--causal] [--no-backward] [--iters 3]
    python gemm4-attention-kernels_b200/profile_case.py --packed 8192,4096,2048,1024,1024 --causal   # packed (varlen) layout
    python gemm4-attention-kernels_b200/profile_case.py --packed-random 32768 --causal              # random packing

Meant as the small, self-terminating command to put under `ncu` (one kernel, a few launches) and as a
quick timing tool. Hq=32, Hkv=4, D=512, bf16, synthetic N(0,1) inputs (the benchmark's shapes).
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from splitd_flash_attn import interface as I  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seqlen", type=int, default=4096)
    ap.add_argument("--heads-q", type=int, default=32)
    ap.add_argument("--heads-kv", type=int, default=4)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--no-backward", action="store_true")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--packed", type=str, default="", help="comma separated sequence lengths: packed (T,H,D) layout")
    ap.add_argument("--packed-random", type=int, default=0,
                    help="packed layout with lengths uniform in [128, 8192] (seed 0) until this many tokens, last one truncated")
    a = ap.parse_args()
    torch.manual_seed(0)
    D = 512
    kw = {}
    if a.packed_random:
        gen, lens = torch.Generator().manual_seed(0), []
        while sum(lens) < a.packed_random:
            lens.append(int(torch.randint(128, 8193, (1,), generator=gen)))
        lens[-1] -= sum(lens) - a.packed_random
        a.packed = ",".join(str(x) for x in lens)
        print("sequence lengths:", a.packed)
    if a.packed:
        lens = [int(x) for x in a.packed.split(",")]
        T = sum(lens)
        mk = lambda h: torch.randn(T, h, D, device="cuda").to(torch.bfloat16)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
        kw = dict(cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens))
        F = sum(4.0 * a.heads_q * s * s * D for s in lens) * (0.5 if a.causal else 1.0)
    else:
        B, S = a.batch, a.seqlen
        mk = lambda h: torch.randn(B, S, h, D, device="cuda").to(torch.bfloat16)
        F = 4.0 * B * a.heads_q * S * S * D * (0.5 if a.causal else 1.0)
    q, k, v, do = mk(a.heads_q), mk(a.heads_kv), mk(a.heads_kv), mk(a.heads_q)
    for it in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out, lse = I._flash_attn_fwd(q, k, v, causal=a.causal, return_lse=True, **kw)
        e1.record()
        evs = []
        if not a.no_backward:
            I._flash_attn_bwd(q, k, v, out, do, lse, causal=a.causal, stage_events=evs, **kw)
        torch.cuda.synchronize()
        line = f"iter {it}: fwd {e0.elapsed_time(e1):.3f} ms ({F / e0.elapsed_time(e1) / 1e9:.0f} TFLOP/s)"
        if evs:
            t = [evs[i].elapsed_time(evs[i + 1]) for i in range(3)]
            line += (f" | preprocess {t[0]:.3f} ms | P/dS tiles {t[1]:.3f} ms ({F / t[1] / 1e9:.0f}) | "
                     f"dQ+dK+dV GEMMs {t[2]:.3f} ms ({1.5 * F / t[2] / 1e9:.0f}) | bwd {2.5 * F / sum(t) / 1e9:.0f} TFLOP/s")
        print(line)
    print("status", I.kernel_status())


if __name__ == "__main__":
    main()
