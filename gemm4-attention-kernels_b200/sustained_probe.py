"""Run cuBLAS, the forward and the backward of one long shape back to back for a few seconds each and report
throughput together with the SM clock and board power sampled meanwhile (NVML, read only).

    python gemm4-attention-kernels_b200/sustained_probe.py [--seconds 3]

A kernel timed alone for a millisecond runs at a clock the board cannot hold; under a seconds-long load the
power cap sets the clock. This tool shows, per kernel, what is left at that point: TFLOP/s, the clock, the
fraction of that clock's tensor ceiling (8192 FLOP/clk/SM x 148 SMs), and TFLOP per joule, with a cuBLAS bf16
GEMM as the yardstick. B=1, S=16384, Hq=32, Hkv=4, D=512, bf16, non-causal, synthetic N(0,1) inputs.
"""
import argparse
import os
import sys
import threading
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from splitd_flash_attn import interface as I  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seconds", type=float, default=3.0)
    args = ap.parse_args()
    import pynvml

    pynvml.nvmlInit()
    handle = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
    B, S, HQ, HKV, D = 1, 16384, 32, 4, 512
    torch.manual_seed(0)
    q = torch.randn(B, S, HQ, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, S, HKV, D, device="cuda", dtype=torch.bfloat16)
    v, do = torch.randn_like(k), torch.randn_like(q)
    out, lse = I._flash_attn_fwd(q, k, v, causal=False, return_lse=True)
    a = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
    F = 4.0 * B * HQ * S * S * D

    def run(name, fn, flops):
        fn()
        torch.cuda.synchronize()
        samples, stop = [], [False]

        def sampler():
            while not stop[0]:
                samples.append((pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM),
                                pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0))
                time.sleep(0.05)

        th = threading.Thread(target=sampler)
        th.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0, n = time.time(), 0
        e0.record()
        while time.time() - t0 < args.seconds:
            for _ in range(4):
                fn()
            n += 4
            torch.cuda.synchronize()
        e1.record()
        torch.cuda.synchronize()
        stop[0] = True
        th.join()
        half = samples[len(samples) // 2:]  # the settled half
        clk = sum(s[0] for s in half) / len(half)
        watts = sum(s[1] for s in half) / len(half)
        tf = flops * n / e0.elapsed_time(e1) / 1e9
        ceiling = 8192 * 148 * clk * 1e6 / 1e12
        print(f"{name:28s} {tf:7.0f} TFLOP/s  clock {clk:6.0f} MHz  power {watts:6.0f} W  -> "
              f"{100 * tf / ceiling:5.1f} % of the clock's tensor ceiling, {tf / watts:5.2f} TFLOP/J")

    run("cuBLAS bf16 8192^3", lambda: torch.matmul(a, b), 2.0 * 8192 ** 3)
    run("forward", lambda: I._flash_attn_fwd(q, k, v, causal=False, return_lse=True), F)
    stages = []

    def bwd():
        evs = []
        I._flash_attn_bwd(q, k, v, out, do, lse, causal=False, stage_events=evs)
        stages.append(evs)

    run("backward (pre+tiles+grads)", bwd, 2.5 * F)
    torch.cuda.synchronize()
    half = stages[len(stages) // 2:]
    t = [sum(e[i].elapsed_time(e[i + 1]) for e in half) / len(half) for i in range(3)]
    print(f"  inside it: preprocess {t[0]:.3f} ms | P/dS tiles {t[1]:.3f} ms ({F / t[1] / 1e9:.0f} TFLOP/s) | "
          f"dQ+dK+dV GEMMs {t[2]:.3f} ms ({1.5 * F / t[2] / 1e9:.0f} TFLOP/s)")
    print("status", I.kernel_status())


if __name__ == "__main__":
    main()
