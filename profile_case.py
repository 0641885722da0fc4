"""Run one kernel of the quantization path on a small seeded case, a few launches, for profilers.

    python profile_case.py hessian --C 2048 --G 4 --tokens 8192 --dtype bf16
    python profile_case.py fwht --rows 65536 --n 12288 --dtype bf16
    python profile_case.py chol --C 2048 --G 4
    python profile_case.py fasterquant --R 4096 --C 2048 --G 4

The inputs exceed the 126 MB L2 but stay within a few GB, so that a multi-pass profiler capture
finishes by itself in a minute or two.  Prints the mean device time per call measured with CUDA
events.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _time(fn, reps):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["hessian", "fwht", "chol", "fasterquant"])
    ap.add_argument("--C", type=int, default=2048)
    ap.add_argument("--R", type=int, default=4096)
    ap.add_argument("--G", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32", "f16"])
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--variant", type=int, default=0)
    a = ap.parse_args()
    from gptq_plus_mp_quant_b200 import ops
    from gptq_plus_mp_quant_b200.gptq_utils import fasterquant_impl as fi
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    dt = {"bf16": torch.bfloat16, "f32": torch.float32, "f16": torch.float16}[a.dtype]
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    if a.case == "hessian":
        x = (torch.randn(a.tokens, a.C, generator=g, device=dev) * torch.exp(torch.randn(a.C, generator=g, device=dev))).to(dt)
        s = torch.exp(3 * torch.randn(a.tokens, a.G, generator=g, device=dev)).clamp(max=1000.0)
        H = torch.zeros(a.G, a.C, a.C, device=dev)
        act = torch.zeros(a.C, device=dev)
        ms = _time(lambda: ops.hessian_accum(x, s, H, act, variant=a.variant), a.reps)
        fl = 2.0 * a.tokens * a.C * a.C * a.G
        print(f"hessian C={a.C} G={a.G} tokens={a.tokens} {a.dtype}: {ms:.3f} ms per call, {fl / ms / 1e9:.1f} algorithmic TFLOP/s")
    elif a.case == "fwht":
        x = torch.randn(a.rows, a.n, generator=g, device=dev).to(dt)
        hadK, K = hu.get_hadK(a.n)
        ms = _time(lambda: hu.matmul_hadU_cuda(x, hadK, K), a.reps)
        by = 2.0 * x.numel() * x.element_size()
        print(f"fwht rows={a.rows} n={a.n} K={K} {a.dtype}: {ms:.3f} ms per call, {by / ms / 1e6:.1f} GB/s")
    elif a.case == "chol":
        x = torch.randn(4 * a.C, a.C, generator=g, device=dev) * torch.exp(torch.randn(a.C, generator=g, device=dev))
        H = (x.t() @ x / x.shape[0]).unsqueeze(0).repeat(a.G, 1, 1).contiguous()
        from gptq_plus_mp_quant_b200 import _lib
        fi.hinv_with_fallback(H, None, 0.01, True)
        _lib.profile_enable(True)
        ms = _time(lambda: fi.hinv_with_fallback(H, None, 0.01, True), a.reps)
        parts = {name: _lib.profile_read(tag)[0] / (a.reps + 1) for name, tag in
                 (("diag", 7), ("panel", 8), ("trailing", 9), ("inverse", 10))}
        _lib.profile_enable(False)
        print(f"chol C={a.C} G={a.G}: {ms:.3f} ms per call, {(2.0 / 3.0) * a.C ** 3 * a.G / ms / 1e9:.2f} TFLOP/s (2/3 C^3 per group); "
              + ", ".join(f"{k} {v:.2f} ms" for k, v in parts.items()))
    else:
        from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
        from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
        x = (torch.randn(a.tokens, a.C, generator=g, device=dev) * torch.exp(torch.randn(a.C, generator=g, device=dev))).to(dt)
        s = torch.exp(3 * torch.randn(1, a.tokens, a.G, generator=g, device=dev)).clamp(max=1000.0)
        W = torch.randn(a.R, a.C, generator=g, device=dev) * 0.02
        grad = torch.randn(a.R, a.C, generator=g, device=dev) * 1e-4
        lin = torch.nn.Linear(a.C, a.R, bias=False, device=dev)

        def run():
            lin.weight.data.copy_(W)
            o = GPTQPlus(lin, s, grad, a.G, 0.25, 0.7)
            o.quantizer = WeightQuantizer()
            o.quantizer.configure(4, perchannel=True, sym=True)
            o.add_batch(x.unsqueeze(0), None)
            o.finalize_hessian()
            o.fasterquant(groupsize=128, actorder=True, static_groups=True)

        ms = _time(run, a.reps)
        print(f"fasterquant R={a.R} C={a.C} G={a.G} (incl. Hessian of {a.tokens} tokens): {ms:.3f} ms per call")


if __name__ == "__main__":
    main()
