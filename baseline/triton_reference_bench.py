"""Time the reference's own Triton kernels (baseline/_ref, see make_ref.py) on one GPU: forward + backward of
`ssd.bi.ssd_combined.bimamba_chunk_scan_combined` at the benchmark shape (batch 8, seqlen 2048, 24 heads x 64,
dstate 128, chunk 256, bf16, z, D, dt_bias, softplus).  Prints one JSON line.  Run in its own process: the package
name `ssd` is the same as this repository's.

    python baseline/triton_reference_bench.py [--steps 50] [--warmup 10] [--batch 8]
"""
import argparse
import json
import math
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "_ref"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--batch", type=int, default=8)
    a = ap.parse_args()
    if not os.path.isdir(os.path.join(HERE, "_ref", "ssd")):
        print(json.dumps({"impl": "triton-reference", "unavailable": "baseline/_ref not installed (run baseline/make_ref.py)"}))
        return
    import torch
    from ssd.bi.ssd_combined import bimamba_chunk_scan_combined
    b, L, H, P, G, N, Q = a.batch, 2048, 24, 64, 1, 128, 256
    g = torch.Generator().manual_seed(0)
    bf, dev = torch.bfloat16, "cuda"
    x = torch.randn(b, L, H, P, generator=g).to(bf).to(dev).requires_grad_(True)
    dt = (torch.randn(b, L, H, generator=g) - 4.0).to(dev).requires_grad_(True)
    A = (-torch.exp(torch.rand(H, generator=g) * math.log(16.0))).to(dev).requires_grad_(True)
    B = torch.randn(b, L, G, N, generator=g).to(bf).to(dev).requires_grad_(True)
    C = torch.randn(b, L, G, N, generator=g).to(bf).to(dev).requires_grad_(True)
    D = torch.randn(H, generator=g).to(dev).requires_grad_(True)
    z = torch.randn(b, L, H, P, generator=g).to(bf).to(dev).requires_grad_(True)
    bias = (-torch.rand(H, generator=g)).to(dev).requires_grad_(True)
    dout = torch.randn(b, L, H, P, generator=g).to(bf).to(dev)
    leaves = (x, dt, A, B, C, D, z, bias)

    def step():
        for t in leaves:
            t.grad = None
        out = bimamba_chunk_scan_combined(x, dt, A, B, C, Q, D=D, z=z, dt_bias=bias, dt_softplus=True)
        out.backward(dout)

    for _ in range(a.warmup):        # includes Triton autotuning of every kernel
        step()
    torch.cuda.synchronize()
    times = []
    for _ in range(a.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    med = times[len(times) // 2]
    import triton
    print(json.dumps({"impl": "triton-reference", "metric": "bi-SSD fwd+bwd tokens/s", "value": b * L / (med * 1e-3),
                      "unit": "tokens/s", "ms_per_step_median": med, "ms_min": times[0], "steps": a.steps,
                      "triton": triton.__version__, "note": "free autotune as shipped; ddt/dA/ddt_bias of the reference "
                      "are invalid at this size (state-passing backward defect) but timing is unaffected"}))


if __name__ == "__main__":
    main()
