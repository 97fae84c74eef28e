"""Time the reference's own Triton kernels (baseline/_ref, see make_ref.py) on one GPU: forward + backward of
`ssd.bi.ssd_combined.bimamba_chunk_scan_combined` at the benchmark shape (batch 8, seqlen 2048, 24 heads x 64,
dstate 128, chunk 256, bf16, z, D, dt_bias, softplus).  Prints one JSON line.  Run in its own process: the package
name `ssd` is the same as this repository's.

    python baseline/triton_reference_bench.py [--protocol free|restricted] [--steps 50] [--warmup 10] [--batch 8]

Protocols:
  free        the reference as shipped: every kernel autotunes over its full configuration list.
  restricted  `_chunk_scan_fwd_kernel` (src/ssd/bi/ssd_chunk_scan.py:24-39) may only pick the two tile shapes that
              compute the right result at chunk 256, (32, 64, 32) and (64, 128, 64); everything else as shipped.

Timing: the same way the new kernels are timed - `steps` passes back to back between two CUDA events after the
warm-up (which includes all autotuning) - plus, for reference, the median of individually timed passes.
"""
import argparse
import json
import math
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "_ref"))

VALID_SCAN_TILES = {(32, 64, 32), (64, 128, 64)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--protocol", default="free", choices=["free", "restricted"])
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--batch", type=int, default=8)
    a = ap.parse_args()
    if not os.path.isdir(os.path.join(HERE, "_ref", "ssd")):
        print(json.dumps({"impl": "triton-reference", "unavailable": "baseline/_ref not installed (run baseline/make_ref.py)"}))
        return
    import torch
    import triton
    from triton.runtime.autotuner import Autotuner
    import ssd.bi.ssd_bmm as m_bmm
    import ssd.bi.ssd_chunk_scan as m_scan
    import ssd.bi.ssd_chunk_state as m_state
    import ssd.bi.ssd_combined as m_comb
    import ssd.bi.ssd_state_passing as m_pass
    from ssd.bi.ssd_combined import bimamba_chunk_scan_combined
    if a.protocol == "restricted":
        k = m_scan._chunk_scan_fwd_kernel
        keep = [c for c in k.configs
                if (c.kwargs["BLOCK_SIZE_M"], c.kwargs["BLOCK_SIZE_N"], c.kwargs["BLOCK_SIZE_K"]) in VALID_SCAN_TILES]
        assert keep, "the reference's configuration list no longer holds the two valid tiles"
        k.configs = keep
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
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms_b2b = e0.elapsed_time(e1) / a.steps
    times = []
    for _ in range(min(a.steps, 20)):
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        step()
        s1.record()
        torch.cuda.synchronize()
        times.append(s0.elapsed_time(s1))
    times.sort()
    picks = {}
    for m in (m_comb, m_scan, m_state, m_pass, m_bmm):
        for name, k in vars(m).items():
            if isinstance(k, Autotuner) and getattr(k, "cache", None):
                picks[name] = sorted({str(c) for c in k.cache.values()})
    print(json.dumps({"impl": "triton-reference", "protocol": a.protocol, "metric": "bi-SSD fwd+bwd tokens/s",
                      "value": b * L / (ms_b2b * 1e-3), "unit": "tokens/s", "ms_per_step": ms_b2b,
                      "ms_per_step_median_single": times[len(times) // 2], "ms_min_single": times[0], "steps": a.steps,
                      "warmup": a.warmup, "batch": b, "triton": triton.__version__,
                      "autotune_picks": {"_chunk_scan_fwd_kernel": picks.get("_chunk_scan_fwd_kernel")},
                      "autotuned_kernels": len(picks),
                      "note": "one-token Triton 3.x compat fix applied to the copy (tl.flip(..., dim=1)); ddt/dA/ddt_bias of "
                              "the reference are invalid at this size (state-passing backward defect), timing is unaffected"}))


if __name__ == "__main__":
    main()
