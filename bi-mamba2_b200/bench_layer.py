"""Time one BiMamba2 layer (forward + backward) and list the library's kernels with their mean launch times.

    python bi-mamba2_b200/bench_layer.py [--batch 16] [--seqlen 4096] [--d-model 1024] [--d-state 64] [--steps 5]

Synthetic input, random-init weights, bf16.  The per-kernel figures come from the library's own CUDA-event brackets
(bissd_trace_enable / bissd_trace_read); the layer time is measured without them.  Prints one JSON line.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from ssd import _cabi  # noqa: E402
from ssd.modules import BiMamba2  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seqlen", type=int, default=4096)
    ap.add_argument("--d-model", type=int, default=1024)
    ap.add_argument("--d-state", type=int, default=64)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    torch.manual_seed(0)
    layer = BiMamba2(d_model=a.d_model, d_state=a.d_state, d_conv=7, expand=2, headdim=64, chunk_size=256).cuda().bfloat16()
    u = torch.randn(a.batch, a.seqlen, a.d_model, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn_like(u)
    for _ in range(a.warmup):
        layer(u).backward(g)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        layer(u).backward(g)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    _cabi.trace_enable(True)
    for _ in range(a.steps):
        layer(u).backward(g)
    torch.cuda.synchronize()
    tr = _cabi.trace_read()
    _cabi.trace_enable(False)
    kernels = {k: {"us_per_step": v[0] / a.steps * 1000.0, "launches_per_step": v[1] / a.steps}
               for k, v in sorted(tr.items(), key=lambda kv: -kv[1][0])}
    print(json.dumps({"metric": "BiMamba2 layer fwd+bwd", "ms_per_step": ms,
                      "tokens_per_s": a.batch * a.seqlen / ms * 1e3, "dtype": "bf16", "data": "synthetic",
                      "config": {"batch": a.batch, "seqlen": a.seqlen, "d_model": a.d_model, "d_state": a.d_state,
                                 "d_conv": 7, "headdim": 64, "chunk_size": 256},
                      "library_kernels_us_per_step": sum(k["us_per_step"] for k in kernels.values()),
                      "kernels": kernels}))


if __name__ == "__main__":
    main()
