"""Child process of tests/test_scan_gpu.py::test_first_call_inside_a_graph_capture.

The very first forward + backward of the process runs inside a CUDA graph capture: the library must not create its
second stream there and keeps every launch on the capturing stream.  The replayed graph is then compared, bit for bit,
with an eager step of the same process, which does use the second stream in its backward pass.  Prints
`CAPTURE_FIRST_CALL bit-equal` or `CAPTURE_FIRST_CALL MISMATCH`."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "bi-mamba2_b200"))
from ssd.bi.ssd_combined import bimamba_chunk_scan_combined  # noqa: E402


def main():
    torch.manual_seed(0)
    b, L, H, P, G, N, Q = 2, 512, 8, 64, 1, 128, 256
    dev = "cuda"
    mk = lambda *s: torch.randn(*s, device=dev)
    x = mk(b, L, H, P).bfloat16().requires_grad_(True)
    z = mk(b, L, H, P).bfloat16().requires_grad_(True)
    B = mk(b, L, G, N).bfloat16().requires_grad_(True)
    C = mk(b, L, G, N).bfloat16().requires_grad_(True)
    dt = (mk(b, L, H) - 4).requires_grad_(True)
    A = (-torch.exp(torch.rand(H, device=dev) * 2)).requires_grad_(True)
    D = mk(H).requires_grad_(True)
    bias = (-torch.rand(H, device=dev)).requires_grad_(True)
    dout = mk(b, L, H, P).bfloat16()
    leaves = (x, z, B, C, dt, A, D, bias)

    def step():
        for t in leaves:
            t.grad = None
        out = bimamba_chunk_scan_combined(x, dt, A, B, C, Q, D=D, z=z, dt_bias=bias, dt_softplus=True)
        out.backward(dout)
        return out

    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            out_captured = step()
    graph.replay()
    torch.cuda.synchronize()
    want = [t.grad.clone() for t in leaves]
    out_want = out_captured.clone()
    out_eager = step()
    torch.cuda.synchronize()
    same = torch.equal(out_eager, out_want) and all(torch.equal(t.grad, w) for t, w in zip(leaves, want))
    print("CAPTURE_FIRST_CALL", "bit-equal" if same else "MISMATCH")


if __name__ == "__main__":
    main()
