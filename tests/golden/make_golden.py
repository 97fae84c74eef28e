"""Generate the golden vectors under tests/golden/ from the REFERENCE implementation itself.

Run once, in a container that has the reference checkout (see --reference) - it is not needed at
test time.  Usage:  python tests/golden/make_golden.py [--reference /path/to/Bi-Mamba2]

Two sources, both the reference's own code:

1. `triton_bi_*.npz` - the reference's bidirectional Triton kernels
   (`ssd.bi.ssd_combined.bimamba_chunk_scan_combined`, src/ssd/bi/ssd_combined.py:577) forward AND backward,
   executed on CPU by Triton's interpreter (TRITON_INTERPRET=1).  To run there, a temporary copy of the
   package gets the one-token fix `tl.flip(..., dim=1)` at src/ssd/bi/ssd_chunk_state.py:91 (Triton 3.x needs
   the argument), `torch.cuda.device` / `get_device_properties` are stubbed, and every autotuner is pinned to
   one configuration that is numerically valid (forward tile (32,64,32); state-passing block >= headdim*dstate).
   The intermediates of the forward chain (dt_out, both cumsums, passed states, final states) are stored too.
2. `torchref_*.npz` - the reference's pure-PyTorch path `ssd_chunk_scan_combined_ref`
   (src/ssd/uni/ssd_combined.py:621) composed as ref(x) + flip(ref(flip x)) + D*x, then *silu(z), forward only
   (its autograd backward is NaN for dt/A/B/C at realistic decays because it masks after exp).

Inputs are stored beside the outputs so the tests need no RNG agreement.
"""
import argparse
import contextlib
import os
import shutil
import sys
import tempfile
import types

import numpy as np


def _patched_copy(ref_root):
    tmp = tempfile.mkdtemp(prefix="bissd_ref_")
    shutil.copytree(os.path.join(ref_root, "src", "ssd"), os.path.join(tmp, "ssd"))
    path = os.path.join(tmp, "ssd", "bi", "ssd_chunk_state.py")
    src = open(path).read()
    needle = "tl.flip(tl.cumsum(tl.flip(dA, dim=1), axis=1))"
    assert needle in src, "reference source changed; update the patch"
    src = src.replace(needle, "tl.flip(tl.cumsum(tl.flip(dA, dim=1), axis=1), dim=1)")
    open(path, "w").write(src)
    return tmp


def _to_np(t):
    return None if t is None else t.detach().cpu().double().numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    args = ap.parse_args()
    here = os.path.dirname(os.path.abspath(__file__))

    os.environ["TRITON_INTERPRET"] = "1"
    tmp = _patched_copy(args.reference)
    sys.path.insert(0, tmp)
    import torch
    torch.cuda.device = lambda idx: contextlib.nullcontext()
    torch.cuda.get_device_properties = lambda d: types.SimpleNamespace(multi_processor_count=148)
    from triton.runtime.autotuner import Autotuner
    import ssd.bi.ssd_combined as m0
    import ssd.bi.ssd_chunk_scan as m1
    import ssd.bi.ssd_chunk_state as m2
    import ssd.bi.ssd_state_passing as m3
    import ssd.bi.ssd_bmm as m4
    import ssd.uni.ssd_combined as u0

    for m in (m0, m1, m2, m3, m4):
        for name, k in vars(m).items():
            if isinstance(k, Autotuner):
                if name == "_chunk_scan_fwd_kernel":
                    pick = [c for c in k.configs if (c.kwargs["BLOCK_SIZE_M"], c.kwargs["BLOCK_SIZE_N"],
                                                     c.kwargs["BLOCK_SIZE_K"]) == (32, 64, 32)]
                elif name.startswith("_state_passing"):
                    pick = [max(k.configs, key=lambda c: c.kwargs["BLOCK_SIZE"])]
                else:
                    pick = [k.configs[0]]
                k.configs = pick[:1]

    def make_inputs(seed, b, L, H, P, G, N, has_D, D_hdim, has_z, has_bias, softplus):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(b, L, H, P, generator=g)
        if softplus:
            dt = 0.5 * torch.randn(b, L, H, generator=g) - 1.0
        else:
            dt = torch.rand(b, L, H, generator=g) * 0.2 + 0.01
        A = -torch.exp(torch.rand(H, generator=g) * 2.0)
        B = torch.randn(b, L, G, N, generator=g)
        C = torch.randn(b, L, G, N, generator=g)
        D = (torch.randn(H, P, generator=g) if D_hdim else torch.randn(H, generator=g)) if has_D else None
        z = torch.randn(b, L, H, P, generator=g) if has_z else None
        dt_bias = 0.5 * torch.randn(H, generator=g) if has_bias else None
        dout = torch.randn(b, L, H, P, generator=g)
        return x, dt, A, B, C, D, z, dt_bias, dout

    # name: (seed, b, L, H, P, G, N, Q, D, D_hdim, z, bias, softplus, dt_limit)
    triton_cases = {
        "triton_bi_plain": (1, 2, 64, 4, 4, 4, 4, 32, False, False, False, True, True, (0.0, float("inf"))),
        "triton_bi_full": (2, 1, 96, 4, 8, 2, 8, 32, True, True, True, True, True, (0.0, float("inf"))),
        "triton_bi_ragged_limit": (3, 1, 80, 2, 8, 1, 8, 32, True, False, False, False, False, (0.03, 0.15)),
    }
    for name, (seed, b, L, H, P, G, N, Q, has_D, D_hdim, has_z, has_bias, softplus, dt_limit) in triton_cases.items():
        x, dt, A, B, C, D, z, dt_bias, dout = make_inputs(seed, b, L, H, P, G, N, has_D, D_hdim, has_z, has_bias, softplus)
        leaves = [t if t is None else t.clone().requires_grad_(True) for t in (x, dt, A, B, C, D, z, dt_bias)]
        lx, ldt, lA, lB, lC, lD, lz, lbias = leaves
        out = m0.bimamba_chunk_scan_combined(lx, ldt, lA, lB, lC, Q, D=lD, z=lz, dt_bias=lbias,
                                             dt_softplus=softplus, dt_limit=dt_limit)
        out.backward(dout)
        with torch.no_grad():
            fwd = m0._mamba_chunk_scan_combined_fwd(x, dt, A, B, C, Q, D=D, z=z, dt_bias=dt_bias,
                                                    dt_softplus=softplus, dt_limit=dt_limit)
        _, out_x, dt_out, cs_f, cs_b, st_f, st_b, fin_f, fin_b = fwd
        arrays = dict(
            meta=np.array([b, L, H, P, G, N, Q, int(softplus)]), dt_limit=np.array(dt_limit),
            x=_to_np(x), dt=_to_np(dt), A=_to_np(A), B=_to_np(B), C=_to_np(C), dout=_to_np(dout),
            out=_to_np(out), dt_out=_to_np(dt_out), cs_f=_to_np(cs_f), cs_b=_to_np(cs_b),
            states_f=_to_np(st_f), states_b=_to_np(st_b), final_f=_to_np(fin_f), final_b=_to_np(fin_b),
            dx=_to_np(lx.grad), ddt=_to_np(ldt.grad), dA=_to_np(lA.grad), dB=_to_np(lB.grad), dC=_to_np(lC.grad),
        )
        for key, val in dict(D=D, z=z, dt_bias=dt_bias, out_x=out_x, dD=None if lD is None else lD.grad,
                             dz=None if lz is None else lz.grad,
                             ddt_bias=None if lbias is None else lbias.grad).items():
            if val is not None:
                arrays[key] = _to_np(val)
        arrays = {k: (v.astype(np.float32) if v.dtype == np.float64 and k not in ("dt_limit",) else v)
                  for k, v in arrays.items()}
        np.savez_compressed(os.path.join(here, name + ".npz"), **arrays)
        print("wrote", name, {k: v.shape for k, v in arrays.items() if k in ("x", "out", "dA")})

    torch_cases = {
        "torchref_small": (11, 2, 128, 4, 8, 2, 16, 32, True, False, True, True, True),
        "torchref_hdimD": (12, 1, 192, 2, 16, 1, 8, 64, True, True, False, False, False),
    }
    for name, (seed, b, L, H, P, G, N, Q, has_D, D_hdim, has_z, has_bias, softplus) in torch_cases.items():
        x, dt, A, B, C, D, z, dt_bias, dout = make_inputs(seed, b, L, H, P, G, N, has_D, D_hdim, has_z, has_bias, softplus)
        with torch.no_grad():
            yf = u0.ssd_chunk_scan_combined_ref(x, dt, A, B, C, Q, D=None, z=None, dt_bias=dt_bias, dt_softplus=softplus)
            yb = u0.ssd_chunk_scan_combined_ref(x.flip(1), dt.flip(1), A, B.flip(1), C.flip(1), Q, D=None, z=None,
                                                dt_bias=dt_bias, dt_softplus=softplus).flip(1)
            y = yf + yb
            if D is not None:
                y = y + x * (D[None, None, :, None] if D.dim() == 1 else D[None, None])
            out = y if z is None else y * torch.nn.functional.silu(z)
        arrays = dict(meta=np.array([b, L, H, P, G, N, Q, int(softplus)]), dt_limit=np.array((0.0, float("inf"))),
                      x=_to_np(x), dt=_to_np(dt), A=_to_np(A), B=_to_np(B), C=_to_np(C), out=_to_np(out))
        for key, val in dict(D=D, z=z, dt_bias=dt_bias).items():
            if val is not None:
                arrays[key] = _to_np(val)
        arrays = {k: (v.astype(np.float32) if v.dtype == np.float64 and k != "dt_limit" else v) for k, v in arrays.items()}
        np.savez_compressed(os.path.join(here, name + ".npz"), **arrays)
        print("wrote", name)
    shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    main()
