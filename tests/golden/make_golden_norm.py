"""Generate tests/golden/rmsnorm_ref_*.npz from the REFERENCE's own `rms_norm_ref`
(src/ssd/bi/layernorm_gated.py:18-41; pure PyTorch, runs on CPU).

Run once where the reference checkout is present (see --reference); it is not needed at test time.
    python tests/golden/make_golden_norm.py [--reference /path/to/Bi-Mamba2]

Each file stores the inputs (x, z, weight, dout - values exactly representable in the case's dtype), the switches,
and the reference's forward result and autograd gradients (dx, dz, dweight), computed by the reference function on
the inputs cast to its working precision.  The cases mirror tests/test_norm_gpu.py (hidden size, group size, gate
order, dtypes) on a handful of rows so that the fixtures stay small.
"""
import argparse
import os
import sys

import numpy as np

# name: (rows shape, hidden, dtype, weight dtype, group_size, norm_before_gate, has_z)
CASES = {
    "rmsnorm_ref_module_shape_bf16": ((2, 3), 2048, "bfloat16", "float32", None, True, True),
    "rmsnorm_ref_fp32_groups": ((5, 2), 1024, "float32", "float32", 256, True, True),
    "rmsnorm_ref_gate_before_norm_fp16": ((9,), 512, "float16", "float16", None, False, True),
    "rmsnorm_ref_no_gate_bf16_weight": ((2, 2), 4096, "bfloat16", "bfloat16", 1024, True, False),
    "rmsnorm_ref_wide_fp32_gate_first": ((5,), 3072, "float32", "float32", 768, False, True),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    args = ap.parse_args()
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(args.reference, "src"))
    import torch
    from ssd.bi.layernorm_gated import rms_norm_ref
    for i, (name, (lead, hidden, dtype, wdtype, group, nbg, has_z)) in enumerate(CASES.items()):
        dt, wdt = getattr(torch, dtype), getattr(torch, wdtype)
        g = torch.Generator().manual_seed(100 + i)
        x = torch.randn(*lead, hidden, generator=g).to(dt)
        z = torch.randn(*lead, hidden, generator=g).to(dt) if has_z else None
        w = (1.0 + 0.3 * torch.randn(hidden, generator=g)).to(wdt)
        dout = torch.randn(*lead, hidden, generator=g).to(dt)
        # forward in the case's dtype exactly as a caller of the reference would get it
        out = rms_norm_ref(x, w, None, z=z, eps=1e-5, group_size=group, norm_before_gate=nbg)
        # gradients of the fp32 evaluation of the same function on the same (rounded) inputs
        leaves = [t.float().clone().requires_grad_(True) if t is not None else None for t in (x, w, z)]
        ref = rms_norm_ref(leaves[0], leaves[1], None, z=leaves[2], eps=1e-5, group_size=group, norm_before_gate=nbg)
        ref.backward(dout.float())
        arrays = dict(x=x.float().numpy(), weight=w.float().numpy(), dout=dout.float().numpy(),
                      out=out.float().numpy(), out_fp32=ref.detach().numpy(), dx=leaves[0].grad.numpy(),
                      dweight=leaves[1].grad.numpy(),
                      meta=np.array([hidden, 0 if group is None else group, int(nbg), int(has_z)]),
                      dtypes=np.array([dtype, wdtype]))
        if has_z:
            arrays["z"] = z.float().numpy()
            arrays["dz"] = leaves[2].grad.numpy()
        np.savez_compressed(os.path.join(here, name + ".npz"), **arrays)
        print("wrote", name, x.shape)


if __name__ == "__main__":
    main()
