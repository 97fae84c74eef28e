"""Pin oracle/layer_oracle.py: the gated RMSNorm restatement against golden vectors written by the reference's own
`rms_norm_ref` (tests/golden/make_golden_norm.py), forward and autograd gradients; the convolution oracle against a
direct evaluation of its defining sum."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR
from oracle.bissd_oracle import max_rel_err
from oracle.layer_oracle import dwconv1d_silu_reference, rms_norm_gated_reference

NORM_GOLDEN = ["rmsnorm_ref_module_shape_bf16", "rmsnorm_ref_fp32_groups", "rmsnorm_ref_gate_before_norm_fp16",
               "rmsnorm_ref_no_gate_bf16_weight", "rmsnorm_ref_wide_fp32_gate_first"]


def load_norm_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    hidden, group, nbg, has_z = (int(v) for v in z["meta"])
    dtype, wdtype = (getattr(torch, str(s)) for s in z["dtypes"])
    t = {k: torch.from_numpy(z[k]) for k in z.files if k not in ("meta", "dtypes")}
    return dict(t, hidden=hidden, group=(group or None), nbg=bool(nbg), has_z=bool(has_z), dtype=dtype, wdtype=wdtype)


@pytest.mark.parametrize("name", NORM_GOLDEN)
def test_norm_oracle_matches_reference_golden(name):
    g = load_norm_golden(name)
    x, w = g["x"].to(g["dtype"]), g["weight"].to(g["wdtype"])
    z = g["z"].to(g["dtype"]) if g["has_z"] else None
    out = rms_norm_gated_reference(x, w, None, z=z, eps=1e-5, group_size=g["group"], norm_before_gate=g["nbg"])
    assert out.dtype == g["dtype"]
    assert torch.equal(out.float(), g["out"])                    # same arithmetic, same rounding: bit for bit
    leaves = [t.float().clone().requires_grad_(True) if t is not None else None for t in (x, w, z)]
    ref = rms_norm_gated_reference(leaves[0], leaves[1], None, z=leaves[2], eps=1e-5, group_size=g["group"],
                                   norm_before_gate=g["nbg"])
    ref.backward(g["dout"])
    assert max_rel_err(ref, g["out_fp32"]) < 1e-6
    assert max_rel_err(leaves[0].grad, g["dx"]) < 1e-5
    assert max_rel_err(leaves[1].grad, g["dweight"]) < 1e-5
    if g["has_z"]:
        assert max_rel_err(leaves[2].grad, g["dz"]) < 1e-5


def test_conv_oracle_matches_its_defining_sum():
    g = torch.Generator().manual_seed(1)
    b, L, C, K = 2, 9, 4, 7
    x, w, bias = torch.randn(b, L, C, generator=g).double(), torch.randn(C, 1, K, generator=g).double(), torch.randn(C, generator=g).double()
    want = torch.zeros(b, L, C, dtype=torch.float64)
    for l in range(L):
        for k in range(K):
            j = l + k - K // 2
            if 0 <= j < L:
                want[:, l] += w[:, 0, k] * x[:, j]
    want = torch.nn.functional.silu(want + bias)
    assert max_rel_err(dwconv1d_silu_reference(x, w, bias), want) < 1e-12
