"""Gated RMSNorm kernels (csrc/norm_kernels.cuh, through the C ABI) against (a) golden vectors written by the
reference's own rms_norm_ref (src/ssd/bi/layernorm_gated.py:18-41; tests/golden/make_golden_norm.py) and (b) the CPU
oracle `rms_norm_gated_reference` (pinned to the same vectors by tests/test_layer_oracle.py) on larger seeded inputs.
Tolerances: max |got - ref| / max |ref| per tensor <= 1e-5 for fp32, 2e-2 for bf16 / fp16 (outputs are rounded to the
16-bit type; the reference of the comparison is computed in fp32 from the same rounded inputs)."""
import pytest
import torch

from oracle.bissd_oracle import max_rel_err
from oracle.layer_oracle import rms_norm_gated_reference
from test_layer_oracle import NORM_GOLDEN, load_norm_golden

pytestmark = pytest.mark.gpu

CASES = [
    # name, (rows shape, hidden), dtype, weight dtype, group, norm_before_gate, has_z
    ("module_shape_bf16", ((2, 300), 2048), torch.bfloat16, torch.float32, None, True, True),
    ("fp32_groups", ((5, 7), 1024), torch.float32, torch.float32, 256, True, True),
    ("gate_before_norm_fp16", ((33,), 512), torch.float16, torch.float16, None, False, True),
    ("no_gate_bf16_weight", ((4, 65), 4096), torch.bfloat16, torch.bfloat16, 1024, True, False),
    ("wide_fp32_gate_first", ((19,), 3072), torch.float32, torch.float32, 768, False, True),
]


@pytest.mark.parametrize("name,shape,dtype,wdtype,group,nbg,has_z", CASES, ids=[c[0] for c in CASES])
def test_forward_and_backward_match_formula(name, shape, dtype, wdtype, group, nbg, has_z):
    from ssd.bi.layernorm_gated import _kernel_ok, rmsnorm_fn
    lead, hidden = shape
    g = torch.Generator().manual_seed(sum(name.encode()))
    x = torch.randn(*lead, hidden, generator=g).to(dtype).cuda()
    z = torch.randn(*lead, hidden, generator=g).to(dtype).cuda() if has_z else None
    w = (1.0 + 0.3 * torch.randn(hidden, generator=g)).to(wdtype).cuda()
    dout = torch.randn(*lead, hidden, generator=g).to(dtype).cuda()
    assert _kernel_ok(x, w, None, z, group)
    leaves = [t.clone().requires_grad_(True) if t is not None else None for t in (x, w, z)]
    out = rmsnorm_fn(leaves[0], leaves[1], None, z=leaves[2], eps=1e-5, group_size=group, norm_before_gate=nbg)
    out.backward(dout)
    ref_leaves = [t.detach().float().cpu().requires_grad_(True) if t is not None else None for t in (x, w, z)]
    ref = rms_norm_gated_reference(ref_leaves[0], ref_leaves[1], None, z=ref_leaves[2], eps=1e-5, group_size=group,
                                   norm_before_gate=nbg)
    ref.backward(dout.float().cpu())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert out.dtype == dtype and out.shape == x.shape
    assert max_rel_err(out, ref) < tol
    for got, want, nm in zip(leaves, ref_leaves, ("dx", "dw", "dz")):
        if got is not None:
            assert got.grad.dtype == got.dtype
            assert max_rel_err(got.grad, want.grad) < (tol if nm != "dw" or dtype == torch.float32 else 2e-2), nm


@pytest.mark.parametrize("name", NORM_GOLDEN)
def test_kernels_match_reference_golden(name):
    """The CUDA kernels on the golden inputs against what the reference function itself returned."""
    from ssd.bi.layernorm_gated import rmsnorm_fn
    g = load_norm_golden(name)
    x = g["x"].to(g["dtype"]).cuda().requires_grad_(True)
    w = g["weight"].to(g["wdtype"]).cuda().requires_grad_(True)
    z = g["z"].to(g["dtype"]).cuda().requires_grad_(True) if g["has_z"] else None
    out = rmsnorm_fn(x, w, None, z=z, eps=1e-5, group_size=g["group"], norm_before_gate=g["nbg"])
    out.backward(g["dout"].to(g["dtype"]).cuda())
    tol = 1e-5 if g["dtype"] == torch.float32 else 2e-2
    assert max_rel_err(out, g["out"]) < tol
    assert max_rel_err(x.grad, g["dx"]) < tol
    assert max_rel_err(w.grad, g["dweight"]) < tol
    if g["has_z"]:
        assert max_rel_err(z.grad, g["dz"]) < tol


def test_strided_rows_and_repeatability():
    from ssd.bi.layernorm_gated import rmsnorm_fn
    g = torch.Generator().manual_seed(3)
    big = torch.randn(64, 3 * 1024, generator=g).bfloat16().cuda()
    x, z = big[:, :1024], big[:, 2048:]                     # row stride 3072, not contiguous
    w = torch.ones(1024, device="cuda")
    a = rmsnorm_fn(x, w, None, z=z, eps=1e-5)
    b = rmsnorm_fn(x, w, None, z=z, eps=1e-5)
    assert torch.equal(a, b)
    assert max_rel_err(a, rms_norm_gated_reference(x.float().cpu(), w.cpu(), None, z=z.float().cpu(), eps=1e-5)) < 2e-2


def test_arguments_outside_the_kernel_range_raise():
    """No eager or CPU path is shipped: unsupported shapes and CPU tensors are errors, not silent detours."""
    from ssd.bi.layernorm_gated import RMSNorm, rmsnorm_fn
    with pytest.raises(RuntimeError, match="multiple of 256"):
        rmsnorm_fn(torch.randn(4, 200, device="cuda"), torch.ones(200, device="cuda"))
    with pytest.raises(RuntimeError, match="CUDA"):
        rmsnorm_fn(torch.randn(4, 256), torch.ones(256))
    with pytest.raises(RuntimeError, match="group size"):
        RMSNorm(512, group_size=128, device="cuda")(torch.randn(2, 512, device="cuda"))
