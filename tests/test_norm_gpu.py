"""Gated RMSNorm kernels (csrc/norm_kernels.cuh, through the C ABI) against the reference formula written with PyTorch
tensor ops in fp32 (`rmsnorm_ref_fn`, a restatement of rms_norm_ref, src/ssd/bi/layernorm_gated.py:18-41).
Tolerances: max |got - ref| / max |ref| per tensor <= 1e-5 for fp32, 2e-2 for bf16 / fp16 (outputs are rounded to the
16-bit type; the reference of the comparison is computed in fp32 from the same rounded inputs)."""
import pytest
import torch

from oracle.bissd_oracle import max_rel_err

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
    from ssd.bi.layernorm_gated import _kernel_ok, rmsnorm_fn, rmsnorm_ref_fn
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
    ref_leaves = [t.detach().float().requires_grad_(True) if t is not None else None for t in (x, w, z)]
    ref = rmsnorm_ref_fn(ref_leaves[0], ref_leaves[1], None, z=ref_leaves[2], eps=1e-5, group_size=group,
                         norm_before_gate=nbg)
    ref.backward(dout.float())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert out.dtype == dtype and out.shape == x.shape
    assert max_rel_err(out, ref) < tol
    for got, want, nm in zip(leaves, ref_leaves, ("dx", "dw", "dz")):
        if got is not None:
            assert got.grad.dtype == got.dtype
            assert max_rel_err(got.grad, want.grad) < (tol if nm != "dw" or dtype == torch.float32 else 2e-2), nm


def test_strided_rows_and_repeatability():
    from ssd.bi.layernorm_gated import rmsnorm_fn, rmsnorm_ref_fn
    g = torch.Generator().manual_seed(3)
    big = torch.randn(64, 3 * 1024, generator=g).bfloat16().cuda()
    x, z = big[:, :1024], big[:, 2048:]                     # row stride 3072, not contiguous
    w = torch.ones(1024, device="cuda")
    a = rmsnorm_fn(x, w, None, z=z, eps=1e-5)
    b = rmsnorm_fn(x, w, None, z=z, eps=1e-5)
    assert torch.equal(a, b)
    assert max_rel_err(a, rmsnorm_ref_fn(x.float(), w, None, z=z.float(), eps=1e-5)) < 2e-2


def test_shapes_outside_the_kernel_range_use_the_formula():
    from ssd.bi.layernorm_gated import _kernel_ok, rmsnorm_fn, rmsnorm_ref_fn
    x = torch.randn(4, 200, device="cuda")                  # hidden not a multiple of 256
    w = torch.ones(200, device="cuda")
    assert not _kernel_ok(x, w, None, None, None)
    assert torch.equal(rmsnorm_fn(x, w), rmsnorm_ref_fn(x, w))
