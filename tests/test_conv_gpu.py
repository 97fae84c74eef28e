"""Depthwise conv1d + SiLU kernels (csrc/conv_kernels.cuh, through the C ABI) against the reference expression
`silu(conv1d(x^T, w, b, padding=K//2, groups=C))^T` evaluated by PyTorch in fp32 on the same (rounded) inputs.
Tolerances: max |got - ref| / max |ref| per tensor <= 1e-5 for fp32, 2e-2 for bf16 / fp16."""
import pytest
import torch

from oracle.bissd_oracle import max_rel_err
from oracle.layer_oracle import dwconv1d_silu_reference

pytestmark = pytest.mark.gpu

CASES = [
    # name, (batch, seqlen, channels), width, dtype, weight dtype, bias
    ("module_shape_bf16", (2, 300, 2304), 7, torch.bfloat16, torch.bfloat16, True),
    ("fp32_width3", (3, 77, 64), 3, torch.float32, torch.float32, True),
    ("fp16_no_bias", (1, 130, 520), 5, torch.float16, torch.float32, False),
    ("short_sequence", (4, 3, 128), 7, torch.float32, torch.float32, True),
    # 16-bit rolling-window kernels at the edges: sequence shorter than the window, ragged last row block
    ("bf16_width3_tiny", (2, 5, 64), 3, torch.bfloat16, torch.bfloat16, True),
    ("bf16_width7_shorter_than_window", (1, 2, 128), 7, torch.bfloat16, torch.float32, True),
    ("fp16_width7_ragged_blocks", (2, 131, 264), 7, torch.float16, torch.float16, False),
]


@pytest.mark.parametrize("name,shape,K,dtype,wdtype,has_bias", CASES, ids=[c[0] for c in CASES])
def test_forward_and_backward_match_reference_expression(name, shape, K, dtype, wdtype, has_bias):
    from ssd.bi.conv_silu import _kernel_ok, dwconv1d_silu
    b, L, C = shape
    g = torch.Generator().manual_seed(sum(name.encode()))
    x = torch.randn(b, L, C, generator=g).to(dtype).cuda()
    w = (0.4 * torch.randn(C, 1, K, generator=g)).to(wdtype).cuda()
    bias = (0.2 * torch.randn(C, generator=g)).to(wdtype).cuda() if has_bias else None
    dout = torch.randn(b, L, C, generator=g).to(dtype).cuda()
    assert _kernel_ok(x, w, bias)
    leaves = [t.clone().requires_grad_(True) if t is not None else None for t in (x, w, bias)]
    out = dwconv1d_silu(*leaves)
    out.backward(dout)
    ref_leaves = [t.detach().float().cpu().requires_grad_(True) if t is not None else None for t in (x, w, bias)]
    ref = dwconv1d_silu_reference(*ref_leaves)
    ref.backward(dout.float().cpu())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert out.dtype == dtype and out.shape == x.shape and out.is_contiguous()
    assert max_rel_err(out, ref) < tol
    for got, want, nm in zip(leaves, ref_leaves, ("dx", "dw", "db")):
        if got is not None:
            assert got.grad.shape == got.shape and got.grad.dtype == got.dtype
            assert max_rel_err(got.grad, want.grad) < tol, nm


def test_strided_input_slice_is_read_in_place_and_results_repeat():
    from ssd.bi.conv_silu import dwconv1d_silu
    g = torch.Generator().manual_seed(5)
    big = torch.randn(2, 200, 1024 + 512 + 24, generator=g).bfloat16().cuda()
    x = big[..., 1024:1536]                                  # what BiMamba2 does: a channel slice of in_proj's output
    w = (0.3 * torch.randn(512, 1, 7, generator=g)).cuda()
    a, b2 = dwconv1d_silu(x, w), dwconv1d_silu(x, w)
    assert torch.equal(a, b2)
    assert max_rel_err(a, dwconv1d_silu_reference(x.float().cpu(), w.cpu())) < 2e-2


def test_arguments_outside_the_kernel_range_raise():
    """No eager or CPU path is shipped: unsupported shapes and CPU tensors are errors, not silent detours."""
    from ssd.bi.conv_silu import dwconv1d_silu
    with pytest.raises(RuntimeError, match="multiple of 8"):
        dwconv1d_silu(torch.randn(1, 16, 12, device="cuda"), torch.randn(12, 1, 3, device="cuda"))
    with pytest.raises(RuntimeError, match="odd"):
        dwconv1d_silu(torch.randn(1, 16, 16, device="cuda"), torch.randn(16, 1, 4, device="cuda"))
    with pytest.raises(RuntimeError, match="CUDA"):
        dwconv1d_silu(torch.randn(1, 16, 16), torch.randn(16, 1, 3))
