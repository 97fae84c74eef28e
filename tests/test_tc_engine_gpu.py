"""The tcgen05 block-GEMM engine (TMEM accumulators, swizzled shared-memory operand staging, both operand majors)
against a host GEMM, through the C ABI's self-test entry point."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("n,k", [(64, 64), (128, 256), (256, 192), (48, 72)])
def test_selftest_gemm(dtype, a_mn, b_mn, n, k):
    from ssd import _cabi
    lib = _cabi.load()
    g = torch.Generator().manual_seed(n * 1000 + k)
    A = torch.randn(128, k, generator=g).to(dtype)
    B = torch.randn(n, k, generator=g).to(dtype)
    ref = A.float() @ B.float().t()
    Ad = (A.t().contiguous() if a_mn else A).cuda()
    Bd = (B.t().contiguous() if b_mn else B).cuda()
    C = torch.zeros(128, n, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    code = _cabi.BF16 if dtype == torch.bfloat16 else _cabi.F16
    _cabi.check(lib.bissd_selftest_gemm(code, int(a_mn), int(b_mn), n, k, Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(),
                                        status.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert status.item() == 0, "a device-side wait ran out"
    err = (C.cpu() - ref).abs().max().item() / ref.abs().max().item()
    assert err < 1e-5, err
