"""The BiMamba2 layer (the operator's caller in the reference, src/ssd/modules.py:17-187): same parameters and
state_dict keys, forward + backward against a restatement of the layer on the CPU built on the oracle's scan (its
O(L^2) definition in fp64 for the small layer, its chunked evaluator in fp32 at config #4's sequence length and
width) and on oracle/layer_oracle.py for the convolution and the gated RMSNorm.  The layers are sized so that the
CUDA norm and convolution kernels run (d_inner a multiple of 256); tolerances are layer-level (several GEMMs in
16-bit around the scan): 2e-3 fp32, 5e-2 bf16."""
import pytest
import torch
import torch.nn.functional as F

from oracle.bissd_oracle import chunked_reference, dense_reference, max_rel_err
from oracle.layer_oracle import dwconv1d_silu_reference, rms_norm_gated_reference

pytestmark = pytest.mark.gpu


def _dense_layer(m, u, d=torch.float64, chunked=False):
    """Restatement of BiMamba2.forward with the module's own parameters (src/ssd/modules.py:118-187) in dtype d."""
    W = {k: v.detach().to("cpu", d).requires_grad_(True) for k, v in m.named_parameters()}
    zxbcdt = u @ W["in_proj.weight"].t()
    A = -torch.exp(W["A_log"])
    z, xBC, dt = torch.split(zxbcdt, [m.d_inner, m.d_inner + 2 * m.ngroups * m.d_state, m.nheads], dim=-1)
    dt = F.softplus(dt + W["dt_bias"])
    xBC = dwconv1d_silu_reference(xBC, W["conv1d.weight"], W["conv1d.bias"])
    x, B, C = torch.split(xBC, [m.d_inner, m.ngroups * m.d_state, m.ngroups * m.d_state], dim=-1)
    b, L = u.shape[:2]
    args = (x.reshape(b, L, m.nheads, m.headdim), dt, A, B.reshape(b, L, m.ngroups, m.d_state),
            C.reshape(b, L, m.ngroups, m.d_state))
    if chunked:
        y = chunked_reference(*args, m.chunk_size, D=W["D"], compute_dtype=d)
    else:
        y = dense_reference(*args, D=W["D"], compute_dtype=d)
    y = rms_norm_gated_reference(y.reshape(b, L, m.d_inner), W["norm.weight"], None, z=z, eps=1e-5)
    return y @ W["out_proj.weight"].t(), W


def test_state_dict_keys_match_reference_layer():
    from ssd.modules import BiMamba2
    m = BiMamba2(64, d_state=16, headdim=16, chunk_size=32)
    assert set(m.state_dict().keys()) == {"dt_bias", "A_log", "D", "in_proj.weight", "conv1d.weight", "conv1d.bias",
                                          "fc_D.weight", "norm.weight", "out_proj.weight"}


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-3), (torch.bfloat16, 5e-2)])
def test_layer_forward_backward_against_dense_restatement(dtype, tol):
    from ssd.modules import BiMamba2
    torch.manual_seed(0)
    m = BiMamba2(128, d_state=64, headdim=64, chunk_size=128, d_conv=7)     # d_inner 256: the CUDA norm's range
    with torch.no_grad():
        m.A_log.uniform_(0.0, 2.0)
        m.D.normal_()
    u = torch.randn(2, 256, 128, dtype=torch.float64)
    gout = torch.randn(2, 256, 128, dtype=torch.float64)
    ref_u = u.clone().requires_grad_(True)
    ref_out, W = _dense_layer(m, ref_u)
    ref_out.backward(gout)
    mg = BiMamba2(128, d_state=64, headdim=64, chunk_size=128, d_conv=7).to("cuda", dtype)
    mg.load_state_dict({k: v.to(dtype) for k, v in m.state_dict().items()})
    ug = u.to("cuda", dtype).requires_grad_(True)
    from ssd import _cabi
    _cabi.trace_enable(True)
    out = mg(ug)
    out.backward(gout.to("cuda", dtype))
    torch.cuda.synchronize()
    ran = set(_cabi.trace_read())
    _cabi.trace_enable(False)
    assert {"rmsnorm_gated_fwd", "rmsnorm_gated_bwd"} <= ran and any(k.startswith("dwconv") for k in ran), ran
    assert max_rel_err(out, ref_out) < tol
    assert max_rel_err(ug.grad, ref_u.grad) < tol
    for k, p in mg.named_parameters():
        if k == "fc_D.weight":            # defined but unused, as in the reference: receives no gradient
            assert p.grad is None
            continue
        assert max_rel_err(p.grad, W[k].grad) < tol, k


def test_config4_layer_slab_against_chunked_restatement():
    """Config #4's layer at its true width and sequence length, one batch row: d_model 1024, d_state 64, d_conv 7,
    expand 2, headdim 64 (32 heads), chunk 256, bf16 module and input of shape (1, 4096, 1024).  The restatement runs
    in fp32 on the CPU from the same bf16-rounded parameters and input."""
    from ssd.modules import BiMamba2
    torch.manual_seed(4)
    dtype = torch.bfloat16
    mg = BiMamba2(1024, d_state=64, d_conv=7, expand=2, headdim=64, ngroups=1, chunk_size=256).to("cuda", dtype)
    with torch.no_grad():
        mg.A_log.uniform_(0.0, 2.0)
        mg.D.normal_()
    u = torch.randn(1, 4096, 1024).to(dtype)
    gout = torch.randn(1, 4096, 1024).to(dtype)
    ref_u = u.float().requires_grad_(True)
    ref_out, W = _dense_layer(mg, ref_u, d=torch.float32, chunked=True)
    ref_out.backward(gout.float())
    ug = u.cuda().requires_grad_(True)
    out = mg(ug)
    out.backward(gout.cuda())
    tol = 5e-2
    assert max_rel_err(out, ref_out) < tol
    assert max_rel_err(ug.grad, ref_u.grad) < tol
    for k, p in mg.named_parameters():
        if k == "fc_D.weight":
            continue
        assert max_rel_err(p.grad, W[k].grad) < tol, k


# ---- the fused, memory-efficient path (the reference's commented-out use_mem_eff_path, src/ssd/modules.py:129-150) ----

def _pair(dtype, d_model=128, **kw):
    """Two layers with the same parameters: the step-by-step path and the single-node path."""
    from ssd.modules import BiMamba2
    torch.manual_seed(1)
    a = BiMamba2(d_model, use_mem_eff_path=False, **kw).to("cuda", dtype)
    with torch.no_grad():
        a.A_log.uniform_(0.0, 2.0)
        a.D.normal_()
    b = BiMamba2(d_model, use_mem_eff_path=True, **kw).to("cuda", dtype)
    b.load_state_dict(a.state_dict())
    return a, b


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mem_eff_path_equals_step_by_step_path(dtype):
    """Same kernels in the same order: the outputs are bit-equal and so are the gradients the library computes; the
    output projection's weight gradient comes from a differently shaped GEMM and is held to a rounding tolerance."""
    a, b = _pair(dtype, d_state=64, headdim=64, chunk_size=128, d_conv=7)
    u = torch.randn(2, 384, 128, device="cuda", dtype=dtype)
    gout = torch.randn_like(u)
    ua, ub = u.clone().requires_grad_(True), u.clone().requires_grad_(True)
    oa, ob = a(ua), b(ub)
    assert torch.equal(oa, ob)
    oa.backward(gout)
    ob.backward(gout)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert max_rel_err(ub.grad, ua.grad) <= tol
    for (k, pa), (_, pb) in zip(a.named_parameters(), b.named_parameters()):
        if k == "fc_D.weight":
            assert pb.grad is None
            continue
        assert pb.grad is not None and pb.grad.shape == pa.grad.shape, k
        assert max_rel_err(pb.grad, pa.grad) <= tol, k
    for k in ("conv1d.weight", "conv1d.bias", "A_log", "D", "dt_bias", "norm.weight"):   # straight from the library
        assert torch.equal(dict(b.named_parameters())[k].grad, dict(a.named_parameters())[k].grad), k


def test_mem_eff_path_against_dense_restatement():
    from ssd.modules import BiMamba2
    torch.manual_seed(0)
    m = BiMamba2(128, d_state=64, headdim=64, chunk_size=128, d_conv=7)
    with torch.no_grad():
        m.A_log.uniform_(0.0, 2.0)
        m.D.normal_()
    u = torch.randn(2, 256, 128, dtype=torch.float64)
    gout = torch.randn(2, 256, 128, dtype=torch.float64)
    ref_u = u.clone().requires_grad_(True)
    ref_out, W = _dense_layer(m, ref_u)
    ref_out.backward(gout)
    mg = BiMamba2(128, d_state=64, headdim=64, chunk_size=128, d_conv=7, use_mem_eff_path=True).to("cuda", torch.float32)
    mg.load_state_dict(m.state_dict())
    ug = u.to("cuda", torch.float32).requires_grad_(True)
    out = mg(ug)
    out.backward(gout.to("cuda", torch.float32))
    tol = 2e-3
    assert max_rel_err(out, ref_out) < tol
    assert max_rel_err(ug.grad, ref_u.grad) < tol
    for k, p in mg.named_parameters():
        if k != "fc_D.weight":
            assert max_rel_err(p.grad, W[k].grad) < tol, k


def test_mem_eff_path_holds_less_memory_between_the_passes():
    a, b = _pair(torch.bfloat16, d_model=512, d_state=64, headdim=64, chunk_size=256, d_conv=7)
    u = torch.randn(4, 2048, 512, device="cuda", dtype=torch.bfloat16)
    held = []
    for m in (a, b):
        torch.cuda.synchronize()
        base = torch.cuda.memory_allocated()
        out = m(u.clone().requires_grad_(True))
        torch.cuda.synchronize()
        held.append(torch.cuda.memory_allocated() - base)
        out.sum().backward()
        del out
    assert held[1] < 0.75 * held[0], held


def test_split_conv1d_scan_function_without_norm_and_projection():
    """The function form with the gate inside the scan and no projections, against the same steps taken one by one."""
    from ssd.bi.conv_silu import dwconv1d_silu
    from ssd.bi.split_conv1d_scan import bimamba_split_conv1d_scan_combined, mamba_split_conv1d_scan_combined
    from ssd.bi.ssd_combined import bimamba_chunk_scan_combined
    assert mamba_split_conv1d_scan_combined is bimamba_split_conv1d_scan_combined
    torch.manual_seed(2)
    b, L, H, P, G, N, K, Q = 2, 256, 8, 32, 2, 32, 5, 64
    dim, dt_ = H * P, torch.bfloat16
    zxbcdt = torch.randn(b, L, 2 * dim + 2 * G * N + H, device="cuda", dtype=dt_)
    cw = (torch.randn(dim + 2 * G * N, 1, K, device="cuda") * 0.3)
    cb = torch.randn(dim + 2 * G * N, device="cuda") * 0.1
    dt_bias = torch.rand(H, device="cuda") - 4.0
    A = -torch.exp(torch.rand(H, device="cuda") * 2.0)
    D = torch.randn(H, P, device="cuda")
    leaves = [t.clone().requires_grad_(True) for t in (zxbcdt, cw, cb, dt_bias, A, D)]
    ref_leaves = [t.clone().requires_grad_(True) for t in (zxbcdt, cw, cb, dt_bias, A, D)]
    out = bimamba_split_conv1d_scan_combined(*leaves, Q, ngroups=G)
    z, xBC, dt = torch.split(ref_leaves[0], [dim, dim + 2 * G * N, H], dim=-1)
    xBC = dwconv1d_silu(xBC, ref_leaves[1], ref_leaves[2])
    x, Bm, Cm = torch.split(xBC, [dim, G * N, G * N], dim=-1)
    ref = bimamba_chunk_scan_combined(x.unflatten(-1, (H, P)), dt, ref_leaves[4], Bm.unflatten(-1, (G, N)),
                                      Cm.unflatten(-1, (G, N)), Q, D=ref_leaves[5], z=z.unflatten(-1, (H, P)),
                                      dt_bias=ref_leaves[3], dt_softplus=True).reshape(b, L, dim)
    assert torch.equal(out, ref)
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g)
    for got, want, name in zip(leaves, ref_leaves, ("zxbcdt", "conv_w", "conv_b", "dt_bias", "A", "D")):
        assert max_rel_err(got.grad, want.grad) <= 1e-6, name
