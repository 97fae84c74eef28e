"""The BiMamba2 layer (the operator's caller in the reference, src/ssd/modules.py:17-187): same parameters and
state_dict keys, forward + backward against a dense restatement of the layer in fp64 built on the oracle's O(L^2)
definition of the scan."""
import pytest
import torch
import torch.nn.functional as F

from oracle.bissd_oracle import dense_reference, max_rel_err

pytestmark = pytest.mark.gpu


def _dense_layer(m, u):
    """fp64 restatement of BiMamba2.forward with the module's own parameters (src/ssd/modules.py:118-187)."""
    d = torch.float64
    W = {k: v.detach().to("cpu", d).requires_grad_(True) for k, v in m.named_parameters()}
    zxbcdt = u @ W["in_proj.weight"].t()
    A = -torch.exp(W["A_log"])
    z, xBC, dt = torch.split(zxbcdt, [m.d_inner, m.d_inner + 2 * m.ngroups * m.d_state, m.nheads], dim=-1)
    dt = F.softplus(dt + W["dt_bias"])
    xBC = F.silu(F.conv1d(xBC.transpose(1, 2), W["conv1d.weight"], W["conv1d.bias"], padding=m.d_conv // 2,
                          groups=xBC.shape[-1]).transpose(1, 2))
    x, B, C = torch.split(xBC, [m.d_inner, m.ngroups * m.d_state, m.ngroups * m.d_state], dim=-1)
    b, L = u.shape[:2]
    y = dense_reference(x.reshape(b, L, m.nheads, m.headdim), dt, A, B.reshape(b, L, m.ngroups, m.d_state),
                        C.reshape(b, L, m.ngroups, m.d_state), D=W["D"])
    y = y.reshape(b, L, m.d_inner)
    y = y * torch.rsqrt(y.square().mean(-1, keepdim=True) + 1e-5) * W["norm.weight"] * F.silu(z)
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
    m = BiMamba2(64, d_state=64, headdim=64, chunk_size=128, d_conv=7)
    with torch.no_grad():
        m.A_log.uniform_(0.0, 2.0)
        m.D.normal_()
    u = torch.randn(2, 256, 64, dtype=torch.float64)
    gout = torch.randn(2, 256, 64, dtype=torch.float64)
    ref_u = u.clone().requires_grad_(True)
    ref_out, W = _dense_layer(m, ref_u)
    ref_out.backward(gout)
    mg = BiMamba2(64, d_state=64, headdim=64, chunk_size=128, d_conv=7).to("cuda", dtype)
    mg.load_state_dict({k: v.to(dtype) for k, v in m.state_dict().items()})
    ug = u.to("cuda", dtype).requires_grad_(True)
    out = mg(ug)
    out.backward(gout.to("cuda", dtype))
    assert max_rel_err(out, ref_out) < tol
    assert max_rel_err(ug.grad, ref_u.grad) < tol
    for k, p in mg.named_parameters():
        if k == "fc_D.weight":            # defined but unused, as in the reference: receives no gradient
            assert p.grad is None
            continue
        assert max_rel_err(p.grad, W[k].grad) < tol, k
