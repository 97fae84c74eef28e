"""Gated RMSNorm used by BiMamba2:  rmsnorm(x) * silu(z)  (norm_before_gate) or rmsnorm(x * silu(z)).

Same class name, constructor and forward signature as the reference's `ssd.bi.layernorm_gated.RMSNorm`
(src/ssd/bi/layernorm_gated.py:415-437); the arithmetic follows its `rms_norm_ref` (:18-41): statistics in fp32,
result cast back to the input dtype.  This layer sits outside the scan operator and is expressed with PyTorch
tensor ops (autograd provides its backward).
"""
import torch
import torch.nn.functional as F


def rmsnorm_fn(x, weight, bias=None, z=None, eps=1e-6, group_size=None, norm_before_gate=True):
    dtype = x.dtype
    xf = x.float()
    zf = z.float() if z is not None else None
    if zf is not None and not norm_before_gate:
        xf = xf * F.silu(zf)
    if group_size is None:
        rstd = torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
        out = xf * rstd * weight.float()
    else:
        xg = xf.unflatten(-1, (-1, group_size))
        rstd = torch.rsqrt(xg.square().mean(dim=-1, keepdim=True) + eps)
        out = (xg * rstd).flatten(-2) * weight.float()
    if bias is not None:
        out = out + bias.float()
    if zf is not None and norm_before_gate:
        out = out * F.silu(zf)
    return out.to(dtype)


class RMSNorm(torch.nn.Module):
    def __init__(self, hidden_size, eps=1e-5, group_size=None, norm_before_gate=True, device=None, dtype=None):
        """group_size=None normalises over the whole hidden dimension; otherwise over groups of that many channels."""
        factory_kwargs = {"device": device, "dtype": dtype}
        super().__init__()
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.empty(hidden_size, **factory_kwargs))
        self.register_parameter("bias", None)
        self.group_size = group_size
        self.norm_before_gate = norm_before_gate
        self.reset_parameters()

    def reset_parameters(self):
        torch.nn.init.ones_(self.weight)

    def forward(self, x, z=None):
        return rmsnorm_fn(x, self.weight, self.bias, z=z, eps=self.eps, group_size=self.group_size,
                          norm_before_gate=self.norm_before_gate)
