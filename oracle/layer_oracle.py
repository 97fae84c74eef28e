"""CPU restatements of the two element-wise neighbours of the scan inside the BiMamba2 layer.

THIS FILE IS TEST INFRASTRUCTURE (see bissd_oracle.py): only the tests import it; the shipped layer never does.

Parity status: PINNED for the gated RMSNorm - `tests/golden/rmsnorm_ref_*.npz` hold inputs, outputs and autograd
gradients of the reference's own `rms_norm_ref` (src/ssd/bi/layernorm_gated.py:18-41), written by
`tests/golden/make_golden_norm.py`; `tests/test_layer_oracle.py` holds `rms_norm_gated_reference` to them.  The
convolution oracle IS the reference expression (src/ssd/modules.py:164-167: nn.Conv1d with groups = channels and
padding = width // 2 on the transposed tensor, then SiLU), evaluated by PyTorch.
"""
import torch
import torch.nn.functional as F


def rms_norm_gated_reference(x, weight, bias=None, z=None, eps=1e-6, group_size=None, norm_before_gate=True):
    """Follows rms_norm_ref (src/ssd/bi/layernorm_gated.py:18-41) with upcast=True: everything in fp32 (or the input's
    wider type), statistics per group of `group_size` channels (the whole row when None), the gate applied before the
    statistics (norm_before_gate=False, :26-27) or after the weight (:38-39), result cast to x's dtype (:40)."""
    dtype = x.dtype
    wide = torch.float64 if dtype == torch.float64 else torch.float32
    xf = x.to(wide)
    zf = z.to(wide) if z is not None else None
    w = weight.to(wide)
    if zf is not None and not norm_before_gate:
        xf = xf * F.silu(zf)
    if group_size is None:
        rstd = 1.0 / torch.sqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
        out = xf * rstd * w
    else:
        xg = xf.unflatten(-1, (-1, group_size))
        rstd = 1.0 / torch.sqrt(xg.square().mean(dim=-1, keepdim=True) + eps)
        out = (xg * rstd).flatten(-2) * w
    if bias is not None:
        out = out + bias.to(wide)
    if zf is not None and norm_before_gate:
        out = out * F.silu(zf)
    return out.to(dtype)


def dwconv1d_silu_reference(x, weight, bias=None):
    """x (batch, seqlen, channels); weight (channels, 1, width) as nn.Conv1d stores it, or (channels, width).
    The expression of src/ssd/modules.py:164-167."""
    w = weight.reshape(weight.shape[0], 1, -1)
    y = F.conv1d(x.transpose(1, 2), w, bias, padding=w.shape[-1] // 2, groups=w.shape[0])
    return F.silu(y).transpose(1, 2)
