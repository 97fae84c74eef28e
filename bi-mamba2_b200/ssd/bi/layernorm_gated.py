"""Gated RMSNorm used by BiMamba2:  rmsnorm(x) * silu(z)  (norm_before_gate) or rmsnorm(x * silu(z)).

Same class name, constructor and forward signature as the reference's `ssd.bi.layernorm_gated.RMSNorm`
(src/ssd/bi/layernorm_gated.py:415-437); the arithmetic follows its `rms_norm_ref` (:18-41): statistics in fp32,
result cast back to the input dtype.

All work is done by libbissd's `bissd_rmsnorm_gated_forward/_backward` (csrc/norm_kernels.cuh).  Their range: CUDA
tensors, fp32 / bf16 / fp16, hidden a multiple of 256 and at most 4096, groups that are multiples of 256, no bias (the
reference's RMSNorm registers none), weight in fp32 or the input's dtype.  There is no eager or CPU path: anything
outside that range raises.
"""
import ctypes

import torch

from ssd import _cabi

_DT = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}


def _why_not(x, weight, bias, z, group_size):
    """None when the kernels cover these arguments, else the reason they do not."""
    hidden = x.shape[-1]
    group = hidden if group_size is None else group_size
    if not x.is_cuda or not weight.is_cuda or (z is not None and not z.is_cuda):
        return "tensors must be on a CUDA device (no CPU implementation is shipped)"
    if bias is not None:
        return "a bias is not supported"
    if x.dtype not in _DT or weight.dtype not in (torch.float32, x.dtype):
        return f"unsupported dtypes: x {x.dtype}, weight {weight.dtype}"
    if hidden % 256 != 0 or hidden > 4096:
        return f"hidden size {hidden} must be a multiple of 256 and at most 4096"
    if group % 256 != 0 or hidden % group != 0:
        return f"group size {group} must be a multiple of 256 that divides the hidden size {hidden}"
    if z is not None and (z.shape != x.shape or z.dtype != x.dtype):
        return "z must have x's shape and dtype"
    if x.numel() == 0:
        return "empty input"
    return None


def _kernel_ok(x, weight, bias, z, group_size):
    return _why_not(x, weight, bias, z, group_size) is None


def _rows(t, hidden):
    t = t.reshape(-1, hidden)
    if t.stride(-1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


def _norm_args(x2, z2, weight, rstd, eps, group_size, norm_before_gate, out=None, dout=None, dx=None, dz=None, dw=None):
    ptr = lambda t: None if t is None else t.data_ptr()
    a = _cabi.NormArgs()
    a.rows, a.hidden = x2.shape
    a.group_size = 0 if group_size is None else int(group_size)
    a.x_dtype, a.w_dtype = _DT[x2.dtype], _DT[weight.dtype]
    a.norm_before_gate, a.eps = int(bool(norm_before_gate)), float(eps)
    a.stride_x = x2.stride(0)
    a.stride_z = z2.stride(0) if z2 is not None else 0
    a.stride_out = (out if out is not None else dout).stride(0)
    a.x, a.z, a.weight, a.out, a.rstd = ptr(x2), ptr(z2), ptr(weight), ptr(out), ptr(rstd)
    a.dout, a.dx, a.dz, a.dweight = ptr(dout), ptr(dx), ptr(dz), ptr(dw)
    return a


def norm_forward(x2, z2, weight, eps, group_size, norm_before_gate, rstd=None):
    """x2, z2: (rows, hidden) with unit inner stride (rows may be strided).  Returns (out (rows, hidden) contiguous,
    rstd (rows, hidden / group) fp32)."""
    lib = _cabi.load()
    rows, hidden = x2.shape
    group = hidden if group_size is None else group_size
    out = torch.empty((rows, hidden), dtype=x2.dtype, device=x2.device)
    if rstd is None:
        rstd = torch.empty((rows, hidden // group), dtype=torch.float32, device=x2.device)
    a = _norm_args(x2, z2, weight, rstd, eps, group_size, norm_before_gate, out=out)
    with torch.cuda.device(x2.device):
        _cabi.check(lib.bissd_rmsnorm_gated_forward(ctypes.byref(a), torch.cuda.current_stream().cuda_stream))
    return out, rstd


def norm_backward(x2, z2, weight, rstd, eps, group_size, norm_before_gate, dout2, dx, dz):
    """Gradients of norm_forward: writes dx (row stride of x2) and dz (row stride of z2; None without z), returns the
    weight gradient.  dout2: (rows, hidden) with unit inner stride."""
    lib = _cabi.load()
    assert dx.stride(0) == x2.stride(0) and (z2 is None or dz.stride(0) == z2.stride(0))
    dw = torch.empty_like(weight)
    a = _norm_args(x2, z2, weight, rstd, eps, group_size, norm_before_gate, dout=dout2, dx=dx, dz=dz, dw=dw)
    need = ctypes.c_size_t()
    _cabi.check(lib.bissd_rmsnorm_gated_workspace_bytes(ctypes.byref(a), ctypes.byref(need)))
    ws = torch.empty(max(need.value, 16), dtype=torch.uint8, device=x2.device)
    with torch.cuda.device(x2.device):
        _cabi.check(lib.bissd_rmsnorm_gated_backward(ctypes.byref(a), ws.data_ptr(), need.value,
                                                     torch.cuda.current_stream().cuda_stream))
    return dw


class _RMSNormGatedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, z, eps, group_size, norm_before_gate):
        hidden = x.shape[-1]
        x2 = _rows(x, hidden)
        z2 = _rows(z, hidden) if z is not None else None
        weight = weight.contiguous()
        out, rstd = norm_forward(x2, z2, weight, eps, group_size, norm_before_gate)
        ctx.save_for_backward(x2, weight, z2, rstd)
        ctx.cfg = (eps, group_size, norm_before_gate, x.shape)
        return out.reshape(x.shape)

    @staticmethod
    def backward(ctx, dout):
        x2, weight, z2, rstd = ctx.saved_tensors
        eps, group_size, norm_before_gate, shape = ctx.cfg
        hidden = x2.shape[1]
        d2 = _rows(dout, hidden)
        dx = torch.empty((x2.shape[0], hidden), dtype=x2.dtype, device=x2.device)
        dz = torch.empty_like(dx) if z2 is not None else None
        # dx / dz are written with x's / z's row strides
        xs = x2 if x2.stride(0) == hidden else x2.contiguous()
        zs = z2 if z2 is None or z2.stride(0) == hidden else z2.contiguous()
        dw = norm_backward(xs, zs, weight, rstd, eps, group_size, norm_before_gate, d2, dx, dz)
        return dx.reshape(shape), dw, (dz.reshape(shape) if dz is not None else None), None, None, None


def rmsnorm_fn(x, weight, bias=None, z=None, eps=1e-6, group_size=None, norm_before_gate=True):
    """Same signature as the reference's rmsnorm_fn (src/ssd/bi/layernorm_gated.py:391-393).  Raises for arguments
    outside the kernels' range (see the module docstring)."""
    why = _why_not(x, weight, bias, z, group_size)
    if why is not None:
        raise RuntimeError(f"rmsnorm_fn: {why}")
    return _RMSNormGatedFn.apply(x, weight, z, eps, group_size, norm_before_gate)


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
