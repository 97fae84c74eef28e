"""Depthwise non-causal conv1d + SiLU over (batch, seqlen, channels) tensors - the front end of BiMamba2.

`dwconv1d_silu(x, weight, bias)` equals `silu(conv1d(x.transpose(1, 2), weight, bias, padding=K // 2, groups=C))
.transpose(1, 2)` (src/ssd/modules.py:164-167) but works channels-last: no transposes, and the result is one
contiguous (batch, seqlen, channels) tensor whose channel slices (x, B, C) the scan reads in place.

All work is done by libbissd (`bissd_dwconv_silu_forward/_backward`, csrc/conv_kernels.cuh).  Their range: CUDA
tensors, fp32 / bf16 / fp16, channels a multiple of 8, odd width up to 7, weight (and bias) in fp32 or the input's dtype.
There is no eager or CPU path: anything outside that range raises.
"""
import ctypes

import torch

from ssd import _cabi

_DT = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}


def _why_not(x, weight, bias):
    """None when the kernels cover these arguments, else the reason they do not."""
    C, K = weight.shape[0], weight.shape[-1]
    if not x.is_cuda or not weight.is_cuda:
        return "tensors must be on a CUDA device (no CPU implementation is shipped)"
    if x.dim() != 3 or x.shape[-1] != C:
        return f"x must be (batch, seqlen, channels) with {C} channels, got {tuple(x.shape)}"
    if x.dtype not in _DT or weight.dtype not in (torch.float32, x.dtype) or (bias is not None and bias.dtype != weight.dtype):
        return f"unsupported dtypes: x {x.dtype}, weight {weight.dtype}"
    if C % 8 != 0:
        return f"channels ({C}) must be a multiple of 8"
    if K % 2 != 1 or K > 7:
        return f"width ({K}) must be odd and at most 7"
    if x.numel() == 0:
        return "empty input"
    return None


def _kernel_ok(x, weight, bias):
    return _why_not(x, weight, bias) is None


def _strided_ok(t):
    return t.stride(-1) == 1 and t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0


def _args(x, weight, bias, out=None, dout=None, dx=None, dw=None, db=None):
    ptr = lambda t: None if t is None else t.data_ptr()
    a = _cabi.ConvArgs()
    a.batch, a.seqlen, a.channels = x.shape
    a.width = weight.shape[-1]
    a.x_dtype, a.w_dtype = _DT[x.dtype], _DT[weight.dtype]
    a.x_stride_batch, a.x_stride_row = x.stride(0), x.stride(1)
    o = out if out is not None else dout
    a.out_stride_batch, a.out_stride_row = o.stride(0), o.stride(1)
    a.x, a.weight, a.bias, a.out = ptr(x), ptr(weight), ptr(bias), ptr(out)
    a.dout, a.dx, a.dweight, a.dbias = ptr(dout), ptr(dx), ptr(dw), ptr(db)
    return a


def conv_forward(x, w2, bias):
    """silu(depthwise conv) of x (batch, seqlen, channels; rows may be strided, see _strided_ok) into a new contiguous
    tensor.  w2: (channels, width) contiguous."""
    lib = _cabi.load()
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    a = _args(x, w2, bias, out=out)
    with torch.cuda.device(x.device):
        _cabi.check(lib.bissd_dwconv_silu_forward(ctypes.byref(a), torch.cuda.current_stream().cuda_stream))
    return out


def conv_backward(x, w2, bias, dout, dx):
    """Gradients of conv_forward: writes dx (same strides as x) and returns (dweight (channels, width), dbias or None).
    dout: contiguous (batch, seqlen, channels)."""
    lib = _cabi.load()
    assert dx.stride() == x.stride() and dout.is_contiguous()
    dw = torch.empty_like(w2)
    db = torch.empty_like(bias) if bias is not None else None
    a = _args(x, w2, bias, dout=dout, dx=dx, dw=dw, db=db)
    need = ctypes.c_size_t()
    _cabi.check(lib.bissd_dwconv_silu_workspace_bytes(ctypes.byref(a), ctypes.byref(need)))
    ws = torch.empty(need.value, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _cabi.check(lib.bissd_dwconv_silu_backward(ctypes.byref(a), ws.data_ptr(), need.value,
                                                   torch.cuda.current_stream().cuda_stream))
    return dw, db


class _DWConvSiLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        if not _strided_ok(x):
            x = x.contiguous()
        w2 = weight.reshape(weight.shape[0], -1).contiguous()
        out = conv_forward(x, w2, bias)
        ctx.save_for_backward(x, w2, bias)
        ctx.wshape = weight.shape
        return out

    @staticmethod
    def backward(ctx, dout):
        x, w2, bias = ctx.saved_tensors
        xc = x if x.is_contiguous() else x.contiguous()          # dx is written with x's strides: use a contiguous pair
        dx = torch.empty_like(xc)
        dw, db = conv_backward(xc, w2, bias, dout.contiguous(), dx)
        return dx, dw.reshape(ctx.wshape), db


def dwconv1d_silu(x, weight, bias=None):
    """x (batch, seqlen, channels), weight (channels, 1, width) as nn.Conv1d stores it (or (channels, width)).
    Raises for arguments outside the kernels' range (see the module docstring)."""
    why = _why_not(x, weight, bias)
    if why is not None:
        raise RuntimeError(f"dwconv1d_silu: {why}")
    return _DWConvSiLUFn.apply(x, weight, bias)
