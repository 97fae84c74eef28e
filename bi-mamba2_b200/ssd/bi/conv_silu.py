"""Depthwise non-causal conv1d + SiLU over (batch, seqlen, channels) tensors - the front end of BiMamba2.

`dwconv1d_silu(x, weight, bias)` equals `silu(conv1d(x.transpose(1, 2), weight, bias, padding=K // 2, groups=C))
.transpose(1, 2)` (src/ssd/modules.py:164-167) but works channels-last: no transposes, and the result is one
contiguous (batch, seqlen, channels) tensor whose channel slices (x, B, C) the scan reads in place.

On CUDA tensors in the kernels' range (channels % 8 == 0, odd width <= 8, channel stride 1) the work is done by
libbissd (`bissd_dwconv_silu_forward/_backward`, csrc/conv_kernels.cuh); otherwise by the PyTorch expression above.
"""
import ctypes

import torch
import torch.nn.functional as F

from ssd import _cabi

_DT = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}


def dwconv1d_silu_ref(x, weight, bias=None):
    """The reference expression; weight (channels, 1, width) or (channels, width)."""
    w = weight.reshape(weight.shape[0], 1, -1)
    y = F.conv1d(x.transpose(1, 2), w, bias, padding=w.shape[-1] // 2, groups=w.shape[0])
    return F.silu(y).transpose(1, 2)


def _kernel_ok(x, weight, bias):
    C, K = weight.shape[0], weight.shape[-1]
    return (x.is_cuda and x.dim() == 3 and x.dtype in _DT and weight.dtype in (torch.float32, x.dtype) and
            (bias is None or bias.dtype == weight.dtype) and C % 8 == 0 and K % 2 == 1 and K <= 8 and
            x.shape[-1] == C and x.numel() > 0)


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


class _DWConvSiLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        lib = _cabi.load()
        if not _strided_ok(x):
            x = x.contiguous()
        w2 = weight.reshape(weight.shape[0], -1).contiguous()
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        a = _args(x, w2, bias, out=out)
        with torch.cuda.device(x.device):
            _cabi.check(lib.bissd_dwconv_silu_forward(ctypes.byref(a), torch.cuda.current_stream().cuda_stream))
        ctx.save_for_backward(x, w2, bias)
        ctx.wshape = weight.shape
        return out

    @staticmethod
    def backward(ctx, dout):
        lib = _cabi.load()
        x, w2, bias = ctx.saved_tensors
        dout = dout.contiguous()
        xc = x if x.is_contiguous() else x.contiguous()          # dx is written with x's strides: use a contiguous pair
        dx = torch.empty_like(xc)
        dw = torch.empty_like(w2)
        db = torch.empty_like(bias) if bias is not None else None
        a = _args(xc, w2, bias, dout=dout, dx=dx, dw=dw, db=db)
        need = ctypes.c_size_t()
        _cabi.check(lib.bissd_dwconv_silu_workspace_bytes(ctypes.byref(a), ctypes.byref(need)))
        ws = torch.empty(need.value, dtype=torch.uint8, device=x.device)
        with torch.cuda.device(x.device):
            _cabi.check(lib.bissd_dwconv_silu_backward(ctypes.byref(a), ws.data_ptr(), need.value,
                                                       torch.cuda.current_stream().cuda_stream))
        return dx, dw.reshape(ctx.wshape), db


def dwconv1d_silu(x, weight, bias=None):
    """x (batch, seqlen, channels), weight (channels, 1, width) as nn.Conv1d stores it (or (channels, width))."""
    if _kernel_ok(x, weight, bias):
        return _DWConvSiLUFn.apply(x, weight, bias)
    return dwconv1d_silu_ref(x, weight, bias)
