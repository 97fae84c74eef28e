"""The layer's fused, memory-efficient path: split of the input projection, depthwise conv1d + SiLU, bidirectional SSD
scan, gated RMSNorm and the output projection as ONE autograd node that keeps only the projection's output, the scan's
output and the norm's statistics, and recomputes the rest in the backward pass.

It is what the reference sketches as `mamba_split_conv1d_scan_combined` (src/ssd/bi/ssd_combined.py:597-773, a copy
of the unidirectional layer's fused function that still calls a causal convolution and passes arguments the
bidirectional scan does not take) and what its layer leaves commented out behind `use_mem_eff_path`
(src/ssd/modules.py:60,129-150).  Here it computes exactly what the layer's step-by-step path computes
(src/ssd/modules.py:152-187): the same kernels of libbissd in the same order, so both paths give the same numbers.

Saved for the backward pass: zxbcdt, the scan's output (the norm's input), rstd and the parameters.  Recomputed there:
the convolution's output (x, B, C), the scan's per-chunk quantities (dt after softplus, the cumulative sums and the
states entering each chunk: the LOCAL phase of the forward library call) and the norm's output (for the output
projection's weight gradient).  Against the step-by-step path this drops the convolution's output, the norm's output
and the scan's saved states from what a layer holds between its forward and backward passes.
"""
import torch
import torch.nn.functional as F

from ssd import _cabi
from ssd.bi import conv_silu, layernorm_gated
from ssd.bi.ssd_combined import _scan_bwd_eager, _scan_fwd_core


def _split_sizes(zxbcdt, conv1d_weight, D, headdim, ngroups):
    if D.dim() == 1:
        if headdim is None:
            raise ValueError("headdim must be given when D has one entry per head")
        nheads = D.shape[0]
    else:
        nheads, headdim = D.shape
    dim = nheads * headdim
    if nheads % ngroups:
        raise ValueError("nheads must be a multiple of ngroups")
    dstate = (conv1d_weight.shape[0] - dim) // ngroups // 2
    if zxbcdt.shape[-1] != 2 * dim + 2 * ngroups * dstate + nheads:
        # the reference's signature allows extra "non-SSM" channels with a SwiGLU branch; BiMamba2 has none
        raise ValueError(f"zxbcdt must have 2*dim + 2*ngroups*dstate + nheads = {2 * dim + 2 * ngroups * dstate + nheads} "
                         f"channels, got {zxbcdt.shape[-1]}")
    return nheads, headdim, dim, dstate


def _views(zxbcdt, nheads, headdim, dim, dstate, ngroups):
    z, xBC, dt = torch.split(zxbcdt, [dim, dim + 2 * ngroups * dstate, nheads], dim=-1)
    return z, xBC, dt


def _in_place_ok(t):
    """A (batch, seqlen, channels) slice of zxbcdt the kernels can read, and write the gradient of, where it lies."""
    return t.stride(-1) == 1 and t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0


def _readable(t):
    return t if _in_place_ok(t) else t.contiguous()


def _writable(slot):
    """The tensor a kernel writes for `slot` (a slice of dzxbcdt): the slice itself, or a contiguous stand-in that is
    copied into it afterwards (returned as the second value)."""
    if _in_place_ok(slot):
        return slot, None
    tmp = torch.empty(slot.shape, dtype=slot.dtype, device=slot.device)
    return tmp, tmp


def _xbc_views(xBC_conv, nheads, headdim, dim, dstate, ngroups):
    x, B, C = torch.split(xBC_conv, [dim, ngroups * dstate, ngroups * dstate], dim=-1)
    return (x.unflatten(-1, (nheads, headdim)), B.unflatten(-1, (ngroups, dstate)), C.unflatten(-1, (ngroups, dstate)))


class BiMambaSplitConv1dScanCombinedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, zxbcdt, conv1d_weight, conv1d_bias, dt_bias, A, D, chunk_size, dt_limit, rmsnorm_weight, rmsnorm_eps,
                outproj_weight, outproj_bias, headdim, ngroups, norm_before_gate, rmsnorm_group_size):
        nheads, headdim, dim, dstate = _split_sizes(zxbcdt, conv1d_weight, D, headdim, ngroups)
        if not zxbcdt.is_contiguous():
            zxbcdt = zxbcdt.contiguous()
        batch, seqlen, _ = zxbcdt.shape
        z, xBC, dt = _views(zxbcdt, nheads, headdim, dim, dstate, ngroups)
        # the slices are read where they lie when their rows are 16-byte aligned (a channel count of zxbcdt that is a
        # multiple of 8), else through a contiguous copy
        z, xBC = _readable(z), _readable(xBC)
        w2 = conv1d_weight.reshape(conv1d_weight.shape[0], -1).contiguous()
        why = conv_silu._why_not(xBC, conv1d_weight, conv1d_bias)
        if why is not None:
            raise RuntimeError(f"bimamba_split_conv1d_scan_combined: convolution: {why}")
        xBC_conv = conv_silu.conv_forward(xBC, w2, conv1d_bias)
        x, B, C = _xbc_views(xBC_conv, nheads, headdim, dim, dstate, ngroups)
        zh = z.unflatten(-1, (nheads, headdim))
        gate_in_scan = rmsnorm_weight is None
        res = _scan_fwd_core(x, dt, A, B, C, chunk_size, D, zh if gate_in_scan else None, dt_bias, None, None, True,
                             dt_limit[0], dt_limit[1], True)
        out, out_x = res[0], res[1]
        rstd = None
        if gate_in_scan:
            y = out.reshape(batch, seqlen, dim)
            saved_scan_out = out_x                               # pre-gate output: what the scan's backward reads
        else:
            group = dim // ngroups if rmsnorm_group_size is None else rmsnorm_group_size
            x2 = out.reshape(batch * seqlen, dim)
            z2 = z.reshape(batch * seqlen, dim)                  # a strided view: rows of zxbcdt
            why = layernorm_gated._why_not(x2, rmsnorm_weight, None, z2, group)
            if why is not None:
                raise RuntimeError(f"bimamba_split_conv1d_scan_combined: norm: {why}")
            rmsnorm_weight = rmsnorm_weight.contiguous()
            y2, rstd = layernorm_gated.norm_forward(x2, z2, rmsnorm_weight, rmsnorm_eps, group, norm_before_gate)
            y = y2.reshape(batch, seqlen, dim)
            saved_scan_out = out
        result = F.linear(y, outproj_weight, outproj_bias) if outproj_weight is not None else y
        ctx.save_for_backward(zxbcdt, conv1d_weight, conv1d_bias, saved_scan_out, A, D, dt_bias, rmsnorm_weight, rstd,
                              outproj_weight, outproj_bias)
        ctx.cfg = (chunk_size, dt_limit, rmsnorm_eps, headdim, ngroups, norm_before_gate, rmsnorm_group_size)
        return result

    @staticmethod
    def backward(ctx, dresult):
        (zxbcdt, conv1d_weight, conv1d_bias, scan_out, A, D, dt_bias, rmsnorm_weight, rstd, outproj_weight,
         outproj_bias) = ctx.saved_tensors
        chunk_size, dt_limit, rmsnorm_eps, headdim, ngroups, norm_before_gate, rmsnorm_group_size = ctx.cfg
        nheads, headdim, dim, dstate = _split_sizes(zxbcdt, conv1d_weight, D, headdim, ngroups)
        batch, seqlen, _ = zxbcdt.shape
        z, xBC, dt = _views(zxbcdt, nheads, headdim, dim, dstate, ngroups)
        z, xBC = _readable(z), _readable(xBC)
        zh = z.unflatten(-1, (nheads, headdim))
        dzxbcdt = torch.empty_like(zxbcdt)
        dz_slot, dxBC_slot, ddt_slot = _views(dzxbcdt, nheads, headdim, dim, dstate, ngroups)
        (dz, dz_tmp), (dxBC, dxBC_tmp) = _writable(dz_slot), _writable(dxBC_slot)
        gate_in_scan = rmsnorm_weight is None
        dresult = dresult.contiguous()
        # recompute x, B, C
        w2 = conv1d_weight.reshape(conv1d_weight.shape[0], -1).contiguous()
        xBC_conv = conv_silu.conv_forward(xBC, w2, conv1d_bias)
        x, B, C = _xbc_views(xBC_conv, nheads, headdim, dim, dstate, ngroups)
        dy = F.linear(dresult, outproj_weight.t()) if outproj_weight is not None else dresult
        dy = dy.reshape(batch, seqlen, dim)
        doutproj_weight = doutproj_bias = drmsnorm_weight = None
        if gate_in_scan:
            dscan_out = dy.unflatten(-1, (nheads, headdim))
        else:
            group = dim // ngroups if rmsnorm_group_size is None else rmsnorm_group_size
            x2 = scan_out.reshape(batch * seqlen, dim)
            z2 = z.reshape(batch * seqlen, dim)
            dy2 = dy.reshape(batch * seqlen, dim)
            dscan2 = torch.empty_like(x2)
            drmsnorm_weight = layernorm_gated.norm_backward(x2, z2, rmsnorm_weight, rstd, rmsnorm_eps, group,
                                                            norm_before_gate, dy2, dscan2,
                                                            dz.reshape(batch * seqlen, dim))
            dscan_out = dscan2.reshape(batch, seqlen, nheads, headdim)
        if outproj_weight is not None:
            if gate_in_scan:
                y = scan_out * F.silu(zh)                        # scan_out is the pre-gate output here
                y = y.reshape(batch, seqlen, dim)
            else:
                y = layernorm_gated.norm_forward(x2, z2, rmsnorm_weight, rmsnorm_eps, group, norm_before_gate,
                                                 rstd=torch.empty_like(rstd))[0].reshape(batch, seqlen, dim)
            doutproj_weight = torch.einsum("bso,bsd->od", dresult, y)
            doutproj_bias = dresult.sum(dim=(0, 1)) if outproj_bias is not None else None
        # recompute what the scan's forward hands to its backward (LOCAL phase: no scan, `out` is not written)
        zs = zh if gate_in_scan else None
        loc = _scan_fwd_core(x, dt, A, B, C, chunk_size, D, zs, dt_bias, None, None, True, dt_limit[0], dt_limit[1], True,
                             phases=_cabi.PHASE_LOCAL, out=dscan_out if dscan_out.is_contiguous() else dscan_out.contiguous())
        dt_out, cs_f, cs_b, states_f, states_b = loc[2:7]
        dx, ddt, dA, dB, dC, dD, dzs, ddt_bias, _, _ = _scan_bwd_eager(
            dscan_out, x, dt, A, B, C, chunk_size, D, zs, dt_bias, scan_out if gate_in_scan else None, dt_out, cs_f, cs_b,
            states_f, states_b, None, None, False, True, dt_limit[0], dt_limit[1])
        if gate_in_scan:
            dz.copy_(dzs.reshape(batch, seqlen, dim))
        ddt_slot.copy_(ddt)
        dxBC_conv = torch.cat([dx.reshape(batch, seqlen, dim), dB.reshape(batch, seqlen, -1),
                               dC.reshape(batch, seqlen, -1)], dim=-1)
        dw2, dconv_bias = conv_silu.conv_backward(xBC, w2, conv1d_bias, dxBC_conv, dxBC)
        if dz_tmp is not None:
            dz_slot.copy_(dz_tmp)
        if dxBC_tmp is not None:
            dxBC_slot.copy_(dxBC_tmp)
        dA = dA.to(A.dtype)
        dD = dD.to(D.dtype)
        ddt_bias = ddt_bias.to(dt_bias.dtype)
        return (dzxbcdt, dw2.reshape(conv1d_weight.shape), dconv_bias, ddt_bias, dA, dD, None, None, drmsnorm_weight, None,
                doutproj_weight, doutproj_bias, None, None, None, None)


def bimamba_split_conv1d_scan_combined(zxbcdt, conv1d_weight, conv1d_bias, dt_bias, A, D, chunk_size,
                                       dt_limit=(0.0, float("inf")), rmsnorm_weight=None, rmsnorm_eps=1e-6,
                                       outproj_weight=None, outproj_bias=None, headdim=None, ngroups=1,
                                       norm_before_gate=True, rmsnorm_group_size=None):
    """
    Argument (names and meaning as the reference's mamba_split_conv1d_scan_combined, src/ssd/bi/ssd_combined.py:758-773):
        zxbcdt: (batch, seqlen, 2 * dim + 2 * ngroups * dstate + nheads) where dim == nheads * headdim; [z | x B C | dt]
        conv1d_weight: (dim + 2 * ngroups * dstate, 1, width) or (.., width); conv1d_bias: (dim + 2 * ngroups * dstate,)
        dt_bias, A: (nheads,);  D: (nheads, headdim) or (nheads,) (then headdim must be given)
        rmsnorm_weight: (dim,) - with it, out = rmsnorm(y, gate z) over groups of rmsnorm_group_size channels
            (default dim // ngroups as in the reference's function; the layer normalises over all of dim); without it
            the gate is applied inside the scan
        outproj_weight: (out_dim, dim), outproj_bias: (out_dim,) - optional final projection
        norm_before_gate: True: rmsnorm(y) * silu(z); False: rmsnorm(y * silu(z))
    Return:
        out: (batch, seqlen, out_dim or dim)
    Differences from that signature: the convolution is the layer's centred (non-causal) one, `initial_states`,
    `seq_idx`, `return_final_states` and extra non-SSM channels are not taken (the bidirectional layer has none), and
    arguments outside the kernels' range raise instead of falling back.
    """
    return BiMambaSplitConv1dScanCombinedFn.apply(zxbcdt, conv1d_weight, conv1d_bias, dt_bias, A, D, chunk_size, dt_limit,
                                                  rmsnorm_weight, rmsnorm_eps, outproj_weight, outproj_bias, headdim,
                                                  ngroups, norm_before_gate, rmsnorm_group_size)


mamba_split_conv1d_scan_combined = bimamba_split_conv1d_scan_combined   # the reference's name for it
