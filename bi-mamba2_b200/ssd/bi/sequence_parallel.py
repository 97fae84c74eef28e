"""Sequence-sharded bidirectional SSD scan: one long sequence split over the ranks of a process group.

Rank r owns tokens [r*L/W, (r+1)*L/W).  Each pass runs in two phases of libbissd (BISSD_PHASE_LOCAL / _FINISH,
include/bissd.h) with ONE exchange in between:

    forward :  LOCAL  -> local final states F_f, F_b (from zero incoming state) and log total decay per (batch, head)
               all-gather, then every rank chains   final_f(r) = Lambda_r * init_f(r) + F_f(r),  init_f(r+1) = final_f(r)
               (mirrored right-to-left for the reverse scan)                      -> FINISH with init_f / init_b
    backward:  LOCAL  -> gradients w.r.t. the incoming states for zero gradient of the outgoing ones
               all-gather, then   dinit_f(r) = dinit_loc_f(r) + Lambda_r * dfinal_f(r),  dfinal_f(r-1) = dinit_f(r)
               (mirrored)                                                        -> FINISH with dfinal_f / dfinal_b

The reference has no multi-GPU path; its single-GPU recurrence over chunks (src/ssd/bi/ssd_state_passing.py:27-92) is
what the chaining above continues across ranks.  The boundary payload per rank and direction is
batch*nheads*headdim*dstate fp32 values.  NCCL (through torch.distributed) carries it; remote data always lands in
local memory before a kernel reads it.
"""
import ctypes
import math

import torch
import torch.distributed as dist

from .. import _cabi
from .ssd_combined import _check_shapes, _check_status, _f32c, _inner_contig, _problem, _ptr, _tensor4, _workspace


# ----------------------------------------------------------------------------------------------------------------
# boundary algebra (pure tensor code: runs on any device, tested on CPU with gloo)
# ----------------------------------------------------------------------------------------------------------------
def chain_forward_boundaries(F_f, F_b, log_decay, rank):
    """F_f, F_b: lists (one per rank) of (b,H,P,N) local final states; log_decay: list of (b,H) = sum of a over the
    rank's tokens.  Returns (init_f, init_b) for `rank`."""
    W = len(F_f)
    lam = [torch.exp(ld)[..., None, None] for ld in log_decay]
    init_f = torch.zeros_like(F_f[0])
    for r in range(rank):                       # left to right: state entering rank r+1
        init_f = lam[r] * init_f + F_f[r]
    init_b = torch.zeros_like(F_b[0])
    for r in range(W - 1, rank, -1):            # right to left
        init_b = lam[r] * init_b + F_b[r]
    return init_f, init_b


def chain_backward_boundaries(dinit_loc_f, dinit_loc_b, log_decay, rank):
    """dinit_loc_*: lists of (b,H,P,N) gradients w.r.t. each rank's incoming states computed with zero gradient of its
    outgoing states.  Returns (dfinal_f, dfinal_b) for `rank`: the gradients of its outgoing states."""
    W = len(dinit_loc_f)
    lam = [torch.exp(ld)[..., None, None] for ld in log_decay]
    dfin = torch.zeros_like(dinit_loc_f[0])     # gradient of final_f of the last rank
    for r in range(W - 1, rank, -1):
        dfin = dinit_loc_f[r] + lam[r] * dfin   # = dinit_f(r) = dfinal_f(r-1)
    dfinal_f = dfin
    dfin = torch.zeros_like(dinit_loc_b[0])     # final_b of rank 0 leaves to the left: no consumer
    for r in range(0, rank):
        dfin = dinit_loc_b[r] + lam[r] * dfin   # = dinit_b(r) = dfinal_b(r+1)
    dfinal_b = dfin
    return dfinal_f, dfinal_b


def _all_gather(t, group):
    W = dist.get_world_size(group)
    out = [torch.empty_like(t) for _ in range(W)]
    dist.all_gather(out, t.contiguous(), group=group)
    return out


# ----------------------------------------------------------------------------------------------------------------
# phased calls into libbissd
# ----------------------------------------------------------------------------------------------------------------
class _Shard:
    """Buffers of one rank's pass; the workspace must survive from the LOCAL to the FINISH phase."""


def local_forward(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, dt_softplus=False,
                  dt_limit=(0.0, float("inf"))):
    _check_shapes(x, dt, A, B, C, chunk_size, D, z)
    lib = _cabi.load()
    st = _Shard()
    st.x, st.B, st.C, st.z = _inner_contig(x), _inner_contig(B), _inner_contig(C), _inner_contig(z)
    st.dt, st.A32, st.D32, st.bias32 = dt, _f32c(A), _f32c(D), _f32c(dt_bias)
    st.chunk_size, st.has = chunk_size, (D is not None, z is not None, dt_bias is not None)
    batch, seqlen, nheads, headdim = x.shape
    dstate = B.shape[3]
    nchunks = math.ceil(seqlen / chunk_size)
    st.p = _problem(x, dt, B, chunk_size, D, z, dt_bias, dt_softplus, dt_limit[0], dt_limit[1])
    dev = x.device
    f32 = dict(dtype=torch.float32, device=dev)
    st.out = torch.empty(x.shape, dtype=x.dtype, device=dev)
    st.out_x = torch.empty(x.shape, dtype=x.dtype, device=dev) if z is not None else None
    st.dt_out = torch.empty(batch, nheads, nchunks, chunk_size, **f32)
    st.cs_f, st.cs_b = torch.empty_like(st.dt_out), torch.empty_like(st.dt_out)
    st.states_f = torch.empty(batch, nchunks, nheads, headdim, dstate, dtype=x.dtype, device=dev)
    st.states_b = torch.empty_like(st.states_f)
    st.final_f = torch.empty(batch, nheads, headdim, dstate, **f32)
    st.final_b = torch.empty_like(st.final_f)
    st.ws, st.ws_bytes = _workspace(st.p, dev, "fwd")
    _forward_call(lib, st, None, None, _cabi.PHASE_LOCAL)
    st.log_decay = st.cs_f[..., -1].sum(dim=-1)             # (b,H): sum of a over this rank's tokens
    return st


def _forward_call(lib, st, init_f, init_b, phases):
    dt = st.dt
    args = _cabi.FwdArgs(st.p, _tensor4(st.x), _tensor4(st.B), _tensor4(st.C), _tensor4(st.z),
                         _cabi.Tensor(dt.data_ptr(), dt.stride(0), dt.stride(1), dt.stride(2)),
                         _ptr(st.A32), _ptr(st.D32), _ptr(st.bias32), _tensor4(st.out), _tensor4(st.out_x),
                         _ptr(st.dt_out), _ptr(st.cs_f), _ptr(st.cs_b), _ptr(st.states_f), _ptr(st.states_b),
                         _ptr(st.final_f), _ptr(st.final_b), _ptr(init_f), _ptr(init_b), phases)
    dev = st.x.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _cabi.check(lib.bissd_forward(ctypes.byref(args), st.ws.data_ptr(), st.ws_bytes, stream))
        _check_status(st.ws, stream)


def finish_forward(st, init_f, init_b):
    st.init_f, st.init_b = _f32c(init_f), _f32c(init_b)
    _forward_call(_cabi.load(), st, st.init_f, st.init_b, _cabi.PHASE_FINISH)
    return st.out


def local_backward(st, dout):
    lib = _cabi.load()
    x, B, C, dt = st.x, st.B, st.C, st.dt
    dev = x.device
    f32 = dict(dtype=torch.float32, device=dev)
    has_D, has_z, has_bias = st.has
    st.dout = _inner_contig(dout)
    st.dx = torch.empty(x.shape, dtype=x.dtype, device=dev)
    st.dz = torch.empty(x.shape, dtype=x.dtype, device=dev) if has_z else None
    st.dB, st.dC = torch.empty(B.shape, dtype=B.dtype, device=dev), torch.empty(C.shape, dtype=C.dtype, device=dev)
    st.ddt = torch.empty(dt.shape, dtype=dt.dtype, device=dev)
    st.dA = torch.empty(x.shape[2], **f32)
    st.dD = torch.empty(st.D32.shape, **f32) if has_D else None
    st.dbias = torch.empty(x.shape[2], **f32) if has_bias else None
    st.dinit_f = torch.empty_like(st.final_f)
    st.dinit_b = torch.empty_like(st.final_f)
    st.bws, st.bws_bytes = _workspace(st.p, dev, "bwd")
    _backward_call(lib, st, None, None, _cabi.PHASE_LOCAL)
    return st.dinit_f, st.dinit_b


def _backward_call(lib, st, dfinal_f, dfinal_b, phases):
    dt = st.dt
    args = _cabi.BwdArgs(st.p, _tensor4(st.x), _tensor4(st.B), _tensor4(st.C), _tensor4(st.z), _tensor4(st.dout),
                         _tensor4(st.out_x), _cabi.Tensor(dt.data_ptr(), dt.stride(0), dt.stride(1), dt.stride(2)),
                         _ptr(st.A32), _ptr(st.D32), _ptr(st.bias32), _ptr(st.dt_out), _ptr(st.cs_f), _ptr(st.cs_b),
                         _ptr(st.states_f), _ptr(st.states_b), _ptr(st.dx), _ptr(st.dz), _ptr(st.dB), _ptr(st.dC),
                         _ptr(st.ddt), _ptr(st.dA), _ptr(st.dD), _ptr(st.dbias), _ptr(dfinal_f), _ptr(dfinal_b),
                         _ptr(st.dinit_f), _ptr(st.dinit_b), phases)
    dev = st.x.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _cabi.check(lib.bissd_backward(ctypes.byref(args), st.bws.data_ptr(), st.bws_bytes, stream))
        _check_status(st.bws, stream)


def finish_backward(st, dfinal_f, dfinal_b):
    """Returns dx, ddt, dA, dB, dC, dD, dz, ddt_bias of this shard (parameter gradients are this rank's partial sums)."""
    st.dfinal_f, st.dfinal_b = _f32c(dfinal_f), _f32c(dfinal_b)
    _backward_call(_cabi.load(), st, st.dfinal_f, st.dfinal_b, _cabi.PHASE_FINISH)
    return st.dx, st.ddt, st.dA, st.dB, st.dC, st.dD, st.dz, st.dbias


# ----------------------------------------------------------------------------------------------------------------
# autograd entry point for real process groups
# ----------------------------------------------------------------------------------------------------------------
class _SeqParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt, A, B, C, chunk_size, D, z, dt_bias, dt_softplus, dt_limit, group):
        st = local_forward(x, dt, A, B, C, chunk_size, D, z, dt_bias, dt_softplus, dt_limit)
        rank = dist.get_rank(group)
        Ff, Fb, ld = _all_gather(st.final_f, group), _all_gather(st.final_b, group), _all_gather(st.log_decay, group)
        init_f, init_b = chain_forward_boundaries(Ff, Fb, ld, rank)
        out = finish_forward(st, init_f, init_b)
        ctx.st, ctx.group, ctx.ld = st, group, ld
        ctx.dtypes = (A.dtype, None if D is None else D.dtype, None if dt_bias is None else dt_bias.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        st, group = ctx.st, ctx.group
        rank = dist.get_rank(group)
        dif, dib = local_backward(st, dout)
        gf, gb = _all_gather(dif, group), _all_gather(dib, group)
        dfinal_f, dfinal_b = chain_backward_boundaries(gf, gb, ctx.ld, rank)
        dx, ddt, dA, dB, dC, dD, dz, dbias = finish_backward(st, dfinal_f, dfinal_b)
        a_dt, d_dt, b_dt = ctx.dtypes
        return (dx, ddt, dA.to(a_dt), dB, dC, None, None if dD is None else dD.to(d_dt), dz,
                None if dbias is None else dbias.to(b_dt), None, None, None)


def bimamba_chunk_scan_combined_seq_parallel(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, dt_softplus=False,
                                             dt_limit=(0.0, float("inf")), group=None):
    """Like bimamba_chunk_scan_combined, for a sequence sharded over `group` (rank order = sequence order; every rank
    passes its own contiguous slice of x, dt, B, C, z).  Gradients of A, D and dt_bias are this rank's partial sums:
    all-reduce them like any data-parallel parameter gradient."""
    return _SeqParallelFn.apply(x, dt, A, B, C, chunk_size, D, z, dt_bias, dt_softplus, dt_limit, group)
