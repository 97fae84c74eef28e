"""Sequence-sharded bidirectional SSD scan: one long sequence split over the ranks of a process group.

Rank r owns tokens [r*L/W, (r+1)*L/W).  Each pass runs in two phases of libbissd (BISSD_PHASE_LOCAL / _FINISH,
include/bissd.h) with ONE exchange in between:

    forward :  LOCAL  -> local final states F_f, F_b (from zero incoming state) and log total decay per (batch, head)
               ONE all-gather of the packed (F_f, F_b, log decay), then every rank chains
               final_f(r) = Lambda_r * init_f(r) + F_f(r),  init_f(r+1) = final_f(r)  (unrolled into one weighted sum;
               mirrored right-to-left for the reverse scan)                       -> FINISH with init_f / init_b
    backward:  LOCAL  -> gradients w.r.t. the incoming states for zero gradient of the outgoing ones
               ONE all-gather, then   dinit_f(r) = dinit_loc_f(r) + Lambda_r * dfinal_f(r),  dfinal_f(r-1) = dinit_f(r)
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
def _chain_weights(log_decay_all, rank):
    """log_decay_all (W,b,H): each rank's sum of a over its tokens.  Returns (w_left, w_right), both (W,b,H) fp32:
    w_left[r']  = exp(sum of log decays of the ranks strictly between r' and `rank`) for r' < rank, else 0;
    w_right[r'] = the same for r' > rank.  Every exponent is a sum of non-positive numbers; the prefix sums are taken
    in fp64 so that their differences stay exact when one rank's decay is huge and its neighbours' are not."""
    W = log_decay_all.shape[0]
    ld = log_decay_all.double()
    c = torch.cat([torch.zeros_like(ld[:1]), torch.cumsum(ld, dim=0)], dim=0)       # c[k] = sum_{j<k} ld[j]
    idx = torch.arange(W, device=ld.device)
    shape = (W,) + (1,) * (ld.dim() - 1)
    left = (idx < rank).view(shape)
    right = (idx > rank).view(shape)
    e_left = c[rank].unsqueeze(0) - c[1:]                                           # span (r', rank)
    e_right = c[:-1] - c[rank + 1].unsqueeze(0)                                     # span (rank, r')
    zero = torch.zeros((), dtype=torch.float64, device=ld.device)
    w_left = torch.where(left, torch.exp(torch.where(left, e_left, zero)), zero)
    w_right = torch.where(right, torch.exp(torch.where(right, e_right, zero)), zero)
    return w_left.to(log_decay_all.dtype), w_right.to(log_decay_all.dtype)


def chain_forward_stacked(F_f, F_b, log_decay, rank):
    """F_f, F_b (W,b,H,P,N): every rank's local final states (from zero incoming state); log_decay (W,b,H).
    Returns (init_f, init_b) for `rank`:  init_f = sum_{r'<rank} (prod_{r'<r''<rank} Lambda_r'') F_f[r'],  init_b the
    mirror image over r' > rank - the recurrence  S <- Lambda_r S + F_r  of the single-GPU chunk loop
    (src/ssd/bi/ssd_state_passing.py:60,81) continued across ranks, unrolled into one weighted sum."""
    w_left, w_right = _chain_weights(log_decay, rank)
    return (w_left[..., None, None] * F_f).sum(dim=0), (w_right[..., None, None] * F_b).sum(dim=0)


def chain_backward_stacked(dinit_loc_f, dinit_loc_b, log_decay, rank):
    """dinit_loc_* (W,b,H,P,N): every rank's gradient w.r.t. its incoming states computed with zero gradient of its
    outgoing states.  Returns (dfinal_f, dfinal_b) for `rank`, the gradients of its outgoing states:
    dfinal_f = sum_{r'>rank} (prod_{rank<r''<r'} Lambda_r'') dinit_loc_f[r'],  dfinal_b the mirror image."""
    w_left, w_right = _chain_weights(log_decay, rank)
    return (w_right[..., None, None] * dinit_loc_f).sum(dim=0), (w_left[..., None, None] * dinit_loc_b).sum(dim=0)


def chain_on_device(left, right, log_decay, rank):
    """The two weighted sums of chain_forward_stacked / chain_backward_stacked in ONE libbissd launch
    (bissd_chain_boundaries) instead of some twenty small tensor kernels.  left, right: (W,b,H,P,N) fp32 CUDA tensors
    (views of a gathered buffer are fine: only the rank stride may differ from contiguous); log_decay (W,b,H).
    Returns (sum over ranks < rank of left, sum over ranks > rank of right), each (b,H,P,N)."""
    W, b, H, P, N = left.shape
    assert left.dtype == torch.float32 and right.dtype == torch.float32 and log_decay.dtype == torch.float32
    assert left[0].is_contiguous() and right[0].is_contiguous() and log_decay[0].is_contiguous()
    assert left.stride(0) == right.stride(0)
    out_l, out_r = torch.empty(2, b, H, P, N, dtype=torch.float32, device=left.device).unbind(0)
    lib = _cabi.load()
    with torch.cuda.device(left.device):
        stream = torch.cuda.current_stream(left.device).cuda_stream
        _cabi.check(lib.bissd_chain_boundaries(left.data_ptr(), right.data_ptr(), log_decay.data_ptr(), left.stride(0),
                                               log_decay.stride(0), W, rank, b * H, P * N, out_l.data_ptr(),
                                               out_r.data_ptr(), stream))
    return out_l, out_r


def chain_forward_boundaries(F_f, F_b, log_decay, rank):
    """List form (one entry per rank) of chain_forward_stacked."""
    return chain_forward_stacked(torch.stack(list(F_f)), torch.stack(list(F_b)), torch.stack(list(log_decay)), rank)


def chain_backward_boundaries(dinit_loc_f, dinit_loc_b, log_decay, rank):
    """List form (one entry per rank) of chain_backward_stacked."""
    return chain_backward_stacked(torch.stack(list(dinit_loc_f)), torch.stack(list(dinit_loc_b)),
                                  torch.stack(list(log_decay)), rank)


def _all_gather(t, group):
    W = dist.get_world_size(group)
    out = [torch.empty_like(t) for _ in range(W)]
    dist.all_gather(out, t.contiguous(), group=group)
    return out


_gather_buffers = {}


def gather_packed(tensors, group):
    """ONE collective for several same-dtype tensors: they are packed into one flat buffer, all-gathered into a
    (W, total) tensor that lands in local memory, and handed back as (W, *shape) views in the order given.

    The send and receive buffers are kept per (device, dtype, size, world size) and reused: a buffer that has been
    through a NCCL call is held back by the caching allocator until the communication stream has released it, so
    fresh ones every pass turn into real cudaMalloc / cudaFree calls - two milliseconds per step at config #3's shard
    size.  The views returned are therefore only valid until the next call with the same sizes: use them at once (the
    chaining does) and copy what must live longer."""
    W = dist.get_world_size(group)
    n = sum(t.numel() for t in tensors)
    ref = tensors[0]
    key = (ref.device, ref.dtype, n, W)
    buf = _gather_buffers.get(key)
    if buf is None:
        buf = (torch.empty(n, dtype=ref.dtype, device=ref.device), torch.empty(W * n, dtype=ref.dtype, device=ref.device))
        _gather_buffers[key] = buf
    flat, out = buf
    torch.cat([t.reshape(-1) for t in tensors], out=flat)
    dist.all_gather_into_tensor(out, flat, group=group)       # rank r's buffer lands at [r * n, (r + 1) * n)
    rows = out.view(W, n)
    views, o = [], 0
    for t in tensors:
        views.append(rows[:, o:o + t.numel()].view((W,) + tuple(t.shape)))
        o += t.numel()
    return views


# Optional CUDA-event brackets around the exchange (collective + chaining) of every pass, for benchmarks.
_exchange_events = None


def record_exchange_events(on):
    """on=True: start collecting (start, end) event pairs around every boundary exchange; on=False: stop and drop."""
    global _exchange_events
    _exchange_events = [] if on else None


def exchange_ms():
    """Sum of the recorded exchange times in ms (synchronises on the recorded events)."""
    total = 0.0
    for e0, e1 in _exchange_events or []:
        e1.synchronize()
        total += e0.elapsed_time(e1)
    return total


class _ExchangeTimer:
    def __init__(self, device):
        self.on = _exchange_events is not None and device.type == "cuda"
        if self.on:
            self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        if self.on:
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if self.on:
            self.e1.record()
            _exchange_events.append((self.e0, self.e1))
        return False


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
        with _ExchangeTimer(x.device):
            Ff, Fb, ld = gather_packed([st.final_f, st.final_b, st.log_decay], group)
            init_f, init_b = chain_on_device(Ff, Fb, ld, rank)
        out = finish_forward(st, init_f, init_b)
        # The shard object lives on the autograd node; it must not hold the output tensor (whose grad_fn is that node):
        # the cycle would keep every buffer of the pass alive until Python's cycle collector runs, and the caching
        # allocator would answer each new pass with fresh cudaMalloc calls.
        st.out = None
        ctx.st, ctx.group, ctx.ld = st, group, ld.clone()        # ld is a view of a reused receive buffer
        ctx.dtypes = (A.dtype, None if D is None else D.dtype, None if dt_bias is None else dt_bias.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        st, group = ctx.st, ctx.group
        rank = dist.get_rank(group)
        dif, dib = local_backward(st, dout)
        with _ExchangeTimer(dout.device):
            gf, gb = gather_packed([dif, dib], group)
            dfinal_b, dfinal_f = chain_on_device(gb, gf, ctx.ld, rank)      # left = dinit_b -> dfinal_b, right = dinit_f -> dfinal_f
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
