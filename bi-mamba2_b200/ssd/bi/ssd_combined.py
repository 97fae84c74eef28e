"""Bidirectional SSD chunk scan  y = SS(x) + flip(SS(flip(x))) + D*x  (optionally gated by z) on B200.

Drop-in for the reference module of the same import path (`ssd.bi.ssd_combined`, Hprairie/Bi-Mamba2
src/ssd/bi/ssd_combined.py): same public function `bimamba_chunk_scan_combined` (:577), same autograd class
name `MambaChunkScanCombinedFn` (:555) and the two private entry points the reference's own tests and
benchmarks call, `_mamba_chunk_scan_combined_fwd` (:297) and `_mamba_chunk_scan_combined_bwd` (:334).

All arithmetic runs in libbissd.so (hand-written CUDA for sm_100a, C ABI in include/bissd.h) through two
PyTorch custom ops, `bissd::scan_fwd` and `bissd::scan_bwd` (in eager mode their implementations are called
directly, skipping the dispatcher).  There is no Triton and no CPU or eager fallback:
without the library, or on CPU tensors, the operator raises.
"""
import math
import os
from typing import Optional, Tuple

import torch

from .. import _cabi

_DTYPES = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}

# With BISSD_CHECK_STATUS=1 every pass is followed by a (synchronising) read of the library's device status word
# and raises if a bounded device-side wait ran out.  Meant for tests and debugging; off by default.
CHECK_STATUS = os.environ.get("BISSD_CHECK_STATUS", "0") == "1"


def _check_status(ws, stream):
    if not CHECK_STATUS:
        return
    import ctypes
    st = ctypes.c_int(0)
    _cabi.check(_cabi.load().bissd_read_status(ws.data_ptr(), stream, ctypes.byref(st)))
    if st.value != 0:
        raise _cabi.BissdError(f"libbissd device status {st.value}: a device-side wait ran out; results are invalid")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _tensor4(t):
    """(batch, seq, heads, inner) tensor with contiguous inner dim -> C struct."""
    if t is None:
        return _cabi.Tensor(None, 0, 0, 0)
    return _cabi.Tensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _problem(x, dt, B, chunk_size, D, z, dt_bias, dt_softplus, dt_min, dt_max):
    batch, seqlen, nheads, headdim = x.shape
    ngroups, dstate = B.shape[2], B.shape[3]
    if x.dtype not in _DTYPES or dt.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype: x {x.dtype}, dt {dt.dtype}")
    return _cabi.Problem(batch, seqlen, nheads, headdim, ngroups, dstate, int(chunk_size), _DTYPES[x.dtype],
                         _DTYPES[dt.dtype], int(D is not None), int(D is not None and D.dim() == 2),
                         int(z is not None), int(dt_bias is not None), int(bool(dt_softplus)),
                         float(dt_min), float(dt_max))


_ws_bytes = {}                                    # problem fields -> (forward bytes, backward bytes)


def _workspace(problem, device, which):
    key = tuple(getattr(problem, name) for name, _ in problem._fields_)
    sizes = _ws_bytes.get(key)
    if sizes is None:
        import ctypes
        f, b = ctypes.c_size_t(0), ctypes.c_size_t(0)
        _cabi.check(_cabi.load().bissd_workspace_bytes(ctypes.byref(problem), ctypes.byref(f), ctypes.byref(b)))
        sizes = _ws_bytes[key] = (f.value, b.value)
    nbytes = sizes[0] if which == "fwd" else sizes[1]
    return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device), nbytes


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("bimamba_chunk_scan_combined runs on CUDA tensors only (no CPU implementation is shipped)")


def _f32c(t):
    if t is None:
        return None
    if t.dtype is torch.float32 and t.is_contiguous():
        return t                                  # only its address is taken: no detach / cast / copy needed
    return t.detach().to(torch.float32).contiguous()


def _inner_contig(t):
    """t as the library reads it in place: unit inner stride and, for 16-bit tensors, 16-byte aligned rows (what the
    tensor-core kernels and the workspace size reported for them assume); anything else is copied."""
    if t is None:
        return t
    if t.stride(-1) != 1:
        return t.contiguous()
    if t.element_size() == 2 and (t.data_ptr() % 16 or any(st % 8 for st in t.stride()[:-1])):
        return t.contiguous()
    return t


def kernel_path(x, dt, B, chunk_size, D=None, z=None, dt_bias=None, dt_softplus=False, dt_limit=(0.0, float("inf"))):
    """Which kernel family libbissd picks for these arguments ("tcgen05" or "simt")."""
    import ctypes
    p = _problem(x, dt, B, chunk_size, D, z, dt_bias, dt_softplus, dt_limit[0], dt_limit[1])
    return _cabi.load().bissd_kernel_path(ctypes.byref(p)).decode()


# ----------------------------------------------------------------------------------------------------------------
# custom ops: thin marshalling around bissd_forward / bissd_backward
#
# `_scan_fwd_core` / `_scan_bwd_core` do the marshalling; `bissd::scan_fwd` / `bissd::scan_bwd` are the same functions
# registered as PyTorch custom ops (with fake kernels) so that torch.compile and the dispatcher see opaque operators.
# In plain eager mode the autograd function below calls the cores directly: a trip through the custom-op machinery
# costs about 0.1 ms of host time per call, a quarter of a forward + backward step of the benchmark shape.
# ----------------------------------------------------------------------------------------------------------------
def _family(n, shape, fused, **kw):
    """n equally shaped buffers: views of one allocation when `fused` (every torch.empty costs a few microseconds of
    host time), separate tensors otherwise (outputs of a custom op may not share storage)."""
    if fused:
        return torch.empty((n,) + tuple(shape), **kw).unbind(0)
    return tuple(torch.empty(shape, **kw) for _ in range(n))


def _scan_fwd_core(x, dt, A, B, C, chunk_size, D, z, dt_bias, init_f, init_b, dt_softplus, dt_min, dt_max, fused,
                   phases=None, out=None):
    """Returns (out, out_x, dt_out, cs_f, cs_b, states_f, states_b, final_f, final_b); out_x is empty without z.
    phases: a BISSD_PHASE_* mask (default all); with PHASE_LOCAL alone only dt_out, the cumulative sums, the entering
    states and the final states are computed and `out` (any tensor of x's shape, never written) must be given."""
    import ctypes
    _require_cuda(x, dt, A, B, C, D, z, dt_bias)
    lib = _cabi.load()
    x, B, C, z = _inner_contig(x), _inner_contig(B), _inner_contig(C), _inner_contig(z)
    A32, D32, bias32 = _f32c(A), _f32c(D), _f32c(dt_bias)
    init_f, init_b = _f32c(init_f), _f32c(init_b)
    batch, seqlen, nheads, headdim = x.shape
    dstate = B.shape[3]
    nchunks = math.ceil(seqlen / chunk_size)
    p = _problem(x, dt, B, chunk_size, D, z, dt_bias, dt_softplus, dt_min, dt_max)
    dev = x.device
    phases = _cabi.PHASE_ALL if phases is None else phases
    if out is None:
        out = torch.empty(x.shape, dtype=x.dtype, device=dev)
    if z is not None and (phases & _cabi.PHASE_FINISH):
        out_x = torch.empty(x.shape, dtype=x.dtype, device=dev)
    else:
        out_x = torch.empty(0, dtype=x.dtype, device=dev) if z is None else out
    dt_out, cs_f, cs_b = _family(3, (batch, nheads, nchunks, chunk_size), fused, dtype=torch.float32, device=dev)
    states_f, states_b = _family(2, (batch, nchunks, nheads, headdim, dstate), fused, dtype=x.dtype, device=dev)
    final_f, final_b = _family(2, (batch, nheads, headdim, dstate), fused, dtype=torch.float32, device=dev)
    ws, nbytes = _workspace(p, dev, "fwd")
    args = _cabi.FwdArgs(p, _tensor4(x), _tensor4(B), _tensor4(C), _tensor4(z),
                         _cabi.Tensor(dt.data_ptr(), dt.stride(0), dt.stride(1), dt.stride(2)),
                         _ptr(A32), _ptr(D32), _ptr(bias32), _tensor4(out), _tensor4(out_x if z is not None else None),
                         _ptr(dt_out), _ptr(cs_f), _ptr(cs_b), _ptr(states_f), _ptr(states_b), _ptr(final_f),
                         _ptr(final_b), _ptr(init_f), _ptr(init_b), phases)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _cabi.check(lib.bissd_forward(ctypes.byref(args), ws.data_ptr(), nbytes, stream))
        _check_status(ws, stream)
    return out, out_x, dt_out, cs_f, cs_b, states_f, states_b, final_f, final_b


def _scan_fwd_impl(x: torch.Tensor, dt: torch.Tensor, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, chunk_size: int,
                   D: Optional[torch.Tensor], z: Optional[torch.Tensor], dt_bias: Optional[torch.Tensor],
                   init_f: Optional[torch.Tensor], init_b: Optional[torch.Tensor], dt_softplus: bool, dt_min: float,
                   dt_max: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                                           torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return _scan_fwd_core(x, dt, A, B, C, chunk_size, D, z, dt_bias, init_f, init_b, dt_softplus, dt_min, dt_max, False)


def _scan_fwd_eager(*args):
    return _scan_fwd_core(*args, True)


scan_fwd = torch.library.custom_op("bissd::scan_fwd", _scan_fwd_impl, mutates_args=())


@scan_fwd.register_fake
def _(x, dt, A, B, C, chunk_size, D, z, dt_bias, init_f, init_b, dt_softplus, dt_min, dt_max):
    batch, seqlen, nheads, headdim = x.shape
    dstate = B.shape[3]
    nchunks = (seqlen + chunk_size - 1) // chunk_size
    f32 = dict(dtype=torch.float32, device=x.device)
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    out_x = torch.empty(x.shape if z is not None else (0,), dtype=x.dtype, device=x.device)
    hq = (batch, nheads, nchunks, chunk_size)
    st = (batch, nchunks, nheads, headdim, dstate)
    fin = (batch, nheads, headdim, dstate)
    return (out, out_x, torch.empty(hq, **f32), torch.empty(hq, **f32), torch.empty(hq, **f32),
            torch.empty(st, dtype=x.dtype, device=x.device), torch.empty(st, dtype=x.dtype, device=x.device),
            torch.empty(fin, **f32), torch.empty(fin, **f32))


def _scan_bwd_core(dout, x, dt, A, B, C, chunk_size, D, z, dt_bias, out_x, dt_out, cs_f, cs_b, states_f, states_b,
                   dfinal_f, dfinal_b, want_dinit, dt_softplus, dt_min, dt_max, fused):
    """Returns (dx, ddt, dA, dB, dC, dD, dz, ddt_bias, dinit_f, dinit_b); absent ones are empty tensors."""
    import ctypes
    _require_cuda(dout, x, dt, A, B, C)
    lib = _cabi.load()
    x, B, C, z, dout, out_x = (_inner_contig(t) for t in (x, B, C, z, dout, out_x))
    A32, D32, bias32 = _f32c(A), _f32c(D), _f32c(dt_bias)
    dfinal_f, dfinal_b = _f32c(dfinal_f), _f32c(dfinal_b)
    batch, seqlen, nheads, headdim = x.shape
    dstate = B.shape[3]
    p = _problem(x, dt, B, chunk_size, D, z, dt_bias, dt_softplus, dt_min, dt_max)
    dev = x.device
    f32 = dict(dtype=torch.float32, device=dev)
    empty = lambda dtype=torch.float32: torch.empty(0, dtype=dtype, device=dev)
    dx = torch.empty(x.shape, dtype=x.dtype, device=dev)
    dz = torch.empty(x.shape, dtype=x.dtype, device=dev) if z is not None else empty(x.dtype)
    dB = torch.empty(B.shape, dtype=B.dtype, device=dev)
    dC = torch.empty(C.shape, dtype=C.dtype, device=dev)
    ddt = torch.empty(dt.shape, dtype=dt.dtype, device=dev)
    if dt_bias is not None:
        dA, ddt_bias = _family(2, (nheads,), fused, **f32)
    else:
        dA, ddt_bias = torch.empty(nheads, **f32), empty()
    dD = torch.empty(D.shape, **f32) if D is not None else empty()
    if want_dinit:
        dinit_f, dinit_b = _family(2, (batch, nheads, headdim, dstate), fused, **f32)
    else:
        dinit_f, dinit_b = empty(), empty()
    ws, nbytes = _workspace(p, dev, "bwd")
    opt = lambda t, present: _ptr(t) if present else None
    args = _cabi.BwdArgs(p, _tensor4(x), _tensor4(B), _tensor4(C), _tensor4(z), _tensor4(dout),
                         _tensor4(out_x if z is not None else None),
                         _cabi.Tensor(dt.data_ptr(), dt.stride(0), dt.stride(1), dt.stride(2)),
                         _ptr(A32), _ptr(D32), _ptr(bias32), _ptr(dt_out), _ptr(cs_f), _ptr(cs_b), _ptr(states_f),
                         _ptr(states_b), _ptr(dx), opt(dz, z is not None), _ptr(dB), _ptr(dC), _ptr(ddt), _ptr(dA),
                         opt(dD, D is not None), opt(ddt_bias, dt_bias is not None), _ptr(dfinal_f), _ptr(dfinal_b),
                         opt(dinit_f, want_dinit), opt(dinit_b, want_dinit), _cabi.PHASE_ALL)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _cabi.check(lib.bissd_backward(ctypes.byref(args), ws.data_ptr(), nbytes, stream))
        _check_status(ws, stream)
    return dx, ddt, dA, dB, dC, dD, dz, ddt_bias, dinit_f, dinit_b


def _scan_bwd_impl(dout: torch.Tensor, x: torch.Tensor, dt: torch.Tensor, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor,
                   chunk_size: int, D: Optional[torch.Tensor], z: Optional[torch.Tensor], dt_bias: Optional[torch.Tensor],
                   out_x: Optional[torch.Tensor], dt_out: torch.Tensor, cs_f: torch.Tensor, cs_b: torch.Tensor,
                   states_f: torch.Tensor, states_b: torch.Tensor, dfinal_f: Optional[torch.Tensor],
                   dfinal_b: Optional[torch.Tensor], want_dinit: bool, dt_softplus: bool, dt_min: float,
                   dt_max: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                                           torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return _scan_bwd_core(dout, x, dt, A, B, C, chunk_size, D, z, dt_bias, out_x, dt_out, cs_f, cs_b, states_f, states_b,
                          dfinal_f, dfinal_b, want_dinit, dt_softplus, dt_min, dt_max, False)


def _scan_bwd_eager(*args):
    return _scan_bwd_core(*args, True)


scan_bwd = torch.library.custom_op("bissd::scan_bwd", _scan_bwd_impl, mutates_args=())


def _ops():
    """(forward, backward) callables: the registered custom ops while torch.compile is tracing, else the plain
    implementations."""
    if torch.compiler.is_compiling():
        return scan_fwd, scan_bwd
    return _scan_fwd_eager, _scan_bwd_eager


@scan_bwd.register_fake
def _(dout, x, dt, A, B, C, chunk_size, D, z, dt_bias, out_x, dt_out, cs_f, cs_b, states_f, states_b, dfinal_f,
      dfinal_b, want_dinit, dt_softplus, dt_min, dt_max):
    dev = x.device
    f32 = dict(dtype=torch.float32, device=dev)
    e = lambda dtype=torch.float32: torch.empty(0, dtype=dtype, device=dev)
    fin = (x.shape[0], x.shape[2], x.shape[3], B.shape[3])
    return (torch.empty_like(x), torch.empty(dt.shape, dtype=dt.dtype, device=dev), torch.empty(x.shape[2], **f32),
            torch.empty_like(B), torch.empty_like(C), torch.empty(D.shape, **f32) if D is not None else e(),
            torch.empty_like(x) if z is not None else e(x.dtype),
            torch.empty(x.shape[2], **f32) if dt_bias is not None else e(),
            torch.empty(fin, **f32) if want_dinit else e(), torch.empty(fin, **f32) if want_dinit else e())


# ----------------------------------------------------------------------------------------------------------------
# reference-compatible surface
# ----------------------------------------------------------------------------------------------------------------
def _check_shapes(x, dt, A, B, C, chunk_size, D, z):
    # same conditions, same exception type as the reference (src/ssd/bi/ssd_combined.py:298-310)
    batch, seqlen, nheads, headdim = x.shape
    _, _, ngroups, dstate = B.shape
    assert nheads % ngroups == 0
    assert B.shape == (batch, seqlen, ngroups, dstate)
    assert dt.shape == (batch, seqlen, nheads)
    assert A.shape == (nheads,)
    assert C.shape == B.shape
    assert chunk_size >= 32, "chunk_size must be >= 32"
    if z is not None:
        assert z.shape == x.shape
    if D is not None:
        assert D.shape == (nheads, headdim) or D.shape == (nheads,)


def _mamba_chunk_scan_combined_fwd(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, dt_softplus=False,
                                   dt_limit=(0.0, float("inf")), initial_states_f=None, initial_states_b=None):
    """Same 9-tuple as the reference (src/ssd/bi/ssd_combined.py:331):
    out, out_x, dt, dA_cumsum_f, dA_cumsum_b, states_f, states_b, final_states_f, final_states_b."""
    _check_shapes(x, dt, A, B, C, chunk_size, D, z)
    out, out_x, dt_out, cs_f, cs_b, st_f, st_b, fin_f, fin_b = _ops()[0](
        x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states_f, initial_states_b, dt_softplus,
        float(dt_limit[0]), float(dt_limit[1]))
    return out, (out_x if z is not None else None), dt_out, cs_f, cs_b, st_f, st_b, fin_f, fin_b


def _mamba_chunk_scan_combined_bwd(dout, x, dt, A, B, C, out, chunk_size, D=None, z=None, dt_bias=None,
                                   dfinal_states=None, dt_softplus=False, dt_limit=(0.0, float("inf")),
                                   dx=None, ddt=None, dB=None, dC=None, dz=None, recompute_output=False):
    """Same 8-tuple as the reference (src/ssd/bi/ssd_combined.py:473): dx, ddt, dA, dB, dC, dD, dz, ddt_bias.
    Like the reference it recomputes the forward intermediates from the raw inputs; `out` is only consulted
    through its recomputed pre-gate value."""
    _check_shapes(x, dt, A, B, C, chunk_size, D, z)
    assert dout.shape == x.shape
    fwd_op, bwd_op = _ops()
    fw = fwd_op(x, dt, A, B, C, chunk_size, D, z, dt_bias, None, None, dt_softplus, float(dt_limit[0]),
                float(dt_limit[1]))
    outz, out_x, dt_out, cs_f, cs_b, st_f, st_b = fw[:7]
    g = bwd_op(dout, x, dt, A, B, C, chunk_size, D, z, dt_bias, out_x if z is not None else None, dt_out, cs_f, cs_b,
                 st_f, st_b, None, None, False, dt_softplus, float(dt_limit[0]), float(dt_limit[1]))
    gdx, gddt, gdA, gdB, gdC, gdD, gdz, gbias = g[:8]
    for given, got in ((dx, gdx), (ddt, gddt), (dB, gdB), (dC, gdC), (dz, gdz)):
        if given is not None:
            given.copy_(got)
    res = (gdx if dx is None else dx, gddt if ddt is None else ddt, gdA, gdB if dB is None else dB,
           gdC if dC is None else dC, gdD.to(D.dtype) if D is not None else None,
           (gdz if dz is None else dz) if z is not None else None, gbias if dt_bias is not None else None)
    return res if not recompute_output else (*res, outz)


class MambaChunkScanCombinedFn(torch.autograd.Function):
    """Autograd wrapper with the argument order of the reference class (src/ssd/bi/ssd_combined.py:555-574), plus
    two optional trailing arguments (incoming boundary states) used by the sequence-sharded driver."""

    @staticmethod
    def forward(ctx, x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, dt_softplus=False,
                dt_limit=(0.0, float("inf")), return_final_states=False, initial_states_f=None, initial_states_b=None):
        _check_shapes(x, dt, A, B, C, chunk_size, D, z)
        out, out_x, dt_out, cs_f, cs_b, st_f, st_b, fin_f, fin_b = _ops()[0](
            x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states_f, initial_states_b, dt_softplus,
            float(dt_limit[0]), float(dt_limit[1]))
        ctx.save_for_backward(out_x if z is not None else None, x, dt, dt_out, cs_f, cs_b, st_f, st_b, A, B, C, D, z,
                              dt_bias)
        ctx.dt_softplus = dt_softplus
        ctx.chunk_size = chunk_size
        ctx.dt_limit = dt_limit
        ctx.return_final_states = return_final_states
        ctx.has_init = initial_states_f is not None or initial_states_b is not None
        ctx.init_given = (initial_states_f is not None, initial_states_b is not None)
        if return_final_states:
            return out, fin_f, fin_b
        return out

    @staticmethod
    def backward(ctx, dout, *args):
        out_x, x, dt, dt_out, cs_f, cs_b, st_f, st_b, A, B, C, D, z, dt_bias = ctx.saved_tensors
        dfin_f = dfin_b = None
        if ctx.return_final_states:
            dfin_f, dfin_b = args[0], args[1]
        g = _ops()[1](dout, x, dt, A, B, C, ctx.chunk_size, D, z, dt_bias, out_x, dt_out, cs_f, cs_b, st_f, st_b,
                      dfin_f, dfin_b, ctx.has_init, ctx.dt_softplus, float(ctx.dt_limit[0]), float(ctx.dt_limit[1]))
        dx, ddt, dA, dB, dC, dD, dz, ddt_bias, dinit_f, dinit_b = g
        return (dx, ddt, dA.to(A.dtype), dB, dC, None,
                dD.to(D.dtype) if D is not None else None,
                dz if z is not None else None,
                ddt_bias.to(dt_bias.dtype) if dt_bias is not None else None,
                None, None, None,
                dinit_f if ctx.init_given[0] else None, dinit_b if ctx.init_given[1] else None)


def bimamba_chunk_scan_combined(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, dt_softplus=False,
                                dt_limit=(0.0, float("inf")), return_final_states=False,
                                initial_states_f=None, initial_states_b=None):
    """
    Argument:
        x: (batch, seqlen, nheads, headdim)
        dt: (batch, seqlen, nheads)
        A: (nheads)
        B: (batch, seqlen, ngroups, dstate)
        C: (batch, seqlen, ngroups, dstate)
        chunk_size: int, 32 ... 256 (the reference accepts any value >= 32; larger chunks are refused here with
            a libbissd shape error)
        D: (nheads, headdim) or (nheads,)
        z: (batch, seqlen, nheads, headdim)
        dt_bias: (nheads,)
        dt_softplus: Whether to apply softplus to dt
        return_final_states: also return (final_states_f, final_states_b), each (batch, nheads, headdim, dstate)
            fp32 - the forward scan's state after the last token and the reverse scan's state at token 0.
            Unlike the reference (src/ssd/bi/ssd_combined.py:571) their gradients are supported.
        initial_states_f / initial_states_b: optional (batch, nheads, headdim, dstate) states entering before
            token 0 (forward scan) and after the last token (reverse scan); not in the reference.
    Return:
        out: (batch, seqlen, nheads, headdim)
    """
    return MambaChunkScanCombinedFn.apply(x, dt, A, B, C, chunk_size, D, z, dt_bias, dt_softplus, dt_limit,
                                          return_final_states, initial_states_f, initial_states_b)
