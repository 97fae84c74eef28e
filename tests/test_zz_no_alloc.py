"""The forward entry point that runs on library-owned scratch (`bissd_forward_static_scratch`).

It exists for hosts that may not allocate device memory where they call the operator (a server that hands out
fixed buffers and bans cudaMalloc after start-up).  Called here through the C ABI with caller-owned inputs and
outputs only, twice in a row with different inputs - the second call meets the scratch as the first left it - and
compared with the ordinary entry point `bissd_forward` given a caller-allocated workspace (the same kernels run
in both, so the results must agree to the tolerance of the other GPU tests - in practice bit for bit) and, so that the
file stands on its own, with the CPU oracle.  The device status word of the library-owned scratch must read 0 after
each call, and the second call must not change the device's free memory.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _buffers(x, B, Q):
    b, L, H, P = x.shape
    N = B.shape[3]
    nc = math.ceil(L / Q)
    dev = x.device
    f32 = dict(dtype=torch.float32, device=dev)
    return dict(out=torch.zeros_like(x), out_x=torch.zeros_like(x),
                dt_out=torch.zeros(b, H, nc, Q, **f32), cs_f=torch.zeros(b, H, nc, Q, **f32),
                cs_b=torch.zeros(b, H, nc, Q, **f32),
                states_f=torch.zeros(b, nc, H, P, N, dtype=x.dtype, device=dev),
                states_b=torch.zeros(b, nc, H, P, N, dtype=x.dtype, device=dev),
                final_f=torch.zeros(b, H, P, N, **f32), final_b=torch.zeros(b, H, P, N, **f32))


def _args(_cabi, inp, Q, buf):
    x, dt, A, B, C, D, z, bias = (inp[k] for k in ("x", "dt", "A", "B", "C", "D", "z", "dt_bias"))
    b, L, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    code = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}
    prob = _cabi.Problem(b, L, H, P, G, N, Q, code[x.dtype], code[dt.dtype], 1, 0, 1, 1, 1, 0.0, float("inf"))
    t4 = lambda t: _cabi.Tensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))
    return _cabi.FwdArgs(prob, t4(x), t4(B), t4(C), t4(z), t4(dt), A.data_ptr(), D.data_ptr(), bias.data_ptr(),
                         t4(buf["out"]), t4(buf["out_x"]), buf["dt_out"].data_ptr(), buf["cs_f"].data_ptr(),
                         buf["cs_b"].data_ptr(), buf["states_f"].data_ptr(), buf["states_b"].data_ptr(),
                         buf["final_f"].data_ptr(), buf["final_b"].data_ptr(), None, None, _cabi.PHASE_ALL), prob


def _inputs(seed, shape, dtype):
    b, L, H, P, G, N = shape
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g)
    return {k: v.cuda() for k, v in dict(
        x=mk(b, L, H, P).to(dtype), dt=mk(b, L, H) - 4.0, A=-torch.exp(torch.rand(H, generator=g) * 2.7),
        B=mk(b, L, G, N).to(dtype), C=mk(b, L, G, N).to(dtype), D=mk(H), z=mk(b, L, H, P).to(dtype),
        dt_bias=-torch.rand(H, generator=g)).items()}


@pytest.mark.parametrize("dtype,shape,Q", [(torch.bfloat16, (1, 512, 4, 64, 1, 128), 256),
                                           (torch.float32, (2, 200, 2, 16, 1, 24), 64)])
def test_static_scratch_forward_matches_workspace_forward(dtype, shape, Q):
    from ssd import _cabi
    lib = _cabi.load()
    stream = torch.cuda.current_stream().cuda_stream
    for call, seed in enumerate((1, 2)):                 # two calls in a row on the shared scratch
        inp = _inputs(seed, shape, dtype)
        ref_buf, new_buf = _buffers(inp["x"], inp["B"], Q), _buffers(inp["x"], inp["B"], Q)
        ref_args, prob = _args(_cabi, inp, Q, ref_buf)
        need = ctypes.c_size_t(0)
        _cabi.check(lib.bissd_workspace_bytes(ctypes.byref(prob), ctypes.byref(need), None))
        assert need.value <= _cabi.STATIC_SCRATCH_BYTES
        ws = torch.empty(need.value, dtype=torch.uint8, device="cuda")
        _cabi.check(lib.bissd_forward(ctypes.byref(ref_args), ws.data_ptr(), need.value, stream))
        new_args, _ = _args(_cabi, inp, Q, new_buf)
        if call == 1:                                    # the second call must leave the device's free memory alone
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
        _cabi.check(lib.bissd_forward_static_scratch(ctypes.byref(new_args), stream))
        torch.cuda.synchronize()
        if call == 1:
            assert torch.cuda.mem_get_info()[0] == free_before, "the no-allocation entry point changed free device memory"
        status = ctypes.c_int(-1)
        _cabi.check(lib.bissd_read_status(None, stream, ctypes.byref(status)))   # NULL = the library-owned scratch
        assert status.value == 0, f"device status word {status.value}: a bounded device-side wait ran out"
        tol = 1e-3 if dtype == torch.float32 else 2e-2
        for k in ref_buf:
            a, r = new_buf[k].float(), ref_buf[k].float()
            assert torch.isfinite(a).all(), (call, k)
            err = (a - r).abs().max().item() / max(r.abs().max().item(), 1e-30)
            assert err <= tol, (call, k, err)
        from oracle.bissd_oracle import chunked_reference, max_rel_err
        c = {k: v.cpu() for k, v in inp.items()}
        want = chunked_reference(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, D=c["D"], z=c["z"], dt_bias=c["dt_bias"],
                                 dt_softplus=True)
        assert max_rel_err(new_buf["out"], want) <= tol, call


def test_static_scratch_refuses_oversized_problem():
    from ssd import _cabi
    lib = _cabi.load()
    inp = _inputs(3, (1, 256, 2, 16, 1, 16), torch.float32)
    buf = _buffers(inp["x"], inp["B"], 64)
    args, _ = _args(_cabi, inp, 64, buf)
    args.p.batch, args.p.seqlen, args.p.nheads, args.p.headdim, args.p.dstate = 8, 2048, 24, 64, 128   # 117 MB scratch
    assert lib.bissd_forward_static_scratch(ctypes.byref(args), None) == _cabi.ERR_TOO_LARGE
    assert b"scratch" in lib.bissd_strerror(_cabi.ERR_TOO_LARGE)
