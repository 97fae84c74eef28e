"""CPU oracle for the bidirectional SSD chunk scan  y = SS(x) + flip(SS(flip(x))) + D*x  (optionally gated by z).

THIS FILE IS TEST INFRASTRUCTURE.  It is the checker for the CUDA path; only the test-suite, the smoke test
and the CPU-baseline leg of the benchmark may import it.  The shipped operator never calls into it.

Parity status: PINNED.  `tests/golden/*.npz` hold outputs of the reference implementation itself (its Triton
kernels executed by Triton's CPU interpreter, and its pure-PyTorch path), produced by
`tests/golden/make_golden.py`; `tests/test_oracle.py` checks every function below against them.

Two evaluators of the same formula are provided:

* `dense_reference`   - the O(L^2) definition, no chunking at all.  Ground truth for L <= ~1024.
* `chunked_reference` - a restatement of the reference's pure-PyTorch chunked path
  (`src/ssd/uni/ssd_combined.py:621-659` -> `src/ssd/uni/ssd_chunk_state.py:964-992`,
  `src/ssd/uni/ssd_state_passing.py:326-347`, `src/ssd/uni/ssd_chunk_scan.py:1791-1832`), composed for both
  directions as the bi operator does (`src/ssd/bi/ssd_combined.py:297-331`).  It differs from the reference
  text in one deliberate way: the causal mask is applied INSIDE the exponent (fill -inf, then exp) instead of
  after it, which is the same function but has finite gradients (the reference's order yields 0*inf = NaN in
  autograd for realistic decays).  It exposes every intermediate the CUDA kernels produce.

Gradients come from autograd on these evaluators.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def _softplus_ref(v: torch.Tensor) -> torch.Tensor:
    # src/ssd/bi/softplus.py:8-11 : identity above 20, log(exp(v)+1) below.
    return torch.where(v <= 20.0, torch.log1p(torch.exp(torch.clamp(v, max=20.0))), v)


def discretize(dt, A, dt_bias=None, dt_softplus=False, dt_limit=(0.0, float("inf")), compute_dtype=torch.float64):
    """dt (b,L,H) -> Delta (b,L,H), a = Delta*A (b,L,H).  Follows _chunk_cumsum_fwd_kernel
    (src/ssd/bi/ssd_chunk_state.py:75-86): bias, softplus, clamp - in this order."""
    d = dt.to(compute_dtype)
    if dt_bias is not None:
        d = d + dt_bias.to(compute_dtype)
    if dt_softplus:
        d = _softplus_ref(d)
    lo, hi = dt_limit
    # the kernel always applies min(max(dt, dt_min), dt_max), also for the default (0, inf)
    # (src/ssd/bi/ssd_chunk_state.py:83); the gradient is zero where the clamp is active (:157-162).
    d = torch.clamp(d, min=lo, max=hi)
    a = d * A.to(compute_dtype)
    return d, a


def dense_reference(x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False,
                    dt_limit=(0.0, float("inf")), compute_dtype=torch.float64,
                    return_final_states=False, initial_states_f=None, initial_states_b=None):
    """O(L^2) evaluation of
        y_t = sum_{s<=t} (C_t.B_s) exp(sum_{r=s+1..t} a_r) Delta_s x_s
            + sum_{s>=t} (C_t.B_s) exp(sum_{r=t..s-1} a_r) Delta_s x_s  + D x_t ,  out = y * silu(z).
    The s == t term is counted once per direction (README.md:15; inclusive masks at
    src/ssd/bi/ssd_chunk_scan.py:140,143).  Shapes as in bimamba_chunk_scan_combined
    (src/ssd/bi/ssd_combined.py:577-593).  initial_states_f enters before token 0, initial_states_b after
    token L-1 (an extension the reference lacks; used to check sequence sharding)."""
    b, L, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    R = H // G
    cd = compute_dtype
    xd, Bd, Cd = x.to(cd), B.to(cd), C.to(cd)
    delta, a = discretize(dt, A, dt_bias, dt_softplus, dt_limit, cd)
    cs = torch.cumsum(a, dim=1)                                  # (b,L,H) inclusive
    # forward direction exponent E_f[t,s] = cs[t]-cs[s] (s<=t); reverse E_b[t,s] = (cs[s]-a[s]) - (cs[t]-a[t]) (s>=t)
    csx = cs - a                                                 # exclusive cumsum
    Ef = cs.unsqueeze(2) - cs.unsqueeze(1)                       # (b,t,s,H)
    Eb = csx.unsqueeze(1) - csx.unsqueeze(2)                     # (b,t,s,H)
    idx = torch.arange(L)
    lower = (idx[:, None] >= idx[None, :])[None, :, :, None]
    upper = (idx[:, None] <= idx[None, :])[None, :, :, None]
    neg_inf = torch.tensor(float("-inf"), dtype=cd)
    Lmat = torch.exp(torch.where(lower, Ef, neg_inf)) + torch.exp(torch.where(upper, Eb, neg_inf))   # (b,t,s,H)
    CB = torch.einsum("btgn,bsgn->btsg", Cd, Bd).repeat_interleave(R, dim=3)                        # (b,t,s,H)
    M = CB * Lmat * delta.unsqueeze(1)
    y = torch.einsum("btsh,bshp->bthp", M, xd)
    Bh = Bd.repeat_interleave(R, dim=2)
    Ch = Cd.repeat_interleave(R, dim=2)
    if initial_states_f is not None:
        y = y + torch.einsum("bthn,bhpn->bthp", Ch, initial_states_f.to(cd)) * torch.exp(cs).unsqueeze(-1)
    if initial_states_b is not None:
        tot = cs[:, -1:, :]
        y = y + torch.einsum("bthn,bhpn->bthp", Ch, initial_states_b.to(cd)) * torch.exp(tot - csx).unsqueeze(-1)
    if D is not None:
        Dd = D.to(cd)
        y = y + xd * (Dd[None, None, :, None] if Dd.dim() == 1 else Dd[None, None])
    out_x = y
    out = y if z is None else y * F.silu(z.to(cd))
    if not return_final_states:
        return out
    # final_f = state after the last token; final_b = state of the reverse scan at token 0
    tot = cs[:, -1:, :]
    wf = torch.exp(tot - cs) * delta                              # decay from s (exclusive) to the end
    wb = torch.exp(csx) * delta                                   # decay from the start to s (exclusive)
    final_f = torch.einsum("bsh,bshp,bshn->bhpn", wf, xd, Bh)
    final_b = torch.einsum("bsh,bshp,bshn->bhpn", wb, xd, Bh)
    if initial_states_f is not None:
        final_f = final_f + initial_states_f.to(cd) * torch.exp(tot[:, 0])[..., None, None]
    if initial_states_b is not None:
        final_b = final_b + initial_states_b.to(cd) * torch.exp(tot[:, 0])[..., None, None]
    return out, final_f, final_b


def chunked_reference(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, dt_softplus=False,
                      dt_limit=(0.0, float("inf")), compute_dtype=torch.float64, return_intermediates=False,
                      initial_states_f=None, initial_states_b=None):
    """Chunked evaluation with every intermediate of the reference's forward chain
    (src/ssd/bi/ssd_combined.py:321-331).  Ragged tails (L % Q != 0) are zero-padded like the reference kernels
    do (src/ssd/bi/ssd_chunk_state.py:73,84)."""
    b, L, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    R = H // G
    Q = chunk_size
    nc = (L + Q - 1) // Q
    pad = nc * Q - L
    cd = compute_dtype
    delta, a = discretize(dt, A, dt_bias, dt_softplus, dt_limit, cd)
    xd, Bd, Cd = x.to(cd), B.to(cd), C.to(cd)
    if pad:
        delta = F.pad(delta, (0, 0, 0, pad))
        a = F.pad(a, (0, 0, 0, pad))
        xd = F.pad(xd, (0, 0, 0, 0, 0, pad))
        Bd = F.pad(Bd, (0, 0, 0, 0, 0, pad))
        Cd = F.pad(Cd, (0, 0, 0, 0, 0, pad))
    dt_out = delta.view(b, nc, Q, H).permute(0, 3, 1, 2)            # (b,H,nc,Q)   src/ssd/bi/ssd_chunk_state.py:85
    ac = a.view(b, nc, Q, H).permute(0, 3, 1, 2)
    cs_f = torch.cumsum(ac, dim=-1)                                 # :88
    cs_b = torch.flip(torch.cumsum(torch.flip(ac, [-1]), dim=-1), [-1])   # :91
    xc = xd.view(b, nc, Q, H, P)
    Bc = Bd.view(b, nc, Q, G, N).repeat_interleave(R, dim=3)        # (b,nc,Q,H,N)
    Cc = Cd.view(b, nc, Q, G, N).repeat_interleave(R, dim=3)
    tot = cs_f[..., -1]                                             # (b,H,nc) == cs_b[...,0]
    # local chunk states, both directions (src/ssd/bi/ssd_chunk_state.py:187-263; uni ref :964-992)
    w_f = torch.exp(tot[..., None] - cs_f) * dt_out                 # (b,H,nc,Q)
    w_b = torch.exp(cs_b[..., :1] - cs_b) * dt_out
    loc_f = torch.einsum("bhcl,bclhp,bclhn->bchpn", w_f, xc, Bc)
    loc_b = torch.einsum("bhcl,bclhp,bclhn->bchpn", w_b, xc, Bc)
    # state passing (src/ssd/bi/ssd_state_passing.py:27-92); S_f[c] enters chunk c from the left,
    # S_b[c] enters chunk c from the right.
    S_f = [None] * nc
    S_b = [None] * nc
    run = torch.zeros(b, H, P, N, dtype=cd) if initial_states_f is None else initial_states_f.to(cd)
    for c in range(nc):
        S_f[c] = run
        run = torch.exp(tot[:, :, c])[..., None, None] * run + loc_f[:, c]
    final_f = run
    run = torch.zeros(b, H, P, N, dtype=cd) if initial_states_b is None else initial_states_b.to(cd)
    for c in range(nc - 1, -1, -1):
        S_b[c] = run
        run = torch.exp(tot[:, :, c])[..., None, None] * run + loc_b[:, c]
    final_b = run
    S_f = torch.stack(S_f, dim=1)                                   # (b,nc,H,P,N)
    S_b = torch.stack(S_b, dim=1)
    # chunk scan (src/ssd/bi/ssd_chunk_scan.py:42-189; uni ref :1791-1832), mask inside the exponent
    CB = torch.einsum("bclgn,bcsgn->bcgls", Cd.view(b, nc, Q, G, N), Bd.view(b, nc, Q, G, N))     # (b,nc,G,Q,Q)
    idx = torch.arange(Q)
    lower = idx[:, None] >= idx[None, :]
    upper = idx[:, None] <= idx[None, :]
    neg_inf = torch.tensor(float("-inf"), dtype=cd)
    seg_f = cs_f[..., :, None] - cs_f[..., None, :]                 # (b,H,nc,l,s)
    seg_b = cs_b[..., :, None] - cs_b[..., None, :]
    Lmat = torch.exp(torch.where(lower, seg_f, neg_inf)) + torch.exp(torch.where(upper, seg_b, neg_inf))
    M = CB.repeat_interleave(R, dim=2).permute(0, 2, 1, 3, 4) * Lmat * dt_out[..., None, :]       # (b,H,nc,l,s)
    y = torch.einsum("bhcls,bcshp->bclhp", M, xc)
    y = y + torch.einsum("bclhn,bchpn->bclhp", Cc, S_f) * torch.exp(cs_f).permute(0, 2, 3, 1)[..., None]
    y = y + torch.einsum("bclhn,bchpn->bclhp", Cc, S_b) * torch.exp(cs_b).permute(0, 2, 3, 1)[..., None]
    y = y.reshape(b, nc * Q, H, P)[:, :L]
    if D is not None:
        Dd = D.to(cd)
        y = y + x.to(cd) * (Dd[None, None, :, None] if Dd.dim() == 1 else Dd[None, None])
    out_x = y
    out = y if z is None else y * F.silu(z.to(cd))
    if not return_intermediates:
        return out
    return dict(out=out, out_x=out_x, dt_out=dt_out, cs_f=cs_f, cs_b=cs_b, loc_f=loc_f, loc_b=loc_b,
                states_f=S_f, states_b=S_b, final_f=final_f, final_b=final_b, CB=CB)


def reference_with_grads(x, dt, A, B, C, chunk_size, dout, D=None, z=None, dt_bias=None, dt_softplus=False,
                         dt_limit=(0.0, float("inf")), compute_dtype=torch.float64, dense=False):
    """Forward + autograd backward of the oracle on (rounded) inputs.  Returns dict with out and the gradients
    the operator's backward returns (src/ssd/bi/ssd_combined.py:574): dx, ddt, dA, dB, dC, dD, dz, ddt_bias."""
    cd = compute_dtype
    leaves = {}
    for name, t in dict(x=x, dt=dt, A=A, B=B, C=C, D=D, z=z, dt_bias=dt_bias).items():
        leaves[name] = None if t is None else t.detach().to(cd).clone().requires_grad_(True)
    if dense:
        out = dense_reference(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], D=leaves["D"],
                              z=leaves["z"], dt_bias=leaves["dt_bias"], dt_softplus=dt_softplus, dt_limit=dt_limit,
                              compute_dtype=cd)
    else:
        out = chunked_reference(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], chunk_size,
                                D=leaves["D"], z=leaves["z"], dt_bias=leaves["dt_bias"], dt_softplus=dt_softplus,
                                dt_limit=dt_limit, compute_dtype=cd)
    out.backward(dout.to(cd))
    res = dict(out=out.detach())
    for name, key in (("x", "dx"), ("dt", "ddt"), ("A", "dA"), ("B", "dB"), ("C", "dC"), ("D", "dD"), ("z", "dz"),
                      ("dt_bias", "ddt_bias")):
        res[key] = None if leaves[name] is None else leaves[name].grad
    return res


def max_rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max|got-ref| / max|ref| - the error metric used for every parity statement in this repository."""
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    denom = ref.abs().max().item()
    if denom == 0.0:
        return (got - ref).abs().max().item()
    return (got - ref).abs().max().item() / denom
