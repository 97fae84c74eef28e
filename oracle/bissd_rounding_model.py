"""Rounding model of the bidirectional SSD chunk scan: the exact formulas of bissd_manual_backward.py, evaluated in
fp64, with a rounding to the 16-bit operand type inserted wherever an implementation stores or feeds a tensor-core
operand in that type.

THIS FILE IS TEST INFRASTRUCTURE (see bissd_oracle.py).  It answers one question on the CPU: how far from the exact
result do the reduced parameter gradients (dA, dD, ddt_bias) land when nothing but the unavoidable 16-bit operand
roundings is applied - and does an implementation that rounds in a few more places land measurably further?

Two placements are modelled:

* "reference" - where the reference's Triton kernels round (all accumulation fp32, modelled as exact):
    B * (decay * dt) -> x dtype before the chunk-state product    src/ssd/bi/ssd_chunk_state.py:241-244
    passed states -> C dtype                                        src/ssd/bi/ssd_combined.py:324-327
    C.B^T kept fp32;  CB * decay * dt -> x dtype (one rounding)     src/ssd/bi/ssd_chunk_scan.py:155-156
    out_x, out -> x dtype
    g = dout * silu(z) -> x dtype                                   src/ssd/bi/ssd_chunk_scan.py:357-440
    g * exp(cs) -> dout dtype before the state-gradient product     src/ssd/bi/ssd_chunk_scan.py:503-504
    passed state gradients -> x dtype                               src/ssd/bi/ssd_combined.py:396
    CB^T * decay -> x dtype before the product with g               src/ssd/bi/ssd_combined.py:59-232
    dCB -> 16-bit before the products with B / C                    src/ssd/bi/ssd_bmm.py:244-245
    the intra-chunk decay terms and the chunk-level <S, g> terms stay fp32

* "kernel" - the placement of this library's TMA-fed / persistent kernels, which differs in:
    x * (decay * dt) (not B * ...) -> x dtype before the chunk-state product
    C.B^T -> bf16 when it is written, then  bf16(CB) * weight -> x dtype   (two roundings where the reference has one)
    the chunk-level <S, g> terms use the 16-bit saved states
    the intra-chunk decay terms are row / column sums of  (g.x^T) * bf16(CB) * weight  rounded to bf16
"""
import torch
import torch.nn.functional as F

from .bissd_oracle import chunked_reference


def _rounder(dtype):
    def q(t):
        return t.to(dtype).to(torch.float64)
    return q


def rounded_forward_backward(x, dt, A, B, C, chunk_size, dout, D=None, z=None, dt_bias=None, dt_softplus=False,
                             placement="reference", cb_single_rounding=False):
    """x, B, C, z, dout are 16-bit tensors (their dtype is the operand type); returns out and the eight gradients as
    fp64 tensors carrying the modelled rounding noise.  `cb_single_rounding` (kernel placement only): form
    bf16(CB) * weight in fp32 and round once, instead of rounding the weight and the product separately."""
    assert placement in ("reference", "kernel")
    kern = placement == "kernel"
    cd = torch.float64
    q = _rounder(x.dtype)
    qcb = _rounder(torch.bfloat16)                                        # the kernels keep C.B^T in bf16 for both operand types
    b, L, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    R = H // G
    Q = chunk_size
    assert L % Q == 0
    nc = L // Q
    fw = chunked_reference(x, dt, A, B, C, Q, D=None, z=None, dt_bias=dt_bias, dt_softplus=dt_softplus,
                           compute_dtype=cd, return_intermediates=True)
    dt_out, cs_f, cs_b = fw["dt_out"], fw["cs_f"], fw["cs_b"]            # exact: fp32 in every implementation
    tot = cs_f[..., -1]
    xc = x.to(cd).view(b, nc, Q, H, P)
    Bc = B.to(cd).view(b, nc, Q, G, N)
    Cc = C.to(cd).view(b, nc, Q, G, N)
    Bh, Ch = Bc.repeat_interleave(R, dim=3), Cc.repeat_interleave(R, dim=3)
    wf = torch.exp(tot[..., None] - cs_f)
    wb = torch.exp(cs_b[..., :1] - cs_b)
    sf = (wf * dt_out).permute(0, 2, 3, 1)[..., None]                    # (b,nc,Q,H,1)
    sb = (wb * dt_out).permute(0, 2, 3, 1)[..., None]
    # ---- chunk states
    if kern:
        loc_f = torch.einsum("bclhp,bclhn->bchpn", q(xc * sf), Bh)
        loc_b = torch.einsum("bclhp,bclhn->bchpn", q(xc * sb), Bh)
    else:
        loc_f = torch.einsum("bclhp,bclhn->bchpn", xc, q(Bh * sf))
        loc_b = torch.einsum("bclhp,bclhn->bchpn", xc, q(Bh * sb))
    S_f, S_b = [None] * nc, [None] * nc
    run = torch.zeros(b, H, P, N, dtype=cd)
    for c in range(nc):
        S_f[c] = run
        run = torch.exp(tot[:, :, c])[..., None, None] * run + loc_f[:, c]
    run = torch.zeros(b, H, P, N, dtype=cd)
    for c in range(nc - 1, -1, -1):
        S_b[c] = run
        run = torch.exp(tot[:, :, c])[..., None, None] * run + loc_b[:, c]
    S_f32, S_b32 = torch.stack(S_f, 1), torch.stack(S_b, 1)               # fp32 states (exact here)
    S_f, S_b = q(S_f32), q(S_b32)                                         # as saved / fed to the tensor core
    # ---- masked-decay tile
    idx = torch.arange(Q)
    lower = idx[:, None] >= idx[None, :]
    upper = idx[:, None] <= idx[None, :]
    ninf = torch.tensor(float("-inf"), dtype=cd)
    Lf = torch.exp(torch.where(lower, cs_f[..., :, None] - cs_f[..., None, :], ninf))
    Lb = torch.exp(torch.where(upper, cs_b[..., :, None] - cs_b[..., None, :], ninf))
    CB = torch.einsum("bclgn,bcsgn->bcgls", Cc, Bc).repeat_interleave(R, dim=2).permute(0, 2, 1, 3, 4)   # (b,H,nc,l,s)
    wgt = (Lf + Lb) * dt_out[..., None, :]

    def tile(cb, w):
        if not kern:
            return q(cb * w)
        if cb_single_rounding:
            return q(qcb(cb) * w)
        return q(qcb(cb) * q(w))

    M = tile(CB, wgt)
    ef = torch.exp(cs_f).permute(0, 2, 3, 1)
    eb = torch.exp(cs_b).permute(0, 2, 3, 1)
    y = torch.einsum("bhcls,bcshp->bclhp", M, xc)
    y = y + torch.einsum("bclhn,bchpn->bclhp", Ch, S_f) * ef[..., None]
    y = y + torch.einsum("bclhn,bchpn->bclhp", Ch, S_b) * eb[..., None]
    y = y.reshape(b, L, H, P)
    xd = x.to(cd)
    if D is not None:
        Dd = D.to(cd)
        y = y + xd * (Dd[None, None, :, None] if Dd.dim() == 1 else Dd[None, None])
    res = {}
    out_x = q(y)
    do = dout.to(cd)
    if z is not None:
        zz = z.to(cd)
        sig = torch.sigmoid(zz)
        res["out"] = q(y * zz * sig)
        res["dz"] = q(do * out_x * sig * (1 + zz * (1 - sig)))
        g = q(do * zz * sig)
    else:
        res["out"] = out_x
        g = do
    if D is not None:
        gx = g * xd
        res["dD"] = gx.sum(dim=(0, 1, 3)) if D.dim() == 1 else gx.sum(dim=(0, 1))
    gc = g.view(b, nc, Q, H, P)
    # ---- state gradients and their recurrence
    Gf = torch.einsum("bclhp,bclhn->bchpn", q(gc * ef[..., None]), Ch)
    Gb = torch.einsum("bclhp,bclhn->bchpn", q(gc * eb[..., None]), Ch)
    E_f, E_b, dT_f, dT_b = [None] * nc, [None] * nc, [None] * nc, [None] * nc
    run = torch.zeros(b, H, P, N, dtype=cd)
    for c in range(nc - 1, -1, -1):
        E_f[c] = run
        dec = torch.exp(tot[:, :, c])
        dT_f[c] = dec * ((S_f if kern else S_f32)[:, c] * run).sum(dim=(-1, -2))
        run = dec[..., None, None] * run + Gf[:, c]
    run = torch.zeros(b, H, P, N, dtype=cd)
    for c in range(nc):
        E_b[c] = run
        dec = torch.exp(tot[:, :, c])
        dT_b[c] = dec * ((S_b if kern else S_b32)[:, c] * run).sum(dim=(-1, -2))
        run = dec[..., None, None] * run + Gb[:, c]
    E_f, E_b = q(torch.stack(E_f, 1)), q(torch.stack(E_b, 1))
    dT_f, dT_b = torch.stack(dT_f, 2), torch.stack(dT_b, 2)
    # ---- dx, ddt_out
    Mt = tile(CB, Lf + Lb)                                                # used transposed: sum_s Mt[s,l] g[s]
    acc = torch.einsum("bclhn,bchpn,bhcl->bclhp", Bh, E_f, wf) + torch.einsum("bclhn,bchpn,bhcl->bclhp", Bh, E_b, wb)
    acc = acc + torch.einsum("bhcsl,bcshp->bclhp", Mt, gc)
    dxc = acc * dt_out.permute(0, 2, 3, 1)[..., None]
    ddt_out = (acc * xc).sum(-1).permute(0, 3, 1, 2)
    dx = dxc.reshape(b, L, H, P)
    if D is not None:
        dx = dx + g * (Dd[None, None, :, None] if Dd.dim() == 1 else Dd[None, None])
    res["dx"] = q(dx)
    # ---- dB / dC state parts and the next / prev terms
    if kern:
        dBf = torch.einsum("bclhp,bchpn->bclhn", q(xc * sf), E_f)
        dBb = torch.einsum("bclhp,bchpn->bclhn", q(xc * sb), E_b)
        dCf = torch.einsum("bclhp,bchpn->bclhn", q(gc * ef[..., None]), S_f)
        dCb = torch.einsum("bclhp,bchpn->bclhn", q(gc * eb[..., None]), S_b)
    else:
        dBf = torch.einsum("bclhp,bchpn->bclhn", xc, E_f) * sf
        dBb = torch.einsum("bclhp,bchpn->bclhn", xc, E_b) * sb
        dCf = torch.einsum("bclhp,bchpn->bclhn", gc, S_f) * ef[..., None]
        dCb = torch.einsum("bclhp,bchpn->bclhn", gc, S_b) * eb[..., None]
    nf = (dBf * Bh).sum(-1).permute(0, 3, 1, 2)
    nb = (dBb * Bh).sum(-1).permute(0, 3, 1, 2)
    pf = (dCf * Ch).sum(-1).permute(0, 3, 1, 2)
    pb = (dCb * Ch).sum(-1).permute(0, 3, 1, 2)
    dB_states = (dBf + dBb).view(b, nc, Q, G, R, N).sum(4)
    dC_states = (dCf + dCb).view(b, nc, Q, G, R, N).sum(4)
    # ---- dCB and the intra-chunk decay terms
    G2 = torch.einsum("bclhp,bcshp->bhcls", gc, xc)
    dts = dt_out[..., None, :]
    dCB = q((G2 * dts * (Lf + Lb)).view(b, G, R, nc, Q, Q).sum(2).permute(0, 2, 1, 3, 4))
    CBw = qcb(CB) if kern else CB                                         # the kernels read the bf16 copy of C.B^T here too
    Wf = G2 * CBw * dts * Lf * (idx[:, None] > idx[None, :])
    Wb = G2 * CBw * dts * Lb * (idx[:, None] < idx[None, :])
    if kern:
        Wf, Wb = qcb(Wf), qcb(Wb)                                         # rounded to bf16 for the column-sum product
    Rf = torch.cumsum(Wf, dim=-1) - Wf
    da_f = (Rf * lower).sum(dim=-2)
    Rb = torch.flip(torch.cumsum(torch.flip(Wb, [-1]), -1), [-1]) - Wb
    da_b = (Rb * upper).sum(dim=-2)
    dBc = torch.einsum("bcgls,bclgn->bcsgn", dCB, Cc) + dB_states
    dCc = torch.einsum("bcgls,bcsgn->bclgn", dCB, Bc) + dC_states
    res["dB"] = q(dBc.reshape(b, L, G, N))
    res["dC"] = q(dCc.reshape(b, L, G, N))
    # ---- assemble d(a), through the discretisation
    pf2 = pf.clone()
    pf2[..., -1] += dT_f
    pb2 = pb.clone()
    pb2[..., 0] += dT_b
    prev_f = torch.flip(torch.cumsum(torch.flip(pf2, [-1]), -1), [-1])
    prev_b = torch.cumsum(pb2, -1)
    next_f = torch.cumsum(nf, -1) - nf
    next_b = torch.flip(torch.cumsum(torch.flip(nb, [-1]), -1), [-1]) - nb
    ddA = da_f + da_b + next_f + next_b + prev_f + prev_b
    ddelta = ddA * A.to(cd)[None, :, None, None] + ddt_out
    ddelta = ddelta.permute(0, 2, 3, 1).reshape(b, L, H)
    pre = dt.to(cd)
    if dt_bias is not None:
        pre = pre + dt_bias.to(cd)
    ddt = ddelta
    if dt_softplus:
        ddt = torch.where(pre <= 20.0, ddt * torch.sigmoid(pre), ddt)
    res["ddt"] = ddt
    res["dA"] = (ddA * dt_out).sum(dim=(0, 2, 3))
    if dt_bias is not None:
        res["ddt_bias"] = ddt.sum(dim=(0, 1))
    return res


def reduced_gradient_scales(x, dt, A, B, C, chunk_size, dout, D=None, z=None, dt_bias=None, dt_softplus=False,
                            dt_limit=(0.0, float("inf"))):
    """Sum of the MAGNITUDES of the terms behind each reduced parameter gradient, per head, in fp64:
        dA[h]       = sum_{b,l} ddA[b,l,h] * Delta[b,l,h]          ->  sum |ddA * Delta|
        dD[h(,p)]   = sum_{b,l(,p)} g[b,l,h,p] * x[b,l,h,p]        ->  sum |g * x|
        ddt_bias[h] = sum_{b,l} ddt[b,l,h]                          ->  sum |ddt|
    A reduced gradient whose value is much smaller than this scale is an ill-conditioned sum: rounding noise of
    relative size u on the terms shows up as u * scale / |value| on the result."""
    from .bissd_manual_backward import manual_backward
    cd = torch.float64
    m = manual_backward(x, dt, A, B, C, chunk_size, dout, D=D, z=z, dt_bias=dt_bias, dt_softplus=dt_softplus,
                        dt_limit=dt_limit)
    fw = chunked_reference(x, dt, A, B, C, chunk_size, dt_bias=dt_bias, dt_softplus=dt_softplus, dt_limit=dt_limit,
                           compute_dtype=cd, return_intermediates=True)
    scales = {"dA": (m["ddA"] * fw["dt_out"]).abs().sum(dim=(0, 2, 3))}
    if D is not None:
        g = dout.to(cd) if z is None else dout.to(cd) * F.silu(z.to(cd))
        gx = (g * x.to(cd)).abs()
        scales["dD"] = gx.sum(dim=(0, 1, 3)) if D.dim() == 1 else gx.sum(dim=(0, 1))
    if dt_bias is not None:
        scales["ddt_bias"] = m["ddt"].abs().sum(dim=(0, 1))
    return scales


# 16-bit operands carry 8 (bf16) or 11 (fp16) significand bits; the kernels keep C.B^T in bf16 for both, so one unit
# in the last place of bf16 is the noise scale of a term.
TERM_NOISE = 2.0 ** -8


def reduced_gradient_ok(got, ref, scale, tol):
    """The acceptance rule for dA / dD / ddt_bias in 16-bit:  |got - ref| <= max(tol * max|ref|, TERM_NOISE * max scale).
    The first bound is the stated tolerance; the second takes over only when the sum is ill-conditioned
    (sum of magnitudes more than tol / TERM_NOISE = 5 times the value at tol = 2e-2)."""
    err = (got.detach().double().cpu() - ref.detach().double().cpu()).abs().max().item()
    bound = max(tol * ref.abs().max().item(), TERM_NOISE * scale.abs().max().item())
    return err <= bound, err, bound
