"""Hand-derived backward of the bidirectional SSD chunk scan, phase by phase, on CPU.

THIS FILE IS TEST INFRASTRUCTURE (see bissd_oracle.py).  It restates, in plain PyTorch, the quantities each
backward CUDA kernel produces, so that (a) the derivation is checked against autograd of the oracle and (b) a
kernel can be compared with its own phase in isolation.  The phases follow the reference's backward chain
(src/ssd/bi/ssd_combined.py:334-475); names on the right are the reference functions computing the same
quantity.

Notation per (batch, head), chunk c, local index l in [0,Q):  Delta = dt_out, a = Delta*A,
cs_f[l] = sum_{j<=l} a_j, cs_b[l] = sum_{j>=l} a_j, T = cs_f[Q-1] = cs_b[0].
"""
import torch
import torch.nn.functional as F

from .bissd_oracle import chunked_reference


def manual_backward(x, dt, A, B, C, chunk_size, dout, D=None, z=None, dt_bias=None, dt_softplus=False,
                    dt_limit=(0.0, float("inf")), compute_dtype=torch.float64, dfinal_f=None, dfinal_b=None,
                    initial_states_f=None, initial_states_b=None):
    cd = compute_dtype
    b, L, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    R = H // G
    Q = chunk_size
    nc = (L + Q - 1) // Q
    pad = nc * Q - L
    fw = chunked_reference(x, dt, A, B, C, Q, D=D, z=z, dt_bias=dt_bias, dt_softplus=dt_softplus, dt_limit=dt_limit,
                           compute_dtype=cd, return_intermediates=True, initial_states_f=initial_states_f,
                           initial_states_b=initial_states_b)
    dt_out, cs_f, cs_b = fw["dt_out"], fw["cs_f"], fw["cs_b"]            # (b,H,nc,Q)
    S_f, S_b = fw["states_f"], fw["states_b"]                             # (b,nc,H,P,N) entering states
    tot = cs_f[..., -1]                                                   # (b,H,nc)

    def chunks(t, last):                                                  # (b,L,h,d) -> (b,nc,Q,h,d) zero padded
        t = t.to(cd)
        if pad:
            t = F.pad(t, (0, 0, 0, 0, 0, pad))
        return t.view(b, nc, Q, t.shape[2], last)

    xc, Bc, Cc = chunks(x, P), chunks(B, N), chunks(C, N)
    Bh, Ch = Bc.repeat_interleave(R, dim=3), Cc.repeat_interleave(R, dim=3)
    # ---- gate: g = d(out)/d(y)   (_chunk_scan_bwd_dz, src/ssd/bi/ssd_chunk_scan.py:357-440)
    do = dout.to(cd)
    res = {}
    if z is not None:
        zz = z.to(cd)
        sig = torch.sigmoid(zz)
        res["dz"] = do * fw["out_x"] * sig * (1 + zz * (1 - sig))
        g = do * zz * sig
    else:
        g = do
    if D is not None:
        gx = g * x.to(cd)
        res["dD"] = gx.sum(dim=(0, 1, 3)) if D.dim() == 1 else gx.sum(dim=(0, 1))
    gc = chunks(g, P)
    # ---- local state gradients (_chunk_scan_bwd_dstates, :457-522)
    ef = torch.exp(cs_f).permute(0, 2, 3, 1)                              # (b,nc,Q,H)
    eb = torch.exp(cs_b).permute(0, 2, 3, 1)
    Gf = torch.einsum("bclhp,bclh,bclhn->bchpn", gc, ef, Ch)
    Gb = torch.einsum("bclhp,bclh,bclhn->bchpn", gc, eb, Ch)
    # ---- state passing backward, both directions (_state_passing_bwd, src/ssd/bi/ssd_state_passing.py:106-187)
    # E_f[c] = gradient w.r.t. the local state of chunk c (forward direction), dT_f[c] = gradient w.r.t. T_c.
    E_f, E_b = [None] * nc, [None] * nc
    dT_f, dT_b = [None] * nc, [None] * nc
    run = torch.zeros(b, H, P, N, dtype=cd) if dfinal_f is None else dfinal_f.to(cd)
    for c in range(nc - 1, -1, -1):
        E_f[c] = run
        dec = torch.exp(tot[:, :, c])
        dT_f[c] = dec * (S_f[:, c] * run).sum(dim=(-1, -2))
        run = dec[..., None, None] * run + Gf[:, c]
    res["dinit_f"] = run
    run = torch.zeros(b, H, P, N, dtype=cd) if dfinal_b is None else dfinal_b.to(cd)
    for c in range(nc):
        E_b[c] = run
        dec = torch.exp(tot[:, :, c])
        dT_b[c] = dec * (S_b[:, c] * run).sum(dim=(-1, -2))
        run = dec[..., None, None] * run + Gb[:, c]
    res["dinit_b"] = run
    E_f, E_b = torch.stack(E_f, 1), torch.stack(E_b, 1)                   # (b,nc,H,P,N)
    dT_f, dT_b = torch.stack(dT_f, 2), torch.stack(dT_b, 2)               # (b,H,nc)
    # ---- decay tables
    wf = torch.exp(tot[..., None] - cs_f)                                 # e^{T-cs_f[l]}  (b,H,nc,Q)
    wb = torch.exp(cs_b[..., :1] - cs_b)                                  # e^{T-cs_b[l]}
    idx = torch.arange(Q)
    lower = idx[:, None] >= idx[None, :]
    upper = idx[:, None] <= idx[None, :]
    ninf = torch.tensor(float("-inf"), dtype=cd)
    Lf = torch.exp(torch.where(lower, cs_f[..., :, None] - cs_f[..., None, :], ninf))        # (b,H,nc,l,s), s<=l
    Lb = torch.exp(torch.where(upper, cs_b[..., :, None] - cs_b[..., None, :], ninf))        # s>=l
    CB = fw["CB"].repeat_interleave(R, dim=2).permute(0, 2, 1, 3, 4)                          # (b,H,nc,l,s)
    # ---- dx, ddt_out  (_chunk_scan_chunk_state_bwd_dx, src/ssd/bi/ssd_combined.py:59-232)
    acc = torch.einsum("bclhn,bchpn,bhcl->bclhp", Bh, E_f, wf) + torch.einsum("bclhn,bchpn,bhcl->bclhp", Bh, E_b, wb)
    acc = acc + torch.einsum("bhcsl,bcshp->bclhp", CB * (Lf + Lb), gc)    # sum_s CB[s,l] (Lf+Lb)[s,l] g[s]
    dxc = acc * dt_out.permute(0, 2, 3, 1)[..., None]
    ddt_out = (acc * xc).sum(-1).permute(0, 3, 1, 2)                      # (b,H,nc,Q)
    dx = dxc.reshape(b, nc * Q, H, P)[:, :L]
    if D is not None:
        Dd = D.to(cd)
        dx = dx + g * (Dd[None, None, :, None] if Dd.dim() == 1 else Dd[None, None])
    res["dx"] = dx
    # ---- dB (states part) + "next" decay terms (_chunk_state_bwd_db, src/ssd/bi/ssd_chunk_state.py:379-495)
    dBf = torch.einsum("bclhp,bchpn->bclhn", xc, E_f) * (dt_out * wf).permute(0, 2, 3, 1)[..., None]
    dBb = torch.einsum("bclhp,bchpn->bclhn", xc, E_b) * (dt_out * wb).permute(0, 2, 3, 1)[..., None]
    nf = (dBf * Bh).sum(-1).permute(0, 3, 1, 2)                           # (b,H,nc,Q)
    nb = (dBb * Bh).sum(-1).permute(0, 3, 1, 2)
    dB_states = (dBf + dBb).view(b, nc, Q, G, R, N).sum(4)
    # ---- dC (states part) + "prev" decay terms (_chunk_scan_bwd_dc, src/ssd/bi/ssd_chunk_scan.py:538-636)
    dCf = torch.einsum("bclhp,bchpn->bclhn", gc, S_f) * ef[..., None]
    dCb = torch.einsum("bclhp,bchpn->bclhn", gc, S_b) * eb[..., None]
    pf = (dCf * Ch).sum(-1).permute(0, 3, 1, 2)
    pb = (dCb * Ch).sum(-1).permute(0, 3, 1, 2)
    dC_states = (dCf + dCb).view(b, nc, Q, G, R, N).sum(4)
    # ---- dCB (_chunk_scan_bwd_dcb, :776-859) and the intra-chunk decay terms (:1361-1446, :1078-1157)
    G2 = torch.einsum("bclhp,bcshp->bhcls", gc, xc)                       # g[l].x[s]
    dts = dt_out[..., None, :]
    dCB_h = G2 * dts * (Lf + Lb)
    dCB = dCB_h.view(b, G, R, nc, Q, Q).sum(2).permute(0, 2, 1, 3, 4)     # (b,nc,G,l,s)
    Wf = G2 * CB * dts * Lf * (idx[:, None] > idx[None, :])               # strictly s<l
    Wb = G2 * CB * dts * Lb * (idx[:, None] < idx[None, :])               # strictly s>l
    # da_f[j] = sum_{l>=j} sum_{s<j} Wf[l,s] ;  da_b[j] = sum_{l<=j} sum_{s>j} Wb[l,s]
    Rf = torch.cumsum(Wf, dim=-1) - Wf                                    # exclusive prefix over s -> index j
    da_f = (Rf * lower).sum(dim=-2)                                       # rows l>=j
    Rb = torch.flip(torch.cumsum(torch.flip(Wb, [-1]), -1), [-1]) - Wb    # exclusive suffix over s -> index j
    da_b = (Rb * upper).sum(dim=-2)                                       # rows l<=j
    # ---- bmm backward (_bmm_chunk_bwd, src/ssd/bi/ssd_bmm.py:108-160)
    dBc = torch.einsum("bcgls,bclgn->bcsgn", dCB, Cc) + dB_states
    dCc = torch.einsum("bcgls,bcsgn->bclgn", dCB, Bc) + dC_states
    res["dB"] = dBc.reshape(b, nc * Q, G, N)[:, :L]
    res["dC"] = dCc.reshape(b, nc * Q, G, N)[:, :L]
    # ---- assemble d(a) (src/ssd/bi/ssd_combined.py:456-466)
    pf2 = pf.clone()
    pf2[..., -1] += dT_f
    pb2 = pb.clone()
    pb2[..., 0] += dT_b
    prev_f = torch.flip(torch.cumsum(torch.flip(pf2, [-1]), -1), [-1])   # reverse inclusive cumsum
    prev_b = torch.cumsum(pb2, -1)
    next_f = torch.cumsum(nf, -1) - nf                                    # exclusive cumsum
    next_b = torch.flip(torch.cumsum(torch.flip(nb, [-1]), -1), [-1]) - nb
    ddA = da_f + da_b + next_f + next_b + prev_f + prev_b                 # (b,H,nc,Q)
    # ---- through the discretisation (_chunk_cumsum_bwd, src/ssd/bi/ssd_chunk_state.py:106-170)
    ddelta = ddA * A.to(cd)[None, :, None, None] + ddt_out
    ddelta = ddelta.permute(0, 2, 3, 1).reshape(b, nc * Q, H)[:, :L]
    pre = dt.to(cd)
    if dt_bias is not None:
        pre = pre + dt_bias.to(cd)
    val = torch.where(pre <= 20.0, torch.log1p(torch.exp(torch.clamp(pre, max=20.0))), pre) if dt_softplus else pre
    clamped = (val < dt_limit[0]) | (val > dt_limit[1])
    ddt = torch.where(clamped, torch.zeros_like(ddelta), ddelta)
    if dt_softplus:
        ddt = torch.where(pre <= 20.0, ddt * torch.sigmoid(pre), ddt)
    res["ddt"] = ddt
    res["dA"] = (ddA * dt_out).sum(dim=(0, 2, 3))
    if dt_bias is not None:
        res["ddt_bias"] = ddt.sum(dim=(0, 1))
    res.update(E_f=E_f, E_b=E_b, dT_f=dT_f, dT_b=dT_b, Gf=Gf, Gb=Gb, ddt_out=ddt_out, nf=nf, nb=nb, pf=pf, pb=pb,
               da_f=da_f, da_b=da_b, Wf=Wf, Wb=Wb, dCB=dCB, ddA=ddA, dB_states=dB_states, dC_states=dC_states)
    return res
