"""Sequence sharding: the boundary-state algebra between ranks.

CPU part (world_size-2 gloo processes): every rank evaluates its shard with the oracle standing in for the kernels,
exchanges boundary states with one packed all-gather per pass and chains them with the functions the GPU driver
uses (ssd.bi.sequence_parallel.gather_packed, chain_*_stacked) and must reproduce the unsharded oracle - outputs and gradients.

GPU part (one GPU, ranks emulated one after the other in one process): the phased C-ABI calls
(BISSD_PHASE_LOCAL / BISSD_PHASE_FINISH) with chained boundaries against the unsharded operator.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.bissd_manual_backward import manual_backward
from oracle.bissd_oracle import dense_reference, max_rel_err, reference_with_grads


def _problem(seed=0, b=1, L=128, H=2, P=4, G=1, N=8):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    x, B, C, dout = mk(b, L, H, P), mk(b, L, G, N), mk(b, L, G, N), mk(b, L, H, P)
    dt = torch.rand(b, L, H, generator=g, dtype=torch.float64) * 0.2
    A = -torch.rand(H, generator=g, dtype=torch.float64) - 0.5
    D = mk(H)
    return x, dt, A, B, C, D, dout


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ssd.bi.sequence_parallel import chain_backward_stacked, chain_forward_stacked, gather_packed
        x, dt, A, B, C, D, dout = _problem()
        Q, L = 32, x.shape[1]
        sl = slice(rank * L // world, (rank + 1) * L // world)
        xs, dts, Bs, Cs, gs = x[:, sl], dt[:, sl], B[:, sl], C[:, sl], dout[:, sl]
        # forward, LOCAL: finals from zero incoming state + log total decay
        _, Ff, Fb = dense_reference(xs, dts, A, Bs, Cs, D=D, return_final_states=True)
        ld = (dts * A).sum(dim=1)
        Ff_all, Fb_all, lds = gather_packed([Ff, Fb, ld], None)          # one collective, as the GPU driver does
        init_f, init_b = chain_forward_stacked(Ff_all, Fb_all, lds, rank)
        out = dense_reference(xs, dts, A, Bs, Cs, D=D, initial_states_f=init_f, initial_states_b=init_b)
        # backward, LOCAL: gradient w.r.t. the incoming states with zero gradient of the outgoing ones
        loc = manual_backward(xs, dts, A, Bs, Cs, Q, gs, D=D, initial_states_f=init_f, initial_states_b=init_b)
        gf_all, gb_all = gather_packed([loc["dinit_f"], loc["dinit_b"]], None)
        dfinal_f, dfinal_b = chain_backward_stacked(gf_all, gb_all, lds, rank)
        fin = manual_backward(xs, dts, A, Bs, Cs, Q, gs, D=D, initial_states_f=init_f, initial_states_b=init_b,
                              dfinal_f=dfinal_f, dfinal_b=dfinal_b)
        # parameter gradients are partial sums over ranks
        dA, dD = fin["dA"].clone(), fin["dD"].clone()
        dist.all_reduce(dA)
        dist.all_reduce(dD)
        full = reference_with_grads(x, dt, A, B, C, Q, dout, D=D, dense=True)
        errs = dict(out=max_rel_err(out, full["out"][:, sl]), dx=max_rel_err(fin["dx"], full["dx"][:, sl]),
                    ddt=max_rel_err(fin["ddt"], full["ddt"][:, sl]), dB=max_rel_err(fin["dB"], full["dB"][:, sl]),
                    dC=max_rel_err(fin["dC"], full["dC"][:, sl]), dA=max_rel_err(dA, full["dA"]),
                    dD=max_rel_err(dD, full["dD"]))
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_boundary_chaining_reproduces_unsharded_result_gloo(world):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0
    for r in range(world):
        assert all(v < 1e-10 for v in ret[r].values()), (r, dict(ret[r]))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-3), (torch.bfloat16, 2e-2)])
def test_phased_calls_with_chained_boundaries_match_unsharded_operator(dtype, tol):
    from ssd.bi import sequence_parallel as sp
    from ssd.bi.ssd_combined import bimamba_chunk_scan_combined
    W, b, L, H, P, G, N, Q = 4, 2, 1024, 4, 64, 2, 64, 128
    g = torch.Generator().manual_seed(3)
    mk = lambda *s: torch.randn(*s, generator=g)
    x, B, C, z, dout = (mk(b, L, H, P).to(dtype).cuda(), mk(b, L, G, N).to(dtype).cuda(), mk(b, L, G, N).to(dtype).cuda(),
                        mk(b, L, H, P).to(dtype).cuda(), mk(b, L, H, P).to(dtype).cuda())
    dt = (mk(b, L, H) - 4.0).cuda()
    A = (-torch.exp(torch.rand(H, generator=g) * 2.0)).cuda()
    D, bias = mk(H).cuda(), (-torch.rand(H, generator=g)).cuda()
    leaves = [t.clone().requires_grad_(True) for t in (x, dt, A, B, C, D, z, bias)]
    ref = bimamba_chunk_scan_combined(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], Q, D=leaves[5], z=leaves[6],
                                      dt_bias=leaves[7], dt_softplus=True)
    ref.backward(dout)
    sl = [slice(r * L // W, (r + 1) * L // W) for r in range(W)]
    shards = [sp.local_forward(x[:, s], dt[:, s], A, B[:, s], C[:, s], Q, D=D, z=z[:, s], dt_bias=bias, dt_softplus=True)
              for s in sl]
    Ff, Fb, ld = [s.final_f.clone() for s in shards], [s.final_b.clone() for s in shards], [s.log_decay for s in shards]
    outs = [sp.finish_forward(shards[r], *sp.chain_forward_boundaries(Ff, Fb, ld, r)) for r in range(W)]
    assert max_rel_err(torch.cat(outs, 1), ref) < tol
    loc = [sp.local_backward(shards[r], dout[:, sl[r]]) for r in range(W)]
    gf, gb = [t[0].clone() for t in loc], [t[1].clone() for t in loc]
    grads = [sp.finish_backward(shards[r], *sp.chain_backward_boundaries(gf, gb, ld, r)) for r in range(W)]
    cat = lambda i: torch.cat([gr[i] for gr in grads], 1)
    tot = lambda i: sum(gr[i] for gr in grads)
    got = dict(dx=cat(0), ddt=cat(1), dA=tot(2), dB=cat(3), dC=cat(4), dD=tot(5), dz=cat(6), ddt_bias=tot(7))
    want = dict(zip(("dx", "ddt", "dA", "dB", "dC", "dD", "dz", "ddt_bias"), (t.grad for t in leaves)))
    want = dict(dx=leaves[0].grad, ddt=leaves[1].grad, dA=leaves[2].grad, dB=leaves[3].grad, dC=leaves[4].grad,
                dD=leaves[5].grad, dz=leaves[6].grad, ddt_bias=leaves[7].grad)
    for k in got:
        assert max_rel_err(got[k], want[k]) < tol, k


def _nccl_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from ssd.bi.sequence_parallel import bimamba_chunk_scan_combined_seq_parallel
        from ssd.bi.ssd_combined import bimamba_chunk_scan_combined
        b, L, H, P, G, N, Q = 1, 2048, 4, 64, 2, 128, 256
        g = torch.Generator().manual_seed(5)
        mk = lambda *s: torch.randn(*s, generator=g)
        bf = torch.bfloat16
        x, B, C, dout = (mk(b, L, H, P).to(bf).cuda(), mk(b, L, G, N).to(bf).cuda(), mk(b, L, G, N).to(bf).cuda(),
                         mk(b, L, H, P).to(bf).cuda())
        dt = (mk(b, L, H) - 5.0).cuda()
        A = (-torch.exp(torch.rand(H, generator=g) * 2.0)).cuda()
        D = mk(H, P).cuda()
        full = [t.clone().requires_grad_(True) for t in (x, dt, A, B, C, D)]
        ref = bimamba_chunk_scan_combined(*full[:5], Q, D=full[5], dt_softplus=True)
        ref.backward(dout)
        sl = slice(rank * L // world, (rank + 1) * L // world)
        mine = [x[:, sl].clone().requires_grad_(True), dt[:, sl].clone().requires_grad_(True), A.clone().requires_grad_(True),
                B[:, sl].clone().requires_grad_(True), C[:, sl].clone().requires_grad_(True), D.clone().requires_grad_(True)]
        out = bimamba_chunk_scan_combined_seq_parallel(*mine[:5], Q, D=mine[5], dt_softplus=True)
        out.backward(dout[:, sl])
        dA, dD = mine[2].grad.clone(), mine[5].grad.clone()
        dist.all_reduce(dA)
        dist.all_reduce(dD)
        torch.cuda.synchronize()
        ret[rank] = dict(out=max_rel_err(out, ref[:, sl]), dx=max_rel_err(mine[0].grad, full[0].grad[:, sl]),
                         ddt=max_rel_err(mine[1].grad, full[1].grad[:, sl]), dB=max_rel_err(mine[3].grad, full[3].grad[:, sl]),
                         dC=max_rel_err(mine[4].grad, full[4].grad[:, sl]), dA=max_rel_err(dA, full[2].grad),
                         dD=max_rel_err(dD, full[5].grad))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_sequence_parallel_over_nccl_matches_single_gpu():
    """Real process group: one rank per GPU, boundary states exchanged with NCCL all-gather."""
    world = min(torch.cuda.device_count(), 8)        # 2048 tokens: one 256-token chunk per rank at 8 ranks
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_nccl_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    for r in range(world):
        assert all(v < 2e-2 for v in ret[r].values()), (r, dict(ret[r]))


@pytest.mark.gpu
def test_chain_kernel_matches_tensor_formulation():
    """bissd_chain_boundaries (one launch) against the torch formulation the CPU tests pin, forward and backward roles,
    including ranks whose decay underflows."""
    from ssd.bi import sequence_parallel as sp
    g = torch.Generator().manual_seed(2)
    W, b, H, P, N = 5, 2, 3, 8, 16
    left = torch.randn(W, b, H, P, N, generator=g).cuda()
    right = torch.randn(W, b, H, P, N, generator=g).cuda()
    ld = (-torch.rand(W, b, H, generator=g) * 3.0)
    ld[2, 0, 1] = -2000.0
    ld = ld.cuda()
    for rank in range(W):
        got_l, got_r = sp.chain_on_device(left, right, ld, rank)
        want_l, want_r = sp.chain_forward_stacked(left, right, ld, rank)
        assert max_rel_err(got_l, want_l) < 1e-5 and max_rel_err(got_r, want_r) < 1e-5, rank
        want_df, want_db = sp.chain_backward_stacked(right, left, ld, rank)   # (dinit_f, dinit_b) = (right, left)
        assert max_rel_err(got_r, want_df) < 1e-5 and max_rel_err(got_l, want_db) < 1e-5, rank
