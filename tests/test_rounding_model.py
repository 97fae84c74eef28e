"""How well can ANY 16-bit implementation reproduce the reduced parameter gradients (dA, dD, ddt_bias)?

The rounding model (oracle/bissd_rounding_model.py) evaluates the exact formulas in fp64 and rounds to bf16 only
where an implementation stores or feeds a tensor-core operand in bf16 - once with the placement of the reference's
Triton kernels, once with the placement of this library's kernels.  On a small two-head problem the reduced
gradients are ill-conditioned sums (sum of magnitudes 5 - 400 times the value), and the reference's own placement
misses the 2e-2 bound on them for some seeds while every element-wise tensor stays far inside it.  These tests pin
that fact, and the acceptance rule the GPU tests apply to the reduced gradients on such shapes:
    |got - ref| <= max(2e-2 * max|ref|, 2^-8 * max over heads of sum|terms|).
"""
import math

import pytest
import torch

from oracle.bissd_oracle import max_rel_err, reference_with_grads
from oracle.bissd_rounding_model import (reduced_gradient_ok, reduced_gradient_scales, rounded_forward_backward)

SHAPE = (1, 512, 2, 64, 1, 128, 256)      # batch, seqlen, heads, headdim, groups, dstate, chunk
SEEDS = range(8)
ELEMENTWISE = ("out", "dx", "ddt", "dB", "dC", "dz")
REDUCED = ("dA", "dD", "ddt_bias")


def two_head_inputs(seed, shape=SHAPE, dtype=torch.bfloat16):
    b, L, H, P, G, N, Q = shape
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(b, L, H, P, generator=g).to(dtype)
    B = torch.randn(b, L, G, N, generator=g).to(dtype)
    C = torch.randn(b, L, G, N, generator=g).to(dtype)
    dt = torch.randn(b, L, H, generator=g) - 4.0
    A = -torch.exp(torch.rand(H, generator=g) * 2.7)
    D = torch.randn(H, generator=g)
    z = torch.randn(b, L, H, P, generator=g).to(dtype)
    bias = -torch.rand(H, generator=g)
    dout = torch.randn(b, L, H, P, generator=g).to(dtype)
    return dict(x=x, dt=dt, A=A, B=B, C=C, D=D, z=z, dt_bias=bias, dout=dout)


@pytest.fixture(scope="module")
def runs():
    torch.set_num_threads(max(1, min(8, torch.get_num_threads())))
    Q = SHAPE[-1]
    res = []
    for seed in SEEDS:
        i = two_head_inputs(seed)
        pos = (i["x"], i["dt"], i["A"], i["B"], i["C"], Q, i["dout"])
        kw = dict(D=i["D"], z=i["z"], dt_bias=i["dt_bias"], dt_softplus=True)
        ref = reference_with_grads(*pos, **kw)
        scales = reduced_gradient_scales(*pos, **kw)
        models = {p: rounded_forward_backward(*pos, placement=p, **kw) for p in ("reference", "kernel")}
        res.append((ref, scales, models))
    return res


def test_elementwise_tensors_stay_inside_the_stated_tolerance(runs):
    for ref, _, models in runs:
        for placement, r in models.items():
            for k in ELEMENTWISE:
                assert max_rel_err(r[k], ref[k]) < 1e-2, (placement, k)


def test_reference_rounding_placement_misses_2e_2_on_an_ill_conditioned_reduced_gradient(runs):
    """With nothing but the reference's own operand roundings, at least one seed of the two-head problem puts a
    reduced gradient outside 2e-2: the bound cannot be asked of such a sum, whatever the implementation."""
    worst = {k: max(max_rel_err(models["reference"][k], ref[k]) for ref, _, models in runs) for k in REDUCED}
    assert max(worst.values()) > 2e-2, worst


def test_both_placements_meet_the_conditioning_aware_rule(runs):
    for seed, (ref, scales, models) in zip(SEEDS, runs):
        for placement, r in models.items():
            for k in REDUCED:
                ok, err, bound = reduced_gradient_ok(r[k], ref[k], scales[k], 2e-2)
                assert ok, (seed, placement, k, err, bound)


def test_kernel_placement_is_not_noisier_than_the_reference_placement(runs):
    """Error relative to the sum of magnitudes, median over the seeds: the library's extra roundings (C.B^T stored in
    bf16, row / column sums of rounded products) must not move the typical noise by more than a small factor."""
    for k in REDUCED:
        rel = {p: sorted((models[p][k] - ref[k]).abs().max().item() / scales[k].max().item() for ref, scales, models in runs)
               for p in ("reference", "kernel")}
        med = {p: 0.5 * (v[len(v) // 2 - 1] + v[len(v) // 2]) for p, v in rel.items()}
        assert med["kernel"] <= 3.0 * med["reference"] + 1e-5, (k, med)
        assert rel["kernel"][-1] <= 2.0 ** -8, (k, rel["kernel"][-1])
