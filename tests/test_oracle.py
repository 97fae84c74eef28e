"""Pin the CPU oracle against golden vectors produced by the reference implementation itself
(tests/golden/make_golden.py): its Triton kernels, forward and backward, and its pure-PyTorch path."""
import pytest
import torch

from conftest import GOLDEN_TORCHREF, GOLDEN_TRITON, load_golden
from oracle.bissd_oracle import chunked_reference, dense_reference, max_rel_err, reference_with_grads

# The golden vectors are fp32 results of fp32 kernels (TF32-free on the interpreter); the oracle runs in fp64.
TOL = 2e-5


def _args(g):
    b, L, H, P, G, N, Q, softplus = g["meta"]
    kw = dict(D=g.get("D"), z=g.get("z"), dt_bias=g.get("dt_bias"), dt_softplus=bool(softplus), dt_limit=g["dt_limit"])
    return (g["x"], g["dt"], g["A"], g["B"], g["C"]), Q, kw


@pytest.mark.parametrize("name", GOLDEN_TRITON)
@pytest.mark.parametrize("dense", [False, True])
def test_oracle_matches_reference_triton_fwd_bwd(name, dense):
    g = load_golden(name)
    pos, Q, kw = _args(g)
    r = reference_with_grads(*pos, Q, g["dout"], dense=dense, **kw)
    for key in ("out", "dx", "ddt", "dA", "dB", "dC", "dD", "dz", "ddt_bias"):
        if key in g:
            assert r[key] is not None
            assert max_rel_err(r[key], g[key]) < TOL, key


@pytest.mark.parametrize("name", GOLDEN_TRITON)
def test_oracle_intermediates_match_reference_triton(name):
    g = load_golden(name)
    pos, Q, kw = _args(g)
    r = chunked_reference(*pos, Q, return_intermediates=True, **kw)
    for key in ("dt_out", "cs_f", "cs_b", "states_f", "states_b", "final_f", "final_b", "out_x"):
        if key in g:
            assert max_rel_err(r[key], g[key]) < TOL, key
    _, ff, fb = dense_reference(*pos, return_final_states=True, **kw)
    assert max_rel_err(ff, g["final_f"]) < TOL
    assert max_rel_err(fb, g["final_b"]) < TOL


@pytest.mark.parametrize("name", GOLDEN_TORCHREF)
def test_oracle_matches_reference_pytorch_path(name):
    g = load_golden(name)
    pos, Q, kw = _args(g)
    assert max_rel_err(chunked_reference(*pos, Q, **kw), g["out"]) < TOL
    assert max_rel_err(dense_reference(*pos, **kw), g["out"]) < TOL


def test_dense_and_chunked_agree_with_initial_states():
    torch.manual_seed(0)
    b, L, H, P, G, N, Q = 1, 96, 2, 4, 1, 8, 32
    x, B, C = torch.randn(b, L, H, P), torch.randn(b, L, G, N), torch.randn(b, L, G, N)
    dt, A = torch.rand(b, L, H) * 0.2, -torch.rand(H) - 0.5
    i_f, i_b = torch.randn(b, H, P, N), torch.randn(b, H, P, N)
    o1, f1, b1 = dense_reference(x, dt, A, B, C, return_final_states=True, initial_states_f=i_f, initial_states_b=i_b)
    r = chunked_reference(x, dt, A, B, C, Q, return_intermediates=True, initial_states_f=i_f, initial_states_b=i_b)
    assert max_rel_err(r["out"], o1) < 1e-12
    assert max_rel_err(r["final_f"], f1) < 1e-12
    assert max_rel_err(r["final_b"], b1) < 1e-12


def test_sequence_split_composes():
    """Splitting the sequence in two and handing boundary states across reproduces the unsplit result -
    the property the sequence-sharded multi-GPU path relies on."""
    torch.manual_seed(1)
    b, L, H, P, G, N, Q = 1, 128, 2, 4, 1, 8, 32
    x, B, C = torch.randn(b, L, H, P), torch.randn(b, L, G, N), torch.randn(b, L, G, N)
    dt, A = torch.rand(b, L, H) * 0.2, -torch.rand(H) - 0.5
    full = dense_reference(x, dt, A, B, C)
    h = L // 2
    _, f_left, _ = dense_reference(x[:, :h], dt[:, :h], A, B[:, :h], C[:, :h], return_final_states=True)
    _, _, b_right = dense_reference(x[:, h:], dt[:, h:], A, B[:, h:], C[:, h:], return_final_states=True)
    left = dense_reference(x[:, :h], dt[:, :h], A, B[:, :h], C[:, :h], initial_states_b=b_right)
    right = dense_reference(x[:, h:], dt[:, h:], A, B[:, h:], C[:, h:], initial_states_f=f_left)
    assert max_rel_err(torch.cat([left, right], 1), full) < 1e-12


def test_decay_gradient_telescopes_into_row_and_column_sums():
    """The identity behind the row/column-sum form of the intra-chunk decay gradient (csrc/tc_intra_sums.cuh):
    da_f[j] = sum_{k<j} (colsum W_f[k] - rowsum W_f[k]),  da_b[j] = sum_{k>j} (colsum W_b[k] - rowsum W_b[k])."""
    from oracle.bissd_manual_backward import manual_backward
    g = torch.Generator().manual_seed(11)
    b, L, H, P, G, N, Q = 2, 96, 4, 8, 2, 8, 32
    mk = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    x, B, C, dout = mk(b, L, H, P), mk(b, L, G, N), mk(b, L, G, N), mk(b, L, H, P)
    dt = torch.rand(b, L, H, generator=g, dtype=torch.float64) * 0.3
    A = -torch.rand(H, generator=g, dtype=torch.float64) - 0.2
    r = manual_backward(x, dt, A, B, C, Q, dout)
    uf = r["Wf"].sum(-2) - r["Wf"].sum(-1)                               # column sums - row sums, (b,H,nc,Q)
    ub = r["Wb"].sum(-2) - r["Wb"].sum(-1)
    da_f = torch.cumsum(uf, -1) - uf                                      # exclusive prefix sum
    da_b = torch.flip(torch.cumsum(torch.flip(ub, [-1]), -1), [-1]) - ub  # exclusive suffix sum
    assert max_rel_err(da_f, r["da_f"]) < 1e-10
    assert max_rel_err(da_b, r["da_b"]) < 1e-10
