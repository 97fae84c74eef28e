"""CPU-side checks of the C-ABI boundary: the library loads, exports what include/bissd.h declares, the ctypes
structs have the C layout, and argument validation answers without touching a GPU."""
import ctypes
import os
import re
import subprocess
import sys
import tempfile

import pytest

from conftest import ROOT

sys.path.insert(0, os.path.join(ROOT, "bi-mamba2_b200"))
from ssd import _cabi  # noqa: E402

HEADER = os.path.join(ROOT, "include", "bissd.h")


@pytest.fixture(scope="module")
def lib():
    import importlib.util
    spec = importlib.util.spec_from_file_location("bissd_build", os.path.join(ROOT, "bi-mamba2_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()
    return _cabi.load()


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bissd_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared_functions()
    assert set(_cabi.EXPORTS) <= set(names)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/bissd.h but not exported by libbissd.so"


def test_abi_version(lib):
    assert lib.bissd_abi_version() == _cabi.ABI_VERSION


def test_struct_layout_matches_c_header():
    src = r'''
#include <stdio.h>
#include <stddef.h>
#include "bissd.h"
int main(void) {
  printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\n", sizeof(bissd_problem), sizeof(bissd_tensor), sizeof(bissd_fwd_args),
         sizeof(bissd_bwd_args), offsetof(bissd_fwd_args, dt_out), offsetof(bissd_fwd_args, phases),
         offsetof(bissd_bwd_args, dx), offsetof(bissd_bwd_args, phases), sizeof(bissd_norm_args),
         offsetof(bissd_norm_args, stride_x), offsetof(bissd_norm_args, dweight));
  return 0; }
'''
    with tempfile.TemporaryDirectory() as td:
        cpath, exe = os.path.join(td, "t.c"), os.path.join(td, "t")
        open(cpath, "w").write(src)
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), cpath, "-o", exe])
        got = [int(v) for v in subprocess.check_output([exe]).split()]
    want = [ctypes.sizeof(_cabi.Problem), ctypes.sizeof(_cabi.Tensor), ctypes.sizeof(_cabi.FwdArgs),
            ctypes.sizeof(_cabi.BwdArgs), _cabi.FwdArgs.dt_out.offset, _cabi.FwdArgs.phases.offset,
            _cabi.BwdArgs.dx.offset, _cabi.BwdArgs.phases.offset, ctypes.sizeof(_cabi.NormArgs),
            _cabi.NormArgs.stride_x.offset, _cabi.NormArgs.dweight.offset]
    assert got == want


def _problem(**kw):
    base = dict(batch=2, seqlen=128, nheads=4, headdim=16, ngroups=2, dstate=16, chunk_size=64, x_dtype=0, dt_dtype=0,
                has_D=1, D_has_hdim=0, has_z=0, has_dt_bias=0, dt_softplus=1, dt_min=0.0, dt_max=float("inf"))
    base.update(kw)
    return _cabi.Problem(**base)


def test_workspace_bytes_and_validation(lib):
    f, b = ctypes.c_size_t(0), ctypes.c_size_t(0)
    assert lib.bissd_workspace_bytes(ctypes.byref(_problem()), ctypes.byref(f), ctypes.byref(b)) == 0
    assert f.value > 0 and b.value > f.value
    assert f.value % 256 == 0 and b.value % 256 == 0
    # nheads not divisible by ngroups; chunk below the reference's minimum of 32; bad dtype
    assert lib.bissd_workspace_bytes(ctypes.byref(_problem(ngroups=3)), None, None) == -2
    assert lib.bissd_workspace_bytes(ctypes.byref(_problem(chunk_size=16)), None, None) == -2
    assert lib.bissd_workspace_bytes(ctypes.byref(_problem(x_dtype=7)), None, None) == -3
    assert lib.bissd_workspace_bytes(None, None, None) == -1


def test_backward_workspace_is_sized_by_kernel_family(lib):
    """16-bit problems report the tensor-core kernels' backward scratch (no fp32 copy of the passed state gradients,
    dB / dC parts per group); 16-bit tensors that miss the alignment rules need the CUDA-core size and are refused
    with less - before anything touches a device."""
    cfg2 = dict(batch=8, seqlen=2048, nheads=24, headdim=64, ngroups=1, dstate=128, chunk_size=256, has_z=1, has_dt_bias=1)
    tc, simt = ctypes.c_size_t(0), ctypes.c_size_t(0)
    assert lib.bissd_workspace_bytes(ctypes.byref(_problem(x_dtype=1, dt_dtype=1, **cfg2)), None, ctypes.byref(tc)) == 0
    assert lib.bissd_workspace_bytes(ctypes.byref(_problem(x_dtype=0, dt_dtype=0, **cfg2)), None, ctypes.byref(simt)) == 0
    assert tc.value < 350e6 < simt.value, (tc.value, simt.value)
    a = _cabi.BwdArgs()
    a.p = _problem(x_dtype=1, dt_dtype=1, **cfg2)
    a.phases = 3
    t = lambda addr: _cabi.Tensor(addr, 2048 * 24 * 64, 24 * 64, 64)
    a.x, a.B, a.C, a.z, a.dout, a.out_x = t(4096 + 2), t(4096), t(4096), t(4096), t(4096), t(4096)   # x 2 bytes off
    a.dt = _cabi.Tensor(4096, 2048 * 24, 24, 1)
    for f in ("A", "D", "dt_bias", "dt_out", "cs_f", "cs_b", "states_f", "states_b", "dx", "dz", "dB", "dC", "ddt", "dA",
              "dD", "ddt_bias"):
        setattr(a, f, 4096)
    assert lib.bissd_backward(ctypes.byref(a), 4096, tc.value, None) == -5     # BISSD_ERR_WORKSPACE


def test_forward_rejects_bad_arguments_before_any_launch(lib):
    args = _cabi.FwdArgs()
    args.p = _problem()
    args.phases = 3
    assert lib.bissd_forward(ctypes.byref(args), None, 0, None) == -1          # NULL tensors
    args.phases = 0
    assert lib.bissd_forward(ctypes.byref(args), None, 0, None) == -8          # bad phase mask
    assert lib.bissd_forward(None, None, 0, None) == -1
    assert b"NULL" in lib.bissd_strerror(-1)


def test_operator_refuses_cpu_tensors(lib):
    import torch
    from ssd.bi.ssd_combined import bimamba_chunk_scan_combined
    x = torch.randn(1, 64, 2, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        bimamba_chunk_scan_combined(x, torch.rand(1, 64, 2), -torch.ones(2), torch.randn(1, 64, 1, 8),
                                    torch.randn(1, 64, 1, 8), 32)


def test_fused_layer_function_refuses_cpu_tensors_and_odd_widths(lib):
    import torch
    from ssd.bi.split_conv1d_scan import bimamba_split_conv1d_scan_combined
    H, P, G, N = 8, 16, 1, 16
    dim = H * P
    args = lambda extra=0: (torch.randn(1, 64, 2 * dim + 2 * G * N + H + extra), torch.randn(dim + 2 * G * N, 1, 3), None,
                            torch.zeros(H), -torch.ones(H), torch.ones(H, P), 32)
    with pytest.raises(RuntimeError, match="CUDA"):
        bimamba_split_conv1d_scan_combined(*args())
    with pytest.raises(ValueError, match="channels"):                             # extra non-SSM channels are not taken
        bimamba_split_conv1d_scan_combined(*args(extra=8))


def test_norm_entry_points_validate_before_any_launch(lib):
    a = _cabi.NormArgs(rows=4, hidden=200, group_size=0, x_dtype=0, w_dtype=0, norm_before_gate=1, eps=1e-5,
                       stride_x=200, stride_z=200, stride_out=200, x=256, weight=256, out=256, rstd=256)
    assert lib.bissd_rmsnorm_gated_forward(ctypes.byref(a), None) == -2          # hidden not a multiple of 256
    a.hidden, a.stride_x, a.stride_out = 512, 512, 512
    a.group_size = 384
    assert lib.bissd_rmsnorm_gated_forward(ctypes.byref(a), None) == -2          # group does not divide hidden
    a.group_size, a.x = 0, None
    assert lib.bissd_rmsnorm_gated_forward(ctypes.byref(a), None) == -1
    a.x, a.w_dtype = 256, 2
    assert lib.bissd_rmsnorm_gated_forward(ctypes.byref(a), None) == -3          # weight dtype neither fp32 nor x's
    need = ctypes.c_size_t()
    a.w_dtype = 0
    assert lib.bissd_rmsnorm_gated_workspace_bytes(ctypes.byref(a), ctypes.byref(need)) == 0 and need.value >= 512 * 4
