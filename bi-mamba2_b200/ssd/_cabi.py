"""ctypes binding of libbissd.so - the structs and prototypes of include/bissd.h, nothing else.

There is no fallback: if the shared library is missing or does not load, importing the operator raises.
"""
import ctypes as C
import os

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_lib", "libbissd.so")

ABI_VERSION = 1
F32, BF16, F16 = 0, 1, 2
PHASE_LOCAL, PHASE_FINISH, PHASE_ALL = 1, 2, 3


class Problem(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("batch", "seqlen", "nheads", "headdim", "ngroups", "dstate", "chunk_size",
                                         "x_dtype", "dt_dtype", "has_D", "D_has_hdim", "has_z", "has_dt_bias",
                                         "dt_softplus")] + [("dt_min", C.c_float), ("dt_max", C.c_float)]


class Tensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_batch", C.c_int64), ("stride_seq", C.c_int64), ("stride_head", C.c_int64)]


class FwdArgs(C.Structure):
    _fields_ = [("p", Problem), ("x", Tensor), ("B", Tensor), ("C", Tensor), ("z", Tensor), ("dt", Tensor),
                ("A", C.c_void_p), ("D", C.c_void_p), ("dt_bias", C.c_void_p),
                ("out", Tensor), ("out_x", Tensor),
                ("dt_out", C.c_void_p), ("cs_f", C.c_void_p), ("cs_b", C.c_void_p),
                ("states_f", C.c_void_p), ("states_b", C.c_void_p),
                ("final_f", C.c_void_p), ("final_b", C.c_void_p),
                ("init_f", C.c_void_p), ("init_b", C.c_void_p),
                ("phases", C.c_int32)]


class BwdArgs(C.Structure):
    _fields_ = [("p", Problem), ("x", Tensor), ("B", Tensor), ("C", Tensor), ("z", Tensor), ("dout", Tensor),
                ("out_x", Tensor), ("dt", Tensor),
                ("A", C.c_void_p), ("D", C.c_void_p), ("dt_bias", C.c_void_p),
                ("dt_out", C.c_void_p), ("cs_f", C.c_void_p), ("cs_b", C.c_void_p),
                ("states_f", C.c_void_p), ("states_b", C.c_void_p),
                ("dx", C.c_void_p), ("dz", C.c_void_p), ("dB", C.c_void_p), ("dC", C.c_void_p), ("ddt", C.c_void_p),
                ("dA", C.c_void_p), ("dD", C.c_void_p), ("ddt_bias", C.c_void_p),
                ("dfinal_f", C.c_void_p), ("dfinal_b", C.c_void_p),
                ("dinit_f", C.c_void_p), ("dinit_b", C.c_void_p),
                ("phases", C.c_int32)]


class NormArgs(C.Structure):
    _fields_ = [("rows", C.c_int64), ("hidden", C.c_int32), ("group_size", C.c_int32), ("x_dtype", C.c_int32),
                ("w_dtype", C.c_int32), ("norm_before_gate", C.c_int32), ("eps", C.c_float),
                ("stride_x", C.c_int64), ("stride_z", C.c_int64), ("stride_out", C.c_int64),
                ("x", C.c_void_p), ("z", C.c_void_p), ("weight", C.c_void_p), ("out", C.c_void_p), ("rstd", C.c_void_p),
                ("dout", C.c_void_p), ("dx", C.c_void_p), ("dz", C.c_void_p), ("dweight", C.c_void_p)]


class ConvArgs(C.Structure):
    _fields_ = [("batch", C.c_int32), ("seqlen", C.c_int32), ("channels", C.c_int32), ("width", C.c_int32),
                ("x_dtype", C.c_int32), ("w_dtype", C.c_int32),
                ("x_stride_batch", C.c_int64), ("x_stride_row", C.c_int64),
                ("out_stride_batch", C.c_int64), ("out_stride_row", C.c_int64),
                ("x", C.c_void_p), ("weight", C.c_void_p), ("bias", C.c_void_p), ("out", C.c_void_p),
                ("dout", C.c_void_p), ("dx", C.c_void_p), ("dweight", C.c_void_p), ("dbias", C.c_void_p)]


EXPORTS = ("bissd_abi_version", "bissd_strerror", "bissd_last_cuda_error", "bissd_workspace_bytes", "bissd_forward",
           "bissd_backward", "bissd_kernel_path", "bissd_launch_count", "bissd_trace_enable", "bissd_trace_read", "bissd_selftest_gemm", "bissd_read_status",
           "bissd_forward_static_scratch", "bissd_chain_boundaries", "bissd_rmsnorm_gated_workspace_bytes", "bissd_rmsnorm_gated_forward",
           "bissd_rmsnorm_gated_backward", "bissd_dwconv_silu_workspace_bytes", "bissd_dwconv_silu_forward",
           "bissd_dwconv_silu_backward")

STATIC_SCRATCH_BYTES = 16 << 20      # BISSD_STATIC_SCRATCH_BYTES
ERR_TOO_LARGE = -9

_lib = None


def lib_path():
    return _LIB_PATH


def load():
    """Load libbissd.so once; raise (never fall back) when it is absent or has the wrong ABI."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise ImportError(f"{_LIB_PATH} not found: build it with `python bi-mamba2_b200/build.py` "
                          "(there is no non-CUDA implementation of this operator)")
    lib = C.CDLL(_LIB_PATH)
    lib.bissd_abi_version.restype = C.c_int
    lib.bissd_strerror.restype = C.c_char_p
    lib.bissd_strerror.argtypes = [C.c_int]
    lib.bissd_last_cuda_error.restype = C.c_char_p
    lib.bissd_workspace_bytes.restype = C.c_int
    lib.bissd_workspace_bytes.argtypes = [C.POINTER(Problem), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
    lib.bissd_forward.restype = C.c_int
    lib.bissd_forward.argtypes = [C.POINTER(FwdArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.bissd_backward.restype = C.c_int
    lib.bissd_backward.argtypes = [C.POINTER(BwdArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.bissd_kernel_path.restype = C.c_char_p
    lib.bissd_kernel_path.argtypes = [C.POINTER(Problem)]
    lib.bissd_launch_count.restype = C.c_ulonglong
    lib.bissd_trace_enable.restype = C.c_int
    lib.bissd_trace_enable.argtypes = [C.c_int]
    lib.bissd_trace_read.restype = C.c_int
    lib.bissd_trace_read.argtypes = [C.c_char_p, C.c_size_t, C.POINTER(C.c_float), C.POINTER(C.c_int), C.c_int,
                                     C.POINTER(C.c_int)]
    lib.bissd_forward_static_scratch.restype = C.c_int
    lib.bissd_forward_static_scratch.argtypes = [C.POINTER(FwdArgs), C.c_void_p]
    lib.bissd_rmsnorm_gated_workspace_bytes.restype = C.c_int
    lib.bissd_rmsnorm_gated_workspace_bytes.argtypes = [C.POINTER(NormArgs), C.POINTER(C.c_size_t)]
    lib.bissd_rmsnorm_gated_forward.restype = C.c_int
    lib.bissd_rmsnorm_gated_forward.argtypes = [C.POINTER(NormArgs), C.c_void_p]
    lib.bissd_rmsnorm_gated_backward.restype = C.c_int
    lib.bissd_rmsnorm_gated_backward.argtypes = [C.POINTER(NormArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.bissd_dwconv_silu_workspace_bytes.restype = C.c_int
    lib.bissd_dwconv_silu_workspace_bytes.argtypes = [C.POINTER(ConvArgs), C.POINTER(C.c_size_t)]
    lib.bissd_dwconv_silu_forward.restype = C.c_int
    lib.bissd_dwconv_silu_forward.argtypes = [C.POINTER(ConvArgs), C.c_void_p]
    lib.bissd_dwconv_silu_backward.restype = C.c_int
    lib.bissd_dwconv_silu_backward.argtypes = [C.POINTER(ConvArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.bissd_chain_boundaries.restype = C.c_int
    lib.bissd_chain_boundaries.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int,
                                           C.c_int64, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.bissd_read_status.restype = C.c_int
    lib.bissd_read_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]
    lib.bissd_selftest_gemm.restype = C.c_int
    lib.bissd_selftest_gemm.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_void_p]
    if lib.bissd_abi_version() != ABI_VERSION:
        raise ImportError(f"libbissd ABI {lib.bissd_abi_version()} != binding ABI {ABI_VERSION}; rebuild the library")
    _lib = lib
    return lib


def launch_count():
    return int(load().bissd_launch_count())


def trace_enable(on):
    check(load().bissd_trace_enable(int(bool(on))))


def trace_read():
    """{kernel name: (total device ms, launches)} for everything recorded since trace_enable(True)."""
    lib = load()
    cap = 64
    names = C.create_string_buffer(4096)
    ms = (C.c_float * cap)()
    cnt = (C.c_int * cap)()
    n = C.c_int(0)
    check(lib.bissd_trace_read(names, 4096, ms, cnt, cap, C.byref(n)))
    keys = [k for k in names.value.decode().split(";") if k]
    return {k: (float(ms[i]), int(cnt[i])) for i, k in enumerate(keys[:n.value])}


class BissdError(RuntimeError):
    pass


def check(status):
    if status != 0:
        lib = load()
        msg = lib.bissd_strerror(status).decode()
        cuda = lib.bissd_last_cuda_error().decode()
        raise BissdError(f"libbissd error {status}: {msg}" + (f" [{cuda}]" if cuda else ""))
