"""ctypes loaders for the native libraries and the error type of the kernels."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

from . import build

_cuda = None
_host = None


class KernelError(RuntimeError):
    """A native entry point returned a non-zero status."""


class CommTimeout(KernelError):
    """A bounded device-side wait ran out (status word written by the kernel)."""


_ERRORS = {-1: "bad argument", -2: "driver call failed (tensor map)", -3: "launch failed",
           -4: "size beyond the built-in maximum", 101: "producer wait timed out",
           102: "MMA wait timed out", 103: "epilogue wait timed out",
           104: "TMEM-empty wait timed out", 105: "peer wait timed out",
           106: "attention wait timed out",
           # checked build (TERAPIPE_CHECKED=1): an index check inside a kernel failed
           121: "checked build: GEMM tile outside the output grid",
           122: "checked build: staging / flag slot beyond its capacity",
           123: "checked build: rank index outside the group",
           124: "checked build: attention row or statistics slot outside the buffers",
           125: "checked build: element range malformed",
           129: "checked build: self-test check failed (as requested)"}
CHECK_CODES = range(121, 130)


class CheckFailed(KernelError):
    """An index check of the checked kernel build failed; the guarded access was skipped."""


def check(status: int, what: str) -> None:
    if status != 0:
        raise KernelError(f"{what}: {_ERRORS.get(status, 'error')} ({status})")


def cuda_lib() -> ctypes.CDLL:
    """The sm_100a kernel library; built on first use when nvcc is present.  With
    ``TERAPIPE_CHECKED=1`` in the environment the checked build is loaded instead: the same
    kernels with index checks that report through the status word (see ``build.py``)."""
    global _cuda
    if _cuda is None:
        checked = os.environ.get("TERAPIPE_CHECKED", "0") == "1"
        path = build.CUDA_LIB_CHECKED if checked else build.CUDA_LIB
        if not path.exists() or os.environ.get("TERAPIPE_REBUILD"):
            build.build_cuda(checked=checked)
        _cuda = ctypes.CDLL(str(path))
        _declare(_cuda)
        if bool(_cuda.tp_checked_build()) != checked:
            raise KernelError(f"{path.name} is not the {'checked' if checked else 'regular'} build")
    return _cuda


def host_lib() -> ctypes.CDLL:
    global _host
    if _host is None:
        build.build_host()      # no-op when the sources are unchanged
        _host = ctypes.CDLL(str(build.HOST_LIB))
        f = _host.tp_plan_slices
        f.restype = ctypes.c_double
        f.argtypes = [c_void_p, c_longlong, c_longlong, c_longlong, c_longlong, c_longlong,
                      ctypes.c_double, c_void_p, c_void_p, c_void_p]
        w = _host.tp_tile_order_walk
        w.restype = c_longlong
        w.argtypes = [c_int, c_int, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p,
                      c_void_p]
    return _host


# Argument types of every entry point of the kernel library that is called through `cuda_lib()`:
# P = pointer, I = int, L = long long, F = float.  tests/test_bindings_cpu.py checks this table
# against the `extern "C"` definitions in csrc/*.cu.
P, I, L, F = c_void_p, c_int, c_longlong, c_float
SIGNATURES = {
    "tp_gemm": [I, I, I, P, L, P, L, P, L, I, I, I, I, I, F, P, P, L, I, P, I, P, L, I, P, P],
    "tp_layernorm_fwd": [I, P, P, P, P, P, P, I, I, F, P],
    "tp_layernorm_bwd_parts": [I],
    "tp_layernorm_bwd": [I, P, P, P, P, P, P, P, P, P, P, I, I, P],
    "tp_layernorm_bwd_accum": [I, P, P, P, P, P, P, P, P, I, I, P],
    "tp_layernorm_bwd_finish": [P, I, I, P, P, P],
    "tp_colsum": [I, P, L, I, I, P, P],
    "tp_adam_tick": [P, F, F, P],
    "tp_fused_adam": [I, P, P, P, P, P, L, P, F, F, F, F, F, F, P],
    "tp_fill": [I, P, L, F, P],
    "tp_gemm_ar": [I, I, P, L, P, L, L, I, I, I, P, P, L, I, I, I, P, I, P, P, P, P, P, P],
    "tp_advance_counter": [P, I, P],
    "tp_gemm_set_pair_default": [I],
    "tp_gemm_set_prefetch": [I],
    "tp_gemm_ar_set_exchange": [I],
    "tp_link_probe": [P, L, I, P],
    "tp_gemm_trace": [I, P, L, P, L, P, L, I, I, I, P, P, P],
    "tp_dp_reduce_adam": [I, I, I, I, P, P, P, P, P, P, P, L, L, P, F, F, F, F, F, F, P, P],
    "tp_set_wait_limit_ns": [L],
    "tp_set_pdl": [I],
    "tp_gemm_ag": [I, I, P, L, P, L, P, L, I, I, I, P, I, P, I, P, L, P, P, I, I, I, P, P],
    "tp_gemm_rs": [I, I, P, L, P, L, P, L, I, I, I, P, P, L, I, I, I, I, P, I, P, P, P, P],
    "tp_layernorm_fwd_push": [I, P, P, P, P, P, P, I, I, F, I, I, P, I, P, P, P],
    "tp_layernorm_bwd_accum_push": [I, P, P, P, P, P, P, P, P, I, I, I, I, P, I, P, P, P],
    "tp_layernorm_bwd_finish_assign": [P, I, I, P, P, P],
    "tp_ag_push": [P, L, P, P, I, I, I, P, P, P],
    "tp_ag_copy": [P, L, P, P, I, I, I, P, P],
    "tp_group_barrier": [P, I, I, I, P, P, P],
    "tp_peer_sum": [P, I, P, I, I, P],
    "tp_attn_fwd": [I, I, P, I, I, I, I, P, L, P, L, P, P],
    "tp_attn_bwd": [I, I, P, I, I, I, I, I, P, L, P, L, P, L, P, P, L, P, P],
    "tp_checked_build": [],
    "tp_checked_selftest": [I, I, P, P],
    "tp_attn_fwd_scaled": [I, I, F, P, I, I, I, I, P, L, P, L, P, P],
    "tp_attn_bwd_scaled": [I, I, F, P, I, I, I, I, I, P, L, P, L, P, L, P, P, L, P, P],
}


def _declare(lib: ctypes.CDLL) -> None:
    for name, argtypes in SIGNATURES.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype = c_int
            fn.argtypes = argtypes
