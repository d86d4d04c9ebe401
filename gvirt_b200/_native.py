"""Loader for the two native libraries (CUDA kernels via ctypes, host runtime via pybind11).

The kernel library is only *required* when a CUDA device is present: on a GPU box a missing
or unloadable ``libgvirt_kernels.so`` is an error, never a silent fall-back to PyTorch ops.
On a CPU-only machine the ops use their fp32 PyTorch definitions (the oracle), and the
kernel library — which still builds there by cross-compilation — is simply not called.
"""
from __future__ import annotations

import ctypes
import os
import importlib.util
import threading
from typing import Any

import torch

from . import build as _build

_lock = threading.Lock()
_kernels: ctypes.CDLL | None = None
_runtime = None


class KernelError(RuntimeError):
    pass


_ERR = {-1: "GV_EINVAL (bad argument)", -2: "GV_ECUDA (CUDA call failed)",
        -3: "GV_EUNSUPPORTED", -4: "GV_ETOOBIG"}


def kernels() -> ctypes.CDLL:
    """The ctypes handle of libgvirt_kernels.so (built on first use if absent)."""
    global _kernels
    if _kernels is None:
        with _lock:
            if _kernels is None:
                path = _build.kernels_lib_path()
                if not path.exists():
                    _build.build_kernels()
                lib = ctypes.CDLL(str(path))
                lib.gv_last_error.restype = ctypes.c_char_p
                lib.gv_status_ptr.restype = ctypes.c_void_p
                lib.gv_gemm_set_splitk.argtypes = [ctypes.c_longlong] * 4
                lib.gv_set_pdl.argtypes = [ctypes.c_longlong]
                lib.gv_set_prefill_tc_warpgroups.argtypes = [ctypes.c_longlong]
                lib.gv_set_prefill_tc_warpgroups.restype = None
                lib.gv_set_decode_variant.argtypes = [ctypes.c_longlong]
                lib.gv_set_decode_variant.restype = None
                lib.gv_set_sm_budget.argtypes = [ctypes.c_longlong]
                lib.gv_set_sm_budget.restype = ctypes.c_longlong
                lib.gv_planned_sms.restype = ctypes.c_longlong
                _kernels = lib
                _load_gemm_table(lib)
    return _kernels


def _load_gemm_table(lib) -> None:
    """Install the per-shape split-K table named by GVIRT_GEMM_TABLE (written by
    ``python -m gvirt_b200.tools.gemm_sweep``)."""
    path = os.environ.get("GVIRT_GEMM_TABLE", "")
    if not path:
        return
    import json
    with open(path) as f:
        table = json.load(f)
    for e in table.get("entries", []):
        lib.gv_gemm_set_splitk(int(e["N"]), int(e["K"]), int(e["bn"]), int(e["splitk"]))


def runtime():
    """The pybind11 module with the C++ host runtime (built on first use if absent)."""
    global _runtime
    if _runtime is None:
        with _lock:
            if _runtime is None:
                path = _build.runtime_lib_path()
                if not path.exists():
                    _build.build_runtime()
                spec = importlib.util.spec_from_file_location("_gvirt_runtime", str(path))
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
                _runtime = mod
    return _runtime


_VOIDP, _LL, _FLT = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_float
_NULL = ctypes.c_void_p(0)
_Tensor = torch.Tensor


class Ptr:
    """Wrap a raw integer address so that it is passed as a pointer, not as a long long."""

    __slots__ = ("addr",)

    def __init__(self, addr: int):
        self.addr = int(addr)


def _conv(a: Any):
    t = type(a)
    if t is _Tensor:
        return _VOIDP(a.data_ptr())
    if t is int or t is bool:
        return _LL(a)
    if t is float:
        return _FLT(a)
    if a is None:
        return _NULL
    if t is Ptr:
        return _VOIDP(a.addr)
    if isinstance(a, _Tensor):
        return _VOIDP(a.data_ptr())
    if isinstance(a, (ctypes._SimpleCData, ctypes.Array, ctypes._Pointer)):
        return a
    raise TypeError(f"cannot pass {t} to a kernel launcher")


LAUNCHES = 0  # launcher calls made by this process (each enqueues >= 1 kernel of this library)
_fn_cache: dict = {}
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def call(name: str, *args: Any, stream: torch.cuda.Stream | None = None) -> None:
    """Call ``gv_<name>(*args, stream)``; raises KernelError on a non-zero return code."""
    global LAUNCHES
    LAUNCHES += 1
    fn = _fn_cache.get(name)
    if fn is None:
        fn = getattr(kernels(), "gv_" + name)
        _fn_cache[name] = fn
    if stream is not None:
        sp = stream.cuda_stream
    elif _raw_stream is not None:
        sp = _raw_stream(torch.cuda.current_device())
    else:
        sp = torch.cuda.current_stream().cuda_stream
    rc = fn(*[_conv(a) for a in args], _VOIDP(sp))
    if rc != 0:
        lib = kernels()
        detail = lib.gv_last_error().decode(errors="replace") if rc in (-2, -4) else ""
        raise KernelError(f"gv_{name} failed: {_ERR.get(rc, rc)} {detail}")


def set_sm_budget(sms: int) -> int:
    """Limit the SM count the launchers called from this host thread plan with (persistent grids,
    split choices); 0 lifts the limit. Returns the previous value. Per thread: two engines sharing
    a GPU from two threads each keep their own share."""
    return int(kernels().gv_set_sm_budget(int(sms)))


def planned_sms() -> int:
    """SM count the calling thread's launchers plan with right now."""
    return int(kernels().gv_planned_sms())


def read_status() -> int:
    """Synchronise the current stream and return the device status word (0 = healthy)."""
    out = ctypes.c_uint(0)
    lib = kernels()
    rc = lib.gv_status_read(ctypes.byref(out), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise KernelError("gv_status_read failed: " + lib.gv_last_error().decode(errors="replace"))
    return int(out.value)


def reset_status() -> None:
    lib = kernels()
    lib.gv_status_reset(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


STATUS_BITS = {1: "TMA wait timed out", 2: "MMA wait timed out", 4: "epilogue wait timed out",
               8: "peer wait timed out", 16: "MoE receive region overflow",
               32: "device metadata index out of range"}


def describe_status(word: int) -> str:
    return ", ".join(v for k, v in STATUS_BITS.items() if word & k) or "ok"
