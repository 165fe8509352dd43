"""ctypes binding of the in-tree sm_100a kernel library.

The library is loaded lazily the first time a CUDA op is dispatched. On a machine
with a GPU a missing or unloadable library is an error (never a silent fallback to
ATen); on a CPU-only machine the ops use their PyTorch reference implementations.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Any

import torch

_LOCK = threading.Lock()
_LIB: ctypes.CDLL | None = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float

EPI_NONE, EPI_GELU, EPI_DGELU, EPI_CE_FWD, EPI_CE_BWD, EPI_GELU_GRAD, EPI_MUL, EPI_SWIGLU, EPI_SWIGLU_BWD = range(9)

STATUS_NAMES = {
    0: "ok",
    1: "consumer gave up waiting for a TMA stage",
    2: "producer gave up waiting for a free smem stage",
    3: "epilogue gave up waiting for an accumulator",
    4: "MMA issuer gave up waiting for a drained accumulator",
    5: "communication kernel gave up waiting for a peer flag",
    6: "generic kernel error",
}


class KernelError(RuntimeError):
    """A launcher rejected its arguments or a kernel recorded an error status."""


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("A", c_void_p),
        ("B", c_void_p),
        ("out", c_void_p),
        ("out2", c_void_p),
        ("bias", c_void_p),
        ("residual", c_void_p),
        ("aux", c_void_p),
        ("M", c_int),
        ("N", c_int),
        ("K", c_int),
        ("batch", c_int),
        ("a_mn", c_int),
        ("b_mn", c_int),
        ("epi", c_int),
        ("out_f32", c_int),
        ("accumulate", c_int),
        ("allow_split_k", c_int),
        ("alpha", c_float),
        ("lda", c_ll),
        ("ldb", c_ll),
        ("ldo", c_ll),
        ("ldo2", c_ll),
        ("ldr", c_ll),
        ("ldaux", c_ll),
        ("bs_a", c_ll),
        ("bs_b", c_ll),
        ("bs_out", c_ll),
        ("bs_out2", c_ll),
        ("bs_res", c_ll),
        ("bs_aux", c_ll),
        ("bs_bias", c_ll),
        ("labels", c_void_p),
        ("forbidden", c_void_p),
        ("inv_temp", c_float),
        ("seed", ctypes.c_ulonglong),
        ("ce_part", c_void_p),
        ("label_logit", c_void_p),
        ("row_lse", c_void_p),
        ("gscale", c_float),
        ("gscale_ptr", c_void_p),
        ("a_sum", c_void_p),
    ]


def cuda_kernels_available() -> bool:
    """True when a GPU is present (the kernel library is then mandatory)."""
    return torch.cuda.is_available()


def lib() -> ctypes.CDLL:
    """Load (building first if stale) and return the kernel library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is None:
            from deberta_b200 import build as _build

            path = _build.build()
            handle = ctypes.CDLL(str(path))
            handle.db200_status_read_and_clear.restype = c_int
            handle.db200_status_ptr.restype = c_void_p
            _LIB = handle
    return _LIB


def stream_ptr() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what}: launcher returned {rc}")


def check_status() -> None:
    """Synchronise and raise if any kernel recorded a bounded-wait failure."""
    code = int(lib().db200_status_read_and_clear())
    if code != 0:
        raise KernelError(f"device status {code}: {STATUS_NAMES.get(code, 'unknown')}")


def set_dependent_launch(on: bool) -> bool:
    """Programmatic dependent launch for the kernels that support it (GEMM, norms, attention, position bias, casts): a
    kernel's set-up runs under the tail of its predecessor in the stream and it waits, before touching global memory,
    until the predecessor has completed. On by default; returns the previous setting."""
    return bool(lib().db200_set_pdl(ctypes.c_int(1 if on else 0)))


LAUNCH_COUNT = 0


def call(name: str, *args: Any) -> None:
    global LAUNCH_COUNT
    LAUNCH_COUNT += 1
    fn = getattr(lib(), name)
    check(int(fn(*args)), name)


def call_rc(name: str, *args: Any, accept: tuple[int, ...] = ()) -> int:
    """Like :func:`call`, but return codes listed in ``accept`` come back to the caller instead of raising."""
    global LAUNCH_COUNT
    rc = int(getattr(lib(), name)(*args))
    if rc == 0:
        LAUNCH_COUNT += 1
    elif rc not in accept:
        check(rc, name)
    return rc
