"""ctypes binding of ``libcoda_b200.so`` (the C ABI declared in ``include/coda_b200.h``).

The library is built in-tree by :mod:`coda_kernels_b200.build`.  There is no
fallback: if the shared object is missing or a symbol cannot be resolved, the
import of this module raises, and every operator built on it fails loudly.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from pathlib import Path

_PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = _PKG_DIR / "libcoda_b200.so"
NATIVE_LIB_PATH = _PKG_DIR / "libcoda_b200_torch.so"  # TORCH_LIBRARY dispatch shim over the same C ABI (see ops.py)

_P = c_void_p
_I = c_int
_L = c_int64
_F = c_float

# name -> (restype, argtypes); mirrors include/coda_b200.h one to one.
SIGNATURES = {
    "coda_b200_version": (_I, []),
    "coda_b200_last_error": (c_char_p, []),
    "coda_b200_set_option": (_I, [c_char_p, _I]),
    "coda_b200_selftest_wait_timeout": (_I, [_P, _L, _P, _P]),
    "coda_b200_status_poll": (_I, [_P, _P]),
    "coda_b200_gemm": (_I, [_P, _L, _L, _P, _L, _L, _P, _L, _I, _I, _I, _I, _P, _P, _P]),
    "coda_b200_gemm_workspace_bytes": (_L, [_I, _I, _I]),
    "coda_b200_gemm_ws": (_I, [_P, _L, _L, _P, _L, _L, _P, _L, _I, _I, _I, _I, _P, _P, _L, _P, _P]),
    "coda_b200_gemm_add": (_I, [_P, _L, _L, _P, _L, _L, _P, _L, _I, _P, _L, _I, _I, _I, _I, _P, _P, _P]),
    "coda_b200_gemm_dsigmoid_dgrad": (_I, [_P, _L, _P, _L, _P, _L, _P, _L, _P, _L, _I, _I, _I, _P, _P]),
    "coda_b200_gemm_sigmoid": (_I, [_P, _L, _L, _P, _L, _L, _P, _L, _I, _I, _I, _I, _P, _P]),
    "coda_b200_gemm_swiglu": (_I, [_P, _L, _L, _P, _L, _L, _P, _L, _P, _L, _I, _I, _I, _P, _P]),
    "coda_b200_gemm_sigmoid_glu": (_I, [_P, _L, _L, _P, _L, _L, _P, _L, _P, _L, _I, _I, _I, _P, _P]),
    "coda_b200_dsigmoid_glu": (_I, [_P, _L, _P, _L, _P, _L, _I, _I, _P]),
    "coda_b200_lse_tiles": (_I, [_I]),
    "coda_b200_gemm_lse": (_I, [_P, _L, _L, _P, _L, _L, _P, _L, _P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "coda_b200_lse_finalize": (_I, [_P, _P, _I, _P, _P, _I, _P, _P, _I, _P]),
    "coda_b200_ce_grad_fixup": (_I, [_P, _L, _P, _I, _P, _P, _I, _I, _I, _P]),
    "coda_b200_gemm_qknorm_rope": (
        _I,
        [_P, _L, _L, _P, _L, _L, _P, _L, _P, _L, _P, _L, _P, _P, _P, _I, _P, _I, _I, _I, _F, _I, _I, _I, _P, _P],
    ),
    "coda_b200_gemm_rmsnorm_swiglu": (_I, [_P, _L, _L, _P, _L, _L, _P, _P, _L, _P, _L, _I, _I, _I, _P, _P]),
    "coda_b200_gemm_rmsnorm_lse": (_I, [_P, _L, _L, _P, _L, _L, _P, _P, _L, _P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "coda_b200_gemm_rmsnorm_qknorm_rope": (
        _I,
        [_P, _L, _L, _P, _L, _L, _P, _P, _L, _P, _L, _P, _L, _P, _P, _P, _I, _P, _I, _I, _I, _F, _I, _I, _I, _P, _P],
    ),
    "coda_b200_gemm_lse_logits": (_I, [_P, _L, _L, _P, _L, _L, _P, _P, _L, _P, _P, _I, _I, _I, _P, _P]),
    "coda_b200_lse_reduce": (_I, [_P, _P, _I, _P, _I, _P]),
    "coda_b200_cross_entropy_fwd_bwd": (_I, [_P, _L, _P, _P, _I, _P, _I, _I, _P]),
    "coda_b200_gemm_residual_partial_rmsnorm": (
        _I, [_P, _L, _L, _P, _L, _L, _P, _L, _P, _F, _P, _L, _P, _L, _P, _P, _I, _I, _I, _P, _P]),
    "coda_b200_gemm_swiglu_bwd_zdz": (
        _I, [_P, _L, _L, _P, _L, _L, _P, _L, _P, _L, _P, _L, _P, _F, _P, _I, _I, _I, _P, _P]),
    "coda_b200_gemm_residual_partial_rmsnorm_bwd": (
        _I, [_P, _L, _L, _P, _L, _L, _P, _P, _L, _P, _P, _P, _P, _L, _I, _P, _P, _L, _P, _I, _I, _I, _P, _P]),
    "coda_b200_partial_rmsnorm": (_I, [_P, _L, _P, _F, _P, _L, _P, _L, _P, _I, _I, _P]),
    "coda_b200_gemm_rmsnorm_rope": (_I, [_P, _L, _L, _P, _L, _L, _P, _P, _L, _P, _I, _P, _I, _I, _I, _P, _P]),
    "coda_b200_rope_bwd_zdz": (_I, [_P, _L, _P, _L, _P, _I, _P, _F, _P, _L, _P, _I, _I, _P]),
    "coda_b200_gemm_rmsnorm_lse_zdz": (_I, [_P, _L, _L, _P, _L, _L, _P, _P, _L, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "coda_b200_lse_finalize_zdz": (_I, [_P, _P, _P, _I, _P, _P, _I, _P, _P, _P, _I, _P]),
    "coda_b200_dswiglu": (_I, [_P, _L, _P, _L, _P, _L, _I, _I, _P]),
    "coda_b200_dsigmoid": (_I, [_P, _L, _I, _P, _L, _P, _L, _I, _I, _P]),
    "coda_b200_qknorm_rope_bwd_scratch_bytes": (_L, [_I, _I]),
    "coda_b200_qknorm_rope_bwd": (
        _I,
        [_P, _L, _P, _L, _P, _L, _I, _P, _L, _P, _P, _P, _I, _P, _I, _I, _I, _F, _P, _L, _P, _P, _L, _I, _P],
    ),
    "coda_b200_qknorm_rope_bwd_noalloc": (
        _I,
        [_P, _L, _P, _L, _P, _L, _I, _P, _L, _P, _P, _P, _I, _P, _I, _I, _I, _F, _P, _L, _P, _I, _P],
    ),
}


def _load() -> ctypes.CDLL:
    if os.environ.get("CODA_B200_BUILD_ON_IMPORT", "1") == "1":
        from . import build as _build

        # Rebuild when the sources changed since the library was built (needs nvcc; skipped silently without it,
        # in which case a missing library is the error reported below).
        if _build.is_stale() and _build.have_nvcc():
            _build.build_library()
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m coda_kernels_b200.build` "
            "(needs nvcc; there is no CPU or eager fallback)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # raises AttributeError if the symbol is absent
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


class CodaB200Error(RuntimeError):
    """A C-ABI call rejected its arguments or a CUDA call failed."""


# Optional callable run after every successful library call; ``ops`` installs a synchronising device-status check
# here when CODA_B200_SYNC_STATUS=1 (debug aid: turns an expired device-side wait into an exception at the call site).
post_call_hook = None


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib.coda_b200_last_error()
        raise CodaB200Error(f"{what} failed (code {rc}): {msg.decode() if msg else ''}")
    if post_call_hook is not None:
        post_call_hook(what)


_option_values: dict[str, int] = {}


def set_option(name: str, value: int) -> None:
    check(lib.coda_b200_set_option(name.encode(), int(value)), f"set_option({name})")
    _option_values[name] = int(value)


class option_override:
    """``with option_override("max_ctas", 128): ...`` sets a library option for the launches issued inside the block and
    puts the previous value (as set through this module; the library's default otherwise) back afterwards.  Options are
    process-wide and read once per launch, so this is for the thread that issues the launches."""

    _defaults = {"max_ctas": 0, "group_m": 0, "tile_n": 0, "cta_group": 2, "epi_tma": 1, "split_tail": 1, "probe_ld_kb": 0, "probe_st_kb": 0}

    def __init__(self, name: str, value: int):
        self.name, self.value = name, int(value)

    def __enter__(self):
        self.previous = _option_values.get(self.name, self._defaults[self.name])
        set_option(self.name, self.value)
        return self

    def __exit__(self, *exc):
        set_option(self.name, self.previous)
        return False


# CODA_B200_OPTIONS="name=value,name=value": library options applied at import (same names as coda_b200_set_option).
for _item in filter(None, (s.strip() for s in os.environ.get("CODA_B200_OPTIONS", "").split(","))):
    _name, _, _value = _item.partition("=")
    set_option(_name.strip(), int(_value))
