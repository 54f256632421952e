"""The C-ABI library loads without a GPU and exports exactly what include/coda_b200.h declares."""

import ctypes
import re
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent


def declared_symbols() -> set[str]:
    text = (REPO / "include" / "coda_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(coda_b200_\w+)\s*\(", text))


def test_header_and_binding_agree():
    from coda_kernels_b200 import _lib

    decl = declared_symbols()
    assert decl, "no declarations found in include/coda_b200.h"
    assert decl == set(_lib.SIGNATURES), f"header vs ctypes table: {decl ^ set(_lib.SIGNATURES)}"


def test_library_exports_every_declared_symbol():
    from coda_kernels_b200 import _lib

    handle = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
    assert handle.coda_b200_version() >= 1


def test_host_side_argument_checks_need_no_gpu():
    from coda_kernels_b200 import _lib

    lib = _lib.lib
    assert lib.coda_b200_set_option(b"no_such_option", 1) == -1
    assert b"unknown option" in lib.coda_b200_last_error()
    assert lib.coda_b200_set_option(b"cta_group", 3) == -1
    assert lib.coda_b200_set_option(b"cta_group", 2) == 0
    # NULL operands are rejected before any CUDA call
    assert lib.coda_b200_gemm(None, 1, 1, None, 1, 1, None, 8, 0, 8, 8, 8, None, None, None) == -1
    assert lib.coda_b200_gemm_swiglu(None, 1, 1, None, 1, 1, None, 8, None, 8, 8, 8, 8, None, None) == -1
    assert lib.coda_b200_dswiglu(None, 8, None, 8, None, 8, 8, 8, None) == -1
    assert lib.coda_b200_lse_tiles(128256) == 501
    assert lib.coda_b200_lse_tiles(16032) == 63
    assert lib.coda_b200_qknorm_rope_bwd_scratch_bytes(16384, 128) == 1024 * 256 * 4
    with pytest.raises(_lib.CodaB200Error):
        _lib.check(-1, "probe")


def test_ops_refuse_cpu_tensors():
    import torch

    import coda_kernels_b200 as ck

    x = torch.zeros(8, 8, dtype=torch.bfloat16)
    w = torch.zeros(16, 8, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        ck.linear_swiglu(x, w)
    with pytest.raises(AssertionError):
        ck.linear_cross_entropy(x, w, torch.zeros(8, dtype=torch.int64))
    with pytest.raises(AssertionError):
        ck.linear_cross_entropy(x, w, torch.zeros(8, dtype=torch.int32), reduction="none")
