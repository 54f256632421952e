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


def test_qknorm_rope_bwd_rejects_rows_that_do_not_fit_their_leading_dimension():
    """The backward kernel reads and writes whole rows with 16-byte accesses: a leading dimension shorter than the row
    is refused on the host (fake, aligned, never dereferenced addresses: no GPU needed)."""
    from coda_kernels_b200 import _lib

    lib = _lib.lib
    p = 1 << 20  # 16-byte aligned stand-in for every device pointer
    hq, hk, d, nv, M = 4, 2, 128, 256, 64
    size_qk = (hq + hk) * d

    def call(ld_dq=hq * d, ld_dk=hk * d, ld_dv=nv, ld_pre=size_qk, ld_grad=size_qk + nv, dv=p, nv_=nv, scratch_bytes=1 << 20):
        return lib.coda_b200_qknorm_rope_bwd(p, ld_dq, p, ld_dk, dv, ld_dv, nv_, p, ld_pre, p, p, p, 0, p, d, hq, hk, 1e-6, p, ld_grad,
                                             p, p, scratch_bytes, M, None)

    for kwargs, text in (
        ({"ld_grad": size_qk + nv - 8}, b"ld_grad"),
        ({"ld_pre": size_qk - 8}, b"ld_pre"),
        ({"ld_dq": hq * d - 8}, b"ld_dq"),
        ({"ld_dk": hk * d - 8}, b"ld_dk"),
        ({"ld_dv": nv - 8}, b"ld_dv"),
        ({"dv": None}, b"dv is required"),
    ):
        assert call(**kwargs) == -1, kwargs
        assert text in lib.coda_b200_last_error(), (kwargs, lib.coda_b200_last_error())
    assert call(scratch_bytes=0) == -1 and b"scratch" in lib.coda_b200_last_error()


def test_options_accept_only_documented_values():
    from coda_kernels_b200 import _lib

    lib = _lib.lib
    for name, bad, good in ((b"tile_n", 96, 0), (b"epi_tma", 2, 1), (b"split_tail", 2, 1), (b"group_m", -1, 0), (b"max_ctas", -5, 0),
                            (b"probe_ld_kb", 1000, 0), (b"probe_st_kb", -1, 0)):
        assert lib.coda_b200_set_option(name, bad) == -1
        assert lib.coda_b200_set_option(name, good) == 0
    assert lib.coda_b200_set_option(b"dbg_lbo_mn", 1) == -1, "bring-up knobs are gone from the ABI"


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


def test_option_override_restores_the_previous_value():
    from coda_kernels_b200 import _lib

    _lib.set_option("max_ctas", 0)
    with _lib.option_override("max_ctas", 116):
        assert _lib._option_values["max_ctas"] == 116
        with _lib.option_override("max_ctas", 64):
            assert _lib._option_values["max_ctas"] == 64
        assert _lib._option_values["max_ctas"] == 116
    assert _lib._option_values["max_ctas"] == 0
    with pytest.raises(_lib.CodaB200Error):
        with _lib.option_override("max_ctas", -7):
            pass
    assert _lib._option_values["max_ctas"] == 0
    # the workspace query is plain host arithmetic (it may look up the SM count, which needs a GPU; without one the
    # library falls back to a B200's 148)
    assert _lib.lib.coda_b200_gemm_workspace_bytes(16384, 64, 4096) == 0, "narrow outputs keep their narrow tiles"
    assert _lib.lib.coda_b200_gemm_workspace_bytes(3584, 4096, 16384) == 2 * 74 * 256 * 256 * 4, "224 tiles on 74 CTA pairs: two tail tiles to cut"
    assert _lib.lib.coda_b200_gemm_workspace_bytes(16384, 4096, 28672) == 0, "62 tail tiles cannot be cut profitably"
    with _lib.option_override("split_tail", 0):
        assert _lib.lib.coda_b200_gemm_workspace_bytes(3584, 4096, 16384) == 0
