"""The C-ABI library loads and exports every symbol include/b200_decode.h declares (CPU, no compute)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT, pkg


def _declared():
    text = open(os.path.join(ROOT, "include", "b200_decode.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared()
    for must in ("b200_paged_attn_decode", "b200_kv_append", "b200_moe_route", "b200_moe_permute",
                 "b200_moe_fp8_gemm_gate_up", "b200_moe_fp8_gemm_down", "b200_moe_combine",
                 "b200_moe_fp8_forward", "b200_strerror"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib_mod = pkg("_lib")
    if not os.path.exists(lib_mod.LIB_PATH):
        pkg("build").build_library()
    lib = ctypes.CDLL(lib_mod.LIB_PATH)
    for name in _declared():
        assert hasattr(lib, name), f"{name} declared in b200_decode.h but not exported"


def test_binding_covers_every_declared_symbol():
    assert sorted(pkg("_lib").SIGNATURES) == _declared()


def test_host_side_calls_that_need_no_gpu():
    lib = pkg("_lib").load()
    assert lib.b200_abi_version() == 1
    assert b"barrier" in lib.b200_strerror(-18)
    assert lib.b200_moe_max_tiles(256, 128, 8) == 256 * 8 // 128 + 128
    n = lib.b200_paged_attn_workspace_bytes(64, 32, 128, 512, 16, 512)
    assert n >= 256 + 64 * 32 * 16 * (8 + 128 * 4)
    assert lib.b200_moe_fp8_workspace_bytes(256, 128, 8, 2048, 768) > 256 * 8 * (2048 * 3 + 768)


def test_null_pointer_is_rejected_on_the_host():
    lib = pkg("_lib").load()
    rc = lib.b200_moe_route(None, 1, 4, 16, 4, 1, None, None, None, None)
    assert rc == -1 and b"null" in lib.b200_last_error_detail()


def test_ops_refuse_cpu_tensors():
    import torch

    ops = pkg("ops")
    with pytest.raises(ValueError, match="CUDA"):
        ops.moe_route(torch.zeros(2, 16), 4)
