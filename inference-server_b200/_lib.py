"""ctypes binding of libb200decode.so.

Every exported symbol of ``include/b200_decode.h`` gets its argument and result
types here.  There is no fallback: if the shared library is missing or a symbol
cannot be resolved, importing callers get a ``RuntimeError`` that says how to
build it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200decode.so")

# name -> (restype, argtypes); order follows include/b200_decode.h
SIGNATURES = {
    "b200_abi_version": (c_int, []),
    "b200_strerror": (c_char_p, [c_int]),
    "b200_last_error_detail": (c_char_p, []),
    "b200_read_status": (c_int, [c_void_p, c_void_p]),
    "b200_paged_attn_workspace_bytes": (c_size_t, [c_int] * 6),
    "b200_paged_attn_decode": (
        c_int,
        [c_void_p] * 7 + [c_size_t] + [c_int] * 7 + [c_float, c_int, c_int, c_void_p],
    ),
    "b200_paged_attn_decode_pairs": (c_int, [c_void_p] * 7 + [c_size_t] + [c_int] * 7 + [c_float, c_int, c_void_p]),
    "b200_paged_attn_prefill": (c_int, [c_void_p] * 6 + [c_int] * 8 + [c_float, c_void_p]),
    "b200_paged_attn_decode_static": (c_int, [c_void_p] * 7 + [c_int] * 7 + [c_float, c_int, c_void_p]),
    "b200_kv_append": (c_int, [c_void_p] * 7 + [c_int] * 7 + [c_void_p]),
    "b200_dense_gemm_workspace_bytes": (c_size_t, [c_int, c_int]),
    "b200_dense_gemm_bf16": (c_int, [c_void_p] * 4 + [c_size_t, c_void_p] + [c_int] * 4 + [c_void_p]),
    "b200_qkv_rope_append_supported": (c_int, [c_int, c_int]),
    "b200_qkv_rope_append_gemm": (c_int, [c_void_p] * 12 + [c_int] * 5 + [c_float] + [c_int] * 4 + [c_void_p]),
    "b200_lm_head_argmax_workspace_bytes": (c_size_t, []),
    "b200_lm_head_argmax": (c_int, [c_void_p] * 4 + [c_size_t, c_void_p] + [c_int] * 3 + [c_void_p]),
    "b200_add_rmsnorm_route_supported": (c_int, [c_int] * 3),
    "b200_add_rmsnorm_route": (c_int, [c_void_p] * 3 + [c_float, c_void_p] + [c_int] * 5 + [c_void_p] * 6),
    "b200_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_void_p]),
    "b200_qk_norm_rope_append": (c_int, [c_void_p] * 11 + [c_int] * 4 + [c_float] + [c_int] * 4 + [c_void_p]),
    "b200_moe_route": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200_moe_permute_workspace_bytes": (c_size_t, [c_int] * 3),
    "b200_moe_max_tiles": (c_int, [c_int] * 3),
    "b200_moe_permute": (
        c_int,
        [c_void_p, c_int, c_int, c_int] + [c_void_p] * 5 + [c_int, c_void_p, c_size_t, c_void_p],
    ),
    "b200_moe_permute_quant": (c_int, [c_void_p, c_void_p] + [c_int] * 4 + [c_void_p] * 8 + [c_size_t, c_void_p]),
    "b200_moe_permute_quant_ep": (c_int, [c_void_p, c_void_p] + [c_int] * 6 + [c_void_p] * 11 + [c_size_t, c_void_p]),
    "b200_gather_rows_fp8": (c_int, [c_void_p] * 3 + [c_int, c_int] + [c_void_p] * 3),
    "b200_act_quant_fp8": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_moe_fp8_gemm_gate_up": (c_int, [c_void_p] * 9 + [c_int] * 5 + [c_void_p]),
    "b200_moe_fp8_gemm_down": (c_int, [c_void_p] * 9 + [c_int] * 5 + [c_void_p]),
    "b200_moe_combine": (c_int, [c_void_p] * 3 + [c_int] * 3 + [c_void_p, c_void_p]),
    "b200_moe_combine_add_rmsnorm": (c_int, [c_void_p] * 5 + [c_float] + [c_int] * 3 + [c_void_p, c_void_p]),
    "b200_moe_fp8_workspace_bytes": (c_size_t, [c_int] * 5),
    "b200_moe_fp8_forward": (c_int, [c_void_p, c_void_p, c_int] + [c_void_p] * 6 + [c_size_t] + [c_int] * 7 + [c_void_p]),
    "b200_moe_fp8_forward_add_rmsnorm": (
        c_int, [c_void_p, c_void_p, c_int] + [c_void_p] * 6 + [c_float] + [c_void_p] * 2 + [c_size_t] + [c_int] * 7 + [c_void_p]),
    "b200_moe_fp8_routed_add_rmsnorm": (
        c_int, [c_void_p] * 9 + [c_float] + [c_void_p] * 2 + [c_size_t] + [c_int] * 6 + [c_void_p]),
    # expert parallelism over peer memory (no counterpart in the reference)
    "b200_moe_permute_quant_ep_p2p": (c_int, [c_void_p, c_void_p] + [c_int] * 7 + [c_void_p] * 11 + [c_size_t, c_void_p]),
    "b200_moe_fp8_gemm_down_p2p": (c_int, [c_void_p] * 9 + [c_int] * 8 + [c_void_p]),
    "b200_moe_permute_gather_fp8": (c_int, [c_void_p] + [c_int] * 3 + [c_void_p, c_void_p, c_int] + [c_void_p] * 8
                                    + [c_size_t, c_void_p]),
    "b200_ep_signal": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "b200_ep_wait": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "b200_ep_barrier": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "b200_ipc_export": (c_int, [c_void_p, c_void_p, c_void_p]),
    "b200_ipc_import": (c_int, [c_void_p, ctypes.c_uint64, c_void_p, c_void_p]),
    "b200_ipc_close": (c_int, [c_void_p]),
}

_lib = None


class B200Error(RuntimeError):
    """A C-ABI call returned a negative code, or the device status word is set."""

    def __init__(self, code: int, where: str, detail: str = ""):
        self.code = code
        text = strerror(code)
        super().__init__(f"{where}: {text} (code {code})" + (f": {detail}" if detail else ""))


def load() -> ctypes.CDLL:
    """Load the library once and type every symbol. Raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing. Build it with `python inference-server_b200/build.py` "
            "(needs nvcc); there is no fallback implementation."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise RuntimeError(f"{LIB_PATH} does not export {name}; rebuild the library") from e
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().b200_strerror(int(code)).decode()


def check(rc: int, where: str) -> None:
    """Raise B200Error when a C-ABI call returned non-zero."""
    if rc != 0:
        detail = load().b200_last_error_detail().decode()
        raise B200Error(rc, where, detail)
