"""ctypes binding of libb200attn.so (the C ABI declared in include/b200_attn.h).

There is no fallback: if the shared library is missing or a call returns non-zero, an exception is raised.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent.parent
LIB_PATH = PKG_DIR / "libb200attn.so"

P, I32, I64 = c_void_p, c_int32, c_int64

# name -> argument types, in the order of include/b200_attn.h
SIGNATURES: dict[str, list] = {
    "b200_paged_kv_append": [P, P, I64, I64, I64, I64, I64, I64, P, I64, I64, P, I64, I64, P, I64, P, I32, I32, I32, P],
    "b200_paged_kv_fill_varlen": [P, P, I64, I64, I64, I64, I64, I64, P, I64, I64, P, I64, I64, P, I64, P,
                                  I32, I32, I32, I32, P],
    "b200_paged_decode_split": [P, I64, I64, P, P, I64, I64, I64, I64, I64, I64, P, I64, P, P, P, P,
                                I32, I32, I32, I32, P],
    "b200_paged_decode_combine": [P, P, P, P, P, I32, I32, I32, P],
    "b200_fused_decode_attention": [P, I64, I64, P, I64, I64, P, I64, I64, P, I64, P, P, I64, I64, I64, I64, I64, I64,
                                    I64, P, I64, P, P, I32, P, P, I32, I32, I32, I32, P],
    "b200_fused_decode_attention_ex": [P, I64, I64, P, I64, I64, P, I64, I64, P, I64, P, P, I64, I64, I64, I64, I64,
                                       I64, I64, P, I64, P, P, I32, P, P, I32, I32, I32, I32, P, P, c_float, I32, I32, P],
    "b200_fused_decode_attention_static": [P, I64, I64, P, I64, I64, P, I64, I64, P, I64, P, P, I64, I64, I64, I64, I64,
                                           I64, I64, P, I64, P, P, I32, P, I32, I32, I32, I32, P],
    "b200_selftest_umma": [I32, P, P, P, P],
    "b200_selftest_wait_timeout": [P, P],
    "b200_gdn_recurrent_decode_form": [I32],
    "b200_set_chain_overlap": [I32],
    "b200_gqa_varlen_causal": [P, I64, I64, P, I64, I64, P, I64, I64, P, I64, I64, P, I32, I32, I32, I32, I32, I32, P],
    "b200_fused_prefill_attention": [P, I64, I64, P, I64, I64, P, I64, I64, P, I64, P, P, I64, I64, I64, I64, I64, I64,
                                     P, I64, P, P, I32, P, I32, P, P, I32, I32, I32, I32, I32, I32, P],
    "b200_partial_rope": [P, I64, I64, I64, P, I64, I64, I64, P, I32, I64, I64, P, I32, I32, I32, I32, I32, P],
    "b200_attention_gate_pack": [P, I64, I64, P, I64, I64, P, I32, I32, I32, P],
    "b200_gdn_recurrent_decode": [P, I64, I64, P, I64, I64, P, I64, I64, P, I64, I64, P, I64, I64, P, I64, I64,
                                  P, I64, I64, I32, I32, I32, I32, P],
    "b200_gdn_recurrent_prefill_sequential": [P, I64, I64, P, I64, I64, P, I64, I64, P, I64, I64, P, I64, I64, P,
                                              I32, I32, P, P, I64, I64, I32, I32, I32, P],
    "b200_gdn_chunk_prepare_wy": [P, I64, I64, P, I64, I64, P, I64, I64, P, I64, I64, P, P, P, I32, I32, I32, I32, P],
    "b200_gdn_chunk_state": [P, I64, I64, P, P, P, P, P, P, I32, I32, I32, I32, P],
    "b200_gdn_chunk_output": [P, I64, I64, P, I64, I64, P, P, P, P, I64, I64, I32, I32, I32, I32, P],
    "b200_gdn_chunked_prefill_packed": [P, I64, I64, P, I64, I64, P, I64, I64, P, I64, I64, P, I64, I64, P, I32, I32, I32,
                                        P, P, P, I64, I64, I32, I32, I32, P],
    "b200_skinny_gemm": [P, I64, P, P, I64, I32, I32, I32, I32, P],
    "b200_skinny_gemm_swiglu": [P, I64, P, P, I64, I32, I32, I32, I32, P],
    "b200_argmax_rows": [P, I64, P, P, I32, I32, I32, P],
    "b200_lm_head_argmax": [P, I64, P, P, P, I32, I32, I32, I32, P],
    "b200_add_rmsnorm": [P, I64, I64, I32, P, I64, P, P, P, I32, I32, c_float, I32, P],
    "b200_swiglu": [P, I64, P, I32, I32, I32, P],
    "b200_gdn_decode_prep": [P, I64, P, P, P, I64, P, I64, P, P, P, P, P, P, P, I32, I32, I32, P],
    "b200_gdn_decode_fused": [P, I64, P, P, P, P, P, P, P, I32, I32, I32, I32, P],
    "b200_gdn_gated_rmsnorm": [P, P, I64, P, P, I32, I32, I32, P],
    "b200_conv4_prefill": [P, I64, P, I64, I64, P, P, I64, I32, I32, P],
    "b200_conv4_decode": [P, I64, P, P, P, I64, I32, I32, P],
    "b200_conv_state_from_packed_prefill": [P, P, I64, P, I32, I32, P],
    "b200_gdn_qk_norm_gates": [P, I64, I64, P, I64, I64, P, I64, P, I64, P, P, P, P, P, P, I32, I32, I32, P],
    "b200_embedding_gather": [P, I32, P, P, I32, I32, P],
    "b200_residual_add": [P, P, P, I64, P],
    "b200_swiglu_pair": [P, I64, P, I64, P, I32, I32, P],
    "b200_gdn_chunked_prefill_fused": [P, I64, I64, P, I64, I64, P, I64, I64, P, I64, I64, P, I64, I64, P, I32, I32,
                                       P, P, I64, I64, I32, I32, I32, P],
}
OTHER = {
    "b200_last_error": ([], c_char_p),
    "b200_abi_version": ([], c_int),
    "b200_wait_timed_out": ([], c_int),
    "b200_fused_decode_workspace_bytes": ([], c_int64),
    "b200_argmax_rows_workspace_bytes": ([], c_int64),
    "b200_gdn_chunked_prefill_packed_workspace_bytes": ([I32, I32, I32], c_int64),
}

_lib = None


class B200Error(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Load the library once; raises if it has not been built (python build.py)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise B200Error(f"{LIB_PATH} not found: build it with `python {PKG_DIR / 'build.py'}`; there is no fallback path")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        for name, (argtypes, restype) in OTHER.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = lib
    return _lib


def exported_symbols() -> list[str]:
    return list(SIGNATURES) + list(OTHER)


def call(name: str, *args) -> None:
    lib = load()
    status = getattr(lib, name)(*args)
    if status != 0:
        raise B200Error(f"{name} failed with status {status}: {lib.b200_last_error().decode()}")
