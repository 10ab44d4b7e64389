"""b200attn: sm_100a CUDA kernels for the attention / Gated-DeltaNet hot path, behind a C ABI
(libb200attn.so, include/b200_attn.h), exposed as the reference's `wy_lib::*` torch operators (ops.py)."""
from ._lib import B200Error, LIB_PATH, exported_symbols, load  # noqa: F401
