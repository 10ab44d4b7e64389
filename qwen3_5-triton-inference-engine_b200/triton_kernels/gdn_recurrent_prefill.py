"""Same public names as the reference's triton_kernels/gdn_recurrent_prefill.py, served by b200attn."""
from b200attn.ops import (  # noqa: F401
    call_gdn_recurrent_prefill_chunked_triton,
    gdn_chunk_output,
    gdn_chunk_prepare_wy,
    gdn_chunk_state,
    gdn_chunked_prefill_packed,
    gdn_recurrent_decode,
    gdn_recurrent_prefill_sequential,
)


def call_gdn_chunk_prepare_wy_triton(k, v, beta, g):
    return gdn_chunk_prepare_wy(k, v, beta, g)


def call_gdn_recurrent_prefill_sequential_triton(q, k, v, beta, g, cu_seqlens=None):
    return gdn_recurrent_prefill_sequential(q, k, v, beta, g, cu_seqlens)


def call_gdn_recurrent_decode_triton(q, k, v, beta, g, state):
    return gdn_recurrent_decode(q, k, v, beta, g, state)
