"""Same public names as the reference's triton_kernels/gdn_recurrent_prefill.py, served by b200attn."""
from b200attn.ops import gdn_recurrent_decode, gdn_recurrent_prefill_sequential  # noqa: F401


def call_gdn_recurrent_prefill_sequential_triton(q, k, v, beta, g, cu_seqlens=None):
    return gdn_recurrent_prefill_sequential(q, k, v, beta, g, cu_seqlens)


def call_gdn_recurrent_decode_triton(q, k, v, beta, g, state):
    return gdn_recurrent_decode(q, k, v, beta, g, state)
