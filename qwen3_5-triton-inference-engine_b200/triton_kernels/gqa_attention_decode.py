"""Same public names as the reference's triton_kernels/gqa_attention_decode.py (the contiguous, single-sequence KV
cache that engine/cache.py allocates when paged=False), served by the paged CUDA operators of b200attn over an identity
page table (b200attn/glue_ops.py)."""
from b200attn.glue_ops import (  # noqa: F401
    allocate_contiguous_split_scratch as allocate_split_scratch,
    allocate_kv_cache,
    allocate_position,
    call_gqa_attention_decode_split_triton,
    kv_cache_from_prefill,
)
from b200attn.ops import MAX_SPLITS  # noqa: F401


def call_gqa_attention_decode_triton(q, k_new, v_new, k_cache, v_cache, past_len):
    """The unsplit form of the reference (triton_kernels/gqa_attention_decode.py:314-327) gives the same result as the
    split form; both are served by the same kernels."""
    return call_gqa_attention_decode_split_triton(q, k_new, v_new, k_cache, v_cache, past_len)
