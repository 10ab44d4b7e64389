"""Same public names as the reference's triton_kernels/gqa_attention_decode_paged.py, served by b200attn."""
from b200attn.ops import (  # noqa: F401
    MAX_SPLITS,
    PAGE_SIZE,
    allocate_paged_kv_cache,
    allocate_split_scratch,
    call_paged_gqa_attention_decode_triton,
    fused_decode_attention,
    fused_decode_workspace,
    paged_gqa_attention_decode_combine,
    paged_gqa_attention_decode_split,
    paged_kv_append,
    paged_kv_fill,
    paged_kv_fill_varlen,
    physical_rows,
)

PAGE = PAGE_SIZE
