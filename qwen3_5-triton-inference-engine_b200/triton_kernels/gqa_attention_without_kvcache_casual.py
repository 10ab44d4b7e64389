"""Same public names as the reference's triton_kernels/gqa_attention_without_kvcache_casual.py, served by the CUDA operators of b200attn (b200attn/glue_ops.py)."""
from b200attn.glue_ops import gqa_attention_without_kvcache_casual  # noqa: F401


def call_gqa_attention_without_kvcache_casual_triton(q, k, v):
    return gqa_attention_without_kvcache_casual(q, k, v)
