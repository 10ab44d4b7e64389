"""Same public names as the reference's triton_kernels/gqa_attention_varlen_causal.py, served by b200attn."""
from b200attn.ops import build_cu_seqlens, fused_prefill_attention, gqa_attention_varlen_causal  # noqa: F401
