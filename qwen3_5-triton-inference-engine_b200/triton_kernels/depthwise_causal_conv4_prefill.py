"""Same module and symbol names as the reference's triton_kernels/depthwise_causal_conv4_prefill.py; the operators here are the plain
PyTorch restatements of b200attn/glue.py (these operators are outside the attention / Gated-DeltaNet path)."""
from b200attn.glue import depthwise_causal_conv4_prefill  # noqa: F401
