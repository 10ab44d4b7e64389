"""Same module and symbol names as the reference's triton_kernels/vocab_argmax.py; the operators here are the plain
PyTorch restatements of b200attn/glue.py (these operators are outside the attention / Gated-DeltaNet path)."""
from b200attn.glue import lm_head_argmax  # noqa: F401
