"""Same module and symbol names as the reference's triton_kernels/embedding_gather.py; the operators here are the plain
PyTorch restatements of b200attn/glue.py (these operators are outside the attention / Gated-DeltaNet path)."""
from b200attn.glue import embedding_gather  # noqa: F401
