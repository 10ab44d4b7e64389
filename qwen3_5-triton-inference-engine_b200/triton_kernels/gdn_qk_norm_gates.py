"""Same module and symbol names as the reference's triton_kernels/gdn_qk_norm_gates.py; the operators here are the plain
PyTorch restatements of b200attn/glue.py (these operators are outside the attention / Gated-DeltaNet path)."""
from b200attn.glue import gdn_qk_norm_gates  # noqa: F401
