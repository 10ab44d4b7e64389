"""Same public names as the reference's triton_kernels/vocab_argmax.py, served by the CUDA operators of b200attn (b200attn/glue_ops.py)."""
from b200attn.glue_ops import lm_head_argmax  # noqa: F401


def call_lm_head_argmax_triton(hidden, weight, last_only=True):
    return lm_head_argmax(hidden, weight, last_only)
