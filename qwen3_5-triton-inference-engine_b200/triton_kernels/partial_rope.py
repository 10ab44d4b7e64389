"""Same public names as the reference's triton_kernels/partial_rope.py, served by b200attn."""
from b200attn.ops import partial_rope  # noqa: F401


def call_partial_rope_triton(x, position_ids, inv_freq, rotary_dim):
    return partial_rope(x, position_ids, inv_freq, rotary_dim)
