"""Same public names as the reference's triton_kernels/residual_add.py, served by the CUDA operators of b200attn (b200attn/glue_ops.py)."""
from b200attn.glue_ops import residual_add  # noqa: F401


def call_residual_add_triton(x, residual):
    return residual_add(x, residual)
