"""Same public names as the reference's triton_kernels/gdn_gated_rmsnorm.py, served by the CUDA operators of b200attn (b200attn/glue_ops.py)."""
from b200attn.glue_ops import gdn_gated_rmsnorm  # noqa: F401


def call_gdn_gated_rmsnorm_triton(x, z, weight):
    return gdn_gated_rmsnorm(x, z, weight)
