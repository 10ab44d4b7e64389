"""Same public names as the reference's triton_kernels/qwen_rmsnorm.py, served by the CUDA operators of b200attn (b200attn/glue_ops.py)."""
from b200attn.glue_ops import qwen_rmsnorm  # noqa: F401


def call_qwen_rmsnorm_triton(x, weight, eps=1e-6):
    return qwen_rmsnorm(x, weight, eps)
