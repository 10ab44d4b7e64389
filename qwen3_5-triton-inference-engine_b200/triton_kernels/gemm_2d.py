"""Same public names as the reference's triton_kernels/gemm_2d.py, served by the CUDA operators of b200attn (b200attn/glue_ops.py)."""
from b200attn.glue_ops import gemm_2d  # noqa: F401


def call_gemm_2d_triton(x, weight):
    return gemm_2d(x, weight)
