"""Same public names as the reference's triton_kernels/swiglu.py, served by the CUDA operators of b200attn (b200attn/glue_ops.py)."""
from b200attn.glue_ops import swiglu  # noqa: F401


def call_swiglu_triton(gate, up):
    return swiglu(gate, up)
