"""Same public names as the reference's triton_kernels/gdn_qk_norm_gates.py, served by the CUDA operators of b200attn (b200attn/glue_ops.py)."""
from b200attn.glue_ops import gdn_qk_norm_gates  # noqa: F401


def call_gdn_qk_norm_gates_triton(q, k, a, b, a_log, dt_bias):
    return gdn_qk_norm_gates(q, k, a, b, a_log, dt_bias)
