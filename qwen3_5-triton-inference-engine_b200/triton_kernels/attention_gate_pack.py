"""Same public names as the reference's triton_kernels/attention_gate_pack.py, served by b200attn."""
from b200attn.ops import attention_gate_pack  # noqa: F401


def call_attention_gate_pack_triton(x, gate):
    return attention_gate_pack(x, gate)
