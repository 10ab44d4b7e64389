"""Same public names as the reference's triton_kernels/depthwise_causal_conv4_decode.py, served by the CUDA operators of b200attn (b200attn/glue_ops.py)."""
from b200attn.glue_ops import (  # noqa: F401
    CONV_KERNEL_SIZE,
    conv_state_from_packed_prefill,
    conv_state_from_prefill,
    conv_weight_for_decode,
    depthwise_causal_conv4_decode,
)


def call_depthwise_causal_conv4_decode_triton(x, state, weight):
    return depthwise_causal_conv4_decode(x, state, weight)
