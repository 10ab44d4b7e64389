"""Same public names as the reference's triton_kernels/depthwise_causal_conv4_prefill.py, served by the CUDA operators of b200attn (b200attn/glue_ops.py)."""
import torch

from b200attn.glue_ops import depthwise_causal_conv4_prefill  # noqa: F401


def call_depthwise_causal_conv4_prefill_triton(x, weight, seq_start=None):
    return depthwise_causal_conv4_prefill(x, weight, seq_start)


def build_seq_start(lengths, *, device="cuda"):
    """Length list -> [total_tokens] int32: for every packed token the first row of its own sequence
    (triton_kernels/depthwise_causal_conv4_prefill.py:195-206)."""
    starts, acc = [], 0
    for n in lengths:
        starts.append(acc)
        acc += n
    return torch.repeat_interleave(torch.tensor(starts, dtype=torch.int32, device=device),
                                   torch.tensor(lengths, device=device))
