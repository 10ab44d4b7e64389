"""Same public names as the reference's triton_kernels/embedding_gather.py, served by the CUDA operators of b200attn (b200attn/glue_ops.py)."""
from b200attn.glue_ops import embedding_gather  # noqa: F401


def call_embedding_gather_triton(input_ids, weight):
    return embedding_gather(input_ids, weight)
