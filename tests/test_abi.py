"""CPU-side checks of the drop-in boundary: the C-ABI library loads and exports every symbol the header declares,
the `wy_lib::*` operators carry the reference's schemas, and nothing runs on CPU tensors (no fallback)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b200_attn.h"

# printed from torch.ops.wy_lib.<op>._schema of the reference package
REFERENCE_SCHEMAS = {
    "paged_kv_append": "wy_lib::paged_kv_append(Tensor(a0!) k_cache, Tensor(a1!) v_cache, Tensor k_new, Tensor v_new, Tensor block_table, Tensor pos) -> ()",
    "paged_kv_fill_varlen": "wy_lib::paged_kv_fill_varlen(Tensor(a0!) k_cache, Tensor(a1!) v_cache, Tensor k_packed, Tensor v_packed, Tensor block_table, Tensor cu_seqlens, SymInt max_seqlen) -> ()",
    "paged_gqa_attention_decode_split": "wy_lib::paged_gqa_attention_decode_split(Tensor q, Tensor k_cache, Tensor v_cache, Tensor block_table, Tensor(a4!) m_partial, Tensor(a5!) l_partial, Tensor(a6!) acc_partial, Tensor pos, SymInt seq_bucket) -> ()",
    "paged_gqa_attention_decode_combine": "wy_lib::paged_gqa_attention_decode_combine(Tensor m_partial, Tensor l_partial, Tensor acc_partial, Tensor pos) -> Tensor",
    "partial_rope": "wy_lib::partial_rope(Tensor x, Tensor position_ids, Tensor inv_freq, SymInt rotary_dim) -> Tensor",
    "attention_gate_pack": "wy_lib::attention_gate_pack(Tensor x, Tensor gate) -> Tensor",
    "gdn_recurrent_decode": "wy_lib::gdn_recurrent_decode(Tensor q, Tensor k, Tensor v, Tensor beta, Tensor g, Tensor(a5!) state) -> Tensor",
    "gdn_recurrent_prefill_sequential": "wy_lib::gdn_recurrent_prefill_sequential(Tensor q, Tensor k, Tensor v, Tensor beta, Tensor g, Tensor? cu_seqlens=None) -> (Tensor, Tensor)",
    "gqa_attention_varlen_causal": "wy_lib::gqa_attention_varlen_causal(Tensor q, Tensor k, Tensor v, Tensor cu_seqlens, SymInt max_seqlen) -> Tensor",
    "gdn_chunk_prepare_wy": "wy_lib::gdn_chunk_prepare_wy(Tensor k, Tensor v, Tensor beta, Tensor g) -> (Tensor, Tensor, Tensor)",
    "gdn_chunk_state": "wy_lib::gdn_chunk_state(Tensor k, Tensor w, Tensor u_base, Tensor g_cumsum) -> (Tensor, Tensor, Tensor)",
    "gdn_chunk_output": "wy_lib::gdn_chunk_output(Tensor q, Tensor k, Tensor delta, Tensor g_cumsum, Tensor chunk_state) -> Tensor",
    # the operators around the path (b200attn/glue_ops.py)
    "conv_state_from_packed_prefill": "wy_lib::conv_state_from_packed_prefill(Tensor(a0!) state, Tensor x, Tensor cu_seqlens) -> ()",
    "depthwise_causal_conv4_decode": "wy_lib::depthwise_causal_conv4_decode(Tensor x, Tensor(a1!) state, Tensor weight) -> Tensor",
    "depthwise_causal_conv4_prefill": "wy_lib::depthwise_causal_conv4_prefill(Tensor x, Tensor weight, Tensor? seq_start=None) -> Tensor",
    "embedding_gather": "wy_lib::embedding_gather(Tensor input_ids, Tensor weight) -> Tensor",
    "gdn_gated_rmsnorm": "wy_lib::gdn_gated_rmsnorm(Tensor x, Tensor z, Tensor weight) -> Tensor",
    "gdn_qk_norm_gates": "wy_lib::gdn_qk_norm_gates(Tensor q, Tensor k, Tensor a, Tensor b, Tensor a_log, Tensor dt_bias) -> (Tensor, Tensor, Tensor, Tensor)",
    "gemm_2d": "wy_lib::gemm_2d(Tensor x, Tensor weight) -> Tensor",
    "gqa_attention_without_kvcache_casual": "wy_lib::gqa_attention_without_kvcache_casual(Tensor q, Tensor k, Tensor v) -> Tensor",
    "lm_head_argmax": "wy_lib::lm_head_argmax(Tensor hidden, Tensor weight, bool last_only=True) -> Tensor",
    "qwen_rmsnorm": "wy_lib::qwen_rmsnorm(Tensor x, Tensor weight, float eps=9.9999999999999995e-07) -> Tensor",
    "residual_add": "wy_lib::residual_add(Tensor x, Tensor residual) -> Tensor",
    "swiglu": "wy_lib::swiglu(Tensor gate, Tensor up) -> Tensor",
}


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import b200attn

    lib = b200attn.load()
    names = declared_symbols()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/b200_attn.h but not exported"
    assert lib.b200_abi_version() == 1
    assert set(b200attn.exported_symbols()) == set(names), "ctypes table and header disagree"
    raw = ctypes.CDLL(str(b200attn.LIB_PATH))
    assert raw.b200_fused_decode_workspace_bytes.restype is not None


def test_operator_schemas_match_reference():
    from b200attn import glue_ops, ops  # noqa: F401  (importing registers the operators)

    for name, schema in REFERENCE_SCHEMAS.items():
        if not hasattr(torch.ops.wy_lib, name):
            pytest.fail(f"wy_lib::{name} is not registered")
        assert str(getattr(torch.ops.wy_lib, name).default._schema) == schema


def test_shim_modules_export_reference_names():
    import importlib

    expected = {
        "gqa_attention_decode_paged": ["PAGE_SIZE", "MAX_SPLITS", "allocate_paged_kv_cache", "allocate_split_scratch",
                                       "physical_rows", "paged_kv_append", "paged_kv_fill", "paged_kv_fill_varlen",
                                       "paged_gqa_attention_decode_split", "paged_gqa_attention_decode_combine",
                                       "call_paged_gqa_attention_decode_triton"],
        "gqa_attention_varlen_causal": ["gqa_attention_varlen_causal", "build_cu_seqlens"],
        "gdn_recurrent_prefill": ["gdn_recurrent_decode", "gdn_recurrent_prefill_sequential", "gdn_chunk_prepare_wy",
                                  "gdn_chunk_state", "gdn_chunk_output", "call_gdn_recurrent_prefill_chunked_triton"],
        "partial_rope": ["partial_rope"],
        "attention_gate_pack": ["attention_gate_pack"],
    }
    for mod, names in expected.items():
        m = importlib.import_module(f"triton_kernels.{mod}")
        for n in names:
            assert hasattr(m, n), f"triton_kernels.{mod}.{n} missing"
    from triton_kernels.gqa_attention_decode_paged import MAX_SPLITS, PAGE_SIZE
    assert (PAGE_SIZE, MAX_SPLITS) == (16, 128)


def test_no_cpu_fallback():
    """CPU tensors must be refused, not silently computed somewhere else."""
    from b200attn import ops

    x = torch.zeros(1, 2, 3, 8, dtype=torch.bfloat16)
    with pytest.raises((NotImplementedError, AssertionError, RuntimeError)):
        ops.partial_rope(x, torch.zeros(1, 3, dtype=torch.int64), torch.ones(2), 4)
    kc = torch.zeros(2, 2, 16, 256, dtype=torch.bfloat16)
    with pytest.raises((NotImplementedError, AssertionError, RuntimeError)):
        ops.paged_kv_append(kc, kc.clone(), kc[:1, :, 0], kc[:1, :, 0], torch.zeros(1, 2, dtype=torch.int32),
                            torch.zeros(1, dtype=torch.int64))


def test_allocators_and_physical_rows():
    from b200attn import ops
    from oracle import reference_ops as O

    k, v = ops.allocate_paged_kv_cache(5, 2, 256, device="cpu")
    assert k.shape == (5, 2, 16, 256) and k.dtype == torch.bfloat16 and not k.any() and v.shape == k.shape
    m, l, acc = ops.allocate_split_scratch(8, 256, batch=3, device="cpu")
    assert m.shape == l.shape == (3, 8, 128) and acc.shape == (3, 8, 128, 256) and acc.dtype == torch.float32
    table = torch.tensor([7, 2, 9], dtype=torch.int32)
    tok = torch.tensor([0, 15, 16, 33, 47], dtype=torch.int64)
    rows = ops.physical_rows(table, tok, 2)
    assert torch.equal(rows, O.physical_rows(table, tok, 2))
    assert rows[3].tolist() == [(9 * 2 + 0) * 16 + 1, (9 * 2 + 1) * 16 + 1]
