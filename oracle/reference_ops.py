"""CPU oracle: a restatement of the reference operators' arithmetic, rounding point by rounding point.

THIS IS TEST INFRASTRUCTURE.  Only tests/, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of bench.py may import it, and only as the checker or the timed CPU
baseline.  The product (the CUDA library and its Python boundary) never calls into this module and has
no CPU fallback.

Parity is PINNED: every function here is checked in tests/test_oracle_golden.py against outputs of the
reference's own operators, produced by tests/golden/make_golden.py (reference kernels executed by the
Triton interpreter on the CPU).

All functions take and return CPU torch tensors.  bf16 rounding is done with ``.to(torch.bfloat16)``
(round-to-nearest-even, same as the kernels' stores).  Citations are ``file:line`` inside the
reference project.
"""
from __future__ import annotations

import math

import torch

PAGE_SIZE = 16     # triton_kernels/gqa_attention_decode_paged.py:91
MAX_SPLITS = 128   # triton_kernels/gqa_attention_decode_paged.py:95
CHUNK = 64         # triton_kernels/gdn_recurrent_prefill.py:722
LOG2E = 1.4426950408889634


def _cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


# =========================================================================== page / index work
def physical_rows(block_table_row: torch.Tensor, token_index: torch.Tensor, num_kv_heads: int):
    """row(t,h) = (block_table[t // PAGE] * H + h) * PAGE + t % PAGE, shape [T, H].
    triton_kernels/gqa_attention_decode_paged.py:127-144."""
    lp = token_index // PAGE_SIZE
    slot = token_index % PAGE_SIZE
    phys = block_table_row.to(torch.int64)[lp]
    heads = torch.arange(num_kv_heads, dtype=torch.int64)
    return (phys[:, None] * num_kv_heads + heads[None, :]) * PAGE_SIZE + slot[:, None]


def paged_kv_append(k_cache, v_cache, k_new, v_new, block_table, pos) -> None:
    """cache[block_table[b, pos[b] // 16], h, pos[b] % 16, :] = new[b, h, :] for K and V, in place.
    triton_kernels/gqa_attention_decode_paged.py:232-250."""
    batch = k_new.shape[0]
    for b in range(batch):
        p = int(pos[b])
        phys = int(block_table[b, p // PAGE_SIZE])
        k_cache[phys, :, p % PAGE_SIZE, :] = k_new[b]
        v_cache[phys, :, p % PAGE_SIZE, :] = v_new[b]


def paged_kv_fill_varlen(k_cache, v_cache, k_packed, v_packed, block_table, cu_seqlens) -> None:
    """Scatter packed [H_kv, T, D] K/V into the pages of each sequence; slots past the sequence end
    keep their old bytes.  triton_kernels/gqa_attention_decode_paged.py:461-489."""
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        start, n = cu[b], cu[b + 1] - cu[b]
        for lp in range(_cdiv(n, PAGE_SIZE)):
            phys = int(block_table[b, lp])
            cnt = min(PAGE_SIZE, n - lp * PAGE_SIZE)
            t0 = start + lp * PAGE_SIZE
            k_cache[phys, :, :cnt, :] = k_packed[:, t0 : t0 + cnt, :]
            v_cache[phys, :, :cnt, :] = v_packed[:, t0 : t0 + cnt, :]


# =========================================================================== paged decode attention
def split_geometry(pos_b: int):
    """(seq_len, pages_used, pages_per_split, num_active) exactly as both kernels recompute them.
    triton_kernels/gqa_attention_decode_paged.py:677-682 and :781-784."""
    seq_len = pos_b + 1
    npu = _cdiv(seq_len, PAGE_SIZE)
    pps = _cdiv(npu, MAX_SPLITS)
    return seq_len, npu, pps, _cdiv(npu, pps)


def paged_decode_split(q, k_cache, v_cache, block_table, m_partial, l_partial, acc_partial, pos) -> None:
    """Split-K online softmax over page ranges; writes (m, l, acc) for ALL 128 splits, empty ones as
    (-inf, 0, 0).  qk in fp32 times scale, p = exp(qk - m) in fp32, p rounded to bf16 for the PV
    product while l sums the unrounded p.  triton_kernels/gqa_attention_decode_paged.py:675-733."""
    batch, hq, d = q.shape
    hkv = k_cache.shape[1]
    group = hq // hkv
    scale = d ** -0.5
    qf = q.float()
    for b in range(batch):
        seq_len, npu, pps, _ = split_geometry(int(pos[b]))
        for h in range(hkv):
            qh = qf[b, h * group : (h + 1) * group]  # [G, D]
            for s in range(MAX_SPLITS):
                m_i = torch.full((group,), -math.inf)
                l_i = torch.zeros(group)
                acc = torch.zeros(group, d)
                for lp in range(s * pps, min(s * pps + pps, npu)):
                    phys = int(block_table[b, lp])
                    k = k_cache[phys, h].float()  # [PAGE, D]
                    v = v_cache[phys, h].float()
                    qk = (qh @ k.t()) * scale
                    tok = lp * PAGE_SIZE + torch.arange(PAGE_SIZE)
                    qk = torch.where(tok[None, :] < seq_len, qk, torch.tensor(-math.inf))
                    m_new = torch.maximum(m_i, qk.max(dim=1).values)
                    alpha = torch.exp(m_i - m_new)
                    p = torch.exp(qk - m_new[:, None])
                    acc = acc * alpha[:, None] + p.to(torch.bfloat16).float() @ v
                    l_i = l_i * alpha + p.sum(dim=1)
                    m_i = m_new
                sl = slice(h * group, (h + 1) * group)
                m_partial[b, sl, s] = m_i
                l_partial[b, sl, s] = l_i
                acc_partial[b, sl, s] = acc


def paged_decode_combine(m_partial, l_partial, acc_partial, pos) -> torch.Tensor:
    """out = sum_s exp(m_s - m) acc_s / sum_s exp(m_s - m) l_s over the first num_active splits, bf16.
    triton_kernels/gqa_attention_decode_paged.py:780-817."""
    batch, hq, _, d = acc_partial.shape
    out = torch.empty(batch, hq, d, dtype=torch.bfloat16)
    for b in range(batch):
        _, _, _, num_active = split_geometry(int(pos[b]))
        m_all = m_partial[b, :, :num_active]
        l_all = l_partial[b, :, :num_active]
        a_all = acc_partial[b, :, :num_active]
        m = m_all.max(dim=-1, keepdim=True).values
        alpha = torch.exp(m_all - m)
        l = (l_all * alpha).sum(dim=-1)
        out[b] = ((a_all * alpha[..., None]).sum(dim=1) / l[:, None]).to(torch.bfloat16)
    return out


def paged_decode(q, k_new, v_new, k_cache, v_cache, block_table, pos, scratch=None) -> torch.Tensor:
    """append -> split -> combine.  triton_kernels/gqa_attention_decode_paged.py:963-994."""
    batch, hq, d = q.shape
    if scratch is None:
        scratch = (
            torch.zeros(batch, hq, MAX_SPLITS), torch.zeros(batch, hq, MAX_SPLITS),
            torch.zeros(batch, hq, MAX_SPLITS, d),
        )
    paged_kv_append(k_cache, v_cache, k_new, v_new, block_table, pos)
    paged_decode_split(q, k_cache, v_cache, block_table, *scratch, pos)
    return paged_decode_combine(*scratch, pos)


def gather_sequence(cache, block_table_row, length: int, num_kv_heads: int):
    """[H_kv, length, D] view of one sequence's cached rows (page table applied)."""
    d = cache.shape[-1]
    rows = physical_rows(block_table_row, torch.arange(length, dtype=torch.int64), num_kv_heads)
    return cache.reshape(-1, d)[rows.t().reshape(-1)].view(num_kv_heads, length, d)


def paged_decode_exact(q, k_cache, v_cache, block_table, lengths) -> torch.Tensor:
    """fp32 softmax attention over the first lengths[b] cached tokens (no bf16 rounding of p), the
    'eager PyTorch-CPU math' form.  triton_kernels/gqa_attention_decode_paged.py:999-1031.
    Returns fp32 [B, H_q, D]."""
    batch, hq, d = q.shape
    hkv = k_cache.shape[1]
    group = hq // hkv
    outs = []
    for b in range(batch):
        t = int(lengths[b])
        k = gather_sequence(k_cache, block_table[b], t, hkv).float().repeat_interleave(group, 0)
        v = gather_sequence(v_cache, block_table[b], t, hkv).float().repeat_interleave(group, 0)
        scores = torch.einsum("hd,htd->ht", q[b].float(), k) * d ** -0.5
        outs.append(torch.einsum("ht,htd->hd", torch.softmax(scores, dim=-1), v))
    return torch.stack(outs)


# =========================================================================== varlen causal prefill
def varlen_causal(q, k, v, cu_seqlens, tile_kv: int = 32, block_q: int = 16) -> torch.Tensor:
    """Packed block-diagonal causal GQA.  q is multiplied by scale*log2(e) and RE-ROUNDED to bf16 before
    QK^T; exp2 softmax tile by tile; p rounded to bf16 for PV, l from fp32 p.
    triton_kernels/gqa_attention_varlen_causal.py:125-210 (tile sizes = its first autotune config)."""
    total, hq, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    qk_scale = (1.0 / math.sqrt(d)) * LOG2E
    out = torch.zeros_like(q)
    cu = cu_seqlens.tolist()
    neg = torch.tensor(-math.inf)
    for b in range(len(cu) - 1):
        s0, n = cu[b], cu[b + 1] - cu[b]
        for h in range(hkv):
            kh = k[s0 : s0 + n, h].float()
            vh = v[s0 : s0 + n, h].float()
            for qb in range(_cdiv(n, block_q)):
                rows = torch.arange(qb * block_q, min((qb + 1) * block_q, n))
                qt = q[s0 + rows, h * group : (h + 1) * group].float()        # [R, G, D]
                qt = (qt * qk_scale).to(torch.bfloat16).float().permute(1, 0, 2)  # [G, R, D]
                m_i = torch.full((group, len(rows)), -math.inf)
                l_i = torch.zeros(group, len(rows))
                acc = torch.zeros(group, len(rows), d)
                for t0 in range(0, (qb + 1) * block_q, tile_kv):
                    cols = torch.arange(t0, t0 + tile_kv)
                    valid = cols < n
                    kt = torch.zeros(tile_kv, d)
                    vt = torch.zeros(tile_kv, d)
                    kt[valid] = kh[cols[valid]]
                    vt[valid] = vh[cols[valid]]
                    qk = qt @ kt.t()  # [G, R, TILE]
                    ok = (rows[:, None] >= cols[None, :]) & valid[None, :]
                    qk = torch.where(ok[None], qk, neg)
                    m_new = torch.maximum(m_i, qk.max(dim=2).values)
                    alpha = torch.exp2(m_i - m_new)
                    p = torch.exp2(qk - m_new[..., None])
                    acc = alpha[..., None] * acc + p.to(torch.bfloat16).float() @ vt
                    l_i = alpha * l_i + p.sum(dim=2)
                    m_i = m_new
                res = (acc / l_i[..., None]).to(torch.bfloat16)  # [G, R, D]
                out[s0 + rows, h * group : (h + 1) * group] = res.permute(1, 0, 2)
    return out


def varlen_causal_exact(q, k, v, cu_seqlens) -> torch.Tensor:
    """fp32 softmax form, returns fp32.  triton_kernels/gqa_attention_varlen_causal.py:301-330."""
    total, hq, d = q.shape
    group = hq // k.shape[1]
    out = torch.zeros(total, hq, d)
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        s0, s1 = cu[b], cu[b + 1]
        n = s1 - s0
        if n == 0:
            continue
        qs = q[s0:s1].permute(1, 0, 2).float()
        ks = k[s0:s1].permute(1, 0, 2).float().repeat_interleave(group, 0)
        vs = v[s0:s1].permute(1, 0, 2).float().repeat_interleave(group, 0)
        scores = qs @ ks.transpose(1, 2) / math.sqrt(d)
        scores = scores + torch.triu(torch.full((n, n), -math.inf), diagonal=1)
        out[s0:s1] = (torch.softmax(scores, dim=-1) @ vs).permute(1, 0, 2)
    return out


# =========================================================================== rope / gate
def partial_rope(x, position_ids, inv_freq, rotary_dim: int) -> torch.Tensor:
    """Half-split rotation of the first rotary_dim dims of x [B,H,T,D]; angles = pos(fp32)*inv_freq in
    fp32; dims >= rotary_dim copied.  triton_kernels/partial_rope.py:56-132, :220-236."""
    half = rotary_dim // 2
    angles = position_ids.to(torch.float32).unsqueeze(-1) * inv_freq.view(1, 1, half)
    cos = torch.cos(angles).unsqueeze(1)
    sin = torch.sin(angles).unsqueeze(1)
    first = x[..., :half].float()
    second = x[..., half:rotary_dim].float()
    out = x.clone()
    out[..., :half] = (first * cos - second * sin).to(x.dtype)
    out[..., half:rotary_dim] = (first * sin + second * cos).to(x.dtype)
    return out


def attention_gate_pack(x, gate) -> torch.Tensor:
    """bf16(x.f32 * sigmoid(gate.f32)), [1,H,T,D] -> [T, H*D].  triton_kernels/attention_gate_pack.py:34-64."""
    b, h, t, d = x.shape
    out = x.float() * torch.sigmoid(gate.float())
    return out.permute(0, 2, 1, 3).reshape(b * t, h * d).to(x.dtype)


# =========================================================================== Gated DeltaNet
def gdn_step(state, q_t, k_t, v_t, beta_t, g_t):
    """One delta-rule step for all heads: state [H,DK,DV] fp32 (returned updated), out [H,DV] fp32.
    Order: decay, mem = k^T S, delta = beta (v - mem), S += k (x) delta, out = q^T S (updated S).
    triton_kernels/gdn_recurrent_prefill.py:106-131, :193-231."""
    state = torch.exp(g_t)[:, None, None] * state
    kf = k_t.float()
    mem = torch.einsum("hk,hkv->hv", kf, state)
    delta = beta_t[:, None] * (v_t.float() - mem)
    state = state + kf[:, :, None] * delta[:, None, :]
    out = torch.einsum("hk,hkv->hv", q_t.float(), state)
    return state, out


def gdn_recurrent_decode(q, k, v, beta, g, state) -> torch.Tensor:
    """One token per sequence; state [B,H,DK,DV] fp32 updated IN PLACE; returns bf16 [B,H,DV].
    triton_kernels/gdn_recurrent_prefill.py:189-246."""
    out = torch.empty(v.shape, dtype=v.dtype)
    for b in range(q.shape[0]):
        new_state, o = gdn_step(state[b], q[b], k[b], v[b], beta[b], g[b])
        state[b] = new_state
        out[b] = o.to(v.dtype)
    return out


def gdn_recurrent_prefill_sequential(q, k, v, beta, g, cu_seqlens=None):
    """Token-serial recurrence over a packed buffer, zero state at each sequence start.  Returns
    (out [T,H,DV] bf16, state [B,H,DK,DV] fp32), or state [H,DK,DV] when cu_seqlens is None.
    triton_kernels/gdn_recurrent_prefill.py:95-143, :1050-1145."""
    total, heads, dk = q.shape
    dv = v.shape[-1]
    squeeze = cu_seqlens is None
    cu = [0, total] if squeeze else cu_seqlens.tolist()
    out = torch.empty(total, heads, dv, dtype=v.dtype)
    states = torch.zeros(len(cu) - 1, heads, dk, dv)
    for b in range(len(cu) - 1):
        s = torch.zeros(heads, dk, dv)
        for t in range(cu[b], cu[b + 1]):
            s, o = gdn_step(s, q[t], k[t], v[t], beta[t], g[t])
            out[t] = o.to(v.dtype)
        states[b] = s
    return out, (states[0] if squeeze else states)


def _pad_chunks(x, num_chunks):
    total = x.shape[0]
    padded = torch.zeros((num_chunks * CHUNK,) + tuple(x.shape[1:]), dtype=torch.float32)
    padded[:total] = x.float()
    return padded.view((num_chunks, CHUNK) + tuple(x.shape[1:]))


def gdn_chunk_prepare_wy(k, v, beta, g):
    """Per 64-token chunk: G = cumsum(g); L[t,i] = beta_t exp(G_t-G_i) <k_t,k_i> (i<t); P = (I+L)^-1 by
    forward substitution; u = P (beta v); w = P (beta exp(G) k).  Padded tokens are all-zero rows.
    Returns w [N,H,64,DK], u_base [N,H,64,DV], g_cumsum [N,H,64] (fp32).
    triton_kernels/gdn_recurrent_prefill.py:289-396."""
    total, heads, dk = k.shape
    n = _cdiv(total, CHUNK)
    kc = _pad_chunks(k, n).permute(0, 2, 1, 3)        # [N,H,64,DK]
    vc = _pad_chunks(v, n).permute(0, 2, 1, 3)
    bc = _pad_chunks(beta, n).permute(0, 2, 1)        # [N,H,64]
    gcs = torch.cumsum(_pad_chunks(g, n), dim=1).permute(0, 2, 1)
    kkt = kc @ kc.transpose(-1, -2)
    strict = torch.tril(torch.ones(CHUNK, CHUNK, dtype=torch.bool), diagonal=-1)
    # the kernel masks pairs that involve a padded token; with zero-padded k those products are 0 anyway
    diff = torch.where(strict, gcs[..., :, None] - gcs[..., None, :], torch.tensor(-math.inf))
    lower = torch.where(strict, bc[..., :, None] * torch.exp(diff) * kkt, torch.tensor(0.0))
    eye = torch.eye(CHUNK)
    inv = eye.expand(n, heads, CHUNK, CHUNK).clone()
    for row in range(1, CHUNK):
        inv[:, :, row, :] = eye[row] - torch.einsum("nhi,nhij->nhj", lower[:, :, row, :row], inv[:, :, :row, :])
    u_base = inv @ (bc[..., None] * vc)
    w = inv @ (bc[..., None] * torch.exp(gcs)[..., None] * kc)
    return w, u_base, gcs.contiguous()


def gdn_chunk_state(k, w, u_base, g_cumsum):
    """Serial scan over chunks: store state_in; delta = u - w state; state = exp(G_last) state +
    k^T (delta * exp(G_last - G)) with padded tokens dropped.  Returns delta [N,H,64,DV],
    chunk_state [N,H,DK,DV] (state ENTERING each chunk), final_state [H,DK,DV].
    triton_kernels/gdn_recurrent_prefill.py:452-537."""
    total, heads, dk = k.shape
    n, _, _, dv = u_base.shape
    kc = _pad_chunks(k, n).permute(0, 2, 1, 3)
    valid = (torch.arange(n * CHUNK) < total).view(n, 1, CHUNK)
    state = torch.zeros(heads, dk, dv)
    delta = torch.empty_like(u_base)
    chunk_state = torch.empty(n, heads, dk, dv)
    for c in range(n):
        chunk_state[c] = state
        delta[c] = u_base[c] - w[c] @ state
        g_last = g_cumsum[c, :, CHUNK - 1]
        to_end = torch.where(valid[c], torch.exp(g_last[:, None] - g_cumsum[c]), torch.tensor(0.0))
        state = torch.exp(g_last)[:, None, None] * state + kc[c].transpose(-1, -2) @ (delta[c] * to_end[..., None])
    return delta, chunk_state, state


def gdn_chunk_output(q, k, delta, g_cumsum, chunk_state) -> torch.Tensor:
    """out_t = exp(G_t) q_t^T S_in + sum_{i<=t} <q_t,k_i> exp(G_t-G_i) delta_i, bf16 [T,H,DV].
    triton_kernels/gdn_recurrent_prefill.py:604-690."""
    total, heads, dk = q.shape
    n, _, _, dv = delta.shape
    qc = _pad_chunks(q, n).permute(0, 2, 1, 3)
    kc = _pad_chunks(k, n).permute(0, 2, 1, 3)
    causal = torch.tril(torch.ones(CHUNK, CHUNK, dtype=torch.bool))
    diff = torch.where(causal, g_cumsum[..., :, None] - g_cumsum[..., None, :], torch.tensor(-math.inf))
    attn = torch.where(causal, (qc @ kc.transpose(-1, -2)) * torch.exp(diff), torch.tensor(0.0))
    out = torch.exp(g_cumsum)[..., None] * (qc @ chunk_state) + attn @ delta  # [N,H,64,DV]
    out = out.permute(0, 2, 1, 3).reshape(n * CHUNK, heads, dv)[:total]
    return out.to(q.dtype)


def gdn_chunked_prefill(q, k, v, beta, g):
    """prepare_wy -> chunk_state -> chunk_output for ONE sequence; returns (out, final_state).
    triton_kernels/gdn_recurrent_prefill.py:1026-1047."""
    w, u_base, gcs = gdn_chunk_prepare_wy(k, v, beta, g)
    delta, chunk_state, final_state = gdn_chunk_state(k, w, u_base, gcs)
    return gdn_chunk_output(q, k, delta, gcs, chunk_state), final_state


def gdn_chunked_prefill_packed(q, k, v, beta, g, cu_seqlens):
    """The packed form the reference cannot do in one call: the chunk-64 pipeline run per sequence, chunk
    grid restarting at every cu_seqlens[b].  Returns (out [T,H,DV] bf16, state [B,H,DK,DV] fp32)."""
    cu = cu_seqlens.tolist()
    outs, states = [], []
    for b in range(len(cu) - 1):
        sl = slice(cu[b], cu[b + 1])
        o, s = gdn_chunked_prefill(q[sl], k[sl], v[sl], beta[sl], g[sl])
        outs.append(o)
        states.append(s)
    return torch.cat(outs, dim=0), torch.stack(states)


# =========================================================================== fused compositions
def fused_decode_attention(q, k_new, v_new, gate, k_cache, v_cache, block_table, pos, inv_freq,
                           rotary_dim: int, exact: bool = False) -> torch.Tensor:
    """The decode attention chain of engine/runner.py:482-517 as one call: partial_rope(q), partial_rope(k)
    at position pos[b]; append; paged attention; gate pack -> [B, H_q*D] bf16.  q/k_new/v_new are the
    post-norm, pre-RoPE [B,H,D] tensors, gate is [B, H_q*D].  Caches are updated in place.
    With exact=True the attention itself uses the fp32-softmax form (large cases)."""
    batch, hq, d = q.shape
    ids = pos.view(batch, 1)
    q_r = partial_rope(q.unsqueeze(2), ids, inv_freq, rotary_dim)[:, :, 0, :]
    k_r = partial_rope(k_new.unsqueeze(2), ids, inv_freq, rotary_dim)[:, :, 0, :]
    if exact:
        paged_kv_append(k_cache, v_cache, k_r, v_new, block_table, pos)
        ctx = paged_decode_exact(q_r, k_cache, v_cache, block_table, (pos + 1).tolist()).to(torch.bfloat16)
    else:
        ctx = paged_decode(q_r, k_r, v_new, k_cache, v_cache, block_table, pos)
    x4 = ctx.permute(1, 0, 2).unsqueeze(0)
    g4 = gate.view(batch, hq, d).permute(1, 0, 2).unsqueeze(0)
    return attention_gate_pack(x4, g4)


def fused_prefill_attention(q, k, v, gate, k_cache, v_cache, block_table, cu_seqlens, position_ids,
                            inv_freq, rotary_dim: int, exact: bool = False) -> torch.Tensor:
    """The packed prefill attention chain of engine/runner.py:339-384 as one call: rope(q), rope(k) with
    per-sequence positions; varlen causal attention; gate pack -> [T, H_q*D]; post-RoPE K and raw V
    scattered into the paged cache.  q [T,H_q,D], k/v [T,H_kv,D], gate [T,H_q*D], position_ids [1,T]."""
    total, hq, d = q.shape
    q_r = partial_rope(q.unsqueeze(0).permute(0, 2, 1, 3), position_ids, inv_freq, rotary_dim)[0].permute(1, 0, 2)
    k_r = partial_rope(k.unsqueeze(0).permute(0, 2, 1, 3), position_ids, inv_freq, rotary_dim)[0].permute(1, 0, 2)
    if exact:
        ctx = varlen_causal_exact(q_r, k_r, v, cu_seqlens).to(torch.bfloat16)
    else:
        ctx = varlen_causal(q_r.contiguous(), k_r.contiguous(), v, cu_seqlens)
    paged_kv_fill_varlen(k_cache, v_cache, k_r.permute(1, 0, 2), v.permute(1, 0, 2), block_table, cu_seqlens)
    x4 = ctx.permute(1, 0, 2).unsqueeze(0)
    g4 = gate.view(1, total, hq, d).permute(0, 2, 1, 3)
    return attention_gate_pack(x4, g4)
