"""Test helpers: the package's seeded input generators plus comparison utilities."""
from __future__ import annotations

import torch

from b200attn.synthetic import PAGE, bf16_randn, cdiv, gdn_inputs, make_paged_case, maxabs, rope_inv_freq  # noqa: F401


def assert_bf16_close(got, want, ulps=1, what="", max_mismatch_frac=1.0):
    """Two bf16 tensors agree to `ulps` units in the last place of the larger magnitude (a bf16 ulp is 2^-8..2^-7
    relative); `max_mismatch_frac` additionally bounds the share of elements that are not bit-equal."""
    g, w = got.detach().float().cpu(), want.detach().float().cpu()
    assert g.shape == w.shape, f"{what}: shape {tuple(g.shape)} vs {tuple(w.shape)}"
    tol = ulps * 2.0 ** -7 * torch.maximum(g.abs(), w.abs()) + 1e-30
    bad = (g - w).abs() > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} elements differ by more than {ulps} bf16 ulp, max abs {float((g - w).abs().max()):.3e}"
    frac = float((g != w).float().mean())
    assert frac <= max_mismatch_frac, f"{what}: {frac:.3%} of the elements are not bit-equal (allowed {max_mismatch_frac:.3%})"
