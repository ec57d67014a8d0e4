"""Parity report of a layer output against the CPU oracle on a fixed token subset (test infrastructure).

The layer is token-wise independent (``pure_torch_mlx/model.py:71-102`` has no cross-token operation), so a run over T
tokens can be checked on any subset of its rows: the oracle is evaluated on those rows only.  For the large
configurations the subset is the first 4096 tokens plus 4096 tokens strided over the rest, which covers the first CTA
wave, the last one and everything in between at a cost of seconds of CPU time.

Acceptance rule (the same in the tests and in the benchmark's report):
  * expert indices equal the reference restatement's, except where the reference's own scores of the two competing
    experts are within ``gap`` (fp32: 1e-6; bf16: one unit in the last place of the largest score) -- such tokens
    are "tie-explained", anything else is "unexplained";
  * on tokens with identical selections: relative Frobenius error and max-abs / max|y| within ``tol``
    (fp32 1e-4, bf16 2e-2) of the reference restatement in the layer dtype;
  * tie-explained tokens are compared with the float64 algebra under the run's own selection (same ``tol``).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .tucker_moe_oracle import classify_topk, layer_forward, layer_forward_f64

F32_TOL = 1e-4
BF16_TOL = 2e-2


def subset_indices(T: int, head: int = 4096, strided: int = 4096) -> torch.Tensor:
    """Token rows to check: all of them up to head + strided tokens, else the first `head` and `strided` rows spread
    evenly over the rest (always including the last row)."""
    if T <= head + strided:
        return torch.arange(T)
    rest = torch.linspace(head, T - 1, strided).round().long()
    return torch.cat([torch.arange(head), torch.unique(rest)])


def score_ulp(scores: torch.Tensor, dtype: torch.dtype) -> float:
    """Selection gap that counts as a tie: 1e-6 in fp32, one bf16 unit in the last place of the largest |score|."""
    if dtype == torch.float32:
        return 1e-6
    m = float(scores.abs().max()) if scores.numel() else 1.0
    return 2.0 ** (torch.tensor(max(m, 1e-30)).log2().floor().item() - 7)


def parity_report(y: torch.Tensor, idx: torch.Tensor, x: torch.Tensor, factors: Dict[str, torch.Tensor], top_k: int,
                  eps: float, dtype: torch.dtype, router=(0, 10.0, 0.5), gap_ulps: float = 1.0,
                  chunk_tokens: int = 256) -> dict:
    """y [n, d_out], idx [n, k] (the run's outputs on the checked rows, any device) against the oracle on x [n, d_in]
    (CPU, layer dtype).  Returns the figures; ``ok`` applies the acceptance rule above."""
    y = y.detach().float().cpu()
    idx = idx.detach().cpu()
    n = x.shape[0]
    tol = F32_TOL if dtype == torch.float32 else BF16_TOL
    if n == 0:
        return {"tokens_checked": 0, "rel_fro": 0.0, "max_abs": 0.0, "max_abs_over_ymax": 0.0, "topk_exact": 0,
                "topk_tie_explained": 0, "topk_unexplained": 0, "tie_tokens_rel_fro": 0.0, "tol": tol, "ok": True}
    y_ref, taps = layer_forward(x, factors, top_k, eps, chunk_tokens=chunk_tokens, return_taps=True, router=router)
    y_ref = y_ref.float()
    # a differing selection is explained by a near-tie of what the reference's top-k compared: its scores, or under rule 1
    # its tempered capped logits (which tie exactly where the cap saturates in bf16)
    gap = gap_ulps * score_ulp(taps["order"].float(), dtype)
    rep = classify_topk(idx, taps["idx"], taps["order"].float(), gap)
    keep = torch.ones(n, dtype=torch.bool)
    keep[rep.mismatch_tokens] = False
    yk, rk = y[keep].double(), y_ref[keep].double()
    den = float(rk.norm())
    rel = float((yk - rk).norm()) / den if den > 0 else float((yk - rk).norm())
    mabs = float((yk - rk).abs().max()) if yk.numel() else 0.0
    ymax = float(rk.abs().max()) if rk.numel() else 1.0
    tie_rel = 0.0
    if rep.mismatch_tokens:
        t = torch.tensor(rep.mismatch_tokens)
        y64, _ = layer_forward_f64(x[t], factors, top_k, eps, idx=idx[t], router=router,
                                   round_scores_to=None if dtype == torch.float32 else dtype)
        tie_rel = float((y[t].double() - y64).norm() / y64.norm())
    out = {"tokens_checked": int(n), "rel_fro": rel, "max_abs": mabs, "max_abs_over_ymax": mabs / max(ymax, 1e-30),
           "topk_exact": rep.exact, "topk_tie_explained": rep.tie_explained, "topk_unexplained": rep.unexplained,
           "tie_tokens_rel_fro": tie_rel, "tol": tol}
    out["ok"] = bool(rep.unexplained == 0 and rel <= tol and out["max_abs_over_ymax"] <= tol and tie_rel <= tol)
    return out


def assert_parity(rep: dict, what: str = "") -> None:
    assert rep["topk_unexplained"] == 0, f"{what}: {rep['topk_unexplained']} selections differ without a score tie: {rep}"
    assert rep["rel_fro"] <= rep["tol"], f"{what}: rel-Fro {rep['rel_fro']:.3e} > {rep['tol']}: {rep}"
    assert rep["max_abs_over_ymax"] <= rep["tol"], f"{what}: max-abs/max|y| {rep['max_abs_over_ymax']:.3e} > {rep['tol']}: {rep}"
    assert rep["tie_tokens_rel_fro"] <= rep["tol"], f"{what}: tie-broken tokens vs float64 {rep['tie_tokens_rel_fro']:.3e}: {rep}"
