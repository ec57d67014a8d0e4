"""CPU oracle for the Tucker-MoE layer forward (test infrastructure, not product code).

Two independent statements of the same layer:

* ``layer_forward``  -- restates the reference module's forward op by op
  (reference ``pure_torch_mlx/model.py:68-102`` and its ``RMSNorm`` at
  ``pure_torch_mlx/model.py:25-27``; second witness
  ``mamba3_mlx/bench_pytorch_ref.py:107-130``) in the tensor dtype it is given, so that it
  rounds where the reference rounds.  It is pinned against outputs of the reference module
  itself: ``tests/golden/make_golden.py`` runs the real module and stores its outputs, and
  ``tests/test_oracle.py`` checks this function against them bit for bit.
* ``layer_forward_f64`` -- float64 evaluation in the coefficient-vector algebra
  ``c = sum_k g_k * U_expert[e_k]``, ``z = sum_a c_a * (h @ core[a])`` that the CUDA kernels
  use.  It arbitrates when a low-precision reference and the kernels disagree.

Also here: the comparison helpers (top-k mismatch classification, relative Frobenius error).  The seeded
synthetic input generator for the benchmark configurations is `mamba_tuckermoe_b200/synthetic.py`, re-exported here.

Only ``tests/``, the smoke check and the benchmark's CPU-baseline leg may import this file.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# Factor container
# --------------------------------------------------------------------------------------

FACTOR_NAMES = ("router_w", "U_in", "inner_norm_w", "U_expert", "core", "U_out", "bias")


from mamba_tuckermoe_b200.synthetic import (BENCH_SHAPES, ZIPF_SHAPES, LayerShape, apply_zipf_router_bias,  # noqa: E402,F401
                                           make_factors, make_tokens)


# --------------------------------------------------------------------------------------
# Restatement of the reference forward
# --------------------------------------------------------------------------------------

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps) * weight`` in x's dtype (model.py:25-27: no fp32 upcast)."""
    denom = x.pow(2).mean(-1, keepdim=True).add(eps).sqrt()
    return (x / denom) * weight


def router_logits(scores: torch.Tensor, cap: float, temperature: float) -> torch.Tensor:
    """Tempered capped logits of the trained checkpoints' router (``sft_cot_bundle/scripts/model.py:320-324``): what their
    softmax and their top-k see.  Both steps are stored in the scores' dtype; in bf16 scores beyond about twice the cap all
    become the same logit."""
    capped = ((2.0 * torch.sigmoid(2.0 * (scores.float() * (1.0 / cap))) - 1.0) * cap).to(scores.dtype)
    return capped / temperature


def capped_softmax_gates(scores: torch.Tensor, top_k: int, cap: float, temperature: float):
    """The trained checkpoints' gate rule, restated from ``sft_cot_bundle/scripts/model.py:318-329`` (same math in
    ``mamba3_mlx/mlx_model/tucker_moe.py:107-114``): soft cap ``cap*tanh(s/cap)`` -- computed in fp32 as
    ``(2*sigmoid(2*s/cap) - 1)*cap`` and stored in the scores' dtype, as the reference's kernel does
    (``model.py:15-18, 32-40``) --, temperature, softmax over ALL experts, top-k of the tempered logits, renormalise the k
    selected probabilities with ``+1e-6``; every step after the cap in the scores' dtype, as in the reference.
    Pinned by ``tests/golden/variant_*.npz``, made by running the reference module itself (its two Triton kernel launches
    replaced by torch statements of their arithmetic: ``tests/golden/make_variant_golden.py``)."""
    logits = router_logits(scores, cap, temperature)
    probs = torch.softmax(logits, dim=-1)
    _, idx = torch.topk(logits, top_k, dim=-1)
    raw = probs.gather(-1, idx)
    return idx, raw / (raw.sum(-1, keepdim=True) + 1e-6)


def _forward_chunk(x_flat: torch.Tensor, f: Dict[str, torch.Tensor], top_k: int, eps: float,
                   taps: Optional[dict], router=(0, 10.0, 0.5)) -> torch.Tensor:
    scores = F.linear(x_flat, f["router_w"])
    if router[0] == 0:
        # model.py:75-77 -- raw scores, top-k on the raw scores, softmax over the k winners only
        sel_val, sel_idx = torch.topk(scores, top_k, dim=-1)
        gates = F.softmax(sel_val, dim=-1)
        order = scores
    else:
        sel_idx, gates = capped_softmax_gates(scores, top_k, router[1], router[2])
        order = router_logits(scores, router[1], router[2])
    # model.py:80-81 -- shared in-projection, then the inner RMSNorm
    h = rms_norm(x_flat @ f["U_in"], f["inner_norm_w"], eps)
    # model.py:87-98 -- per selected expert: mix the core slices, contract, weight, accumulate
    r2 = f["U_out"].shape[0]
    acc = h.new_zeros(x_flat.shape[0], r2)
    for j in range(top_k):
        coeff = f["U_expert"][sel_idx[:, j]]                       # [T, r1]
        mixed = torch.einsum("br,rst->bst", coeff, f["core"])      # [T, r3, r2]
        mid = torch.bmm(h.unsqueeze(1), mixed).squeeze(1)          # [T, r2]
        acc.add_(gates[:, j].unsqueeze(1) * mid)
    # model.py:101
    y = acc @ f["U_out"] + f["bias"]
    if taps is not None:
        # "order": the values the top-k compared (scores under rule 0, tempered capped logits under rule 1)
        for name, val in (("scores", scores), ("order", order), ("idx", sel_idx), ("gates", gates), ("h", h),
                          ("z", acc), ("y", y)):
            taps.setdefault(name, []).append(val)
    return y


@torch.no_grad()
def layer_forward(x: torch.Tensor, factors: Dict[str, torch.Tensor], top_k: int, eps: float,
                  chunk_tokens: int = 256, return_taps: bool = False, router=(0, 10.0, 0.5)):
    """Reference-order forward on CPU.  ``x``: (..., d_in) -> (..., d_out).

    Tokens are processed in chunks because the reference materialises a ``[T, r3, r2]``
    tensor per selected expert (model.py:95); the layer is token-wise independent so
    chunking does not change any result.
    """
    *batch, d_in = x.shape
    x_flat = x.reshape(-1, d_in)
    T = x_flat.shape[0]
    d_out = factors["U_out"].shape[1]
    taps: Optional[dict] = {} if return_taps else None
    outs = []
    for t0 in range(0, T, chunk_tokens):
        outs.append(_forward_chunk(x_flat[t0:t0 + chunk_tokens], factors, top_k, eps, taps, router))
    y = torch.cat(outs, 0) if outs else x_flat.new_zeros(0, d_out)
    y = y.reshape(*batch, d_out)
    if return_taps:
        merged = {k: torch.cat(v, 0) for k, v in taps.items()} if taps else {}
        return y, merged
    return y


@torch.no_grad()
def layer_forward_f64(x: torch.Tensor, factors: Dict[str, torch.Tensor], top_k: int, eps: float,
                      idx: Optional[torch.Tensor] = None, round_scores_to: Optional[torch.dtype] = None,
                      chunk_tokens: int = 2048, router=(0, 10.0, 0.5)):
    """float64 forward in the coefficient-vector algebra.

    ``idx`` (optional, [T, k]) forces the selected experts so that outputs can be compared
    token by token with an implementation that broke a tie differently.
    ``round_scores_to`` rounds the raw scores to a storage dtype before selection and
    softmax, which is what the reference does when its parameters are bf16.
    Returns (y, taps) with taps = idx, gates, c, h, z in float64.
    """
    *batch, d_in = x.shape
    xf = x.reshape(-1, d_in).double()
    f = {k: v.double() for k, v in factors.items()}
    T = xf.shape[0]
    r1, r3, r2 = f["core"].shape
    core_flat = f["core"].reshape(r1, r3 * r2)
    ys, taps = [], {"idx": [], "gates": [], "c": [], "h": [], "z": [], "scores": []}
    for t0 in range(0, T, chunk_tokens):
        xc = xf[t0:t0 + chunk_tokens]
        scores = xc @ f["router_w"].t()
        if round_scores_to is not None:
            scores = scores.to(round_scores_to).double()
        order = scores
        if router[0] != 0:
            capped = router[1] * torch.tanh(scores / router[1])
            if round_scores_to is not None:   # the reference keeps the capped scores and the logits in the layer dtype
                capped = capped.to(round_scores_to).double()
            logits = capped / router[2]
            if round_scores_to is not None:
                logits = logits.to(round_scores_to).double()
            order = logits                    # its top-k runs on the logits (model.py:327)
        if idx is None:   # higher value first, equal values -> lower expert index first
            sel_idx = torch.sort(order, dim=-1, descending=True, stable=True).indices[:, :top_k]
        else:
            sel_idx = idx[t0:t0 + chunk_tokens].long()
        sel_val = torch.gather(scores, 1, sel_idx)
        if router[0] == 0:
            gates = torch.softmax(sel_val, -1)
        else:  # capped / tempered softmax over all experts, renormalised over the selection (+1e-6)
            raw = torch.softmax(logits, -1).gather(-1, sel_idx)
            gates = raw / (raw.sum(-1, keepdim=True) + 1e-6)
        c = torch.einsum("tk,tkr->tr", gates, f["U_expert"][sel_idx])         # [t, r1]
        h = xc @ f["U_in"]
        h = h / torch.sqrt(h.pow(2).mean(-1, keepdim=True) + eps) * f["inner_norm_w"]
        # z[t, s] = sum_a c[t, a] * (h[t, :] @ core[a])[s]
        p = (h @ f["core"].permute(1, 0, 2).reshape(r3, r1 * r2)).reshape(-1, r1, r2)
        z = torch.einsum("ta,tas->ts", c, p)
        ys.append(z @ f["U_out"] + f["bias"])
        for name, val in (("idx", sel_idx), ("gates", gates), ("c", c), ("h", h), ("z", z),
                          ("scores", scores)):
            taps[name].append(val)
    del core_flat
    d_out = f["U_out"].shape[1]
    y = torch.cat(ys, 0) if ys else xf.new_zeros(0, d_out)
    merged = {k: (torch.cat(v, 0) if v else None) for k, v in taps.items()}
    return y.reshape(*batch, d_out), merged


# --------------------------------------------------------------------------------------
# Seeded synthetic inputs
# --------------------------------------------------------------------------------------

# make_factors, make_tokens, apply_zipf_router_bias, BENCH_SHAPES and ZIPF_SHAPES live in
# mamba_tuckermoe_b200/synthetic.py (the benchmark draws its inputs from there too, so that it does not have to import
# this file); they are re-exported above for the tests.


# --------------------------------------------------------------------------------------
# Comparison helpers
# --------------------------------------------------------------------------------------

def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    """||a - b||_F / ||b||_F in float64 (0 for two empty tensors)."""
    a64, b64 = a.double(), b.double()
    den = float(b64.norm())
    return float((a64 - b64).norm()) / den if den > 0 else float((a64 - b64).norm())


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    if a.numel() == 0:
        return 0.0
    return float((a.double() - b.double()).abs().max())


@dataclass
class TopkReport:
    tokens: int
    exact: int                 # ordered index lists identical
    tie_explained: int         # differ, but every differing position is within `gap` in the checker's scores
    unexplained: int
    mismatch_tokens: list = field(default_factory=list)


def classify_topk(idx_test: torch.Tensor, idx_ref: torch.Tensor, scores_ref: torch.Tensor,
                  gap: float) -> TopkReport:
    """Compare ordered top-k index lists token by token.

    A token whose lists differ counts as tie-explained when, at every position where the
    two lists disagree, the checker's own scores of the two competing experts are within
    ``gap`` of each other (fp32: 1e-6; bf16: one unit in the last place of the score).
    """
    idx_test = idx_test.long().cpu()
    idx_ref = idx_ref.long().cpu()
    s = scores_ref.double().cpu()
    T = idx_ref.shape[0]
    same = (idx_test == idx_ref).all(-1)
    exact = int(same.sum())
    tie, bad, toks = 0, 0, []
    for t in torch.nonzero(~same).flatten().tolist():
        ok = True
        for j in range(idx_ref.shape[1]):
            a, b = int(idx_test[t, j]), int(idx_ref[t, j])
            if a != b and abs(float(s[t, a]) - float(s[t, b])) > gap:
                ok = False
        tie += int(ok)
        bad += int(not ok)
        toks.append(t)
    return TopkReport(T, exact, tie, bad, toks)
