"""The CPU oracle against the golden outputs of the real reference module (no GPU needed)."""
import pytest
import torch

from golden_cases import ALL_CASES, F32_CASES, load_case
from oracle.tucker_moe_oracle import (classify_topk, layer_forward, layer_forward_f64, max_abs,
                                      rel_fro)


@pytest.mark.parametrize("name", ALL_CASES)
def test_restatement_is_bit_exact(name):
    """The op-by-op restatement reproduces the reference module's output bit for bit."""
    shape, x, f, dtype, g = load_case(name)
    y, taps = layer_forward(x, f, shape.top_k, shape.eps, return_taps=True)
    assert y.shape == g["y"].shape and y.dtype == dtype
    assert torch.equal(y.float(), g["y"])
    if x.numel():
        assert torch.equal(taps["idx"], g["idx"])
        assert torch.equal(taps["gates"].float(), g["gates"])
        assert torch.equal(taps["scores"].float(), g["scores"])


@pytest.mark.parametrize("chunk", [1, 3, 1000])
def test_chunking_does_not_change_results(chunk):
    shape, x, f, _, g = load_case("ragged_e64_k8_f32")
    y = layer_forward(x, f, shape.top_k, shape.eps, chunk_tokens=chunk)
    assert max_abs(y, g["y"]) < 5e-5  # BLAS blocks differently per chunk size; |y|max is ~6


@pytest.mark.parametrize("name", F32_CASES)
def test_f64_algebra_matches_reference_fp32(name):
    """The coefficient-vector algebra in float64 agrees with the fp32 reference to 1e-5 rel-Fro
    (bound stated for fp32 round-off of the reference itself) with identical selections."""
    shape, x, f, _, g = load_case(name)
    y64, taps = layer_forward_f64(x, f, shape.top_k, shape.eps)
    if x.numel() == 0:
        assert y64.shape == g["y"].shape
        return
    rep = classify_topk(taps["idx"], g["idx"], g["scores"], gap=1e-6)
    assert rep.unexplained == 0
    y64b, _ = layer_forward_f64(x, f, shape.top_k, shape.eps, idx=g["idx"])
    assert rel_fro(y64b, g["y"]) < 1e-5


def test_bf16_reference_vs_f64_with_forced_selection():
    """bf16 reference is low precision end to end; with its own selection forced and scores
    rounded to bf16, float64 algebra stays within the 2e-2 budget."""
    shape, x, f, _, g = load_case("cfg2_head_bf16")
    y64, _ = layer_forward_f64(x, f, shape.top_k, shape.eps, idx=g["idx"], round_scores_to=torch.bfloat16)
    assert rel_fro(y64, g["y"]) < 2e-2


def test_classify_topk_flags_real_mismatch():
    s = torch.tensor([[0.0, 1.0, 2.0, 3.0]])
    ref = torch.tensor([[3, 2]])
    assert classify_topk(torch.tensor([[3, 2]]), ref, s, 1e-6).exact == 1
    assert classify_topk(torch.tensor([[3, 1]]), ref, s, 1e-6).unexplained == 1
    s2 = torch.tensor([[0.0, 2.0, 2.0, 3.0]])
    assert classify_topk(torch.tensor([[3, 1]]), ref, s2, 1e-6).tie_explained == 1


def test_capped_softmax_rule_properties():
    """The second gate rule has no golden vectors (its reference file cannot run here); check the restatement's
    defining properties: same selection as the raw scores, gates proportional to the full-softmax probabilities,
    sum = S / (S + 1e-6), and agreement between the dtype-faithful and the float64 statements."""
    shape, x, f, _, g = load_case("ragged_e64_k8_f32")
    router = (1, 10.0, 0.5)
    y, taps = layer_forward(x, f, shape.top_k, shape.eps, return_taps=True, router=router)
    assert torch.equal(taps["idx"], g["idx"])          # tanh and 1/T are monotone: same experts, same order
    logits = 10.0 * torch.tanh(taps["scores"] / 10.0) / 0.5
    p = torch.softmax(logits, -1).gather(-1, taps["idx"])
    s = p.sum(-1, keepdim=True)
    assert torch.allclose(taps["gates"], p / (s + 1e-6), atol=1e-7)
    assert torch.allclose(taps["gates"].sum(-1, keepdim=True), s / (s + 1e-6), atol=1e-6)
    y64, t64 = layer_forward_f64(x, f, shape.top_k, shape.eps, router=router)
    assert rel_fro(y64, y) < 1e-5
    assert not torch.allclose(y, g["y"], atol=1e-3)    # and it is a different function from rule 0


def test_parity_report_rules():
    """The acceptance rule used by the GPU tests and the benchmark report, on the oracle's own outputs."""
    from oracle.parity import parity_report, subset_indices
    sub = subset_indices(131072)
    assert sub[0] == 0 and sub[4095] == 4095 and sub[-1] == 131071 and 8000 < len(sub) <= 8192
    assert torch.equal(subset_indices(100), torch.arange(100))
    shape, x, f, dtype, g = load_case("ragged_e64_k8_f32")
    y, taps = layer_forward(x, f, shape.top_k, shape.eps, return_taps=True)
    rep = parity_report(y, taps["idx"], x, f, shape.top_k, shape.eps, dtype)
    assert rep["ok"] and rep["topk_exact"] == x.shape[0] and rep["rel_fro"] == 0.0
    # a wrong expert without a score tie is reported as unexplained; a wrong output breaks the tolerance
    bad_idx = taps["idx"].clone()
    bad_idx[0, 0] = (bad_idx[0, 0] + 1) % shape.E if int((bad_idx[0, 0] + 1) % shape.E) not in bad_idx[0, 1:].tolist() else (bad_idx[0, 0] + 2) % shape.E
    rep = parity_report(y, bad_idx, x, f, shape.top_k, shape.eps, dtype)
    assert rep["topk_unexplained"] == 1 and not rep["ok"]
    rep = parity_report(y * 1.01, taps["idx"], x, f, shape.top_k, shape.eps, dtype)
    assert not rep["ok"] and rep["rel_fro"] > 1e-3
