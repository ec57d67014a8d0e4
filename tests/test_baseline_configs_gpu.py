"""The benchmark configurations at their own sizes through ``TuckerMoE.forward`` (AUTO path), checked against the CPU
oracle on a fixed token subset (first 4096 + 4096 strided tokens; everything for small T).

These are the launches the benchmark times: at T = 32768 the prefill configuration runs 256 token tiles in two waves
with the out-projection on CTA pairs, the expert sweep at E = 256 / 1024 takes the separate scores GEMM + select route
at the full d_in, and the skewed configuration runs r3 = 512 with its Zipf router bias in bf16.
"""
import ctypes as C

import pytest
import torch

from gpu_util import build_module
from mamba_tuckermoe_b200 import PATH_AUTO, _lib, read_device_status
from mamba_tuckermoe_b200.synthetic import BENCH_SHAPES, ZIPF_SHAPES, apply_zipf_router_bias, make_factors, make_tokens
from oracle.parity import assert_parity, parity_report, subset_indices

pytestmark = pytest.mark.gpu


def _case(key, T=None):
    shape, T0, dtype, seed, rstd = BENCH_SHAPES[key]
    T = T0 if T is None else T
    f32 = make_factors(shape, seed, torch.float32, rstd)
    x = make_tokens(T, shape.d_in, seed, torch.float32)
    if key in ZIPF_SHAPES:
        x, f32 = apply_zipf_router_bias(x, f32, seed)
    f = {k: v.to(dtype) for k, v in f32.items()}
    return shape, T, dtype, x.to(dtype), f


def _run_and_check(key, T=None, lead=None, head=4096, strided=4096):
    shape, T, dtype, x, f = _case(key, T)
    m = build_module(shape, f, dtype, path=PATH_AUTO)
    xd = x.cuda()
    if lead is not None:
        xd = xd.reshape(*lead, shape.d_in)
    with torch.no_grad():
        y, (idx, gates, c) = m.forward_with_routing(xd)
        y_plain = m(xd)
    torch.cuda.synchronize()
    assert read_device_status() == (0, 0, 0, 0)
    assert y.shape == ((*lead, shape.d_out) if lead is not None else (T, shape.d_out)) and y.dtype == dtype
    y2 = y.reshape(T, shape.d_out)
    assert torch.equal(y_plain.reshape(T, shape.d_out), y2), "plain forward and tapped forward differ"
    sub = subset_indices(T, head, strided)
    rep = parity_report(y2[sub.cuda()], idx[sub.cuda()], x[sub], f, shape.top_k, shape.eps, dtype)
    assert_parity(rep, key)
    # gates are a softmax: they sum to one (bf16 gates are rounded to 8 bits each)
    gs = gates[sub.cuda()].sum(-1)
    assert float((gs - 1).abs().max()) < (1e-5 if dtype == torch.float32 else 1e-2 * shape.top_k)
    return rep


def test_cfg0_fp32_full():
    rep = _run_and_check("cfg0", lead=(1, 512))
    assert rep["tokens_checked"] == 512


@pytest.mark.parametrize("T", [1, 8, 64])
def test_cfg1_decode_shapes(T):
    rep = _run_and_check("cfg1", T=T, lead=(T, 1))
    assert rep["tokens_checked"] == T


def test_cfg2_prefill_full():
    """T = 32768: two waves of token tiles, out-projection on CTA pairs -- the launch the headline number times."""
    shape, T, dtype, _, _ = _case("cfg2", T=8)   # sizes only
    L = _lib.layer_struct(shape, dtype)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert (32768 + 127) // 128 > sms, "the case is meant to need more than one wave of token tiles"
    assert _lib.load().tmoe_resolve_path(C.byref(L), 32768, 0) == 2
    rep = _run_and_check("cfg2", lead=(8, 4096))
    assert rep["tokens_checked"] == 8192


@pytest.mark.parametrize("E", [8, 64, 256, 1024])
@pytest.mark.parametrize("k", [2, 8])
def test_cfg3_expert_sweep_full(E, k):
    rep = _run_and_check(f"cfg3_e{E}_k{k}", head=2048, strided=2048)
    assert rep["tokens_checked"] == 4096


def test_cfg4_skewed_full():
    """T = 131072, d_in = 3072, E = 256, top-8, r = (8, 512, 2048), Zipf(1.2) router bias through input channel 0, bf16."""
    rep = _run_and_check("cfg4", lead=(32, 4096), head=2048, strided=2048)
    assert rep["tokens_checked"] == 4096
    # the skew is real: the reference's own selections concentrate on few experts
    shape, T, dtype, x, f = _case("cfg4", T=2048)
    from oracle.tucker_moe_oracle import layer_forward
    _, taps = layer_forward(x, f, shape.top_k, shape.eps, return_taps=True)
    counts = torch.bincount(taps["idx"].flatten(), minlength=shape.E).float()
    assert float(counts.max()) > 20 * float(counts.median().clamp(min=1))
