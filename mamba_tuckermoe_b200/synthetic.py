"""Seeded synthetic inputs for the benchmark and the tests: layer sizes of the benchmark configurations, factor and token
draws with the distributions those configurations name, and the skewed-routing construction.

The reference ships no weights or activations, and its published shapes come with distributions rather than data
(``x ~ N(0,1)``, router logits ~N(0,1) or N(0, 0.02 sqrt(d_in)), Zipf(1.2) expert popularity), so both the benchmark and
the parity tests draw from here; every draw is fp32 on a CPU generator with a fixed order and is cast afterwards.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch


@dataclass
class LayerShape:
    """Sizes of one Tucker-MoE layer (names follow ``pure_torch_mlx/model.py:44-58``)."""
    d_in: int
    d_out: int
    E: int
    top_k: int
    r1: int
    r3: int
    r2: int
    eps: float = 1e-6

    def flops_per_token(self) -> int:
        """Algorithmic FLOPs per token in the coefficient-vector formulation."""
        return (2 * self.d_in * self.E + 2 * self.d_in * self.r3 + 2 * self.r3 * self.r1 * self.r2
                + 2 * self.r1 * self.r2 + 2 * self.r2 * self.d_out)

    def factor_elems(self) -> int:
        return (self.E * self.d_in + self.d_in * self.r3 + self.r3 + self.E * self.r1
                + self.r1 * self.r3 * self.r2 + self.r2 * self.d_out + self.d_out)



def make_factors(shape: LayerShape, seed: int, dtype: torch.dtype = torch.float32,
                 router_std: Optional[float] = 0.02, bias_std: float = 0.0) -> Dict[str, torch.Tensor]:
    """Seeded factors.  Draw order is fixed: W_r, U_expert, U_in, core, U_out, (bias).

    ``router_std=None`` means ``1/sqrt(d_in)`` so that the logits of N(0,1) inputs are ~N(0,1).
    All draws are fp32 on a CPU generator and are cast to ``dtype`` afterwards.
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    s = shape
    rstd = (1.0 / math.sqrt(s.d_in)) if router_std is None else router_std
    f = {
        "router_w": torch.randn(s.E, s.d_in, generator=g) * rstd,
        "U_expert": torch.randn(s.E, s.r1, generator=g),
        "U_in": torch.randn(s.d_in, s.r3, generator=g) / math.sqrt(s.d_in),
        "core": torch.randn(s.r1, s.r3, s.r2, generator=g) / math.sqrt(s.r3),
        "U_out": torch.randn(s.r2, s.d_out, generator=g) / math.sqrt(s.r2),
        "inner_norm_w": torch.ones(s.r3),
    }
    f["bias"] = (torch.randn(s.d_out, generator=g) * bias_std) if bias_std > 0 else torch.zeros(s.d_out)
    return {k: v.to(dtype).contiguous() for k, v in f.items()}


def make_tokens(T: int, d_in: int, seed: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """x ~ N(0,1), fp32 draw on a CPU generator, cast afterwards.  Independent of the factor seed."""
    g = torch.Generator(device="cpu").manual_seed(seed + 7_000_003)
    return torch.randn(T, d_in, generator=g).to(dtype).contiguous()


def apply_zipf_router_bias(x: torch.Tensor, factors: Dict[str, torch.Tensor], seed: int, s: float = 1.2):
    """Skewed routing inside the bias-free router API (model.py:60 has ``bias=False``).

    Input channel 0 becomes the constant 1 and ``W_r[:, 0]`` the per-expert bias
    ``log p_e - mean(log p)`` with ``p_e ~ rank^-s`` under a seeded expert permutation.
    """
    E = factors["router_w"].shape[0]
    g = torch.Generator(device="cpu").manual_seed(seed + 99)
    perm = torch.randperm(E, generator=g)
    logp = -s * torch.log(torch.arange(1, E + 1, dtype=torch.float32))
    logp = logp - logp.mean()
    b = torch.empty(E)
    b[perm] = logp
    factors["router_w"][:, 0] = b.to(factors["router_w"].dtype)
    x[..., 0] = 1.0
    return x, factors


BENCH_SHAPES = {
    # name: (LayerShape, T, dtype, factor seed, router_std)
    "cfg0": (LayerShape(1536, 2304, 8, 2, 4, 256, 1024), 512, torch.float32, 1000, 0.02),
    "cfg1": (LayerShape(1536, 2304, 8, 2, 4, 256, 1024), 64, torch.bfloat16, 1001, 0.02),
    "cfg2": (LayerShape(1536, 2304, 64, 2, 4, 256, 1024), 32768, torch.bfloat16, 1002, None),
    "cfg3": (LayerShape(1536, 2304, 64, 2, 4, 256, 1024), 16384, torch.bfloat16, 1003, 0.02),
    "cfg4": (LayerShape(3072, 4608, 256, 8, 8, 512, 2048), 131072, torch.bfloat16, 1004, 0.02),
}
# expert-count sweep: E x top-k at T=16384
for _e in (8, 64, 256, 1024):
    for _k in (2, 8):
        BENCH_SHAPES[f"cfg3_e{_e}_k{_k}"] = (LayerShape(1536, 2304, _e, _k, 4, 256, 1024), 16384, torch.bfloat16,
                                              1003, 0.02)
# prefill-sized calls of the reference language model's four layer shapes at its shipped ranks (r1, r2, r3) = (32, 512, 256)
for _n, _di, _do in (("x_up", 1536, 6144), ("out_proj", 768, 768), ("ffn_up", 768, 4608), ("ffn_down", 4608, 768)):
    BENCH_SHAPES[f"shipped_{_n}"] = (LayerShape(_di, _do, 8, 2, 32, 256, 512, 1e-5), 16384, torch.bfloat16, 1005, 0.02)
ZIPF_SHAPES = {"cfg4"}  # skewed routing through apply_zipf_router_bias
