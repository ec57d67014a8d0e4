"""Checkpoint key map (no GPU needed)."""
import numpy as np
import pytest
import torch

from mamba_tuckermoe_b200 import TuckerMoE, TuckerMoEConfig
from mamba_tuckermoe_b200.checkpoint import SUFFIXES, export_tucker, load_tucker, tucker_prefixes


def test_prefixes_follow_the_block_pattern():
    types = (["mamba"] * 4 + ["transformer"]) * 6          # the reference's 30-block layout
    p = tucker_prefixes(types)
    assert len(p) == 24 * 2 + 6 * 3                          # 66 Tucker-MoE layers per model
    assert p[0] == "backbone.layers.0.block.x_up_proj" and p[1] == "backbone.layers.0.block.out_proj"
    assert p[8:11] == ["backbone.layers.4.block.ffn.gate_proj", "backbone.layers.4.block.ffn.up_proj",
                       "backbone.layers.4.block.ffn.down_proj"]


def test_load_and_export_round_trip():
    cfg = TuckerMoEConfig(8, 2, 4, 64, 32, 1e-5)
    a, b = TuckerMoE(64, 96, cfg), TuckerMoE(64, 96, cfg)
    g = torch.Generator().manual_seed(0)
    with torch.no_grad():
        for p in a.parameters():
            p.copy_(torch.randn(p.shape, generator=g))
    ck = export_tucker(a, "backbone.layers.3.block.out_proj")
    assert sorted(ck) == sorted(f"backbone.layers.3.block.out_proj.{s}" for s in SUFFIXES)
    assert all(isinstance(v, np.ndarray) and v.dtype == np.float32 for v in ck.values())
    load_tucker(b, ck, "backbone.layers.3.block.out_proj")
    for (na, pa), (nb, pb) in zip(a.state_dict().items(), b.state_dict().items()):
        assert na == nb and torch.equal(pa, pb)
    with pytest.raises(KeyError):
        load_tucker(b, ck, "backbone.layers.4.block.out_proj")
    bad = dict(ck); bad["backbone.layers.3.block.out_proj.core"] = np.zeros((4, 32, 63), np.float32)
    with pytest.raises(ValueError):
        load_tucker(b, bad, "backbone.layers.3.block.out_proj")
