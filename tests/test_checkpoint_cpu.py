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


def _bf16_layer():
    cfg = TuckerMoEConfig(8, 2, 4, 128, 64, 1e-5)
    m = TuckerMoE(64, 96, cfg)
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for p in m.parameters():
            p.copy_(torch.randn(p.shape, generator=g))
    return m.to(torch.bfloat16)


def _write_sidecar(path, m, **override):
    """A sidecar as save_prepared_sidecar writes it (the blob's content does not matter for the acceptance checks)."""
    from mamba_tuckermoe_b200 import _lib
    from mamba_tuckermoe_b200 import checkpoint as ck
    fields = dict(prepared=np.zeros(ck._prepared_bytes(m), np.uint8), fingerprint=np.array(ck._fingerprint(m)),
                  top_k=np.array(m.top_k), eps=np.array(m.inner_norm.eps, dtype=np.float64),
                  abi=np.array(_lib.load().tmoe_version()), layout=np.array(ck.PREPARED_LAYOUT_VERSION),
                  layer=np.array(ck._layer_tuple(m), dtype=object).astype(str))
    fields.update(override)
    np.savez(path, **{k: v for k, v in fields.items() if v is not None})


def test_prepared_sidecar_is_refused_unless_everything_matches(tmp_path):
    """The kernels read the prepared set through raw offsets: a file from another layout version, another ABI, another
    layer shape, with fewer bytes than the library expects, or from other parameter values must not be installed."""
    from mamba_tuckermoe_b200 import checkpoint as ck
    m = _bf16_layer()
    assert ck._prepared_bytes(m) > 0
    good = str(tmp_path / "good.npz")
    _write_sidecar(good, m)
    assert ck.load_prepared_sidecar(m, good) and m._prep is not None and m._prep.numel() == ck._prepared_bytes(m)
    cases = {
        "truncated": dict(prepared=np.zeros(ck._prepared_bytes(m) - 1024, np.uint8)),
        "longer": dict(prepared=np.zeros(ck._prepared_bytes(m) + 1024, np.uint8)),
        "layout": dict(layout=np.array(ck.PREPARED_LAYOUT_VERSION + 1)),
        "abi": dict(abi=np.array(99)),
        "shape": dict(layer=np.array([64, 96, 8, 4, 256, 64, "torch.bfloat16"], dtype=object).astype(str)),
        "top_k": dict(top_k=np.array(3)),
        "values": dict(fingerprint=np.array("0" * 64)),
        "old_format": dict(abi=None, layout=None, layer=None),
    }
    for name, ov in cases.items():
        fresh = _bf16_layer()
        path = str(tmp_path / f"{name}.npz")
        _write_sidecar(path, fresh, **ov)
        assert not ck.load_prepared_sidecar(fresh, path), name
        assert fresh._prep is None, name
