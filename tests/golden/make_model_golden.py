"""Golden vectors of the Tucker-MoE layers INSIDE the reference language model, made by running the REAL model.

    python tests/golden/make_model_golden.py --reference /path/to/Mamba-TuckerMoE

Builds ``pure_torch_mlx.model.Mamba3LM`` from that checkout (nothing is copied) with one Mamba block and one
transformer block at the shipped widths and ranks (d_model 768, Tucker ranks (32, 512, 256), 8 experts, top-2), fills
the five Tucker-MoE layers through the reference's own ``_load_tucker`` (``pure_torch_mlx/weights.py:74-81``) from
seeded factors, gives every other parameter a seeded value, and runs ``decode_step`` for a few tokens on CPU in fp32.
Forward hooks record, per step,

* the input and output of each Tucker-MoE layer (``model.py:192, 259, 338-340``), and
* the callers' compositions around them: ``mid -> mid + ls_out_proj(out_proj(norm_out_proj(mid)))`` (``model.py:258-260``)
  and ``x_res -> x_res + ls_ffn(ffn_down(silu(ffn_gate(x_f)) * ffn_up(x_f)))`` (``model.py:337-341``).

The fixture ``model_decode_f32.npz`` stores those activations, the two norm weights and LayerScale vectors, and a
SHA-256 of every Tucker factor (the factors themselves are regenerated from their seeds by the tests).
"""
from __future__ import annotations

import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from mamba_tuckermoe_b200.synthetic import LayerShape, make_factors  # noqa: E402

STEPS = (3, 5)           # token ids of the decode steps
SEED = 4242
# (attribute path inside the block, checkpoint suffix, d_in, d_out, factor seed)
MAMBA_LAYERS = (("x_up_proj", "x_up_proj", 1536, 6144, 9001), ("out_proj", "out_proj", 768, 768, 9002))
XFMR_LAYERS = (("ffn_gate", "ffn.gate_proj", 768, 4608, 9003), ("ffn_up", "ffn.up_proj", 768, 4608, 9004),
               ("ffn_down", "ffn.down_proj", 4608, 768, 9005))
SUFFIX = {"router_w": "router.weight", "U_in": "U_in", "inner_norm_w": "inner_norm.weight", "U_expert": "U_expert",
          "core": "core", "U_out": "U_out", "bias": "bias"}


def layer_factors(d_in, d_out, seed):
    """Seeded fp32 factors of one layer at the shipped ranks; the inner-norm weight and the bias are made non-trivial."""
    shape = LayerShape(d_in, d_out, 8, 2, 32, 256, 512, 1e-5)
    f = make_factors(shape, seed, torch.float32, 0.05, 0.1)
    g = torch.Generator().manual_seed(seed + 1)
    f["inner_norm_w"] = (1 + 0.2 * torch.randn(256, generator=g)).contiguous()
    return shape, f


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from pure_torch_mlx.config import Mamba3Config
    from pure_torch_mlx.model import Mamba3LM
    from pure_torch_mlx.weights import _load_tucker

    cfg = Mamba3Config(num_layers=1, mamba_ratio=1, vocab_size=64)
    torch.manual_seed(SEED)
    model = Mamba3LM(cfg).eval()
    g = torch.Generator().manual_seed(SEED)
    with torch.no_grad():
        for name, p in model.named_parameters():   # everything that is not a Tucker factor: seeded, modest scale
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) / (p.shape[-1] ** 0.5))
            elif name.endswith("gamma"):
                p.copy_(0.5 + 0.2 * torch.randn(p.shape, generator=g))
            elif name.endswith("norm.weight") or ".norm_" in name or name.startswith("norm"):
                p.copy_(1 + 0.1 * torch.randn(p.shape, generator=g))
            elif name.endswith("bias"):
                p.copy_(0.05 * torch.randn(p.shape, generator=g))
    mamba, xfmr = model.blocks[0], model.blocks[1]
    out = {"steps": np.array(STEPS)}
    for blk, pfx, layers in ((mamba, "backbone.layers.0.block", MAMBA_LAYERS), (xfmr, "backbone.layers.1.block", XFMR_LAYERS)):
        for attr, suffix, d_in, d_out, seed in layers:
            shape, f = layer_factors(d_in, d_out, seed)
            w = {f"{pfx}.{suffix}.{SUFFIX[k]}": v for k, v in f.items()}
            _load_tucker(getattr(blk, attr), w, f"{pfx}.{suffix}")          # the reference's own loader
            for k, v in f.items():
                out[f"sha.{attr}.{k}"] = np.array(sha(v))

    rec = {}

    def tap(name):
        def hook(mod, inp, res):
            rec.setdefault(name + ".x", []).append(inp[0].detach().reshape(-1).clone())
            rec.setdefault(name + ".y", []).append(res.detach().reshape(-1).clone())
        return hook

    for attr, *_ in MAMBA_LAYERS:
        getattr(mamba, attr).register_forward_hook(tap(attr))
    for attr, *_ in XFMR_LAYERS:
        getattr(xfmr, attr).register_forward_hook(tap(attr))
    mamba.norm_out_proj.register_forward_hook(lambda m, i, r: rec.setdefault("mid", []).append(i[0].detach().reshape(-1).clone()))
    mamba.register_forward_hook(lambda m, i, r: rec.setdefault("mamba_out", []).append(r[0].detach().reshape(-1).clone()))
    xfmr.norm_ffn.register_forward_hook(lambda m, i, r: rec.setdefault("x_res", []).append(i[0].detach().reshape(-1).clone()))
    xfmr.register_forward_hook(lambda m, i, r: rec.setdefault("xfmr_out", []).append(r[0].detach().reshape(-1).clone()))
    # decode() is what the model calls, not forward(): route the block hooks through it
    for blk in (mamba, xfmr):
        blk.forward = blk.decode

    with torch.no_grad():
        states = model.init_states(kv_len=8)
        for tok in STEPS:
            x = model.embed.weight[tok].view(1, 1, -1)
            for i, blk in enumerate(model.blocks):
                x, states[i] = blk(x, states[i])

    for k, v in rec.items():
        out[k] = torch.stack(v).numpy().astype(np.float32)
    out["norm_out_proj.weight"] = mamba.norm_out_proj.weight.detach().numpy()
    out["ls_out_proj.gamma"] = mamba.ls_out_proj.gamma.detach().numpy()
    out["norm_ffn.weight"] = xfmr.norm_ffn.weight.detach().numpy()
    out["ls_ffn.gamma"] = xfmr.ls_ffn.gamma.detach().numpy()
    out["eps"] = np.array(cfg.rms_norm_eps)
    path = os.path.join(HERE, "model_decode_f32.npz")
    np.savez(path, **out)
    print(path, os.path.getsize(path), "bytes;", {k: tuple(v.shape) for k, v in out.items() if hasattr(v, "shape") and v.ndim == 2})


if __name__ == "__main__":
    main()
