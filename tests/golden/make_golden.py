"""Generate the golden fixtures in this directory by running the REAL reference module.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py --reference /path/to/Mamba-TuckerMoE

It imports ``pure_torch_mlx.model.TuckerMoE`` from that checkout (nothing is copied), fills
it with the seeded factors of ``oracle.tucker_moe_oracle``, runs ``forward`` under
``torch.no_grad()`` on CPU and stores, per case, the module's output together with the
intermediate router results recomputed with the module's own parameters.  Small cases store
their inputs; large ones store only the seeds plus a SHA-256 of every input tensor so that a
regenerated input can be verified before it is trusted.

The tests never need the reference checkout: they read the ``.npz`` files written here.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import sys
from types import SimpleNamespace

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle.tucker_moe_oracle import (LayerShape, apply_zipf_router_bias, make_factors,  # noqa: E402
                                      make_tokens)

# name: (shape, T, x leading shape or None, dtype, seed, router_std, bias_std, store_inputs, zipf)
CASES = {
    "tiny_f32": (LayerShape(64, 96, 8, 2, 4, 32, 64, 1e-5), 16, None, "float32", 11, 0.02, 0.1, True, False),
    "tiny_bf16": (LayerShape(64, 96, 8, 2, 4, 32, 64, 1e-5), 16, None, "bfloat16", 12, 0.02, 0.1, True, False),
    "ragged_e64_k8_f32": (LayerShape(256, 384, 64, 8, 8, 64, 128, 1e-6), 33, None, "float32", 13, None, 0.1, True, False),
    "shipped_r1_32_f32": (LayerShape(768, 768, 8, 2, 32, 256, 512, 1e-5), 5, (5, 1), "float32", 14, 0.02, 0.0, False, False),
    "single_token_f32": (LayerShape(64, 96, 8, 2, 4, 32, 64, 1e-5), 1, (1, 1), "float32", 15, 0.02, 0.1, True, False),
    "empty_f32": (LayerShape(64, 96, 8, 2, 4, 32, 64, 1e-5), 0, (0,), "float32", 16, 0.02, 0.1, True, False),
    "topk_equals_e_f32": (LayerShape(64, 96, 4, 4, 2, 32, 64, 1e-6), 9, None, "float32", 17, 0.02, 0.0, True, False),
    "cfg0_head_f32": (LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6), 16, (1, 16), "float32", 1000, 0.02, 0.0, False, False),
    "cfg1_head_bf16": (LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6), 8, (8, 1), "bfloat16", 1001, 0.02, 0.0, False, False),
    "cfg2_head_bf16": (LayerShape(1536, 2304, 64, 2, 4, 256, 1024, 1e-6), 32, None, "bfloat16", 1002, None, 0.0, False, False),
    "cfg2_head_f32": (LayerShape(1536, 2304, 64, 2, 4, 256, 1024, 1e-6), 32, None, "float32", 1002, None, 0.0, False, False),
    "cfg4_head_f32": (LayerShape(3072, 4608, 256, 8, 8, 512, 2048, 1e-6), 4, None, "float32", 1004, 0.02, 0.0, False, True),
}


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def build_case(name):
    shape, T, lead, dtype_name, seed, rstd, bstd, store, zipf = CASES[name]
    dtype = getattr(torch, dtype_name)
    f = make_factors(shape, seed, torch.float32, rstd, bstd)
    x = make_tokens(T, shape.d_in, seed, torch.float32)
    if zipf:
        x, f = apply_zipf_router_bias(x, f, seed)
    f = {k: v.to(dtype) for k, v in f.items()}
    x = x.to(dtype)
    if lead is not None:
        x = x.reshape(*lead, shape.d_in)
    return shape, x, f, dtype, store


def run_reference(ref_root, shape, x, f, dtype):
    sys.path.insert(0, ref_root)
    from pure_torch_mlx.model import TuckerMoE  # the real reference module
    cfg = SimpleNamespace(kmoe_num_experts=shape.E, kmoe_top_k=shape.top_k, kmoe_r1=shape.r1,
                          kmoe_r2=shape.r2, kmoe_r3=shape.r3, rms_norm_eps=shape.eps)
    m = TuckerMoE(shape.d_in, shape.d_out, cfg).to(dtype)
    with torch.no_grad():
        m.router.weight.copy_(f["router_w"]); m.U_in.copy_(f["U_in"])
        m.inner_norm.weight.copy_(f["inner_norm_w"]); m.U_expert.copy_(f["U_expert"])
        m.core.copy_(f["core"]); m.U_out.copy_(f["U_out"]); m.bias.copy_(f["bias"])
        y = m(x)
        xf = x.reshape(-1, shape.d_in)
        scores = m.router(xf)
        val, idx = torch.topk(scores, m.top_k, dim=-1)
        gates = torch.softmax(val, -1)
    return y, scores, idx, gates


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a checkout of the reference project (s990093/Mamba-TuckerMoE)")
    ap.add_argument("--only", default=None)
    a = ap.parse_args()
    torch.manual_seed(0)
    for name in CASES:
        if a.only and name != a.only:
            continue
        shape, x, f, dtype, store = build_case(name)
        y, scores, idx, gates = run_reference(a.reference, shape, x, f, dtype)
        out = {
            "y": y.float().numpy(), "scores": scores.float().numpy(), "idx": idx.numpy(),
            "gates": gates.float().numpy(),
            "sha_x": np.array(sha(x)), "x_shape": np.array(x.shape, dtype=np.int64),
        }
        for k, v in f.items():
            out["sha_" + k] = np.array(sha(v))
        if store:
            out["x"] = x.float().numpy()
            for k, v in f.items():
                out["f_" + k] = v.float().numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(f"{name}: x{tuple(x.shape)} -> y{tuple(y.shape)} |y|max={float(y.float().abs().max()) if y.numel() else 0:.4f}")


if __name__ == "__main__":
    main()
