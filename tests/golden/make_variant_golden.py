"""Golden vectors of the TRAINED-CHECKPOINT variant of the layer (``sft_cot_bundle/scripts/model.py:291-346``,
``TritonTuckerMoE``): capped and tempered router, softmax over all experts, renormalised top-k.

    python tests/golden/make_variant_golden.py --reference /path/to/Mamba-TuckerMoE

The module is imported from the checkout and its own ``forward`` runs on CPU.  That forward launches two Triton kernels,
which need a GPU; for this run the two launchers are replaced by torch statements of exactly what the kernels compute:

* ``fast_scaled_tanh(x, s)`` (``model.py:32-40, 69-70``): ``(2 * sigmoid(2 * (x * (1 / s))) - 1) * s`` in fp32, stored in x's dtype;
* ``FusedLatentMoE.apply(x_shared, G, idx, p)`` (``model.py:165-185, 224-238``): ``sum_k p[b, k] * (x_shared[b] @ G[idx[b, k]])``
  accumulated in fp32, stored in x_shared's dtype.

Everything else is the reference's code as it stands: the router ``nn.Linear``, the temperature (``get_router_temperature(None)``
= 0.5), the softmax, ``torch.topk``, the ``+1e-6`` renormalisation, ``x @ U_in``, ``nn.RMSNorm`` (eps 1e-5), the
``einsum`` that builds the per-expert cores, ``@ U_out`` and the bias.  The stand-ins also record what the module handed
them: the raw logits, the selected experts and their renormalised probabilities.  So the fixtures pin the variant's
router and layer algebra to the reference's own PyTorch code; the arithmetic inside its two Triton kernels is restated.
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

from oracle.tucker_moe_oracle import LayerShape, make_factors, make_tokens  # noqa: E402

# name: (shape, T, dtype, seed, router_std)   -- eps is nn.RMSNorm's 1e-5 in the variant
CASES = {
    "variant_tiny_f32": (LayerShape(64, 96, 8, 2, 4, 32, 64, 1e-5), 24, "float32", 2101, 1.0),
    "variant_e64_k8_f32": (LayerShape(256, 384, 64, 8, 8, 64, 128, 1e-5), 40, "float32", 2102, 0.5),
    "variant_shipped_f32": (LayerShape(768, 768, 8, 2, 32, 256, 512, 1e-5), 6, "float32", 2103, 0.3),
    "variant_e64_k2_bf16": (LayerShape(256, 384, 64, 2, 4, 128, 256, 1e-5), 300, "bfloat16", 2104, 0.5),
    "variant_shipped_bf16": (LayerShape(768, 768, 8, 2, 32, 256, 512, 1e-5), 64, "bfloat16", 2105, 0.3),
    # 512 tokens or more in bf16: the stand-alone router runs on the tensor cores
    "variant_e256_k8_bf16": (LayerShape(256, 128, 256, 8, 8, 64, 128, 1e-5), 600, "bfloat16", 2106, 0.3),
}


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def build_case(name):
    """Seeded inputs of a case (the router rows are wide enough for the tanh cap at 10 to matter for some tokens)."""
    shape, T, dtype_name, seed, rstd = CASES[name]
    dtype = getattr(torch, dtype_name)
    f = make_factors(shape, seed, torch.float32, rstd, 0.1)
    x = make_tokens(T, shape.d_in, seed, torch.float32)
    return shape, x.to(dtype), {k: v.to(dtype) for k, v in f.items()}, dtype


def run_reference(ref_root, shape, x, f, dtype):
    sys.path.insert(0, os.path.join(ref_root, "sft_cot_bundle", "scripts"))
    import model as ref  # the reference's trained-checkpoint model file

    seen = {}

    def scaled_tanh(v, scale=10.0):
        seen["scores"] = v.detach().clone()
        return ((2.0 * torch.sigmoid(2.0 * (v.float() * (1.0 / scale))) - 1.0) * scale).to(v.dtype)

    class Core:
        @staticmethod
        def apply(x_shared, g_experts, idx, probs):
            seen["idx"], seen["gates"] = idx.detach().clone(), probs.detach().clone()
            acc = torch.zeros(x_shared.shape[0], g_experts.shape[2], dtype=torch.float32)
            for k in range(idx.shape[1]):
                g = g_experts[idx[:, k]].float()                                  # [B, r3, r2]
                acc += probs[:, k:k + 1].float() * torch.einsum("br,brs->bs", x_shared.float(), g)
            return acc.to(x_shared.dtype)

    ref.fast_scaled_tanh, ref.FusedLatentMoE = scaled_tanh, Core
    m = ref.TritonTuckerMoE(shape.d_in, shape.d_out, num_experts=shape.E, top_k=shape.top_k, r1=shape.r1, r2=shape.r2,
                            r3=shape.r3).to(dtype).eval()
    with torch.no_grad():
        m.router.weight.copy_(f["router_w"]); m.U_in.copy_(f["U_in"])
        m.inner_norm.weight.copy_(f["inner_norm_w"]); m.U_expert.copy_(f["U_expert"])
        m.core.copy_(f["core"]); m.U_out.copy_(f["U_out"]); m.bias.copy_(f["bias"])
        y, _, _ = m(x)
    return y, seen["scores"], seen["idx"], seen["gates"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a checkout of the reference project (s990093/Mamba-TuckerMoE)")
    a = ap.parse_args()
    for name in CASES:
        shape, x, f, dtype = build_case(name)
        y, scores, idx, gates = run_reference(a.reference, shape, x, f, dtype)
        out = {"y": y.float().numpy(), "scores": scores.float().numpy(), "idx": idx.numpy(), "gates": gates.float().numpy(),
               "sha_x": np.array(sha(x))}
        for k, v in f.items():
            out["sha_" + k] = np.array(sha(v))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        capped = int((scores.float().abs() > 5).sum())
        print(f"{name}: x{tuple(x.shape)} -> y{tuple(y.shape)} |y|max={float(y.float().abs().max()):.4f} "
              f"|score|max={float(scores.float().abs().max()):.2f} ({capped} scores beyond 5)")


if __name__ == "__main__":
    main()
