"""The trained-checkpoint variant of the layer (capped / tempered router, softmax over all experts, renormalised top-k:
``sft_cot_bundle/scripts/model.py:313-346``) against golden vectors made by running the reference's own module
(``tests/golden/make_variant_golden.py``; its two Triton kernel launches were replaced by torch statements of their
arithmetic for that run, everything else is the reference's code).

CPU: the oracle's restatement of that rule reproduces the fixtures.  GPU: the kernels with ``router_mode = 1`` do."""
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
sys.path.insert(0, os.path.dirname(HERE))

from make_variant_golden import CASES, build_case, sha  # noqa: E402
from oracle.tucker_moe_oracle import classify_topk, layer_forward, max_abs, rel_fro, router_logits  # noqa: E402

ROUTER = (1, 10.0, 0.5)   # rule 1, tanh cap 10, temperature get_router_temperature(None) = 0.5


def load(name):
    shape, x, f, dtype = build_case(name)
    z = np.load(os.path.join(HERE, "golden", name + ".npz"))
    assert sha(x) == str(z["sha_x"]), "regenerated x differs from the fixture's input"
    for k, v in f.items():
        assert sha(v) == str(z["sha_" + k]), f"regenerated factor {k} differs from the fixture's"
    g = {k: torch.from_numpy(z[k]) for k in ("y", "scores", "idx", "gates")}
    return shape, x, f, dtype, g


def reference_logits(scores, dtype):
    """What the reference's top-k orders by (model.py:320-327): cap * tanh(score / cap) and the division by the temperature,
    each stored in the layer dtype."""
    return router_logits(scores.to(dtype), ROUTER[1], ROUTER[2]).float()


def compare(name, y, idx, gates, g, dtype, y_tol, gate_tol):
    """Selections equal the reference's except at near-ties of ITS logits (within 2e-5 in fp32, one bf16 step of a logit of
    16-20 in bf16; exact ties, which the cap produces in bf16, go to the lower expert index on both sides); on tokens with
    the same selection the gates and the output agree within the tolerance."""
    gap = 2e-5 if dtype == torch.float32 else 2.0 ** -3
    rep = classify_topk(idx, g["idx"], reference_logits(g["scores"], dtype), gap)
    assert rep.unexplained == 0, (name, rep)
    same = (idx.long().cpu() == g["idx"].long()).all(-1)
    assert int(same.sum()) >= 0.9 * same.numel(), (name, rep)
    assert max_abs(gates.float().cpu()[same], g["gates"][same]) < gate_tol
    assert rel_fro(y.float().cpu()[same], g["y"][same]) < y_tol
    scale = float(g["y"].abs().max())
    assert max_abs(y.float().cpu()[same], g["y"][same]) < y_tol * scale * (1 if dtype == torch.float32 else 2)


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_reproduces_the_variant_module(name):
    shape, x, f, dtype, g = load(name)
    y, taps = layer_forward(x, f, shape.top_k, shape.eps, return_taps=True, router=ROUTER)
    # the raw logits are the same nn.Linear
    assert rel_fro(taps["scores"].float(), g["scores"]) < (1e-6 if dtype == torch.float32 else 1e-2)
    compare(name, y, taps["idx"], taps["gates"], g, dtype, 1e-5 if dtype == torch.float32 else 2e-2,
            2e-6 if dtype == torch.float32 else 8e-3)
    # the probabilities of a token sum to one up to the reference's +1e-6 in the denominator
    assert max_abs(taps["gates"].float().sum(-1), torch.ones(x.shape[0])) < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
def test_kernels_reproduce_the_variant_module(name):
    from gpu_util import build_module
    from mamba_tuckermoe_b200 import PATH_AUTO, read_device_status
    shape, x, f, dtype, g = load(name)
    m = build_module(shape, f, dtype, path=PATH_AUTO)
    m.router_mode = 1
    y, (idx, gates, _) = m.forward_with_routing(x.cuda())
    torch.cuda.synchronize()
    assert read_device_status() == (0, 0, 0, 0)
    compare(name, y, idx, gates, g, dtype, 1e-4 if dtype == torch.float32 else 2e-2, 4e-6 if dtype == torch.float32 else 8e-3)
