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
from oracle.tucker_moe_oracle import classify_topk, layer_forward, layer_forward_f64, max_abs, rel_fro, router_logits  # noqa: E402

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


def compare(name, y, idx, gates, g, dtype, y_tol, gate_tol, case=None):
    """Selections equal the reference's except at near-ties of ITS logits (within 2e-5 in fp32, one bf16 step of a logit of
    16-20 in bf16; exact ties, which the cap produces in bf16, go to the lower expert index here and to whichever
    ``torch.topk`` met first there); on tokens with the same selection the gates and the output agree within the tolerance.
    Tokens whose selection differs by such a tie (``case`` = (shape, x, f) given): the sorted gates still agree -- tied logits
    have equal probabilities -- and the output agrees with the float64 statement evaluated on this run's selection."""
    gap = 2e-5 if dtype == torch.float32 else 2.0 ** -3
    idx, gates, y = idx.long().cpu(), gates.float().cpu(), y.float().cpu()
    rep = classify_topk(idx, g["idx"], reference_logits(g["scores"], dtype), gap)
    assert rep.unexplained == 0, (name, rep)
    same = (idx == g["idx"].long()).all(-1)
    assert int(same.sum()) >= 0.6 * same.numel(), (name, rep)
    assert max_abs(gates[same], g["gates"][same]) < gate_tol
    assert rel_fro(y[same], g["y"][same]) < y_tol
    scale = float(g["y"].abs().max())
    assert max_abs(y[same], g["y"][same]) < y_tol * scale * (1 if dtype == torch.float32 else 2)
    if case is not None and not bool(same.all()):
        shape, x, f = case
        t = torch.nonzero(~same).flatten()
        # a near-tie (not an exact one) moves a gate by up to the gap's worth of probability
        slack = gate_tol if dtype == torch.float32 else 0.07
        assert max_abs(gates[t].sort(-1).values, g["gates"][t].sort(-1).values) < slack
        y64, _ = layer_forward_f64(x[t], f, shape.top_k, shape.eps, idx=idx[t], router=ROUTER,
                                   round_scores_to=None if dtype == torch.float32 else dtype)
        assert rel_fro(y[t], y64) < y_tol


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_reproduces_the_variant_module(name):
    shape, x, f, dtype, g = load(name)
    y, taps = layer_forward(x, f, shape.top_k, shape.eps, return_taps=True, router=ROUTER)
    # the raw logits are the same nn.Linear
    assert rel_fro(taps["scores"].float(), g["scores"]) < (1e-6 if dtype == torch.float32 else 1e-2)
    compare(name, y, taps["idx"], taps["gates"], g, dtype, 1e-5 if dtype == torch.float32 else 2e-2,
            2e-6 if dtype == torch.float32 else 8e-3, (shape, x, f))
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
    compare(name, y, idx, gates, g, dtype, 1e-4 if dtype == torch.float32 else 2e-2, 4e-6 if dtype == torch.float32 else 8e-3,
            (shape, x, f))


@pytest.mark.gpu
@pytest.mark.parametrize("name,T", [("variant_e64_k2_bf16", 1), ("variant_e64_k2_bf16", 4), ("variant_e64_k2_bf16", 7),
                                    ("variant_shipped_bf16", 3), ("variant_shipped_bf16", 8), ("variant_e256_k8_bf16", 2),
                                    ("variant_e256_k8_bf16", 33)])
def test_decode_kernels_reproduce_the_variant_module(name, T):
    """The first T tokens of a bf16 fixture through the decode-shaped kernels (one launch up to 4 tokens, three up to 64):
    the layer is token-wise independent, so the fixture's rows are the answer."""
    from gpu_util import build_module
    from mamba_tuckermoe_b200 import PATH_DECODE, read_device_status
    shape, x, f, dtype, g = load(name)
    m = build_module(shape, f, dtype, path=PATH_DECODE)
    m.router_mode = 1
    y, (idx, gates, _) = m.forward_with_routing(x[:T].cuda())
    torch.cuda.synchronize()
    assert read_device_status() == (0, 0, 0, 0)
    compare(name, y, idx, gates, {k: v[:T] for k, v in g.items()}, dtype, 2e-2, 8e-3, (shape, x[:T], f))


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["variant_e256_k8_bf16", "variant_e64_k2_bf16", "variant_e64_k8_f32"])
def test_router_stage_reproduces_the_variant_module(name):
    """``tmoe_router`` by itself under rule 1: the persistent tensor-core kernel (bf16, 512 tokens or more), the fused
    CUDA-core kernel below that and in fp32."""
    import ctypes as C
    from gpu_util import alloc_workspace, cuda_stream_ptr, factors_struct, layer_struct
    from mamba_tuckermoe_b200 import _lib
    shape, x, f, dtype, g = load(name)
    lib = _lib.load()
    T = x.shape[0]
    fd = {k: v.cuda() for k, v in f.items()}
    L, F = layer_struct(shape, dtype), factors_struct(fd)
    L.router_mode, L.router_cap, L.router_temperature = 1, ROUTER[1], ROUTER[2]
    ws = alloc_workspace(lib, L, T, 1)
    idx = torch.empty(T, shape.top_k, dtype=torch.int32, device="cuda")
    gates = torch.empty(T, shape.top_k, dtype=torch.float32, device="cuda")
    c = torch.empty(T, shape.r1, dtype=torch.float32, device="cuda")
    xd = x.cuda()
    rc = lib.tmoe_router(C.byref(L), C.byref(F), xd.data_ptr(), T, idx.data_ptr(), gates.data_ptr(), c.data_ptr(),
                         ws.data_ptr(), ws.numel(), cuda_stream_ptr())
    assert rc == 0, _lib.status_string(rc)
    torch.cuda.synchronize()
    idx, gates = idx.long().cpu(), gates.cpu()
    gap = 2e-5 if dtype == torch.float32 else 2.0 ** -3
    rep = classify_topk(idx, g["idx"], reference_logits(g["scores"], dtype), gap)
    assert rep.unexplained == 0, (name, rep)
    same = (idx == g["idx"].long()).all(-1)
    assert int(same.sum()) >= 0.6 * T
    assert max_abs(gates[same], g["gates"][same]) < (4e-6 if dtype == torch.float32 else 8e-3)
    # c is the gate-weighted sum of the selected rows of U_expert
    c_ref = torch.einsum("tk,tkr->tr", gates.double(), f["U_expert"].double()[idx])
    assert max_abs(c.cpu(), c_ref) < 1e-5
