"""The drop-in layer where the reference model uses it: inside ``Mamba3Block`` / ``TransformerBlock`` of
``pure_torch_mlx/model.py`` and behind the reference's checkpoint loader.

``tests/golden/model_decode_f32.npz`` was recorded from the REAL reference model (one Mamba block + one transformer
block at the shipped widths and ranks) running ``decode`` for two tokens: the input and output of each of its five
Tucker-MoE layers, and the callers' compositions around them (``model.py:258-260`` and ``model.py:337-341``).  The CPU
tests pin that fixture to the oracle and, when the reference checkout is present, build the reference model with the
drop-in class in place of its own.  The GPU tests replay the recorded activations through the drop-in.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

from make_model_golden import MAMBA_LAYERS, XFMR_LAYERS, layer_factors, sha  # noqa: E402
from oracle.tucker_moe_oracle import layer_forward, layer_forward_f64, max_abs, rel_fro, rms_norm as ref_norm  # noqa: E402

# the reference checkout: TMOE_REFERENCE_DIR, or a directory named "reference" beside this repository
REFERENCE = os.environ.get("TMOE_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
ALL_LAYERS = MAMBA_LAYERS + XFMR_LAYERS


@pytest.fixture(scope="module")
def golden():
    z = np.load(os.path.join(HERE, "golden", "model_decode_f32.npz"))
    g = {k: (torch.from_numpy(z[k]) if z[k].ndim else z[k]) for k in z.files}
    layers = {}
    for attr, _, d_in, d_out, seed in ALL_LAYERS:
        shape, f = layer_factors(d_in, d_out, seed)
        for k, v in f.items():
            assert sha(v) == str(g[f"sha.{attr}.{k}"]), f"regenerated factor {attr}.{k} differs from the fixture's"
        layers[attr] = (shape, f)
    g["layers"] = layers
    g["eps"] = float(g["eps"])
    return g


# ------------------------------------------------------------------------------------------ CPU
@pytest.mark.parametrize("attr", [a for a, *_ in ALL_LAYERS])
def test_oracle_reproduces_the_layers_inside_the_real_model(golden, attr):
    """The restatement gives, on the activations the real model fed its layers, what the real model's layers gave."""
    shape, f = golden["layers"][attr]
    y = layer_forward(golden[attr + ".x"], f, shape.top_k, shape.eps)
    assert max_abs(y, golden[attr + ".y"]) <= 1e-5 * float(golden[attr + ".y"].abs().max())


def test_recorded_compositions_are_the_callers_formulas(golden):
    """mid + gamma * out_proj(norm(mid)) and x_res + gamma * ffn_down(silu(gate) * up) (model.py:258-260, 337-341)."""
    eps = golden["eps"]
    proj = golden["out_proj.y"]
    assert torch.allclose(golden["out_proj.x"], ref_norm(golden["mid"], golden["norm_out_proj.weight"], eps), atol=1e-5)
    assert torch.allclose(golden["mamba_out"], golden["mid"] + golden["ls_out_proj.gamma"] * proj, atol=1e-5)
    assert torch.allclose(golden["ffn_gate.x"], ref_norm(golden["x_res"], golden["norm_ffn.weight"], eps), atol=1e-5)
    assert torch.allclose(golden["ffn_down.x"], F.silu(golden["ffn_gate.y"]) * golden["ffn_up.y"], atol=1e-4)
    assert torch.allclose(golden["xfmr_out"], golden["x_res"] + golden["ls_ffn.gamma"] * golden["ffn_down.y"], atol=1e-4)


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "pure_torch_mlx")), reason="reference checkout not present")
def test_drop_in_class_inside_the_reference_model():
    """Swap the class in the reference's own module, build its language model, fill every Tucker layer through the
    reference's own loader: same state_dict keys and shapes as the unpatched model, same values after loading."""
    sys.path.insert(0, REFERENCE)
    import pure_torch_mlx.model as ref_model
    from pure_torch_mlx.config import Mamba3Config
    from pure_torch_mlx.weights import _load_tucker
    from mamba_tuckermoe_b200 import TuckerMoE
    from mamba_tuckermoe_b200.checkpoint import export_tucker, tucker_prefixes
    cfg = Mamba3Config(num_layers=1, mamba_ratio=2, vocab_size=32, kmoe_r1=4, kmoe_r2=64, kmoe_r3=32)
    plain = ref_model.Mamba3LM(cfg)
    original = ref_model.TuckerMoE
    ref_model.TuckerMoE = TuckerMoE
    try:
        swapped = ref_model.Mamba3LM(cfg)
    finally:
        ref_model.TuckerMoE = original
    n_tucker = sum(isinstance(m, TuckerMoE) for m in swapped.modules())
    assert n_tucker == 2 * 2 + 3 and not any(isinstance(m, original) for m in swapped.modules())
    a, b = plain.state_dict(), swapped.state_dict()
    assert list(a.keys()) == list(b.keys())
    assert all(a[k].shape == b[k].shape and a[k].dtype == b[k].dtype for k in a)
    # the reference's loader, layer by layer, from a checkpoint dict in its key layout
    prefixes = tucker_prefixes(cfg.block_types())
    assert len(prefixes) == n_tucker
    g = torch.Generator().manual_seed(0)
    with torch.no_grad():
        for m in plain.modules():
            if isinstance(m, original):
                for p in m.parameters():
                    p.copy_(torch.randn(p.shape, generator=g))
    def tucker_modules(model, cls):
        out = []
        for blk in model.blocks:
            names = ("x_up_proj", "out_proj") if hasattr(blk, "x_up_proj") else ("ffn_gate", "ffn_up", "ffn_down")
            out += [getattr(blk, n) for n in names]
        assert all(isinstance(m, cls) for m in out)
        return out
    src, dst = tucker_modules(plain, original), tucker_modules(swapped, TuckerMoE)
    for pfx, ms, md in zip(prefixes, src, dst):
        w = {k: torch.from_numpy(v) for k, v in export_tucker(ms, pfx).items()}
        _load_tucker(md, w, pfx)
        for (ka, va), (kb, vb) in zip(ms.state_dict().items(), md.state_dict().items()):
            assert ka == kb and torch.equal(va, vb)
    # a forward on CPU tensors is refused loudly (no fallback hides a missing GPU)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        dst[0](torch.randn(1, 1, dst[0].U_in.shape[0]))


def test_load_state_dict_drops_the_prepared_cache():
    """Parameters replaced through load_state_dict must not leave a stale prepared factor set behind."""
    from mamba_tuckermoe_b200 import TuckerMoE, TuckerMoEConfig
    m = TuckerMoE(64, 96, TuckerMoEConfig(8, 2, 4, 64, 32, 1e-5))
    m._prep, m._prep_key, m._plan = torch.zeros(4), ("stale",), object()
    m.load_state_dict(m.state_dict())
    assert m._prep is None and m._prep_key is None and m._plan is None


# ------------------------------------------------------------------------------------------ GPU
def _module(shape, f, dtype):
    from gpu_util import build_module
    return build_module(shape, {k: v.to(dtype) for k, v in f.items()}, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("attr", [a for a, *_ in ALL_LAYERS])
def test_drop_in_on_the_real_models_activations_fp32(golden, attr):
    shape, f = golden["layers"][attr]
    m = _module(shape, f, torch.float32)
    x = golden[attr + ".x"].reshape(-1, 1, 1, shape.d_in)            # the model calls the layer with (1, 1, d) inputs
    want = golden[attr + ".y"]
    for s in range(x.shape[0]):
        y = m(x[s].cuda())
        assert y.shape == (1, 1, shape.d_out)
        got = y.reshape(-1).cpu()
        assert rel_fro(got, want[s]) <= 1e-4
        assert max_abs(got, want[s]) <= 1e-4 * float(want[s].abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("attr", [a for a, *_ in ALL_LAYERS])
def test_drop_in_on_the_real_models_activations_bf16(golden, attr):
    """bf16 weights and activations (decode kernels, T = 1): against the bf16 reference restatement under the parity rule."""
    from mamba_tuckermoe_b200 import read_device_status
    from oracle.parity import assert_parity, parity_report
    shape, f = golden["layers"][attr]
    fb = {k: v.bfloat16() for k, v in f.items()}
    m = _module(shape, f, torch.bfloat16)
    xb = golden[attr + ".x"].bfloat16()
    ys, idxs = [], []
    for s in range(xb.shape[0]):
        y, (idx, _, _) = m.forward_with_routing(xb[s:s + 1].cuda())
        ys.append(y); idxs.append(idx)
    torch.cuda.synchronize()
    assert read_device_status() == (0, 0, 0, 0)
    rep = parity_report(torch.cat(ys), torch.cat(idxs), xb, fb, shape.top_k, shape.eps, torch.bfloat16)
    assert_parity(rep, attr)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_block_tails_match_the_real_model(golden, dtype):
    """fused_out_proj and fused_ffn on the recorded block-internal activations against what the real blocks returned."""
    from mamba_tuckermoe_b200 import fused_ffn, fused_out_proj
    eps = golden["eps"]
    mods = {a: _module(*golden["layers"][a], dtype) for a, *_ in ALL_LAYERS}
    dev = lambda t: t.to(dtype).cuda()
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for s in range(golden["mid"].shape[0]):
        mid = golden["mid"][s].reshape(1, 1, -1)
        got = fused_out_proj(mods["out_proj"], dev(mid), (dev(golden["norm_out_proj.weight"]), eps), dev(golden["ls_out_proj.gamma"]))
        x_res = golden["x_res"][s].reshape(1, 1, -1)
        got2 = fused_ffn(mods["ffn_gate"], mods["ffn_up"], mods["ffn_down"], dev(x_res),
                         (dev(golden["norm_ffn.weight"]), eps), dev(golden["ls_ffn.gamma"]))
        for g, want, name in ((got, golden["mamba_out"][s], "out_proj tail"), (got2, golden["xfmr_out"][s], "ffn")):
            g = g.reshape(-1).float().cpu()
            if dtype == torch.float32:
                assert rel_fro(g, want) <= tol, name
                assert max_abs(g, want) <= tol * float(want.abs().max()), name
            else:
                # bf16 end to end against the fp32 model: rounding of weights and activations, no selection flips expected
                # to matter at 2e-2 unless two scores tie -- report which composition if so
                lim = tol if name == "out_proj tail" else 3e-2   # three chained bf16 layers in the FFN
                assert rel_fro(g, want) <= lim, f"{name}: {rel_fro(g, want):.3e}"


@pytest.mark.gpu
def test_in_place_weight_load_needs_invalidate_cache(golden):
    """The reference's loader writes through ``.data.copy_`` (weights.py:74-81), which does not change tensor versions.
    Before the first forward that is harmless; after it, the cached prepared factor set is stale until
    ``invalidate_cache()`` is called.  ``load_state_dict`` and ``checkpoint.load_tucker`` invalidate by themselves."""
    from mamba_tuckermoe_b200.checkpoint import export_tucker, load_tucker
    shape, f = golden["layers"]["out_proj"]
    f2 = layer_factors(768, 768, 777)[1]
    m = _module(shape, f, torch.bfloat16)
    x = golden["out_proj.x"].bfloat16().cuda()
    y_old = m(x)
    ref_new = layer_forward_f64(x.cpu(), {k: v.bfloat16() for k, v in f2.items()}, shape.top_k, shape.eps,
                                round_scores_to=torch.bfloat16)[0]
    targets = dict(zip(("router_w", "U_in", "inner_norm_w", "U_expert", "core", "U_out", "bias"), m._params()))
    versions = [p._version for p in m._params()]
    for k, p in targets.items():                         # what _load_tucker does
        p.data.copy_(f2[k].to(p.dtype))
    assert [p._version for p in m._params()] == versions  # ... invisible to the version counters
    y_stale = m(x)
    assert torch.equal(y_stale, y_old), "the hazard: the cached prepared factors still serve the old values"
    m.invalidate_cache()
    y_new = m(x)
    assert rel_fro(y_new.float().cpu(), ref_new) < 2e-2 and not torch.equal(y_new, y_old)
    # the library's own loader and load_state_dict need no manual step
    m2 = _module(shape, f, torch.bfloat16)
    m2(x)
    load_tucker(m2, {f"p.{k}": v for k, v in zip(("router.weight", "U_in", "inner_norm.weight", "U_expert", "core", "U_out", "bias"),
                                                  (f2["router_w"], f2["U_in"], f2["inner_norm_w"], f2["U_expert"], f2["core"], f2["U_out"], f2["bias"]))}, "p")
    assert torch.equal(m2(x), y_new)
    m3 = _module(shape, f, torch.bfloat16)
    m3(x)
    m3.load_state_dict(m2.state_dict())
    assert torch.equal(m3(x), y_new)
