"""Host-side checks that need no GPU: the library loads, exports every declared symbol, validates
its arguments before touching CUDA, and the module mirrors the reference's interface."""
import ctypes as C
import os
import re

import pytest
import torch

import mamba_tuckermoe_b200 as pkg
from mamba_tuckermoe_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _layer(**kw):
    base = dict(d_in=64, d_out=96, n_experts=8, top_k=2, r1=4, r2=64, r3=32, dtype=_lib.TMOE_F32, eps=1e-5,
                router_mode=0, router_cap=10.0, router_temperature=0.5)
    base.update(kw)
    return _lib.Layer(**base)


def test_header_symbols_are_exported():
    text = open(os.path.join(ROOT, "include", "tmoe_b200.h")).read()
    declared = set(re.findall(r"\b(tmoe_[a-z_]+)\s*\(", text))
    assert declared == set(_lib.EXPORTS)
    lib = _lib.load()
    for s in declared:
        assert hasattr(lib, s), s
    assert lib.tmoe_version() == _lib.ABI_VERSION == 2


def test_status_strings():
    for code in range(0, -10, -1):
        assert _lib.status_string(code) != "unknown status"
    assert _lib.status_string(-99) == "unknown status"


@pytest.mark.parametrize("kw,code", [
    (dict(d_in=0), -2), (dict(top_k=9), -2), (dict(d_in=60), -2), (dict(dtype=7), -3),
    (dict(top_k=17, n_experts=32), -2), (dict(r1=65), -2),
])
def test_invalid_layers_are_rejected(kw, code):
    lib = _lib.load()
    L = _layer(**kw)
    assert lib.tmoe_workspace_bytes(C.byref(L), 16, 0) == code
    assert lib.tmoe_prepared_bytes(C.byref(L)) == code
    assert lib.tmoe_resolve_path(C.byref(L), 16, 0) == code


def test_router_rule_parameters_are_validated():
    """An unknown gate rule, or a cap / temperature the capped rule cannot divide by, is an error, not a silent default."""
    lib = _lib.load()
    assert lib.tmoe_workspace_bytes(C.byref(_layer(router_mode=2)), 16, 0) == -6
    assert lib.tmoe_workspace_bytes(C.byref(_layer(router_mode=-1)), 16, 0) == -6
    for kw in (dict(router_cap=0.0), dict(router_cap=-1.0), dict(router_temperature=0.0), dict(router_cap=float("nan")),
               dict(router_temperature=float("inf"))):
        assert lib.tmoe_workspace_bytes(C.byref(_layer(router_mode=1, **kw)), 16, 0) == -2, kw
        assert lib.tmoe_workspace_bytes(C.byref(_layer(router_mode=0, **kw)), 16, 0) > 0, kw   # rule 0 ignores them
    assert lib.tmoe_workspace_bytes(C.byref(_layer(router_mode=1)), 16, 0) > 0
    # top_k is not clamped to the expert count (the trained-checkpoint module clamps; callers pass min(top_k, E))
    assert lib.tmoe_workspace_bytes(C.byref(_layer(top_k=9, n_experts=8)), 16, 0) == -2


def test_token_count_bound():
    lib = _lib.load()
    L = _layer()
    F = _lib.Factors(*[4096] * 7)
    assert lib.tmoe_workspace_bytes(C.byref(L), 1 << 30, 1) > 0
    assert lib.tmoe_workspace_bytes(C.byref(L), (1 << 30) + 1, 1) == -2
    assert lib.tmoe_resolve_path(C.byref(L), 1 << 40, 0) == -2
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, 4096, (1 << 30) + 1, 4096, None, 4096, 1 << 20, 1, None) == -2
    assert lib.tmoe_router(C.byref(L), C.byref(F), 4096, 1 << 31, 4096, 4096, 4096, 4096, 1 << 20, None) == -2


def test_static_scratch_validates_before_enqueueing():
    lib = _lib.load()
    L = _layer()
    F = _lib.Factors(*[4096] * 7)
    # also at T == 0: bad factors, then a clean no-op
    assert lib.tmoe_forward_static_scratch(C.byref(L), None, 4096, 0, 4096, None, None) == -1
    Fbad = _lib.Factors(4096, 4096, 4100, 4096, 4096, 4096, 4096)
    assert lib.tmoe_forward_static_scratch(C.byref(L), C.byref(Fbad), 4096, 0, 4096, None, None) == -4
    assert lib.tmoe_forward_static_scratch(C.byref(L), C.byref(F), 4096, 0, 4096, None, None) == 0
    assert lib.tmoe_forward_static_scratch(C.byref(L), C.byref(F), None, 4, 4096, None, None) == -1
    assert lib.tmoe_forward_static_scratch(C.byref(L), C.byref(F), 4100, 4, 4096, None, None) == -4
    # the largest T that fits is what tmoe_workspace_bytes says, and one more token is refused
    t = 1
    while lib.tmoe_workspace_bytes(C.byref(L), t + 1, 1) <= _lib.STATIC_SCRATCH_BYTES:
        t += 1 if t < 64 else t // 16
    while lib.tmoe_workspace_bytes(C.byref(L), t, 1) > _lib.STATIC_SCRATCH_BYTES:
        t -= 1
    assert lib.tmoe_workspace_bytes(C.byref(L), t, 1) <= _lib.STATIC_SCRATCH_BYTES < lib.tmoe_workspace_bytes(C.byref(L), t + 1, 1)
    assert lib.tmoe_forward_static_scratch(C.byref(L), C.byref(F), 4096, t + 1, 4096, None, None) == -5


def test_null_and_alignment_errors_before_any_cuda_call():
    lib = _lib.load()
    L = _layer()
    F = _lib.Factors(*[4096] * 7)
    assert lib.tmoe_forward(C.byref(L), None, None, 4096, 4, 4096, None, 4096, 1 << 20, 1, None) == -1
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, None, 4, 4096, None, 4096, 1 << 20, 1, None) == -1
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, 4100, 4, 4096, None, 4096, 1 << 20, 1, None) == -4
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, 4096, 4, 4096, None, 4096, 16, 1, None) == -5
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, 4096, -1, 4096, None, 4096, 1 << 20, 1, None) == -2
    # the tensor-core path does not cover fp32 layers; T == 0 enqueues nothing
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, 4096, 4, 4096, None, 4096, 1 << 20, 2, None) == -6
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, 4096, 0, 4096, None, 4096, 1 << 20, 1, None) == 0
    Fbad = _lib.Factors(4096, 4096, 4100, 4096, 4096, 4096, 4096)
    assert lib.tmoe_forward(C.byref(L), C.byref(Fbad), None, 4096, 4, 4096, None, 4096, 1 << 20, 1, None) == -4
    ex = _lib.Extras(residual=4096)
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, 4096, 4, 4096, C.byref(ex), 4096, 1 << 20, 1, None) == -1
    # further result buffers: count in range, every pointer present and aligned, tensor-core path only
    ex = _lib.Extras(n_peer_y=8)
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, 4096, 4, 4096, C.byref(ex), 4096, 1 << 20, 1, None) == -2
    ex = _lib.Extras(n_peer_y=2)
    ex.peer_y[0] = 4096
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, 4096, 4, 4096, C.byref(ex), 4096, 1 << 20, 1, None) == -1
    ex.peer_y[1] = 4100
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, 4096, 4, 4096, C.byref(ex), 4096, 1 << 20, 1, None) == -4
    ex.peer_y[1] = 8192
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, 4096, 4, 4096, C.byref(ex), 4096, 1 << 20, 1, None) == -6


def test_peer_buffer_entry_points_validate():
    lib = _lib.load()
    p, h = C.c_void_p(), (C.c_ubyte * _lib.PEER_HANDLE_BYTES)()
    assert lib.tmoe_peer_alloc(0, C.byref(p), h) == -2
    assert lib.tmoe_peer_alloc(1 << 20, None, h) == -1
    assert lib.tmoe_peer_open(None, C.byref(p)) == -1
    assert lib.tmoe_peer_close(None) == -1 and lib.tmoe_peer_free(None) == -1
    assert lib.tmoe_peer_push(None, 0, None, 0, None) == 0
    assert lib.tmoe_peer_push(None, 2, None, 64, None) == -1
    assert lib.tmoe_peer_push(None, -1, None, 64, None) == -2


def test_path_resolution_and_sizes():
    lib = _lib.load()
    cfg2 = _layer(d_in=1536, d_out=2304, n_experts=64, top_k=2, r1=4, r2=1024, r3=256, dtype=_lib.TMOE_BF16, eps=1e-6)
    assert lib.tmoe_resolve_path(C.byref(cfg2), 32768, 0) == 2
    assert lib.tmoe_resolve_path(C.byref(cfg2), 8, 0) == 3      # decode-shaped kernels up to 8 tokens
    assert lib.tmoe_resolve_path(C.byref(cfg2), 9, 0) == 2      # one tensor-core tile (shared between CTAs) from there
    assert lib.tmoe_resolve_path(C.byref(cfg2), 64, 3) == 3     # still available on request up to 64
    assert lib.tmoe_resolve_path(C.byref(cfg2), 65, 3) == -6
    assert lib.tmoe_resolve_path(C.byref(cfg2), 1, 3) == 3
    assert lib.tmoe_resolve_path(C.byref(cfg2), 64, 2) == 2
    f32 = _layer(d_in=1536, d_out=2304, r2=1024, r3=256)
    assert lib.tmoe_resolve_path(C.byref(f32), 32768, 0) == 1
    assert lib.tmoe_resolve_path(C.byref(f32), 8, 3) == -6
    assert lib.tmoe_prepared_bytes(C.byref(f32)) == 0
    n = lib.tmoe_prepared_bytes(C.byref(cfg2))
    raw = 2 * (256 * 1536 + 64 * 1536 + 4 * 1024 * 256 + 2304 * 1024) + 4 * (256 + 2304 + 64 * 4)
    assert raw <= n <= raw + 8 * 1024
    ws = lib.tmoe_workspace_bytes(C.byref(cfg2), 32768, 0)
    assert ws >= 32768 * 1024 * 2 + 256
    # few token tiles: the tensor-core path keeps one [T, r1] block of c per CTA sharing a tile (up to 16) plus the visible one
    small, big = lib.tmoe_workspace_bytes(C.byref(cfg2), 64, 2), lib.tmoe_workspace_bytes(C.byref(cfg2), 64 * 300, 2)
    assert small >= 17 * 64 * 4 * 4 + 64 * 1024 * 2
    assert big < 300 * small                      # ... and only for small calls
    shipped = _layer(d_in=768, d_out=768, r1=32, r2=512, r3=256, dtype=_lib.TMOE_BF16)
    assert lib.tmoe_resolve_path(C.byref(shipped), 4096, 0) == 2      # r1=32: tensor-core kernels (8-column slices)
    assert lib.tmoe_resolve_path(C.byref(shipped), 4096, 2) == 2
    assert lib.tmoe_resolve_path(C.byref(shipped), 1, 0) == 3          # ... and the decode kernels up to 8 tokens
    odd = _layer(d_in=768, d_out=768, r1=3, r2=512, r3=256, dtype=_lib.TMOE_BF16)
    assert lib.tmoe_resolve_path(C.byref(odd), 4096, 0) == 1           # other r1: CUDA-core path
    assert lib.tmoe_resolve_path(C.byref(odd), 4096, 2) == -6
    assert lib.tmoe_prepared_bytes(C.byref(shipped)) > 0


def test_module_mirrors_reference_interface():
    cfg = pkg.TuckerMoEConfig(kmoe_num_experts=8, kmoe_top_k=2, kmoe_r1=4, kmoe_r2=64, kmoe_r3=32, rms_norm_eps=1e-5)
    m = pkg.TuckerMoE(64, 96, cfg)
    assert list(m.state_dict().keys()) == ["U_in", "U_expert", "core", "U_out", "bias", "router.weight",
                                           "inner_norm.weight"]
    shapes = {k: tuple(v.shape) for k, v in m.state_dict().items()}
    assert shapes == {"U_in": (64, 32), "U_expert": (8, 4), "core": (4, 32, 64), "U_out": (64, 96), "bias": (96,),
                      "router.weight": (8, 64), "inner_norm.weight": (32,)}
    assert m.top_k == 2 and m.inner_norm.eps == 1e-5
    assert torch.equal(m.bias, torch.zeros(96)) and torch.equal(m.inner_norm.weight, torch.ones(32))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        m(torch.randn(3, 64))


def test_fake_kernel_gives_shapes_without_a_gpu():
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(2, 5, 64)
        y = torch.ops.tmoe_b200.forward(x, torch.empty(8, 64), torch.empty(64, 32), torch.empty(32), 1e-5,
                                        torch.empty(8, 4), torch.empty(4, 32, 64), torch.empty(64, 96),
                                        torch.empty(96), 2, 0, None, None, None, None, 0, 10.0, 0.5)
    assert y.shape == (2, 5, 96)


def test_module_copies_and_pickles_without_its_caches():
    import copy
    import pickle
    import torch
    from mamba_tuckermoe_b200 import TuckerMoE, TuckerMoEConfig
    m = TuckerMoE(64, 72, TuckerMoEConfig(8, 2, 4, 64, 64, 1e-5))
    with torch.no_grad():
        for q in m.parameters():
            q.normal_()
    m._plan = object()          # stands for the C structs a CUDA call leaves behind
    for c in (copy.deepcopy(m), pickle.loads(pickle.dumps(m))):
        assert c._plan is None
        assert all(torch.equal(a, b) for a, b in zip(c.state_dict().values(), m.state_dict().values()))
