"""Helpers shared by the GPU parity tests."""
from __future__ import annotations

import torch

from mamba_tuckermoe_b200 import TuckerMoE, TuckerMoEConfig, _lib
from oracle.tucker_moe_oracle import LayerShape

STATE_KEYS = {"router_w": "router.weight", "U_in": "U_in", "inner_norm_w": "inner_norm.weight",
              "U_expert": "U_expert", "core": "core", "U_out": "U_out", "bias": "bias"}


def build_module(shape: LayerShape, factors, dtype, device="cuda", path=0) -> TuckerMoE:
    cfg = TuckerMoEConfig(shape.E, shape.top_k, shape.r1, shape.r2, shape.r3, shape.eps)
    m = TuckerMoE(shape.d_in, shape.d_out, cfg)
    m.load_state_dict({STATE_KEYS[k]: v.float() for k, v in factors.items()})
    m = m.to(device=device, dtype=dtype)
    m.path = path
    return m


def layer_struct(shape, dtype):
    return _lib.layer_struct(shape, dtype)


def factors_struct(dev_factors):
    return _lib.factors_struct(dev_factors)


def cuda_stream_ptr():
    return _lib.current_stream_ptr()


def alloc_workspace(lib, layer, T, path):
    return _lib.alloc_workspace(layer, T, path)


def alloc_prepared(lib, layer, factors):
    return _lib.alloc_prepared(layer, factors)
