"""Checkpoint formats on either side of the layer.

* ``.npz`` key map of the reference checkpoints: every Tucker-MoE layer is stored under a prefix
  with the seven suffixes ``router.weight, U_in, inner_norm.weight, U_expert, core, U_out, bias``
  (``pure_torch_mlx/weights.py:74-81``); the prefixes inside a model are
  ``backbone.layers.{i}.block.{x_up_proj,out_proj}`` for Mamba blocks and
  ``backbone.layers.{i}.block.ffn.{gate_proj,up_proj,down_proj}`` for transformer blocks
  (``weights.py:31-41, 67-69``).
* a "prepared factors" sidecar: the K-major bf16 re-layout that the tensor-core and decode
  kernels read, saved next to a checkpoint so that a server does not redo it at start-up
  (the role the ``.mlx_bf16.npz`` sidecar plays for the reference's MLX loader,
  ``mamba3_mlx/mlx_model/weights.py:34-46``).
"""
from __future__ import annotations

import hashlib
from typing import Dict, Iterable, List, Mapping

import numpy as np
import torch

from .tucker_moe import TuckerMoE, _param_key, prepare_factors

SUFFIXES = ("router.weight", "U_in", "inner_norm.weight", "U_expert", "core", "U_out", "bias")


def tucker_prefixes(block_types: Iterable[str]) -> List[str]:
    """Checkpoint prefixes of every Tucker-MoE layer of a model whose blocks are 'mamba' / 'transformer'
    in the given order (``Mamba3Config.block_types()``, ``pure_torch_mlx/config.py:35-42``)."""
    out = []
    for i, t in enumerate(block_types):
        pfx = f"backbone.layers.{i}.block"
        if t == "mamba":
            out += [f"{pfx}.x_up_proj", f"{pfx}.out_proj"]
        else:
            out += [f"{pfx}.ffn.gate_proj", f"{pfx}.ffn.up_proj", f"{pfx}.ffn.down_proj"]
    return out


def _as_tensor(v, dtype, device) -> torch.Tensor:
    if isinstance(v, np.ndarray):
        v = torch.from_numpy(v.astype(np.float32) if v.dtype != np.float32 else v)
    return v.to(device=device, dtype=dtype)


def load_tucker(layer: TuckerMoE, weights: Mapping[str, object], prefix: str) -> None:
    """Fills one layer from a mapping of checkpoint keys (numpy arrays or tensors), the job of
    ``_load_tucker`` (``pure_torch_mlx/weights.py:74-81``); cached prepared factors are dropped."""
    targets = (layer.router.weight, layer.U_in, layer.inner_norm.weight, layer.U_expert, layer.core, layer.U_out,
               layer.bias)
    with torch.no_grad():
        for suffix, p in zip(SUFFIXES, targets):
            key = f"{prefix}.{suffix}"
            if key not in weights:
                raise KeyError(f"checkpoint has no '{key}'")
            src = _as_tensor(weights[key], p.dtype, p.device)
            if tuple(src.shape) != tuple(p.shape):
                raise ValueError(f"'{key}' has shape {tuple(src.shape)}, the layer expects {tuple(p.shape)}")
            p.copy_(src)
    layer.invalidate_cache()


def export_tucker(layer: TuckerMoE, prefix: str) -> Dict[str, np.ndarray]:
    """The inverse of load_tucker: fp32 numpy arrays under the reference's key names."""
    targets = (layer.router.weight, layer.U_in, layer.inner_norm.weight, layer.U_expert, layer.core, layer.U_out,
               layer.bias)
    return {f"{prefix}.{s}": p.detach().float().cpu().numpy() for s, p in zip(SUFFIXES, targets)}


def _fingerprint(layer: TuckerMoE) -> str:
    h = hashlib.sha256()
    for p in layer._params():
        h.update(str((tuple(p.shape), str(p.dtype))).encode())
        h.update(p.detach().contiguous().view(torch.uint8).cpu().numpy().tobytes())
    return h.hexdigest()


# Version of the byte layout that tmoe_prepare_factors writes (block order, tile interleave of the core, padding).  Bump it
# whenever csrc/prepare.cu's layout changes: a sidecar written for another layout is then refused instead of being read
# through the wrong offsets.
PREPARED_LAYOUT_VERSION = 1


def _layer_tuple(layer: TuckerMoE):
    r1, r3, r2 = layer.core.shape
    return [int(layer.U_in.shape[0]), int(layer.U_out.shape[1]), int(layer.router.weight.shape[0]), int(r1), int(r2),
            int(r3), str(layer.U_in.dtype)]


def _prepared_bytes(layer: TuckerMoE) -> int:
    """Size the library expects of this layer's prepared set (0: shape / dtype not covered).  Host-side query."""
    import ctypes as C
    from . import _lib
    from .tucker_moe import _layer_struct
    if layer.U_in.dtype not in (torch.float32, torch.bfloat16):
        return 0
    L = _layer_struct(layer.U_in, layer.router.weight, layer.U_in, layer.U_expert, layer.core, layer.U_out, layer.top_k,
                      layer.inner_norm.eps)
    return int(_lib.load().tmoe_prepared_bytes(C.byref(L)))


def save_prepared_sidecar(layer: TuckerMoE, path: str) -> None:
    """Writes the layer's prepared factor set with what a loader needs to decide whether it may install it: a
    fingerprint of the parameters it was made from, the library's ABI version, the layout version and the layer sizes."""
    from . import _lib
    ps = layer._params()
    prep = prepare_factors(ps[0], ps[1], ps[2], layer.inner_norm.eps, ps[3], ps[4], ps[5], ps[6], layer.top_k)
    if prep is None:
        raise RuntimeError("tmoe_b200: this layer's shape/dtype is not covered by the prepared-factor kernels")
    torch.cuda.current_stream(prep.device).synchronize()
    np.savez(path, prepared=prep.cpu().numpy(), fingerprint=np.array(_fingerprint(layer)),
             top_k=np.array(layer.top_k), eps=np.array(layer.inner_norm.eps, dtype=np.float64),
             abi=np.array(_lib.load().tmoe_version()), layout=np.array(PREPARED_LAYOUT_VERSION),
             layer=np.array(_layer_tuple(layer), dtype=object).astype(str))


def load_prepared_sidecar(layer: TuckerMoE, path: str) -> bool:
    """Installs a saved prepared factor set if it was written for this library build's layout, for a layer of these
    sizes, from exactly the layer's current parameters, and has the size the kernels will read.  Returns False (and
    leaves the layer untouched) otherwise: the kernels address the buffer through raw offsets, so a set from another
    layout or a truncated file must never reach them."""
    from . import _lib
    z = np.load(path if str(path).endswith(".npz") else str(path) + ".npz")
    need = ("prepared", "fingerprint", "top_k", "abi", "layout", "layer")
    if any(k not in z.files for k in need):
        return False
    if int(z["abi"]) != _lib.load().tmoe_version() or int(z["layout"]) != PREPARED_LAYOUT_VERSION:
        return False
    if [str(v) for v in z["layer"].tolist()] != [str(v) for v in _layer_tuple(layer)] or int(z["top_k"]) != layer.top_k:
        return False
    prepared = z["prepared"]
    expect = _prepared_bytes(layer)
    if expect <= 0 or prepared.dtype != np.uint8 or prepared.ndim != 1 or prepared.size != expect:
        return False
    if str(z["fingerprint"]) != _fingerprint(layer):
        return False
    dev = layer.U_in.device
    layer._prep = torch.from_numpy(prepared).to(dev)
    layer._prep_key = _param_key(layer._params())
    layer._plan = None
    return True
