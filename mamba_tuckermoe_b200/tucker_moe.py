"""Drop-in replacement for the reference ``TuckerMoE`` layer, forward only, on B200.

Mirrors ``pure_torch_mlx/model.py:41-102``: same constructor ``TuckerMoE(d_in, d_out, cfg)``,
same parameter names and shapes (so ``state_dict`` keys and the checkpoint loader of
``pure_torch_mlx/weights.py:74-81`` work unchanged), same ``forward(x: (..., d_in)) -> (..., d_out)``
and the public ``top_k`` attribute.  ``forward`` calls the torch custom op
``tmoe_b200::forward`` which hands raw device pointers and the current CUDA stream to the
C-ABI library; there is no PyTorch or CPU fallback for the computation.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import _lib
from ._lib import PATH_AUTO, PATH_DECODE, PATH_SIMT, PATH_TENSOR, Extras, Factors, Layer

__all__ = ["TuckerMoE", "TuckerMoEConfig", "RMSNorm", "tucker_moe_forward", "tucker_moe_forward_taps", "prepare_factors",
           "rms_norm", "fused_ffn", "fused_out_proj",
           "PATH_AUTO", "PATH_SIMT", "PATH_TENSOR", "PATH_DECODE"]


@dataclass
class TuckerMoEConfig:
    """The six fields of the reference ``Mamba3Config`` that the layer reads
    (``pure_torch_mlx/config.py:18-24``, read at ``model.py:56-58,62``), with its defaults.
    Any object with these attributes (the reference dataclass itself included) is accepted."""
    kmoe_num_experts: int = 8
    kmoe_top_k: int = 2
    kmoe_r1: int = 32
    kmoe_r2: int = 512
    kmoe_r3: int = 256
    rms_norm_eps: float = 1e-5


class RMSNorm(nn.Module):
    """Parameter holder with the reference's attribute names (``model.py:19-27``).  Its forward
    is only used outside the fused layer (the layer applies the norm inside its kernels)."""

    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rms = x.pow(2).mean(-1, keepdim=True).add(self.eps).sqrt()
        return (x / rms) * self.weight


_DTYPES = {torch.float32: _lib.TMOE_F32, torch.bfloat16: _lib.TMOE_BF16}

# ------------------------------------------------------------------------------------------
# per-(device, stream) scratch.  Prepared factor sets are NOT cached globally: a key made of
# addresses and versions can collide once a freed parameter's memory is reused, so the cache
# lives on the module that owns the parameters (TuckerMoE._prepared_for).
# ------------------------------------------------------------------------------------------
_cache_lock = threading.Lock()
_workspaces = {}   # (device index, stream handle) -> uint8 tensor


def _workspace(device: torch.device, nbytes: int, stream: Optional[int] = None) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream if stream is None else stream)
    with _cache_lock:
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            # grow geometrically; zero so that the status words start clear
            ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            _workspaces[key] = ws
    return ws


def _param_key(tensors) -> tuple:
    return tuple((t.data_ptr(), t._version, t.dtype, tuple(t.shape)) for t in tensors)


def clear_caches() -> None:
    """Drops the cached per-stream workspaces."""
    with _cache_lock:
        _workspaces.clear()


def prepare_factors(router_w, U_in, inner_norm_w, eps, U_expert, core, U_out, bias, top_k,
                    pre_norm_weight: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Re-laid-out factor set for the tensor-core path (``tmoe_prepare_factors``), or None when
    that path does not cover the layer.  Valid until any of the seven tensors changes.
    With ``pre_norm_weight`` ([d_in]) the callers' RMSNorm weight is folded into the U_in / router copies
    (``tmoe_prepare_factors_prenorm``); such a set is only for forwards that apply the pre-norm in-kernel."""
    params = tuple(p if p.is_contiguous() else p.contiguous()
                   for p in (router_w, U_in, inner_norm_w, U_expert, core, U_out, bias))
    if not params[0].is_cuda or params[0].dtype not in _DTYPES:
        return None
    lib = _lib.load()
    layer = _layer_struct(params[0], params[0], params[1], params[3], params[4], params[5], top_k, eps)
    nbytes = _lib.check(lib.tmoe_prepared_bytes(C.byref(layer)), "tmoe_prepared_bytes")
    if nbytes == 0:
        return None
    dev = params[0].device
    with torch.cuda.device(dev):
        prep = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        factors = Factors(*[p.data_ptr() for p in params])
        stream = torch.cuda.current_stream(dev).cuda_stream
        if pre_norm_weight is None:
            _lib.check(lib.tmoe_prepare_factors(C.byref(layer), C.byref(factors), prep.data_ptr(), nbytes, stream),
                       "tmoe_prepare_factors")
        else:
            w = pre_norm_weight.contiguous()
            if w.dtype != params[0].dtype or w.device != dev or w.shape != (params[1].shape[0],):
                raise RuntimeError("tmoe_b200: pre-norm weight must be (d_in,) in the layer's dtype on its device")
            _lib.check(lib.tmoe_prepare_factors_prenorm(C.byref(layer), C.byref(factors), w.data_ptr(), prep.data_ptr(),
                                                        nbytes, stream), "tmoe_prepare_factors_prenorm")
    return prep


_DEFAULT_ROUTER = (0, 10.0, 0.5)  # (mode, soft cap, temperature); mode 0 ignores the other two


def _layer_struct(x, router_w, U_in, U_expert, core, U_out, top_k, eps, router=_DEFAULT_ROUTER) -> Layer:
    r1, r3, r2 = core.shape
    return Layer(int(U_in.shape[0]), int(U_out.shape[1]), int(router_w.shape[0]), int(top_k), int(r1), int(r2),
                 int(r3), _DTYPES[x.dtype], float(eps), int(router[0]), float(router[1]), float(router[2]))


def _validate(x, params, top_k):
    router_w, U_in, inner_norm_w, U_expert, core, U_out, bias = params
    if not x.is_cuda:
        raise RuntimeError("tmoe_b200: the layer forward runs on CUDA tensors only (no CPU fallback)")
    if x.dtype not in _DTYPES:
        raise RuntimeError(f"tmoe_b200: unsupported dtype {x.dtype} (float32 and bfloat16 only)")
    for name, t in zip(("router.weight", "U_in", "inner_norm.weight", "U_expert", "core", "U_out", "bias"), params):
        if t.device != x.device or t.dtype != x.dtype:
            raise RuntimeError(f"tmoe_b200: parameter {name} is {t.dtype} on {t.device}, x is {x.dtype} on {x.device}")
    E, d_in = router_w.shape
    r1, r3, r2 = core.shape
    if x.shape[-1] != d_in or U_in.shape != (d_in, r3) or inner_norm_w.shape != (r3,) or \
            U_expert.shape != (E, r1) or U_out.shape[0] != r2 or bias.shape != (U_out.shape[1],):
        raise RuntimeError("tmoe_b200: parameter shapes are inconsistent with TuckerMoE's layout")
    if not 0 < top_k <= E:
        raise RuntimeError(f"tmoe_b200: top_k={top_k} must be in 1..{E}")


def _run(x, router_w, U_in, inner_norm_w, eps, U_expert, core, U_out, bias, top_k, path,
         residual=None, layer_scale=None, want_taps=False, prepared=None, silu_gate=None, router=_DEFAULT_ROUTER,
         pre_norm_eps=None):
    params = (router_w, U_in, inner_norm_w, U_expert, core, U_out, bias)
    _validate(x, params, top_k)
    lib = _lib.load()
    d_in = x.shape[-1]
    d_out = U_out.shape[1]
    lead = x.shape[:-1]
    x2 = x.reshape(-1, d_in)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    T = x2.shape[0]
    dev = x.device
    y = torch.empty((T, d_out), dtype=x.dtype, device=dev)
    taps = None
    if T == 0:
        if want_taps:
            taps = (torch.empty((0, top_k), dtype=torch.int32, device=dev),
                    torch.empty((0, top_k), dtype=torch.float32, device=dev),
                    torch.empty((0, core.shape[0]), dtype=torch.float32, device=dev))
        return y.reshape(*lead, d_out), taps
    params = tuple(p if p.is_contiguous() else p.contiguous() for p in params)
    router_w, U_in, inner_norm_w, U_expert, core, U_out, bias = params
    layer = _layer_struct(x, router_w, U_in, U_expert, core, U_out, top_k, eps, router)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        rpath = _lib.check(lib.tmoe_resolve_path(C.byref(layer), T, path), "tmoe_resolve_path")
        factors = Factors(*[p.data_ptr() for p in params])
        prepared_ptr = None
        if rpath in (PATH_TENSOR, PATH_DECODE):
            if prepared is None:  # functional call without a cached set: prepare for this call
                prepared = prepare_factors(router_w, U_in, inner_norm_w, eps, U_expert, core, U_out, bias, top_k)
            prepared_ptr = prepared.data_ptr()
        ws_bytes = _lib.check(lib.tmoe_workspace_bytes(C.byref(layer), T, rpath), "tmoe_workspace_bytes")
        ws = _workspace(dev, ws_bytes)
        extras = Extras()
        keep = []
        if residual is not None:
            res2 = residual.reshape(-1, d_out).contiguous()
            ls = layer_scale.contiguous()
            if res2.shape[0] != T or res2.dtype != x.dtype or ls.dtype != x.dtype or ls.shape != (d_out,):
                raise RuntimeError("tmoe_b200: residual must be (..., d_out) and layer_scale (d_out,) in x's dtype")
            extras.residual, extras.layer_scale = res2.data_ptr(), ls.data_ptr()
            keep += [res2, ls]
        if silu_gate is not None:
            g2 = silu_gate.reshape(-1, d_out).contiguous()
            if g2.shape[0] != T or g2.dtype != x.dtype or g2.device != dev:
                raise RuntimeError("tmoe_b200: silu_gate must be (..., d_out) in x's dtype on x's device")
            extras.silu_gate = g2.data_ptr()
            keep.append(g2)
        if pre_norm_eps is not None:  # `prepared` carries the folded norm weight (prepare_factors(pre_norm_weight=...))
            extras.pre_norm, extras.pre_norm_eps = 1, float(pre_norm_eps)
        if want_taps:
            taps = (torch.empty((T, top_k), dtype=torch.int32, device=dev),
                    torch.empty((T, top_k), dtype=torch.float32, device=dev),
                    torch.empty((T, core.shape[0]), dtype=torch.float32, device=dev))
            extras.idx_out, extras.gates_out, extras.c_out = (t.data_ptr() for t in taps)
        _lib.check(lib.tmoe_forward(C.byref(layer), C.byref(factors), prepared_ptr, x2.data_ptr(), T, y.data_ptr(),
                                    C.byref(extras), ws.data_ptr(), ws.numel(), rpath, stream), "tmoe_forward")
    return y.reshape(*lead, d_out), taps


def read_device_status(device=None) -> Tuple[int, int, int, int]:
    """Synchronises the current stream and returns the four status words of its workspace
    (all zero unless a bounded wait inside a kernel expired)."""
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    with _cache_lock:
        ws = _workspaces.get(key)
    if ws is None:
        return (0, 0, 0, 0)
    out = (C.c_int32 * 4)()
    with torch.cuda.device(dev):
        _lib.check(lib.tmoe_read_device_status(ws.data_ptr(), out, key[1]), "tmoe_read_device_status")
    return tuple(int(v) for v in out)


# ------------------------------------------------------------------------------------------
# torch custom op
# ------------------------------------------------------------------------------------------
@torch.library.custom_op("tmoe_b200::forward", mutates_args=())
def _forward_op(x: torch.Tensor, router_w: torch.Tensor, U_in: torch.Tensor, inner_norm_w: torch.Tensor, eps: float,
                U_expert: torch.Tensor, core: torch.Tensor, U_out: torch.Tensor, bias: torch.Tensor, top_k: int,
                path: int, residual: Optional[torch.Tensor], layer_scale: Optional[torch.Tensor],
                prepared: Optional[torch.Tensor], silu_gate: Optional[torch.Tensor], router_mode: int,
                router_cap: float, router_temperature: float) -> torch.Tensor:
    y, _ = _run(x, router_w, U_in, inner_norm_w, eps, U_expert, core, U_out, bias, top_k, path, residual, layer_scale,
                prepared=prepared, silu_gate=silu_gate, router=(router_mode, router_cap, router_temperature))
    return y


@_forward_op.register_fake
def _(x, router_w, U_in, inner_norm_w, eps, U_expert, core, U_out, bias, top_k, path, residual, layer_scale, prepared,
      silu_gate, router_mode, router_cap, router_temperature):
    return x.new_empty((*x.shape[:-1], U_out.shape[1]))


@torch.library.custom_op("tmoe_b200::rms_norm", mutates_args=())
def _rms_norm_op(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    if not x.is_cuda or x.dtype not in _DTYPES:
        raise RuntimeError("tmoe_b200: rms_norm runs on float32 / bfloat16 CUDA tensors only (no CPU fallback)")
    if weight.dtype != x.dtype or weight.device != x.device or weight.shape != (x.shape[-1],):
        raise RuntimeError("tmoe_b200: rms_norm weight must be (d,) in x's dtype on x's device")
    lib = _lib.load()
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    w = weight if weight.is_contiguous() else weight.contiguous()
    y = torch.empty_like(x2)
    with torch.cuda.device(x.device):
        _lib.check(lib.tmoe_rms_norm(_DTYPES[x.dtype], x2.data_ptr(), w.data_ptr(), float(eps), x2.shape[0], d,
                                     y.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream), "tmoe_rms_norm")
    return y.reshape(x.shape)


@_rms_norm_op.register_fake
def _(x, weight, eps):
    return torch.empty_like(x)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps) * weight`` (the reference ``RMSNorm.forward``, ``model.py:25-27``)."""
    return torch.ops.tmoe_b200.rms_norm(x, weight, float(eps))


def tucker_moe_forward(x, router_w, U_in, inner_norm_w, eps, U_expert, core, U_out, bias, top_k, *, path=PATH_AUTO,
                       residual=None, layer_scale=None, prepared=None, silu_gate=None, router=_DEFAULT_ROUTER):
    """Functional form of the layer (parameter order of ``pure_torch_mlx/weights.py:74-81``).
    With ``residual``/``layer_scale`` it returns ``residual + layer_scale * layer(x)``
    (the callers' epilogue, ``model.py:260, 341``).  ``prepared`` is an optional result of
    ``prepare_factors`` for the same seven tensors; without it the tensor-core path re-lays the
    factors out on every call.  With ``silu_gate`` the result is ``silu(silu_gate) * layer(x)`` (the FFN's
    ``silu(gate) * up``, ``model.py:338-340``), applied before the residual epilogue.  ``router`` is
    ``(mode, cap, temperature)``: mode 0 is the pure-PyTorch rule (top-k of the raw scores, softmax over the
    winners), mode 1 the trained checkpoints' rule (``sft_cot_bundle/scripts/model.py:318-329``)."""
    if (residual is None) != (layer_scale is None):
        raise RuntimeError("tmoe_b200: residual and layer_scale go together")
    return torch.ops.tmoe_b200.forward(x, router_w, U_in, inner_norm_w, float(eps), U_expert, core, U_out, bias,
                                       int(top_k), int(path), residual, layer_scale, prepared, silu_gate, int(router[0]),
                                       float(router[1]), float(router[2]))


def tucker_moe_forward_taps(x, router_w, U_in, inner_norm_w, eps, U_expert, core, U_out, bias, top_k, *,
                            path=PATH_AUTO, prepared=None, router=_DEFAULT_ROUTER):
    """Forward that also returns the routing results (idx int32 [T,k], gates fp32 [T,k], c fp32 [T,r1])."""
    y, taps = _run(x, router_w, U_in, inner_norm_w, float(eps), U_expert, core, U_out, bias, int(top_k), int(path),
                   want_taps=True, prepared=prepared, router=router)
    return y, taps


class _Plan:
    """Everything about a (module, dtype, device, path) combination that does not change from call to call:
    validated contiguous parameters, the C structs, the prepared factor set and, per token count, the resolved
    kernel path and workspace size.  Rebuilt when a parameter's storage or version changes."""
    __slots__ = ("key", "params", "layer", "factors", "layer_ref", "factors_ref", "prepared", "prepared_ptr", "per_T",
                 "dev", "d_in", "d_out", "lib", "pn")


def _drop_caches_after_load(module, incompatible_keys) -> None:
    """load_state_dict post-hook: whatever was derived from the old parameter values is dropped."""
    module.invalidate_cache()


class TuckerMoE(nn.Module):
    """Low-rank Tucker-decomposed Mixture-of-Experts, B200 forward.

    Parameter shapes (identical to the reference, ``model.py:44-52``):
      router.weight (E, d_in)   U_in (d_in, r3)   inner_norm.weight (r3,)   U_expert (E, r1)
      core (r1, r3, r2)         U_out (r2, d_out)  bias (d_out,)
    """

    def __init__(self, d_in: int, d_out: int, cfg):
        super().__init__()
        E = cfg.kmoe_num_experts
        r1, r2, r3 = cfg.kmoe_r1, cfg.kmoe_r2, cfg.kmoe_r3
        self.top_k = cfg.kmoe_top_k
        self.router = nn.Linear(d_in, E, bias=False)
        self.U_in = nn.Parameter(torch.empty(d_in, r3))
        self.inner_norm = RMSNorm(r3, eps=cfg.rms_norm_eps)
        self.U_expert = nn.Parameter(torch.empty(E, r1))
        self.core = nn.Parameter(torch.empty(r1, r3, r2))
        self.U_out = nn.Parameter(torch.empty(r2, d_out))
        self.bias = nn.Parameter(torch.zeros(d_out))
        self.path = PATH_AUTO
        # gate rule: 0 = this module's reference (model.py:75-77); 1 = capped / tempered softmax over all experts,
        # the rule the trained checkpoints were produced with (sft_cot_bundle/scripts/model.py:318-329)
        self.router_mode = int(getattr(cfg, "kmoe_router_mode", 0))
        self.router_cap = float(getattr(cfg, "kmoe_router_cap", 10.0))
        self.router_temperature = float(getattr(cfg, "kmoe_router_temperature", 0.5))
        self._prep_key = None
        self._prep = None
        self._prep_pn_key = None
        self._prep_pn = None
        self._plan = None
        self.register_load_state_dict_post_hook(_drop_caches_after_load)

    def _prepared_for(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """Prepared factor set for the tensor-core path, rebuilt when a parameter's storage,
        version, dtype or device changes; None when this call will not use that path."""
        if not x.is_cuda or x.dtype != torch.bfloat16:
            return None
        if self.path == PATH_SIMT:
            return None
        ps = self._params()
        key = _param_key(ps)
        if key != self._prep_key or os.environ.get("TMOE_ALWAYS_PREPARE") == "1":
            self._prep = prepare_factors(ps[0], ps[1], ps[2], self.inner_norm.eps, ps[3], ps[4], ps[5], ps[6], self.top_k)
            self._prep_key = key
        return self._prep

    def _prenorm_path(self, x: torch.Tensor) -> int:
        """Kernel path on which a call with this x can apply the callers' pre-norm in-kernel (0: none): the decode
        path, or the tensor-core path with its in-kernel router (E <= 256, top_k <= 8, r3 <= 256)."""
        if not x.is_cuda or x.dtype != torch.bfloat16:
            return 0
        T = x.numel() // max(x.shape[-1], 1)
        if T == 0 or self.path == PATH_SIMT:
            return 0
        L = _layer_struct(x, self.router.weight, self.U_in, self.U_expert, self.core, self.U_out, self.top_k,
                          self.inner_norm.eps)
        rp = _lib.load().tmoe_resolve_path(C.byref(L), T, self.path)
        if rp == PATH_DECODE:
            return PATH_DECODE
        r1, r3, _ = self.core.shape
        E = self.router.weight.shape[0]
        if rp == PATH_TENSOR and r3 <= 256 and (E + 15) // 16 * 16 <= 256 and self.top_k <= 8:
            return PATH_TENSOR
        return 0

    def _prepared_prenorm_for(self, x: torch.Tensor, norm_weight: torch.Tensor) -> Optional[torch.Tensor]:
        """Prepared factors with `norm_weight` folded in when this call can run the pre-norm inside the kernels
        (``_prenorm_path``); else None."""
        if self._prenorm_path(x) == 0:
            return None
        ps = self._params()
        key = _param_key(ps) + _param_key((norm_weight,))
        if key != self._prep_pn_key:
            self._prep_pn = prepare_factors(ps[0], ps[1], ps[2], self.inner_norm.eps, ps[3], ps[4], ps[5], ps[6], self.top_k,
                                            pre_norm_weight=norm_weight)
            self._prep_pn_key = key
        return self._prep_pn

    def _params(self):
        return (self.router.weight, self.U_in, self.inner_norm.weight, self.U_expert, self.core, self.U_out, self.bias)

    def _router(self):
        return (self.router_mode, self.router_cap, self.router_temperature)

    def _plan_for(self, x: torch.Tensor) -> _Plan:
        ps = self._params()
        key = (x.dtype, x.device, self.path, self.top_k, self.inner_norm.eps) + self._router() + tuple((p.data_ptr(), p._version) for p in ps)
        plan = self._plan
        if plan is not None and plan.key == key:
            return plan
        _validate(x, ps, self.top_k)
        plan = _Plan()
        plan.key = key
        plan.lib = _lib.load()
        plan.params = tuple(p if p.is_contiguous() else p.contiguous() for p in ps)
        rw, ui, nw, ue, co, uo, b = plan.params
        plan.layer = _layer_struct(x, rw, ui, ue, co, uo, self.top_k, self.inner_norm.eps, self._router())
        plan.factors = Factors(*[p.data_ptr() for p in plan.params])
        plan.layer_ref, plan.factors_ref = C.byref(plan.layer), C.byref(plan.factors)
        plan.prepared = self._prepared_for(x)
        plan.prepared_ptr = plan.prepared.data_ptr() if plan.prepared is not None else None
        plan.per_T = {}
        plan.pn = {}
        plan.dev, plan.d_in, plan.d_out = x.device, ui.shape[0], uo.shape[1]
        self._plan = plan
        return plan

    def _fast_prenorm(self, plan: _Plan, x: torch.Tensor, w: torch.Tensor, T: int):
        """(prepared set with `w` folded in, kernel path) when a call of T tokens can apply the pre-norm in-kernel, else
        None; remembered per (norm weight, T) on the plan."""
        key = (w.data_ptr(), w._version, T)
        hit = plan.pn.get(key)
        if hit is None:
            prep = self._prepared_prenorm_for(x, w)
            hit = (prep, self._prenorm_path(x)) if prep is not None else (None, 0)
            if len(plan.pn) < 64:
                plan.pn[key] = hit
        return hit if hit[0] is not None else None

    def _fast_forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                      layer_scale: Optional[torch.Tensor] = None, silu_gate: Optional[torch.Tensor] = None,
                      pre_norm=None, out: Optional[torch.Tensor] = None, peer_ptrs=None) -> torch.Tensor:
        """Eager call without the dispatcher: the same C entry point as the custom op, with the per-call
        Python work cut to a cache lookup (decode-sized calls cost more in Python than on the GPU).
        The optional arguments are those of ``forward_fused`` (``pre_norm`` as a ``(weight, eps)`` pair);
        ``out`` is an optional contiguous (T, d_out) result buffer; ``peer_ptrs`` are device addresses of further
        (T, d_out) buffers that receive the same result (``tmoe_extras_t.n_peer_y``)."""
        plan = self._plan_for(x)
        if x.shape[-1] != plan.d_in:
            raise RuntimeError(f"tmoe_b200: x has {x.shape[-1]} features, the layer expects {plan.d_in}")
        x2 = x.reshape(-1, plan.d_in)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        if out is None:
            y = torch.empty((T, plan.d_out), dtype=x.dtype, device=x.device)
        else:
            if out.numel() != T * plan.d_out or out.dtype != x.dtype or out.device != x.device or not out.is_contiguous() \
                    or (out.data_ptr() & 15):
                raise RuntimeError("tmoe_b200: `out` must be a contiguous, 16-byte aligned (..., d_out) tensor of x's dtype on x's device")
            y = out
        if T:
            lib, dev = plan.lib, plan.dev
            prepared_ptr, force_path, ex_ref, keep = plan.prepared_ptr, None, None, None
            if residual is not None or silu_gate is not None or pre_norm is not None or peer_ptrs:
                ex = Extras()
                keep = []
                if peer_ptrs:
                    if len(peer_ptrs) > _lib.MAX_PEERS:
                        raise RuntimeError(f"tmoe_b200: at most {_lib.MAX_PEERS} further result buffers")
                    ex.n_peer_y = len(peer_ptrs)
                    for i, ptr in enumerate(peer_ptrs):
                        ex.peer_y[i] = ptr
                if pre_norm is not None:
                    w, e = pre_norm
                    pn = self._fast_prenorm(plan, x, w, T)
                    if pn is None:
                        x2 = rms_norm(x2, w, e)
                    else:
                        prepared_ptr, force_path = pn[0].data_ptr(), pn[1]
                        ex.pre_norm, ex.pre_norm_eps = 1, float(e)
                if residual is not None:
                    res2 = residual.reshape(-1, plan.d_out)
                    if not res2.is_contiguous():
                        res2 = res2.contiguous()
                    ls = layer_scale if layer_scale.is_contiguous() else layer_scale.contiguous()
                    if res2.shape[0] != T or res2.dtype != x.dtype or ls.dtype != x.dtype or ls.shape != (plan.d_out,) \
                            or res2.device != dev or ls.device != dev:
                        raise RuntimeError("tmoe_b200: residual must be (..., d_out) and layer_scale (d_out,) in x's dtype")
                    ex.residual, ex.layer_scale = res2.data_ptr(), ls.data_ptr()
                    keep += [res2, ls]
                if silu_gate is not None:
                    g2 = silu_gate.reshape(-1, plan.d_out)
                    if not g2.is_contiguous():
                        g2 = g2.contiguous()
                    if g2.shape[0] != T or g2.dtype != x.dtype or g2.device != dev:
                        raise RuntimeError("tmoe_b200: silu_gate must be (..., d_out) in x's dtype on x's device")
                    ex.silu_gate = g2.data_ptr()
                    keep.append(g2)
                ex_ref = C.byref(ex)
            info = plan.per_T.get((T, force_path))
            if info is None:
                rpath = _lib.check(lib.tmoe_resolve_path(plan.layer_ref, T, self.path if force_path is None else force_path),
                                   "tmoe_resolve_path")
                info = (rpath, _lib.check(lib.tmoe_workspace_bytes(plan.layer_ref, T, rpath), "tmoe_workspace_bytes"))
                if len(plan.per_T) < 4096:
                    plan.per_T[(T, force_path)] = info
            rpath, ws_bytes = info
            if torch.cuda.current_device() == dev.index:
                stream = torch.cuda.current_stream().cuda_stream
                ws = _workspace(dev, ws_bytes, stream)
                rc = lib.tmoe_forward(plan.layer_ref, plan.factors_ref, prepared_ptr, x2.data_ptr(), T, y.data_ptr(),
                                      ex_ref, ws.data_ptr(), ws.numel(), rpath, stream)
            else:
                with torch.cuda.device(dev):
                    stream = torch.cuda.current_stream(dev).cuda_stream
                    ws = _workspace(dev, ws_bytes, stream)
                    rc = lib.tmoe_forward(plan.layer_ref, plan.factors_ref, prepared_ptr, x2.data_ptr(), T,
                                          y.data_ptr(), ex_ref, ws.data_ptr(), ws.numel(), rpath, stream)
            if rc < 0:
                _lib.check(rc, "tmoe_forward")
        return y.reshape(*x.shape[:-1], plan.d_out)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x: (..., d_in) -> (..., d_out)"""
        if x.is_cuda and not torch.compiler.is_compiling():
            return self._fast_forward(x)
        rw, ui, nw, ue, co, uo, b = self._params()
        return tucker_moe_forward(x, rw, ui, nw, self.inner_norm.eps, ue, co, uo, b, self.top_k, path=self.path,
                                  prepared=self._prepared_for(x), router=self._router())

    def forward_into(self, x: torch.Tensor, out: torch.Tensor, peer_ptrs=None) -> torch.Tensor:
        """``forward`` with the result written into ``out`` (contiguous, (..., d_out), x's dtype and device): lets a
        caller place the output where the next step wants it, e.g. in its slot of an all-gather buffer.  ``peer_ptrs``:
        device addresses of up to 7 more buffers of out's shape (e.g. the same slot in other GPUs' mapped buffers) that
        the out-projection writes tile by tile as well; raises ``TmoeError`` with status ``ERR_UNSUPPORTED`` before
        anything is enqueued when the call does not take the tensor-core path."""
        if not x.is_cuda:
            raise RuntimeError("tmoe_b200: the layer forward runs on CUDA tensors only (no CPU fallback)")
        self._fast_forward(x, out=out, peer_ptrs=peer_ptrs)
        return out

    def forward_fused(self, x: torch.Tensor, *, pre_norm=None, residual: Optional[torch.Tensor] = None,
                      layer_scale: Optional[torch.Tensor] = None, silu_gate: Optional[torch.Tensor] = None,
                      return_routing: bool = False):
        """The layer with the callers' element-wise work attached:

        ``pre_norm``  an RMSNorm module (anything with ``.weight`` and ``.eps``) or a ``(weight, eps)`` pair
                      applied to ``x`` first (``norm_out_proj`` / ``norm_ffn``, ``model.py:258, 337``);
        ``silu_gate`` ``silu(silu_gate) * layer(...)`` in the out-projection's epilogue (``model.py:340``);
        ``residual``, ``layer_scale``  ``residual + layer_scale * (...)`` in the same epilogue (``model.py:260, 341``).
        ``return_routing``  also return ``(idx, gates, c)`` of the call (same kernels, same output).
        """
        if pre_norm is not None and hasattr(pre_norm, "weight"):
            pre_norm = (pre_norm.weight, pre_norm.eps)
        if (residual is None) != (layer_scale is None):
            raise RuntimeError("tmoe_b200: residual and layer_scale go together")
        if return_routing:
            rw, ui, nw, ue, co, uo, b = self._params()
            path, prep, pn_eps = self.path, None, None
            if pre_norm is not None:
                w, e = pre_norm
                prep = self._prepared_prenorm_for(x, w)
                if prep is not None:
                    path, pn_eps = self._prenorm_path(x), float(e)
                else:
                    x = rms_norm(x, w, e)
            if prep is None:
                prep = self._prepared_for(x)
            return _run(x, rw, ui, nw, self.inner_norm.eps, ue, co, uo, b, self.top_k, path, residual, layer_scale,
                        want_taps=True, prepared=prep, silu_gate=silu_gate, router=self._router(), pre_norm_eps=pn_eps)
        if x.is_cuda and not torch.compiler.is_compiling():
            return self._fast_forward(x, residual, layer_scale, silu_gate, pre_norm)
        rw, ui, nw, ue, co, uo, b = self._params()
        if pre_norm is not None:
            w, e = pre_norm
            prep_pn = self._prepared_prenorm_for(x, w)
            if prep_pn is not None:
                # norm weight folded into the prepared factors, 1/rms(x) found inside the in-projection kernel
                T_ = x.numel() // max(x.shape[-1], 1)
                y, _ = _run(x, rw, ui, nw, self.inner_norm.eps, ue, co, uo, b, self.top_k, self._prenorm_path(x), residual,
                            layer_scale, prepared=prep_pn, silu_gate=silu_gate, router=self._router(),
                            pre_norm_eps=float(e))
                return y
            x = rms_norm(x, w, e)
        return tucker_moe_forward(x, rw, ui, nw, self.inner_norm.eps, ue, co, uo, b, self.top_k, path=self.path,
                                  residual=residual, layer_scale=layer_scale, silu_gate=silu_gate,
                                  prepared=self._prepared_for(x), router=self._router())

    def forward_fused_residual(self, x: torch.Tensor, residual: torch.Tensor, layer_scale: torch.Tensor) -> torch.Tensor:
        """``residual + layer_scale * self(x)`` with the epilogue fused into the out-projection
        (what the callers compute at ``model.py:259-260`` and ``model.py:340-341``)."""
        rw, ui, nw, ue, co, uo, b = self._params()
        return tucker_moe_forward(x, rw, ui, nw, self.inner_norm.eps, ue, co, uo, b, self.top_k, path=self.path,
                                  residual=residual, layer_scale=layer_scale, prepared=self._prepared_for(x),
                                  router=self._router())

    def forward_with_routing(self, x: torch.Tensor):
        rw, ui, nw, ue, co, uo, b = self._params()
        return tucker_moe_forward_taps(x, rw, ui, nw, self.inner_norm.eps, ue, co, uo, b, self.top_k, path=self.path,
                                       prepared=self._prepared_for(x), router=self._router())

    @torch.no_grad()
    def forward_host(self, x_host: torch.Tensor, out: Optional[torch.Tensor] = None,
                     chunk_tokens: int = 4096, pipelined: bool = False) -> torch.Tensor:
        """Forward for activations that live in host memory: ``x_host`` (..., d_in) on the CPU (pinned
        memory for full copy speed) -> CPU tensor (..., d_out).

        The token range is cut into chunks; the host->device copy of chunk i+1, the kernels of chunk i
        and the device->host copy of chunk i-1 run on three streams, so one call costs about the longer
        of the two PCIe transfers instead of their sum plus the compute.  The result is complete when
        the current stream has caught up (``torch.cuda.current_stream().synchronize()``).

        ``pipelined=True`` is for a loop of calls: the host->device copies no longer wait for the work already
        queued on the current stream (which includes the previous call's device->host copies), so the input
        copy of one call overlaps the output copy of the one before and a step costs about one PCIe direction.
        The caller then guarantees that ``x_host`` is ready on the host when the call is made (it was not
        filled by a copy still in flight on the current stream) and passes a different ``out`` if the previous
        result has not been consumed yet."""
        dev = self.U_in.device
        if dev.type != "cuda":
            raise RuntimeError("tmoe_b200: move the layer to a CUDA device first (no CPU fallback)")
        d_in, d_out = self.U_in.shape[0], self.U_out.shape[1]
        lead = x_host.shape[:-1]
        xh = x_host.reshape(-1, d_in)
        T = xh.shape[0]
        if out is None:
            out = torch.empty((T, d_out), dtype=xh.dtype, pin_memory=True)
        oh = out.reshape(-1, d_out)
        if oh.shape[0] != T or oh.dtype != xh.dtype or oh.device.type != "cpu":
            raise RuntimeError("tmoe_b200: `out` must be a CPU tensor (..., d_out) of x's dtype")
        if T == 0:
            return out.reshape(*lead, d_out)
        with torch.cuda.device(dev):
            cur = torch.cuda.current_stream(dev)
            st = getattr(self, "_host_state", None)
            if st is None or st["dev"] != dev:
                # two device input buffers used in turn (the copy of one call may run under the kernels of the one
                # before), each with the event after which its last readers are done
                st = {"dev": dev, "streams": (torch.cuda.Stream(dev), torch.cuda.Stream(dev)), "buf": [None, None],
                      "free": [None, None], "n": 0}
                self._host_state = st
            h2d, d2h = st["streams"]
            b = st["n"] & 1
            st["n"] += 1
            xb = st["buf"][b]
            if xb is None or xb.dtype != xh.dtype or xb.numel() < T * d_in:
                if xb is not None:
                    xb.record_stream(h2d)
                xb = torch.empty(T * d_in, dtype=xh.dtype, device=dev)
                st["buf"][b] = xb
                st["free"][b] = None
                h2d.wait_stream(cur)          # a fresh block from the caching allocator is ordered on the current stream
            elif not pipelined:
                h2d.wait_stream(cur)
            if st["free"][b] is not None:
                h2d.wait_event(st["free"][b])  # the kernels of the call that last read this buffer
            d2h.wait_stream(cur)
            x_dev = xb[: T * d_in].view(T, d_in)
            step = max(1, int(chunk_tokens))
            copied = []
            for lo in range(0, T, step):
                hi = min(T, lo + step)
                with torch.cuda.stream(h2d):
                    x_dev[lo:hi].copy_(xh[lo:hi], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(h2d)
                copied.append((lo, hi, ev))
            for lo, hi, ev in copied:
                cur.wait_event(ev)
                y = self.forward(x_dev[lo:hi])
                done = torch.cuda.Event()
                done.record(cur)
                with torch.cuda.stream(d2h):
                    d2h.wait_event(done)
                    oh[lo:hi].copy_(y, non_blocking=True)
                y.record_stream(d2h)
            st["free"][b] = done
            cur.wait_stream(d2h)
        return out.reshape(*lead, d_out)

    def invalidate_cache(self) -> None:
        """Call after writing parameters through ``.data`` once the layer has already run
        (such writes do not change tensor versions, which key the prepared-factor cache)."""
        self._prep_key, self._prep, self._plan = None, None, None
        self._prep_pn_key, self._prep_pn = None, None

    def __getstate__(self):
        """Copies and pickles carry the parameters, not what was derived from them (C structs, prepared buffers)."""
        state = self.__dict__.copy()
        for k in ("_plan", "_prep", "_prep_key", "_prep_pn", "_prep_pn_key"):
            if k in state:
                state[k] = None
        return state


def fused_out_proj(out_proj: TuckerMoE, mid: torch.Tensor, norm, layer_scale: torch.Tensor) -> torch.Tensor:
    """``mid + gamma * out_proj(norm(mid))`` -- the tail of the reference's Mamba block (``model.py:258-260``)
    as one normalisation kernel and one layer call whose epilogue adds the scaled result to ``mid``."""
    return out_proj.forward_fused(mid, pre_norm=norm, residual=mid, layer_scale=layer_scale)


def _gate_up_one_launch(ffn_gate: TuckerMoE, ffn_up: TuckerMoE, x: torch.Tensor, norm_w: torch.Tensor, norm_eps: float):
    """``silu(ffn_gate(norm(x))) * ffn_up(norm(x))`` through ``tmoe_ffn_gate_up`` (the two layers' in-projection / core
    stages in one launch, ``model.py:337-340``), or None when that entry point does not cover the call: other kernel
    paths (few tokens, fp32), different layer sizes, a router the tensor-core kernel does not run in-kernel."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or torch.compiler.is_compiling():
        return None
    T = x.numel() // max(x.shape[-1], 1)
    if T == 0 or ffn_gate.path not in (PATH_AUTO, PATH_TENSOR) or ffn_up.path != ffn_gate.path:
        return None
    shapes = [tuple(p.shape) for p in ffn_gate._params()]
    if shapes != [tuple(p.shape) for p in ffn_up._params()] or ffn_gate.top_k != ffn_up.top_k \
            or ffn_gate.inner_norm.eps != ffn_up.inner_norm.eps or ffn_gate._router() != ffn_up._router():
        return None
    if ffn_gate._prenorm_path(x) != PATH_TENSOR or ffn_up._prenorm_path(x) != PATH_TENSOR:
        return None
    pg, pu = ffn_gate._prepared_prenorm_for(x, norm_w), ffn_up._prepared_prenorm_for(x, norm_w)
    if pg is None or pu is None:
        return None
    lib = _lib.load()
    rw, ui, nw, ue, co, uo, b = ffn_gate._params()
    layer = _layer_struct(x, rw, ui, ue, co, uo, ffn_gate.top_k, ffn_gate.inner_norm.eps, ffn_gate._router())
    d_in, d_out = ui.shape[0], uo.shape[1]
    x2 = x.reshape(-1, d_in)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    dev = x.device
    with torch.cuda.device(dev):
        ws_one = _lib.check(lib.tmoe_workspace_bytes(C.byref(layer), T, PATH_TENSOR), "tmoe_workspace_bytes")
        ws = _workspace(dev, 2 * ((ws_one + 255) // 256 * 256))
        gate = torch.empty((T, d_out), dtype=x.dtype, device=dev)
        act = torch.empty((T, d_out), dtype=x.dtype, device=dev)
        ex = Extras()
        ex.pre_norm, ex.pre_norm_eps = 1, float(norm_eps)
        rc = lib.tmoe_ffn_gate_up(C.byref(layer), pg.data_ptr(), pu.data_ptr(), x2.data_ptr(), T, gate.data_ptr(),
                                  act.data_ptr(), C.byref(ex), ws.data_ptr(), ws.numel(),
                                  torch.cuda.current_stream(dev).cuda_stream)
    if rc == -6:     # TMOE_ERR_UNSUPPORTED: the caller composes the two layers itself
        return None
    _lib.check(rc, "tmoe_ffn_gate_up")
    return act.reshape(*x.shape[:-1], d_out)


def fused_ffn(ffn_gate: TuckerMoE, ffn_up: TuckerMoE, ffn_down: TuckerMoE, x_res: torch.Tensor, norm,
              layer_scale: torch.Tensor) -> torch.Tensor:
    """``x_res + gamma * ffn_down(silu(ffn_gate(x_f)) * ffn_up(x_f))`` with ``x_f = norm(x_res)`` -- the FFN of the
    reference's transformer block (``model.py:337-341``).  The norm runs inside the gate and up layers' in-projection kernels where those
    support it (else ``x_f`` is computed once and shared); on the tensor-core path the two layers' in-projection / core stages are one
    launch that reads each tile of ``x_res`` from HBM once, ``silu(gate) * up`` is the epilogue of the up layer and the residual add is the epilogue of the down
    layer, so no element-wise pass over the 6x-wide activations remains."""
    w, e = (norm.weight, norm.eps) if hasattr(norm, "weight") else norm
    act = _gate_up_one_launch(ffn_gate, ffn_up, x_res, w, e)
    if act is not None:
        return ffn_down.forward_fused(act, residual=x_res, layer_scale=layer_scale)
    if ffn_gate._prepared_prenorm_for(x_res, w) is not None and ffn_up._prepared_prenorm_for(x_res, w) is not None:
        # both layers apply the norm inside their in-projection kernels: no separate pass over x_res
        gate = ffn_gate.forward_fused(x_res, pre_norm=(w, e))
        act = ffn_up.forward_fused(x_res, pre_norm=(w, e), silu_gate=gate)
    else:
        x_f = rms_norm(x_res, w, e)
        gate = ffn_gate(x_f)
        act = ffn_up.forward_fused(x_f, silu_gate=gate)
    return ffn_down.forward_fused(act, residual=x_res, layer_scale=layer_scale)
