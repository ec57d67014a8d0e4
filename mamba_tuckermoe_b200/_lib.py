"""ctypes binding of ``lib/libtmoe_b200.so`` (the C ABI declared in ``include/tmoe_b200.h``)."""
from __future__ import annotations

import ctypes as C
import os
import threading

PKG = os.path.dirname(os.path.abspath(__file__))
# TMOE_LIB_PATH lets a developer point the binding at another build of the same ABI (A/B timing of kernels)
LIB_PATH = os.environ.get("TMOE_LIB_PATH") or os.path.join(PKG, "lib", "libtmoe_b200.so")

TMOE_F32, TMOE_BF16 = 0, 1
PATH_AUTO, PATH_SIMT, PATH_TENSOR, PATH_DECODE = 0, 1, 2, 3
ROUTER_TOPK_SOFTMAX, ROUTER_CAPPED_SOFTMAX = 0, 1
ABI_VERSION = 2   # TMOE_ABI_VERSION of the header this binding mirrors
ERR_UNSUPPORTED = -6
ERR_DEVICE_WAIT = -9
MAX_PEERS = 7

# every symbol the header declares; checked when the library is loaded
EXPORTS = (
    "tmoe_version", "tmoe_status_string", "tmoe_resolve_path", "tmoe_prepared_bytes",
    "tmoe_prepare_factors", "tmoe_workspace_bytes", "tmoe_router", "tmoe_in_core", "tmoe_out",
    "tmoe_forward", "tmoe_read_device_status", "tmoe_launch_count", "tmoe_forward_static_scratch", "tmoe_rms_norm", "tmoe_handoff_plan",
    "tmoe_prepare_factors_prenorm", "tmoe_selftest_bounded_wait", "tmoe_ffn_gate_up",
    "tmoe_peer_alloc", "tmoe_peer_open", "tmoe_peer_close", "tmoe_peer_free", "tmoe_peer_push",
)
PEER_HANDLE_BYTES = 64
STATIC_SCRATCH_BYTES = 4 << 20


class Layer(C.Structure):
    _fields_ = [("d_in", C.c_int32), ("d_out", C.c_int32), ("n_experts", C.c_int32), ("top_k", C.c_int32),
                ("r1", C.c_int32), ("r2", C.c_int32), ("r3", C.c_int32), ("dtype", C.c_int32),
                ("eps", C.c_float), ("router_mode", C.c_int32), ("router_cap", C.c_float),
                ("router_temperature", C.c_float)]


class Factors(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("router_w", "U_in", "inner_norm_w", "U_expert", "core", "U_out", "bias")]


class Extras(C.Structure):
    _fields_ = [("residual", C.c_void_p), ("layer_scale", C.c_void_p), ("idx_out", C.c_void_p),
                ("gates_out", C.c_void_p), ("c_out", C.c_void_p), ("silu_gate", C.c_void_p),
                ("pre_norm", C.c_int32), ("pre_norm_eps", C.c_float),
                ("n_peer_y", C.c_int32), ("reserved0", C.c_int32), ("peer_y", C.c_void_p * 7)]


class TmoeError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {status_string(status)} (status {status})")


_lock = threading.Lock()
_lib = None


def load():
    """Loads the library once.  Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m mamba_tuckermoe_b200.build` "
                "(there is no CPU or PyTorch fallback for the layer forward)")
        lib = C.CDLL(LIB_PATH)
        missing = [s for s in EXPORTS if not hasattr(lib, s)]
        if missing:
            raise RuntimeError(f"{LIB_PATH} does not export {missing}")
        vp, i32, i64 = C.c_void_p, C.c_int, C.c_int64
        LP, FP, EP = C.POINTER(Layer), C.POINTER(Factors), C.POINTER(Extras)
        lib.tmoe_version.restype = i32
        lib.tmoe_status_string.restype = C.c_char_p
        lib.tmoe_status_string.argtypes = [i32]
        lib.tmoe_resolve_path.restype = i32
        lib.tmoe_resolve_path.argtypes = [LP, i64, i32]
        lib.tmoe_prepared_bytes.restype = i64
        lib.tmoe_prepared_bytes.argtypes = [LP]
        lib.tmoe_prepare_factors.restype = i32
        lib.tmoe_prepare_factors.argtypes = [LP, FP, vp, i64, vp]
        lib.tmoe_prepare_factors_prenorm.restype = i32
        lib.tmoe_prepare_factors_prenorm.argtypes = [LP, FP, vp, vp, i64, vp]
        lib.tmoe_workspace_bytes.restype = i64
        lib.tmoe_workspace_bytes.argtypes = [LP, i64, i32]
        lib.tmoe_router.restype = i32
        lib.tmoe_router.argtypes = [LP, FP, vp, i64, vp, vp, vp, vp, i64, vp]
        lib.tmoe_in_core.restype = i32
        lib.tmoe_in_core.argtypes = [LP, FP, vp, vp, i64, vp, vp, vp, i64, i32, vp]
        lib.tmoe_out.restype = i32
        lib.tmoe_out.argtypes = [LP, FP, vp, vp, i64, vp, EP, vp, i64, i32, vp]
        lib.tmoe_forward.restype = i32
        lib.tmoe_forward.argtypes = [LP, FP, vp, vp, i64, vp, EP, vp, i64, i32, vp]
        lib.tmoe_ffn_gate_up.restype = i32
        lib.tmoe_ffn_gate_up.argtypes = [LP, vp, vp, vp, i64, vp, vp, EP, vp, i64, vp]
        lib.tmoe_forward_static_scratch.restype = i32
        lib.tmoe_forward_static_scratch.argtypes = [LP, FP, vp, i64, vp, EP, vp]
        lib.tmoe_rms_norm.restype = i32
        lib.tmoe_rms_norm.argtypes = [i32, vp, vp, C.c_float, i64, C.c_int32, vp, vp]
        lib.tmoe_read_device_status.restype = i32
        lib.tmoe_read_device_status.argtypes = [vp, C.POINTER(C.c_int32), vp]
        lib.tmoe_launch_count.restype = i64
        lib.tmoe_selftest_bounded_wait.restype = i32
        lib.tmoe_selftest_bounded_wait.argtypes = [vp, i64, vp]
        lib.tmoe_handoff_plan.restype = i32
        lib.tmoe_handoff_plan.argtypes = [LP, i64, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
        VPP, HP = C.POINTER(vp), C.POINTER(C.c_ubyte)
        lib.tmoe_peer_alloc.restype = i32
        lib.tmoe_peer_alloc.argtypes = [i64, VPP, HP]
        lib.tmoe_peer_open.restype = i32
        lib.tmoe_peer_open.argtypes = [HP, VPP]
        lib.tmoe_peer_close.restype = i32
        lib.tmoe_peer_close.argtypes = [vp]
        lib.tmoe_peer_free.restype = i32
        lib.tmoe_peer_free.argtypes = [vp]
        lib.tmoe_peer_push.restype = i32
        lib.tmoe_peer_push.argtypes = [VPP, C.c_int32, vp, i64, VPP]
        if lib.tmoe_version() != ABI_VERSION:
            raise RuntimeError("libtmoe_b200.so has an ABI version this binding does not know")
        _lib = lib
    return _lib


def status_string(status: int) -> str:
    return load().tmoe_status_string(int(status)).decode()


def check(status: int, where: str) -> int:
    if status < 0:
        raise TmoeError(int(status), where)
    return int(status)


# ---------------------------------------------------------------------------------------
# small conveniences for callers that drive the stage entry points directly
# ---------------------------------------------------------------------------------------
FACTOR_ORDER = ("router_w", "U_in", "inner_norm_w", "U_expert", "core", "U_out", "bias")


def layer_struct(shape, dtype, router_mode: int = 0, router_cap: float = 10.0, router_temperature: float = 0.5) -> Layer:
    """``shape`` has d_in, d_out, E, top_k, r1, r2, r3, eps; ``dtype`` is a torch dtype."""
    import torch
    return Layer(shape.d_in, shape.d_out, shape.E, shape.top_k, shape.r1, shape.r2, shape.r3,
                 TMOE_BF16 if dtype == torch.bfloat16 else TMOE_F32, shape.eps, router_mode, router_cap,
                 router_temperature)


def factors_struct(dev_factors) -> Factors:
    """``dev_factors``: mapping of FACTOR_ORDER names to contiguous device tensors."""
    return Factors(*[dev_factors[k].data_ptr() for k in FACTOR_ORDER])


def current_stream_ptr():
    import torch
    return torch.cuda.current_stream().cuda_stream


def alloc_workspace(layer: Layer, T: int, path: int):
    import torch
    n = check(load().tmoe_workspace_bytes(C.byref(layer), T, path), "tmoe_workspace_bytes")
    return torch.zeros(max(n, 256), dtype=torch.uint8, device="cuda")


def alloc_prepared(layer: Layer, factors: Factors):
    import torch
    lib = load()
    n = check(lib.tmoe_prepared_bytes(C.byref(layer)), "tmoe_prepared_bytes")
    buf = torch.zeros(max(n, 256), dtype=torch.uint8, device="cuda")
    check(lib.tmoe_prepare_factors(C.byref(layer), C.byref(factors), buf.data_ptr(), buf.numel(),
                                   current_stream_ptr()), "tmoe_prepare_factors")
    return buf
