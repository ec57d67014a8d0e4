"""The three C-ABI stages (router, in-projection + core, out-projection) one by one against the
float64 oracle taps, on both paths."""
import ctypes as C

import pytest
import torch

from gpu_util import alloc_prepared, alloc_workspace, cuda_stream_ptr, factors_struct, layer_struct
from mamba_tuckermoe_b200 import _lib
from oracle.tucker_moe_oracle import LayerShape, classify_topk, layer_forward_f64, make_factors, make_tokens, max_abs, rel_fro

pytestmark = pytest.mark.gpu

CASES = [
    (LayerShape(64, 96, 8, 2, 4, 32, 64, 1e-5), 37, torch.float32),
    (LayerShape(256, 384, 64, 8, 8, 64, 128, 1e-6), 300, torch.float32),     # tiled scores + select kernel
    (LayerShape(256, 384, 1024, 16, 3, 64, 128, 1e-6), 290, torch.float32),  # top-16 of 1024, odd r1
    (LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6), 8, torch.bfloat16),
    (LayerShape(1536, 2304, 64, 2, 4, 256, 1024, 1e-6), 257, torch.bfloat16),
    # bf16 with >= 512 tokens: the scores come from the tensor cores (router_w is the K-major operand as stored); top-k > 8
    # through the GEMM kernel + the keyed select kernel
    (LayerShape(1536, 2304, 64, 2, 4, 256, 1024, 1e-6), 2100, torch.bfloat16),
    (LayerShape(256, 384, 1024, 16, 4, 64, 128, 1e-6), 600, torch.bfloat16),   # top-16 of 1024
    (LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6), 777, torch.bfloat16),   # E = 8: a 128-column tile, 8 of them used
    # the persistent tensor-core router: one expert chunk (E <= 256) and several (E <= 1024, top-k list carried across)
    (LayerShape(512, 384, 256, 8, 8, 64, 128, 1e-6), 40000, torch.bfloat16),   # more tiles than SMs: every CTA walks on
    (LayerShape(512, 384, 1024, 8, 4, 64, 128, 1e-6), 1000, torch.bfloat16),   # four chunks of 256 experts
    (LayerShape(512, 384, 328, 2, 32, 64, 128, 1e-6), 700, torch.bfloat16),    # two chunks, the second mostly padding
    (LayerShape(512, 384, 104, 8, 16, 64, 128, 1e-6), 513, torch.bfloat16),    # 104 experts padded to 112 columns
]


def _setup(shape, T, dtype, seed=31):
    f = make_factors(shape, seed, dtype, None if shape.E >= 64 else 0.02, 0.1)
    x = make_tokens(T, shape.d_in, seed, dtype)
    fd = {k: v.cuda() for k, v in f.items()}
    return x, f, fd


@pytest.mark.parametrize("shape,T,dtype", CASES)
def test_router_stage(shape, T, dtype):
    lib = _lib.load()
    x, f, fd = _setup(shape, T, dtype)
    L, F = layer_struct(shape, dtype), factors_struct(fd)
    ws = alloc_workspace(lib, L, T, 1)
    idx = torch.empty(T, shape.top_k, dtype=torch.int32, device="cuda")
    gates = torch.empty(T, shape.top_k, dtype=torch.float32, device="cuda")
    c = torch.empty(T, shape.r1, dtype=torch.float32, device="cuda")
    xd = x.cuda()
    rc = lib.tmoe_router(C.byref(L), C.byref(F), xd.data_ptr(), T, idx.data_ptr(), gates.data_ptr(), c.data_ptr(),
                         ws.data_ptr(), ws.numel(), cuda_stream_ptr())
    assert rc == 0, _lib.status_string(rc)
    torch.cuda.synchronize()
    rnd = None if dtype == torch.float32 else torch.bfloat16
    _, taps = layer_forward_f64(x, f, shape.top_k, shape.eps, round_scores_to=rnd)
    gap = 1e-6 if dtype == torch.float32 else 2.0 ** -5
    rep = classify_topk(idx.cpu(), taps["idx"], taps["scores"], gap)
    assert rep.unexplained == 0
    # with this run's own selection, gates and c agree with float64
    _, own = layer_forward_f64(x, f, shape.top_k, shape.eps, idx=idx.cpu(), round_scores_to=rnd)
    tol = 2e-6 if dtype == torch.float32 else 4e-3
    assert max_abs(gates.cpu(), own["gates"]) < tol
    assert max_abs(c.cpu(), own["c"]) < tol * 8
    # descending order of the selected scores (in bf16 the kernel sorts by ITS rounding of a score, which may sit one ulp
    # from the float64 statement's rounding: neighbours may then appear swapped by at most that ulp), indices distinct
    s_sel = torch.gather(own["scores"], 1, idx.cpu().long())
    slack = 0.0 if dtype == torch.float32 else 2.0 ** -7
    assert bool((s_sel[:, :-1] >= s_sel[:, 1:] - slack * s_sel[:, 1:].abs()).all())
    srt = torch.sort(idx.cpu(), dim=1).values
    assert bool((srt[:, 1:] != srt[:, :-1]).all())


@pytest.mark.parametrize("shape,T,dtype", CASES)
@pytest.mark.parametrize("path", [1, 2])
def test_in_core_and_out_stages(shape, T, dtype, path):
    lib = _lib.load()
    L = layer_struct(shape, dtype)
    if path == 2 and lib.tmoe_resolve_path(C.byref(L), T, 2) < 0:
        pytest.skip("shape not covered by the tensor-core path")
    x, f, fd = _setup(shape, T, dtype)
    F = factors_struct(fd)
    ws = alloc_workspace(lib, L, T, path)
    prep = alloc_prepared(lib, L, F) if path == 2 else None
    prep_ptr = prep.data_ptr() if prep is not None else None
    rnd = None if dtype == torch.float32 else torch.bfloat16
    y64, taps = layer_forward_f64(x, f, shape.top_k, shape.eps, round_scores_to=rnd)
    c = taps["c"].float().cuda().contiguous()
    zdtype = torch.float32 if path == 1 else torch.bfloat16
    z = torch.empty(T, shape.r2, dtype=zdtype, device="cuda")
    xd = x.cuda()
    rc = lib.tmoe_in_core(C.byref(L), C.byref(F), prep_ptr, xd.data_ptr(), T, c.data_ptr(), z.data_ptr(),
                          ws.data_ptr(), ws.numel(), path, cuda_stream_ptr())
    assert rc == 0, _lib.status_string(rc)
    torch.cuda.synchronize()
    st = (C.c_int32 * 4)()
    assert lib.tmoe_read_device_status(ws.data_ptr(), st, cuda_stream_ptr()) == 0 and list(st) == [0, 0, 0, 0]
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert rel_fro(z.float().cpu(), taps["z"]) < tol
    # out stage on the oracle's z
    z_in = taps["z"].to(zdtype).cuda().contiguous()
    y = torch.empty(T, shape.d_out, dtype=dtype, device="cuda")
    rc = lib.tmoe_out(C.byref(L), C.byref(F), prep_ptr, z_in.data_ptr(), T, y.data_ptr(), None, ws.data_ptr(),
                      ws.numel(), path, cuda_stream_ptr())
    assert rc == 0, _lib.status_string(rc)
    torch.cuda.synchronize()
    assert lib.tmoe_read_device_status(ws.data_ptr(), st, cuda_stream_ptr()) == 0 and list(st) == [0, 0, 0, 0]
    assert rel_fro(y.float().cpu(), y64) < (1e-5 if dtype == torch.float32 else 1e-2)


def test_bounded_wait_reports_and_returns():
    """A wait that can never be satisfied gives up by itself after its limit, records where it gave up in the status
    words and leaves the context usable; tmoe_read_device_status returns the words and clears them."""
    lib = _lib.load()
    shape = LayerShape(64, 96, 8, 2, 4, 32, 64, 1e-5)
    L = layer_struct(shape, torch.float32)
    ws = alloc_workspace(lib, L, 16, 1)
    st = (C.c_int32 * 4)()
    assert lib.tmoe_read_device_status(ws.data_ptr(), st, cuda_stream_ptr()) == 0 and list(st) == [0, 0, 0, 0]
    assert lib.tmoe_selftest_bounded_wait(ws.data_ptr(), 2_000_000, cuda_stream_ptr()) == 0    # ~1 ms
    assert lib.tmoe_read_device_status(ws.data_ptr(), st, cuda_stream_ptr()) == 0
    assert list(st) == [_lib.ERR_DEVICE_WAIT, 9, 42, 0]
    assert "bounded wait" in _lib.status_string(st[0])
    assert lib.tmoe_read_device_status(ws.data_ptr(), st, cuda_stream_ptr()) == 0 and list(st) == [0, 0, 0, 0]
    # the context is healthy: an ordinary forward on the same workspace still works
    x, f, fd = _setup(shape, 16, torch.float32)
    F = factors_struct(fd)
    y = torch.empty(16, shape.d_out, device="cuda")
    xd = x.cuda()
    assert lib.tmoe_forward(C.byref(L), C.byref(F), None, xd.data_ptr(), 16, y.data_ptr(), None, ws.data_ptr(), ws.numel(),
                            1, cuda_stream_ptr()) == 0
    torch.cuda.synchronize()
    y64, _ = layer_forward_f64(x, f, shape.top_k, shape.eps)
    assert rel_fro(y.cpu(), y64) < 1e-5


@pytest.mark.parametrize("shape", [LayerShape(512, 384, 8, 2, 4, 64, 256, 1e-6),     # 64 z columns per core tile and thread
                                   LayerShape(512, 384, 8, 2, 32, 64, 256, 1e-6)])   # r1 = 32: 8 columns, stores paired up
def test_in_core_writes_the_same_z_at_any_16_byte_alignment(shape):
    """The in-projection/core kernel stores z with 256-bit stores when z is 32-byte aligned and with 16-byte stores
    otherwise (the ABI asks for 16 bytes): same bits either way."""
    lib = _lib.load()
    T, dtype = 300, torch.bfloat16
    L = layer_struct(shape, dtype)
    x, f, fd = _setup(shape, T, dtype)
    F = factors_struct(fd)
    ws, prep = alloc_workspace(lib, L, T, 2), alloc_prepared(lib, L, F)
    _, taps = layer_forward_f64(x, f, shape.top_k, shape.eps, round_scores_to=torch.bfloat16)
    c = taps["c"].float().cuda().contiguous()
    xd = x.cuda()
    raw = torch.zeros(T * shape.r2 + 64, dtype=dtype, device="cuda")
    outs = []
    for off in (0, 8):   # elements: 0 and 16 bytes past a 256-byte aligned address
        z = raw[off:off + T * shape.r2].view(T, shape.r2)
        assert z.data_ptr() % 32 == (16 if off else 0)
        raw.zero_()
        rc = lib.tmoe_in_core(C.byref(L), C.byref(F), prep.data_ptr(), xd.data_ptr(), T, c.data_ptr(), z.data_ptr(),
                              ws.data_ptr(), ws.numel(), 2, cuda_stream_ptr())
        assert rc == 0, _lib.status_string(rc)
        torch.cuda.synchronize()
        outs.append(z.clone())
        assert bool((raw[:off] == 0).all()) and bool((raw[off + T * shape.r2:] == 0).all())
    assert torch.equal(outs[0], outs[1])
    assert rel_fro(outs[0].float().cpu(), taps["z"]) < 1e-2
