"""The allocation-free entry point, called through the C ABI (collected last on purpose).

`tmoe_forward_static_scratch` serves hosts that cannot hand the library a workspace when the layer
runs (all device memory already belongs to their own arena, or an allocation's device-wide
synchronisation is not acceptable in their loop): its scratch is a fixed array inside the library.
It must give exactly what `tmoe_forward` gives on the CUDA-core path with a caller workspace, and it
must keep doing so when the shared array still holds the previous call's intermediates.
"""
import ctypes as C

import pytest
import torch

from mamba_tuckermoe_b200 import _lib
from oracle.tucker_moe_oracle import LayerShape, make_factors, make_tokens

pytestmark = pytest.mark.gpu


def _forward_with_workspace(lib, L, F, x, y):
    T = x.shape[0]
    ws = _lib.alloc_workspace(L, T, _lib.PATH_SIMT)
    rc = lib.tmoe_forward(C.byref(L), C.byref(F), None, x.data_ptr(), T, y.data_ptr(), None, ws.data_ptr(),
                          ws.numel(), _lib.PATH_SIMT, _lib.current_stream_ptr())
    assert rc == 0, _lib.status_string(rc)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_matches_workspace_forward_twice(dtype):
    lib = _lib.load()
    shape = LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6)
    f = {k: v.cuda() for k, v in make_factors(shape, 41, dtype, 0.02, 0.1).items()}
    L, F = _lib.layer_struct(shape, dtype), _lib.factors_struct(f)
    # two calls in a row with different token counts and values: the second one finds the array dirty
    for call, T in enumerate((64, 37)):
        x = make_tokens(T, shape.d_in, 100 + call, dtype).cuda()
        y_ref = torch.empty(T, shape.d_out, dtype=dtype, device="cuda")
        y_new = torch.full((T, shape.d_out), float("nan"), dtype=dtype, device="cuda")
        _forward_with_workspace(lib, L, F, x, y_ref)
        before = torch.cuda.memory_allocated()
        rc = lib.tmoe_forward_static_scratch(C.byref(L), C.byref(F), x.data_ptr(), T, y_new.data_ptr(), None,
                                             _lib.current_stream_ptr())
        assert rc == 0, _lib.status_string(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before      # torch's allocator was not involved
        # same kernels, same inputs: fp32 1e-4 / bf16 2e-2 are the suite's tolerances; equality is expected
        tol = 1e-4 if dtype == torch.float32 else 2e-2
        err = (y_new.float() - y_ref.float()).norm() / y_ref.float().norm()
        assert float(err) <= tol
        assert torch.equal(y_new, y_ref)


def test_static_scratch_rejects_sizes_beyond_the_array():
    lib = _lib.load()
    shape = LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6)
    L = _lib.layer_struct(shape, torch.float32)
    F = _lib.Factors(*[4096] * 7)
    too_many = 4096
    assert lib.tmoe_workspace_bytes(C.byref(L), too_many, _lib.PATH_SIMT) > _lib.STATIC_SCRATCH_BYTES
    assert lib.tmoe_forward_static_scratch(C.byref(L), C.byref(F), 4096, too_many, 4096, None, None) == -5
    assert "too small" in _lib.status_string(-5)
    bad = _lib.layer_struct(LayerShape(1530, 2304, 8, 2, 4, 256, 1024, 1e-6), torch.float32)
    assert lib.tmoe_forward_static_scratch(C.byref(bad), C.byref(F), 4096, 8, 4096, None, None) == -2


def test_static_scratch_largest_call_that_fits():
    """The limit is the one tmoe_workspace_bytes states: the largest token count that fits runs and agrees with the
    workspace forward, one more token is refused."""
    lib = _lib.load()
    shape = LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6)
    dtype = torch.bfloat16
    f = {k: v.cuda() for k, v in make_factors(shape, 43, dtype, 0.02, 0.1).items()}
    L, F = _lib.layer_struct(shape, dtype), _lib.factors_struct(f)
    T = 1
    while lib.tmoe_workspace_bytes(C.byref(L), T + 1, _lib.PATH_SIMT) <= _lib.STATIC_SCRATCH_BYTES:
        T += 1
    assert 600 < T < 1000
    x = make_tokens(T + 1, shape.d_in, 7, dtype).cuda()
    y_ref = torch.empty(T, shape.d_out, dtype=dtype, device="cuda")
    y_new = torch.full((T + 1, shape.d_out), float("nan"), dtype=dtype, device="cuda")
    _forward_with_workspace(lib, L, F, x[:T].contiguous(), y_ref)
    rc = lib.tmoe_forward_static_scratch(C.byref(L), C.byref(F), x.data_ptr(), T, y_new.data_ptr(), None,
                                         _lib.current_stream_ptr())
    assert rc == 0, _lib.status_string(rc)
    torch.cuda.synchronize()
    assert torch.equal(y_new[:T], y_ref) and bool(torch.isnan(y_new[T].float()).all())
    assert lib.tmoe_forward_static_scratch(C.byref(L), C.byref(F), x.data_ptr(), T + 1, y_new.data_ptr(), None,
                                           _lib.current_stream_ptr()) == -5
