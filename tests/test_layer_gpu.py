"""GPU parity of the drop-in layer against the golden outputs of the reference module and
against the float64 oracle.  Everything goes through the C ABI (module -> custom op -> ctypes).

Tolerances: fp32 -- relative Frobenius error and max-abs/max|y| <= 1e-4, expert indices equal
except where the reference's own scores tie within 1e-6.  bf16 -- <= 2e-2 on tokens whose
selection matches (index differences must be explained by scores within one bf16 ulp).
"""
import pytest
import torch

from golden_cases import ALL_CASES, BF16_CASES, F32_CASES, load_case
from gpu_util import build_module
from mamba_tuckermoe_b200 import PATH_AUTO, PATH_DECODE, PATH_SIMT, PATH_TENSOR, read_device_status
from oracle.tucker_moe_oracle import (LayerShape, classify_topk, layer_forward, layer_forward_f64, make_factors,
                                      make_tokens, max_abs, rel_fro)

pytestmark = pytest.mark.gpu

F32_TOL = 1e-4
BF16_TOL = 2e-2


def bf16_ulp(scores):
    """One unit in the last place of a bf16 number of the scores' magnitude (8 significand bits)."""
    m = float(scores.abs().max()) if scores.numel() else 1.0
    return 2.0 ** (torch.tensor(max(m, 1e-30)).log2().floor().item() - 7)


def check_against(y, taps, y_ref, idx_ref, scores_ref, dtype, x, f, shape):
    idx, gates, c = taps
    gap = 1e-6 if dtype == torch.float32 else bf16_ulp(scores_ref)
    rep = classify_topk(idx.cpu(), idx_ref, scores_ref, gap)
    assert rep.unexplained == 0, f"unexplained top-k mismatches at tokens {rep.mismatch_tokens}"
    keep = torch.ones(idx_ref.shape[0], dtype=torch.bool)
    keep[rep.mismatch_tokens] = False
    yk, rk = y.float().cpu().reshape(-1, shape.d_out)[keep], y_ref.float().reshape(-1, shape.d_out)[keep]
    tol = F32_TOL if dtype == torch.float32 else BF16_TOL
    scale = float(rk.abs().max()) if rk.numel() else 1.0
    assert rel_fro(yk, rk) <= tol, f"rel-Fro {rel_fro(yk, rk):.3e} (max-abs {max_abs(yk, rk):.3e})"
    assert max_abs(yk, rk) <= tol * max(scale, 1.0), f"max-abs {max_abs(yk, rk):.3e} vs |y|max {scale:.3f}"
    # tokens that broke a tie differently: compare with the float64 oracle under this run's own selection
    if rep.mismatch_tokens:
        t = torch.tensor(rep.mismatch_tokens)
        y64, _ = layer_forward_f64(x.reshape(-1, shape.d_in)[t], f, shape.top_k, shape.eps, idx=idx.cpu()[t],
                                   round_scores_to=None if dtype == torch.float32 else torch.bfloat16)
        assert rel_fro(y.float().cpu().reshape(-1, shape.d_out)[t], y64) <= tol


@pytest.mark.parametrize("name", ALL_CASES)
def test_simt_path_matches_reference_golden(name):
    shape, x, f, dtype, g = load_case(name)
    m = build_module(shape, f, dtype, path=PATH_SIMT)
    y, taps = m.forward_with_routing(x.cuda())
    assert y.shape == g["y"].shape and y.dtype == dtype
    assert read_device_status() == (0, 0, 0, 0)
    if x.numel() == 0:
        return
    check_against(y, taps, g["y"], g["idx"], g["scores"], dtype, x, f, shape)
    # plain forward (custom op) returns the same tensor as the tapped call
    assert torch.equal(m(x.cuda()), y)


@pytest.mark.parametrize("name", F32_CASES)
def test_fp32_gates_and_coefficients(name):
    shape, x, f, dtype, g = load_case(name)
    if x.numel() == 0:
        return
    m = build_module(shape, f, dtype, path=PATH_SIMT)
    _, (idx, gates, c) = m.forward_with_routing(x.cuda())
    same = (idx.cpu().long() == g["idx"]).all(-1)
    assert max_abs(gates.cpu()[same], g["gates"][same]) < 2e-6
    c_ref = torch.einsum("tk,tkr->tr", g["gates"].double(), f["U_expert"].double()[g["idx"]])
    assert max_abs(c.cpu()[same], c_ref[same]) < 1e-5


def _tensor_case(shape, T, seed, router_std=0.02, bias_std=0.1, lead=None):
    f = make_factors(shape, seed, torch.bfloat16, router_std, bias_std)
    x = make_tokens(T, shape.d_in, seed, torch.bfloat16)
    if lead:
        x = x.reshape(*lead, shape.d_in)
    return x, f


TENSOR_SHAPES = [
    # (shape, T) -- ragged token counts, several r1 / r3 / E, in-kernel and separate routing
    (LayerShape(128, 64, 16, 2, 4, 64, 128, 1e-6), 300),
    (LayerShape(256, 264, 8, 2, 2, 128, 256, 1e-5), 129),
    (LayerShape(192, 320, 40, 8, 8, 192, 192, 1e-6), 77),
    (LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6), 64),
    (LayerShape(1536, 2304, 64, 2, 4, 256, 1024, 1e-6), 1000),
    (LayerShape(256, 128, 512, 8, 4, 64, 128, 1e-6), 200),   # E > 256: scores by the GEMM kernel + select kernel
    (LayerShape(512, 384, 256, 8, 8, 512, 256, 1e-6), 200),  # r3 = 512: h fills all of TMEM, scores by a separate GEMM
    (LayerShape(3072, 4608, 256, 8, 8, 512, 2048, 1e-6), 130),  # the large skewed configuration's shapes
    (LayerShape(768, 1536, 8, 2, 16, 256, 512, 1e-5), 300),     # r1 = 16: sixteen 16-column slices per accumulator
    (LayerShape(768, 4608, 8, 2, 32, 256, 512, 1e-5), 333),     # r1 = 32 (the shipped model's ranks): 8-column slices
    (LayerShape(4608, 768, 8, 2, 32, 256, 512, 1e-5), 19000),   # ... more token tiles than SMs
    (LayerShape(192, 72, 300, 8, 32, 64, 64, 1e-6), 140),       # r1 = 32, one 64-column unit of z, routing by the select kernel
]


@pytest.mark.parametrize("shape,T", TENSOR_SHAPES)
def test_tensor_path_matches_oracle(shape, T):
    """tcgen05 path vs (a) the bf16 reference restatement and (b) float64 algebra on the run's own selection."""
    x, f = _tensor_case(shape, T, seed=4000 + T, router_std=None if shape.E >= 40 else 0.02)
    m = build_module(shape, f, torch.bfloat16, path=PATH_TENSOR)
    y, taps = m.forward_with_routing(x.cuda())
    torch.cuda.synchronize()
    assert read_device_status() == (0, 0, 0, 0)
    y_ref, rt = layer_forward(x, f, shape.top_k, shape.eps, return_taps=True)
    check_against(y, taps, y_ref, rt["idx"], rt["scores"], torch.bfloat16, x, f, shape)
    y64, _ = layer_forward_f64(x, f, shape.top_k, shape.eps, idx=taps[0].cpu(), round_scores_to=torch.bfloat16)
    assert rel_fro(y.float().cpu(), y64) <= 1e-2, "tensor path vs float64 algebra with its own selection"
    assert torch.equal(m(x.cuda()), y)


@pytest.mark.parametrize("shape,T", [
    (LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6), 9),
    (LayerShape(768, 1536, 8, 2, 16, 256, 512, 1e-5), 300),
    (LayerShape(256, 264, 8, 2, 2, 128, 256, 1e-5), 1100),
    (LayerShape(256, 128, 512, 8, 8, 64, 128, 1e-6), 2500),   # routing by the select kernel (c arrives from memory)
    (LayerShape(768, 768, 8, 2, 32, 256, 512, 1e-5), 70),     # r1 = 32
])
def test_token_tiles_shared_between_ctas(shape, T):
    """With few token tiles each tile's core tiles are split over several CTAs: same bits as the same tokens at the
    head of a batch large enough that every tile has a CTA of its own."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    T_big = 128 * (sms // 2 + 6)
    x, f = _tensor_case(shape, T_big, seed=515)
    m = build_module(shape, f, torch.bfloat16, path=PATH_TENSOR)
    xd = x.cuda()
    y_big, taps_big = m.forward_with_routing(xd)
    y, taps = m.forward_with_routing(xd[:T].contiguous())
    torch.cuda.synchronize()
    assert read_device_status() == (0, 0, 0, 0)
    assert torch.equal(y, y_big[:T])
    for a, b in zip(taps, taps_big):
        assert torch.equal(a, b[:T])
    assert torch.equal(m(xd[:T].contiguous()), y)


HANDOFF_SHAPES = [
    # more 128-token tiles than SMs and an out-projection large enough for the CTA-pair kernel: the out-projection starts on
    # the SMs that the last, partial wave of token tiles leaves free and takes finished token tiles one by one (tmoe_handoff_plan)
    (LayerShape(256, 512, 16, 2, 4, 64, 128, 1e-6), 20037),
    (LayerShape(256, 520, 8, 2, 8, 128, 256, 1e-6), 19333),
    (LayerShape(128, 1032, 300, 8, 4, 64, 64, 1e-6), 19001),   # routing by the separate GEMM + select kernels in front
]


@pytest.fixture
def hand_over_on(monkeypatch):
    """The tile-by-tile hand-over is opt-in (TMOE_HANDOFF=1, read by the library on every call)."""
    import ctypes
    monkeypatch.setenv("TMOE_HANDOFF", "1")
    ctypes.CDLL(None).setenv(b"TMOE_HANDOFF", b"1", 1)      # the C library's view of the environment
    yield
    ctypes.CDLL(None).unsetenv(b"TMOE_HANDOFF")


@pytest.mark.parametrize("shape,T", HANDOFF_SHAPES)
def test_out_projection_takes_token_tiles_as_they_finish(shape, T, hand_over_on):
    """Forward with the tile-by-tile hand-over vs the oracle, and bit-for-bit vs the two stages called separately (the stage
    entry points run the same kernels one after the other, without the hand-over)."""
    import ctypes as C
    from mamba_tuckermoe_b200 import _lib
    from gpu_util import layer_struct
    lib = _lib.load()
    nh, nt = C.c_int32(0), C.c_int32(0)
    L = layer_struct(shape, torch.bfloat16)
    assert lib.tmoe_handoff_plan(C.byref(L), T, C.byref(nh), C.byref(nt)) == 0
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    if (T + 127) // 128 <= sms:
        pytest.skip("this device has more SMs than the case has token tiles")
    assert nh.value > 0 and nt.value >= sms, "the case is meant to exercise the hand-over"
    x, f = _tensor_case(shape, T, seed=77, router_std=None if shape.E >= 64 else 0.02)
    m = build_module(shape, f, torch.bfloat16, path=PATH_TENSOR)
    xd = x.cuda()
    y, taps = m.forward_with_routing(xd)
    torch.cuda.synchronize()
    assert read_device_status() == (0, 0, 0, 0)
    y_ref, rt = layer_forward(x, f, shape.top_k, shape.eps, return_taps=True, chunk_tokens=1024)
    check_against(y, taps, y_ref, rt["idx"], rt["scores"], torch.bfloat16, x, f, shape)
    # repeated calls re-tag the hand-over words (nothing is cleared between forwards); a smaller call in between does not
    # use them and must not disturb them
    y_small = m(xd[:4000].contiguous())
    for _ in range(3):
        y2 = m(xd)
    torch.cuda.synchronize()
    assert torch.equal(y2, y) and torch.equal(y_small, y[:4000])
    assert read_device_status() == (0, 0, 0, 0)
    # the stage entry points: same kernels, same arithmetic per output tile
    from gpu_util import factors_struct, alloc_workspace, alloc_prepared, cuda_stream_ptr
    fd = {k: v.cuda() for k, v in f.items()}
    F = factors_struct(fd)
    ws = alloc_workspace(lib, L, T, PATH_TENSOR)
    prep = alloc_prepared(lib, L, F)
    z = torch.empty(T, shape.r2, dtype=torch.bfloat16, device="cuda")
    y3 = torch.empty(T, shape.d_out, dtype=torch.bfloat16, device="cuda")
    c = taps[2].float().contiguous()
    assert lib.tmoe_in_core(C.byref(L), C.byref(F), prep.data_ptr(), xd.data_ptr(), T, c.data_ptr(), z.data_ptr(),
                            ws.data_ptr(), ws.numel(), PATH_TENSOR, cuda_stream_ptr()) == 0
    assert lib.tmoe_out(C.byref(L), C.byref(F), prep.data_ptr(), z.data_ptr(), T, y3.data_ptr(), None, ws.data_ptr(),
                        ws.numel(), PATH_TENSOR, cuda_stream_ptr()) == 0
    torch.cuda.synchronize()
    assert torch.equal(y3, y.reshape(T, shape.d_out))


def test_hand_over_survives_a_dirty_workspace(hand_over_on):
    """The hand-over words are compared with a per-forward epoch and never cleared, so whatever an earlier forward (or
    another layer using the same stream's workspace) left in them must not release a tile early."""
    shape, T = HANDOFF_SHAPES[0]
    x, f = _tensor_case(shape, T, seed=78)
    m = build_module(shape, f, torch.bfloat16, path=PATH_TENSOR)
    xd = x.cuda()
    y = m(xd)
    torch.cuda.synchronize()
    # another layer with other sizes on the same stream (same cached workspace), then the first one again
    shape2 = LayerShape(256, 520, 8, 2, 8, 128, 256, 1e-6)
    x2, f2 = _tensor_case(shape2, 19333, seed=79)
    m2 = build_module(shape2, f2, torch.bfloat16, path=PATH_TENSOR)
    y_other = m2(x2.cuda())
    y_again = m(xd)
    torch.cuda.synchronize()
    assert read_device_status() == (0, 0, 0, 0)
    assert torch.equal(y_again, y)
    assert torch.equal(m2(x2.cuda()), y_other)


DECODE_SHAPES = [
    (LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6), 1),
    (LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6), 8),
    (LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6), 64),
    (LayerShape(1536, 2304, 64, 2, 4, 256, 1024, 1e-6), 33),
    (LayerShape(192, 320, 40, 8, 8, 192, 192, 1e-6), 5),
    (LayerShape(256, 264, 24, 12, 2, 128, 256, 1e-5), 9),
    (LayerShape(3072, 4608, 256, 8, 8, 256, 2048, 1e-6), 17),   # r2 > one staged chunk of z
    (LayerShape(3072, 4608, 256, 8, 8, 512, 2048, 1e-6), 9),    # r3 = 512
    (LayerShape(768, 768, 8, 2, 32, 256, 512, 1e-5), 1),        # the shipped model configuration (r1 = 32), one token
    (LayerShape(768, 4608, 8, 2, 32, 256, 512, 1e-5), 7),
    (LayerShape(4608, 768, 8, 2, 16, 256, 512, 1e-5), 33),
]


@pytest.mark.parametrize("shape,T", DECODE_SHAPES)
def test_decode_path_matches_oracle(shape, T):
    """Bandwidth-shaped kernels for T <= 64 vs the bf16 reference restatement and float64 algebra."""
    x, f = _tensor_case(shape, T, seed=6000 + T, router_std=None if shape.E >= 40 else 0.02)
    m = build_module(shape, f, torch.bfloat16, path=PATH_DECODE)
    y, taps = m.forward_with_routing(x.cuda())
    torch.cuda.synchronize()
    y_ref, rt = layer_forward(x, f, shape.top_k, shape.eps, return_taps=True)
    check_against(y, taps, y_ref, rt["idx"], rt["scores"], torch.bfloat16, x, f, shape)
    y64, _ = layer_forward_f64(x, f, shape.top_k, shape.eps, idx=taps[0].cpu(), round_scores_to=torch.bfloat16)
    assert rel_fro(y.float().cpu(), y64) <= 1e-2
    # AUTO picks the same kernels for these sizes; calling twice gives identical bits up to the atomics' order
    m.path = PATH_AUTO
    assert rel_fro(m(x.cuda()).float().cpu(), y.float().cpu()) < 5e-3


FUSED_DECODE_SHAPES = [
    # T <= 4: the whole forward is one launch of thread-block clusters
    (LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6), 1),
    (LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6), 2),
    (LayerShape(1536, 2304, 64, 2, 4, 256, 1024, 1e-6), 3),
    (LayerShape(1536, 6144, 8, 2, 32, 256, 512, 1e-5), 1),      # the shipped model's widest layer
    (LayerShape(4608, 768, 8, 2, 32, 256, 512, 1e-5), 4),       # ... and its deepest contraction
    (LayerShape(768, 768, 8, 2, 16, 256, 512, 1e-5), 4),
    (LayerShape(3072, 4608, 256, 8, 8, 512, 2048, 1e-6), 3),    # r3 = 512, top-8 of 256
    (LayerShape(256, 264, 1024, 16, 2, 64, 128, 1e-5), 2),      # top-16 of 1024, the smallest ranks, d_out not a multiple of 16
    (LayerShape(256, 264, 100, 8, 2, 64, 128, 1e-5), 4),        # 100 experts: four keys per lane in the routing
    (LayerShape(128, 72, 8, 2, 8, 128, 192, 1e-6), 4),
    (LayerShape(768, 768, 8, 2, 16, 256, 512, 1e-5), 8),        # 5 - 8 tokens: the three-kernel form
    (LayerShape(128, 72, 8, 2, 8, 128, 192, 1e-6), 7),
]


@pytest.mark.parametrize("shape,T", FUSED_DECODE_SHAPES)
def test_one_launch_decode_forward(shape, T):
    """One launch per call, the same result on every call (its partial sums are added in a fixed order and its counters
    are left cleared), epilogues included."""
    import ctypes as C
    from mamba_tuckermoe_b200 import _lib
    x, f = _tensor_case(shape, T, seed=8000 + T, router_std=None if shape.E >= 64 else 0.02)
    m = build_module(shape, f, torch.bfloat16, path=PATH_DECODE)
    lib = _lib.load()
    xd = x.cuda()
    m(xd)
    n0 = lib.tmoe_launch_count()
    y1 = m(xd)
    assert lib.tmoe_launch_count() - n0 == (1 if T <= 4 else 3), "up to 4 tokens are meant to be a single launch"
    y, taps = m.forward_with_routing(xd)
    y2 = m(xd)
    torch.cuda.synchronize()
    assert torch.equal(y1, y) and torch.equal(y2, y)
    y_ref, rt = layer_forward(x, f, shape.top_k, shape.eps, return_taps=True)
    check_against(y, taps, y_ref, rt["idx"], rt["scores"], torch.bfloat16, x, f, shape)
    y64, own = layer_forward_f64(x, f, shape.top_k, shape.eps, idx=taps[0].cpu(), round_scores_to=torch.bfloat16)
    assert rel_fro(y.float().cpu(), y64) <= 1e-2
    assert max_abs(taps[1].cpu(), own["gates"]) < 4e-3 and max_abs(taps[2].cpu(), own["c"]) < 4e-2
    # silu-gate and residual epilogues in the same launch
    g = torch.Generator().manual_seed(T)
    gate = torch.randn(T, shape.d_out, generator=g).bfloat16().cuda()
    res = torch.randn(T, shape.d_out, generator=g).bfloat16().cuda()
    gamma = (1 + 0.1 * torch.randn(shape.d_out, generator=g)).bfloat16().cuda()
    fused = m.forward_fused(xd, silu_gate=gate, residual=res, layer_scale=gamma).float()
    expect = res.float() + gamma.float() * (torch.nn.functional.silu(gate.float()) * y64.float().cuda())
    assert rel_fro(fused.cpu(), expect.cpu()) < 1e-2


@pytest.mark.parametrize("shape,T", [
    (LayerShape(256, 264, 8, 2, 4, 128, 256, 1e-5), 300),       # single-CTA GEMM, ragged last tile, d_out not a multiple of 64
    (LayerShape(1536, 2304, 64, 2, 4, 256, 1024, 1e-6), 20000),  # CTA pairs, ragged last tile
])
def test_out_projection_writes_every_destination(shape, T):
    """tmoe_extras_t.peer_y: the out-projection stores each tile to y and to the further buffers (here on the same GPU;
    across GPUs they are the peers' mapped result buffers).  Rows beyond T of a destination stay untouched."""
    from mamba_tuckermoe_b200 import _lib
    x, f = _tensor_case(shape, T, seed=31 + T)
    m = build_module(shape, f, torch.bfloat16, path=PATH_AUTO)
    xd = x.cuda()
    ref = m(xd)
    out = torch.empty_like(ref)
    big = [torch.full((T + 40, shape.d_out), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(_lib.MAX_PEERS)]
    for n in (1, 3, _lib.MAX_PEERS):
        for b in big:
            b.fill_(float("nan"))
        m.forward_into(xd, out, peer_ptrs=[b.data_ptr() for b in big[:n]])
        torch.cuda.synchronize()
        assert torch.equal(out, ref)
        for i, b in enumerate(big):
            if i < n:
                assert torch.equal(b[:T], ref) and bool(torch.isnan(b[T:]).all())
            else:
                assert bool(torch.isnan(b).all())
    assert read_device_status() == (0, 0, 0, 0)
    # the other paths refuse before anything is enqueued
    small = build_module(shape, f, torch.bfloat16, path=PATH_DECODE)
    with pytest.raises(_lib.TmoeError) as e:
        small.forward_into(xd[:4], out[:4], peer_ptrs=[big[0].data_ptr()])
    assert e.value.status == _lib.ERR_UNSUPPORTED


@pytest.mark.parametrize("name", BF16_CASES)
def test_decode_path_matches_reference_golden(name):
    shape, x, f, dtype, g = load_case(name)
    if shape.r3 % 64 or x.numel() // shape.d_in > 64:
        pytest.skip("shape not covered by the decode path")
    m = build_module(shape, f, dtype, path=PATH_DECODE)
    y, taps = m.forward_with_routing(x.cuda())
    check_against(y, taps, g["y"], g["idx"], g["scores"], dtype, x, f, shape)


@pytest.mark.parametrize("name", BF16_CASES)
def test_tensor_path_matches_reference_golden(name):
    shape, x, f, dtype, g = load_case(name)
    if shape.r3 % 64:
        pytest.skip("shape not covered by the tensor-core path")
    m = build_module(shape, f, dtype, path=PATH_TENSOR)
    y, taps = m.forward_with_routing(x.cuda())
    assert read_device_status() == (0, 0, 0, 0)
    check_against(y, taps, g["y"], g["idx"], g["scores"], dtype, x, f, shape)


def assert_selection_explained(idx_run, x_in, f, shape, ulps=1.0, router=(0, 10.0, 0.5)):
    """Every selection that differs from the float64 oracle's (scores rounded to bf16, computed from the very input the
    layer was given) must be a near-tie: the competing experts' scores within `ulps` bf16 units in the last place."""
    _, nat = layer_forward_f64(x_in, f, shape.top_k, shape.eps, round_scores_to=torch.bfloat16, router=router)
    rep = classify_topk(idx_run.cpu(), nat["idx"], nat["scores"], ulps * bf16_ulp(nat["scores"]))
    assert rep.unexplained == 0, f"{rep.unexplained} selections differ without a score tie (tokens {rep.mismatch_tokens[:8]})"
    return rep


def assert_tokens_close(a, b, tol):
    """Error of EVERY token, relative to the token's own norm or to the median token norm, whichever is larger (a token
    whose two experts' contributions nearly cancel has a small norm and a correspondingly large relative error; measured
    against the typical norm it still has to be as accurate as the others, and a wrong token is off by ~100 %)."""
    nb = b.double().norm(dim=-1)
    err = (a.double() - b.double()).norm(dim=-1) / torch.maximum(nb, nb.median()).clamp(min=1e-30)
    assert float(err.max()) < tol, f"token {int(err.argmax())} is off by {float(err.max()):.3e} (tolerance {tol})"


def test_tensor_and_simt_paths_agree():
    shape = LayerShape(1536, 2304, 64, 2, 4, 256, 1024, 1e-6)
    x, f = _tensor_case(shape, 515, seed=77, router_std=None)
    a, ta = build_module(shape, f, torch.bfloat16, path=PATH_TENSOR).forward_with_routing(x.cuda())
    b, tb = build_module(shape, f, torch.bfloat16, path=PATH_SIMT).forward_with_routing(x.cuda())
    # the two paths sum the router dot products in different orders: a selection may differ only at a bf16 near-tie
    assert_selection_explained(ta[0], x, f, shape)
    assert_selection_explained(tb[0], x, f, shape)
    same = (ta[0] == tb[0]).all(-1).cpu()
    assert rel_fro(a.float().cpu()[same], b.float().cpu()[same]) < 1e-2
    for y, taps in ((a, ta), (b, tb)):   # the tie-broken tokens, each against float64 under its own selection
        if not bool(same.all()):
            t = torch.nonzero(~same).flatten()
            y64, _ = layer_forward_f64(x[t], f, shape.top_k, shape.eps, idx=taps[0].cpu()[t], round_scores_to=torch.bfloat16)
            assert_tokens_close(y.float().cpu()[t], y64, BF16_TOL)


@pytest.mark.parametrize("path", [PATH_SIMT, PATH_TENSOR, PATH_DECODE])
def test_fused_residual_epilogue(path):
    """residual + layer_scale * layer(x) equals the callers' composition (model.py:259-260, 340-341)."""
    shape = LayerShape(128, 64, 16, 2, 4, 64, 128, 1e-6)
    n_tok = 40 if path == PATH_DECODE else 130
    x, f = _tensor_case(shape, n_tok, seed=5)
    m = build_module(shape, f, torch.bfloat16, path=path)
    g = torch.Generator().manual_seed(1)
    res = torch.randn(n_tok, shape.d_out, generator=g).bfloat16().cuda()
    gamma = (1 + 0.1 * torch.randn(shape.d_out, generator=g)).bfloat16().cuda()
    y = m(x.cuda()).float()
    fused = m.forward_fused_residual(x.cuda(), res, gamma).float()
    expect = res.float() + gamma.float() * y
    assert rel_fro(fused.cpu(), expect.cpu()) < 1e-2


def test_auto_path_and_leading_shapes():
    shape = LayerShape(1536, 2304, 8, 2, 4, 256, 1024, 1e-6)
    x, f = _tensor_case(shape, 96, seed=9, lead=(2, 48))
    m = build_module(shape, f, torch.bfloat16, path=PATH_AUTO)
    y = m(x.cuda())
    assert y.shape == (2, 48, 2304)
    y1 = m(x.cuda()[0, :1])     # T=1 -> decode-shaped kernels
    assert y1.shape == (1, 2304)
    y_ref = layer_forward(x, f, shape.top_k, shape.eps)
    assert rel_fro(y.float().cpu(), y_ref.float()) < 3e-2


def test_noncontiguous_input_and_worker_thread():
    """The reference calls the layer from worker threads under no_grad (generate.py:107, server.py:125)."""
    import threading
    shape, x, f, dtype, g = load_case("tiny_f32")
    m = build_module(shape, f, dtype)
    xt = torch.cat([x, x], -1).cuda()[:, : shape.d_in]  # non-contiguous view
    out = {}

    def work():
        with torch.no_grad():
            out["y"] = m(xt)
        torch.cuda.synchronize()

    t = threading.Thread(target=work)
    t.start(); t.join()
    assert rel_fro(out["y"].cpu(), g["y"]) < F32_TOL


def test_linearity_in_out_projection_and_bias():
    """Size-independent property at a benchmark-sized T: y(x; bias) - y(x; 0) == bias for every token."""
    shape = LayerShape(1536, 2304, 64, 2, 4, 256, 1024, 1e-6)
    x, f = _tensor_case(shape, 8192, seed=21, router_std=None, bias_std=0.0)
    m0 = build_module(shape, f, torch.bfloat16)
    y0 = m0(x.cuda()).float()
    f2 = dict(f); f2["bias"] = torch.full((shape.d_out,), 0.5).bfloat16()
    y1 = build_module(shape, f2, torch.bfloat16)(x.cuda()).float()
    assert read_device_status() == (0, 0, 0, 0)
    d = (y1 - y0 - 0.5).abs()
    assert float(d.max()) <= 0.07 and float(d.mean()) < 0.01   # one bf16 rounding of |y| <= 16
    # token-wise independence: permuting tokens permutes outputs bit for bit
    perm = torch.randperm(8192, generator=torch.Generator().manual_seed(3)).cuda()
    assert torch.equal(m0(x.cuda()[perm]).float(), y0[perm])


@pytest.mark.parametrize("T,chunk", [(700, 256), (64, 8192), (3000, 1024)])
def test_forward_host_equals_device_forward(T, chunk):
    """Host-resident activations: the chunk-pipelined call returns what the device call returns."""
    shape = LayerShape(256, 264, 8, 2, 4, 128, 256, 1e-5)
    x, f = _tensor_case(shape, T, seed=99)
    m = build_module(shape, f, torch.bfloat16)
    xh = x.pin_memory()
    out = torch.empty(T, shape.d_out, dtype=torch.bfloat16).pin_memory()
    y_host = m.forward_host(xh, out=out, chunk_tokens=chunk)
    torch.cuda.current_stream().synchronize()
    assert y_host.data_ptr() == out.data_ptr()
    y_ref = layer_forward(x, f, shape.top_k, shape.eps)
    assert rel_fro(y_host.float(), y_ref.float()) < 3e-2
    # each chunk is an independent forward on its tokens; chunks above 64 tokens use the tensor-core kernels
    parts = [m(x[lo:lo + chunk].cuda()).cpu() for lo in range(0, T, chunk)]
    assert torch.equal(torch.cat(parts), y_host) or rel_fro(torch.cat(parts).float(), y_host.float()) < 5e-3
    y2 = m.forward_host(x.reshape(1, T, -1))   # unpinned input, allocated output, leading shape kept
    torch.cuda.current_stream().synchronize()
    assert y2.shape == (1, T, shape.d_out) and rel_fro(y2.float().reshape(T, -1), y_host.float()) < 5e-3


def test_forward_host_pipelined_loop():
    """A loop of pipelined host calls (input copy of one call under the output copy of the one before, two device input
    buffers used in turn, growing token counts) returns, per call, what the plain call returns."""
    shape = LayerShape(256, 264, 8, 2, 4, 128, 256, 1e-5)
    m = None
    xs, outs = [], []
    for i, T in enumerate([500, 1300, 900, 1300, 70]):
        x, f = _tensor_case(shape, T, seed=300 + i)
        if m is None:
            m = build_module(shape, make_factors(shape, 300, torch.bfloat16, 0.02, 0.1), torch.bfloat16)
        xs.append(x.pin_memory())
        outs.append(torch.empty(T, shape.d_out, dtype=torch.bfloat16).pin_memory())
    for xh, out in zip(xs, outs):
        m.forward_host(xh, out=out, chunk_tokens=384, pipelined=True)
    torch.cuda.current_stream().synchronize()
    for xh, out in zip(xs, outs):
        ref = m.forward_host(xh, chunk_tokens=384)
        torch.cuda.current_stream().synchronize()
        assert torch.equal(ref, out)


@pytest.mark.parametrize("dtype,T", [(torch.float32, 50), (torch.bfloat16, 300), (torch.bfloat16, 7)])
def test_rms_norm_matches_reference_formula(dtype, T):
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(T, 768, generator=g) * 3).to(dtype)
    w = (1 + 0.2 * torch.randn(768, generator=g)).to(dtype)
    from mamba_tuckermoe_b200 import rms_norm
    from oracle.tucker_moe_oracle import rms_norm as ref_norm
    y = rms_norm(x.cuda(), w.cuda(), 1e-5).cpu()
    ref = ref_norm(x, w, 1e-5)                         # the reference's formula in the tensor dtype (model.py:25-27)
    tol = 2e-6 if dtype == torch.float32 else 1e-2     # bf16: the reference rounds after every step, the kernel once
    assert rel_fro(y.float(), ref.float()) < tol
    ref64 = x.double() / torch.sqrt(x.double().pow(2).mean(-1, keepdim=True) + 1e-5) * w.double()
    assert rel_fro(y.float(), ref64) < (1e-6 if dtype == torch.float32 else 4e-3)


@pytest.mark.parametrize("T", [5, 200])
def test_fused_ffn_and_out_proj_match_callers_composition(T):
    """fused_ffn / fused_out_proj against the literal composition of model.py:337-341 and 258-260 in float64.

    Three bf16 layers in a chain: a token whose rounded scores tie may pick another expert than float64 does.  Every
    such difference is classified (it must be a near-tie in the float64 scores of the layer's actual input), and the
    float64 chain is then evaluated under the run's own selections, where every token has to agree."""
    import torch.nn.functional as F
    from mamba_tuckermoe_b200 import fused_ffn, fused_out_proj
    from oracle.tucker_moe_oracle import rms_norm as ref_norm
    d, dff = 256, 768
    s_up = LayerShape(d, dff, 8, 2, 4, 128, 256, 1e-5)
    s_dn = LayerShape(dff, d, 8, 2, 4, 128, 256, 1e-5)
    fg, fu, fd = (make_factors(s, 70 + i, torch.bfloat16, 0.02, 0.05) for i, s in enumerate((s_up, s_up, s_dn)))
    g = torch.Generator().manual_seed(8)
    x = torch.randn(T, d, generator=g).bfloat16()
    nw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16()
    gamma = (0.5 + 0.1 * torch.randn(d, generator=g)).bfloat16()
    mg, mu, md = build_module(s_up, fg, torch.bfloat16), build_module(s_up, fu, torch.bfloat16), build_module(s_dn, fd, torch.bfloat16)
    norm = (nw.cuda(), 1e-5)
    out = fused_ffn(mg, mu, md, x.cuda(), norm, gamma.cuda())
    # the same three calls one by one, with their routing results
    gate, tg = mg.forward_fused(x.cuda(), pre_norm=norm, return_routing=True)
    act, tu = mu.forward_fused(x.cuda(), pre_norm=norm, silu_gate=gate, return_routing=True)
    out2, td = md.forward_fused(act, residual=x.cuda(), layer_scale=gamma.cuda(), return_routing=True)
    assert torch.equal(out2, out)
    xf = ref_norm(x.double(), nw.double(), 1e-5)
    # the norm weight is folded into bf16 copies of the router rows, which moves a score by a fraction of an ulp
    assert_selection_explained(tg[0], xf, fg, s_up, ulps=2)
    assert_selection_explained(tu[0], xf, fu, s_up, ulps=2)
    assert_selection_explained(td[0], act.double().cpu(), fd, s_dn)
    lay = lambda t, f, s, idx: layer_forward_f64(t, f, s.top_k, s.eps, idx=idx.cpu(), round_scores_to=torch.bfloat16)[0]
    ref = x.double() + gamma.double() * lay(F.silu(lay(xf, fg, s_up, tg[0])) * lay(xf, fu, s_up, tu[0]), fd, s_dn, td[0])
    assert_tokens_close(out.float().cpu(), ref, 3e-2)
    # out_proj tail: mid + gamma * layer(norm(mid))
    s_o = LayerShape(d, d, 8, 2, 4, 128, 256, 1e-5)
    fo = make_factors(s_o, 90, torch.bfloat16, 0.02, 0.05)
    mo = build_module(s_o, fo, torch.bfloat16)
    got = fused_out_proj(mo, x.cuda(), norm, gamma.cuda())
    got2, to = mo.forward_fused(x.cuda(), pre_norm=norm, residual=x.cuda(), layer_scale=gamma.cuda(), return_routing=True)
    assert torch.equal(got2, got)
    assert_selection_explained(to[0], xf, fo, s_o, ulps=2)
    want = x.double() + gamma.double() * lay(xf, fo, s_o, to[0])
    assert_tokens_close(got.float().cpu(), want, BF16_TOL)


@pytest.mark.parametrize("T", [70, 300, 20000])
def test_ffn_gate_and_up_in_one_launch(T):
    """fused_ffn on the tensor-core path: the gate and up layers' in-projection / core stages are one launch whose CTAs
    alternate between the two layers (each tile of x comes from HBM once); five launches for the whole FFN instead of
    six, and the same bits as the three layers called one by one."""
    import ctypes as C
    from mamba_tuckermoe_b200 import _lib, fused_ffn
    d, dff = 256, 768
    s_up = LayerShape(d, dff, 8, 2, 4, 128, 256, 1e-5)
    s_dn = LayerShape(dff, d, 8, 2, 4, 128, 256, 1e-5)
    fg, fu, fd = (make_factors(s, 170 + i, torch.bfloat16, 0.02, 0.05) for i, s in enumerate((s_up, s_up, s_dn)))
    g = torch.Generator().manual_seed(18)
    x = torch.randn(T, d, generator=g).bfloat16().cuda()
    nw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16().cuda()
    gamma = (0.5 + 0.1 * torch.randn(d, generator=g)).bfloat16().cuda()
    mg, mu, md = build_module(s_up, fg, torch.bfloat16), build_module(s_up, fu, torch.bfloat16), build_module(s_dn, fd, torch.bfloat16)
    lib = _lib.load()
    out = fused_ffn(mg, mu, md, x, (nw, 1e-5), gamma)          # prepares the factor sets
    n0 = lib.tmoe_launch_count()
    out = fused_ffn(mg, mu, md, x, (nw, 1e-5), gamma)
    assert lib.tmoe_launch_count() - n0 == 5
    torch.cuda.synchronize()
    assert read_device_status() == (0, 0, 0, 0)
    gate = mg.forward_fused(x, pre_norm=(nw, 1e-5))
    act = mu.forward_fused(x, pre_norm=(nw, 1e-5), silu_gate=gate)
    ref = md.forward_fused(act, residual=x, layer_scale=gamma)
    assert torch.equal(out, ref)
    # different sizes of the two layers: the composition of separate calls is used and gives the usual result
    s_other = LayerShape(d, dff, 8, 2, 4, 64, 256, 1e-5)
    mo = build_module(s_other, make_factors(s_other, 173, torch.bfloat16, 0.02, 0.05), torch.bfloat16)
    out2 = fused_ffn(mo, mu, md, x, (nw, 1e-5), gamma)
    gate2 = mo.forward_fused(x, pre_norm=(nw, 1e-5))
    assert torch.equal(out2, md.forward_fused(mu.forward_fused(x, pre_norm=(nw, 1e-5), silu_gate=gate2), residual=x, layer_scale=gamma))


@pytest.mark.parametrize("dtype,path,T", [
    (torch.float32, PATH_SIMT, 33), (torch.float32, PATH_SIMT, 300), (torch.bfloat16, PATH_SIMT, 40),
    (torch.bfloat16, PATH_TENSOR, 300), (torch.bfloat16, PATH_DECODE, 9), (torch.bfloat16, PATH_DECODE, 64)])
def test_capped_softmax_router_rule(dtype, path, T):
    """router_mode = 1 (tanh cap, temperature, softmax over all experts, renormalised top-k) on every kernel path,
    against the oracle's restatement of sft_cot_bundle/scripts/model.py:318-329 (pinned to the reference module by
    tests/test_variant_golden.py)."""
    small = T != 300 or dtype == torch.float32
    shape = LayerShape(256, 384, 64, 8, 8, 64, 128, 1e-6) if small else LayerShape(1536, 2304, 64, 2, 4, 256, 1024, 1e-6)
    f = make_factors(shape, 123, dtype, None, 0.1)
    f["router_w"] = (f["router_w"].float() * 4).to(dtype)          # scores of a few units so that the cap matters
    x = make_tokens(T, shape.d_in, 123, dtype)
    m = build_module(shape, f, dtype, path=path)
    m.router_mode, m.router_cap, m.router_temperature = 1, 10.0, 0.5
    router = (1, 10.0, 0.5)
    y, taps = m.forward_with_routing(x.cuda())
    torch.cuda.synchronize()
    rnd = None if dtype == torch.float32 else torch.bfloat16
    y_ref, rt = layer_forward(x, f, shape.top_k, shape.eps, return_taps=True, router=router)
    # the top-k of this rule compares the tempered capped logits ("order"); two competing bf16 values may each round one ulp
    # differently in the two implementations, so an order flip is explained by a gap of up to two ulps
    gap = 2e-5 if dtype == torch.float32 else 2 * bf16_ulp(rt["order"])
    rep = classify_topk(taps[0].cpu(), rt["idx"], rt["order"], gap)
    assert rep.unexplained == 0
    y64, own = layer_forward_f64(x, f, shape.top_k, shape.eps, idx=taps[0].cpu(), round_scores_to=rnd, router=router)
    tol = F32_TOL if dtype == torch.float32 else 1e-2
    assert rel_fro(y.float().cpu(), y64) <= tol
    # tempered logits reach ~20, so fp32 exp/tanh round-off of 1e-7 relative becomes a few 1e-6 in a gate
    assert max_abs(taps[1].cpu(), own["gates"]) < (1e-5 if dtype == torch.float32 else 4e-3)
    assert torch.equal(m(x.cuda()), y)                              # eager fast path uses the same rule
    # rule 0 on the same module gives a different answer
    m.router_mode = 0
    assert rel_fro(m(x.cuda()).float().cpu(), y64) > 3 * tol


@pytest.mark.parametrize("T", [1, 8, 40, 65, 700])
def test_in_kernel_pre_norm_matches_separate_norm(T):
    """forward_fused(pre_norm=...) on the tensor-core path (T > 64) and the decode path (T <= 64) folds the norm weight
    into the prepared factors and finds 1/rms(x) in-kernel; it must agree with RMSNorm-then-layer (model.py:258-259, 337-339) in float64 and with the
    two-kernel composition of this library."""
    from oracle.tucker_moe_oracle import rms_norm as ref_norm
    shape = LayerShape(1536, 2304, 64, 2, 4, 256, 1024, 1e-6)
    x, f = _tensor_case(shape, T + 2, seed=31, router_std=None)
    x = x[2:].contiguous()                                        # (the first token of this draw sits on a near-tie of two scores)
    x = (x.float() * 2.5 + 0.3).bfloat16()                       # rms(x) clearly different from 1
    g = torch.Generator().manual_seed(2)
    nw = (1 + 0.3 * torch.randn(shape.d_in, generator=g)).bfloat16()
    m = build_module(shape, f, torch.bfloat16)
    y_fused, taps = m.forward_fused(x.cuda(), pre_norm=(nw.cuda(), 1e-5), return_routing=True)
    torch.cuda.synchronize()
    assert read_device_status() == (0, 0, 0, 0)
    assert m._prep_pn is not None                                  # the in-kernel route was taken
    assert torch.equal(m.forward_fused(x.cuda(), pre_norm=(nw.cuda(), 1e-5)), y_fused)
    from mamba_tuckermoe_b200 import rms_norm
    xn = rms_norm(x.cuda(), nw.cuda(), 1e-5)
    y_two, taps_two = m.forward_with_routing(xn)
    xn64 = ref_norm(x.double(), nw.double(), 1e-5)
    # selections: the fused call against float64 of the exact normalised input (the bf16 fold of the norm weight into
    # the router rows moves a score by a fraction of an ulp), the two-kernel call against float64 of ITS input
    assert_selection_explained(taps[0], xn64, f, shape, ulps=2)
    assert_selection_explained(taps_two[0], xn.double().cpu(), f, shape)
    y64, _ = layer_forward_f64(xn64, f, shape.top_k, shape.eps, idx=taps[0].cpu(), round_scores_to=torch.bfloat16)
    # overall at half the contract's tolerance; token by token at 2.5 times it: the scores here reach 4, where one bf16
    # ulp is 0.03 -- a selected score that rounds the other way moves its gate by 0.8 %, and the two experts' outputs can
    # differ by a multiple of their weighted sum.  A wrong expert or a wrong row would be off by ~100 %.
    assert rel_fro(y_fused.float().cpu(), y64) < 1e-2
    assert_tokens_close(y_fused.float().cpu(), y64, 2.5 * BF16_TOL)
    same = (taps[0] == taps_two[0]).all(-1)
    if bool(same.any()):
        assert rel_fro(y_fused.float()[same].cpu(), y_two.float()[same].cpu()) < 1e-2
        assert_tokens_close(y_fused.float()[same].cpu(), y_two.float()[same].cpu(), 2.5 * BF16_TOL)
    # residual + silu epilogues ride along unchanged
    res = torch.randn(T, shape.d_out, generator=g).bfloat16().cuda()
    gam = torch.ones(shape.d_out).bfloat16().cuda()
    y_r = m.forward_fused(x.cuda(), pre_norm=(nw.cuda(), 1e-5), residual=res, layer_scale=gam)
    assert rel_fro((y_r.float() - res.float()).cpu(), y_fused.float().cpu()) < 1e-2


def test_prepared_sidecar_round_trip(tmp_path):
    """The prepared-factor sidecar installs only on a layer whose parameters match its fingerprint."""
    from mamba_tuckermoe_b200.checkpoint import load_prepared_sidecar, save_prepared_sidecar
    shape = LayerShape(256, 264, 8, 2, 4, 128, 256, 1e-5)
    x, f = _tensor_case(shape, 200, seed=3)
    a = build_module(shape, f, torch.bfloat16)
    y = a(x.cuda())
    path = str(tmp_path / "layer0.prepared.npz")
    save_prepared_sidecar(a, path)
    b = build_module(shape, f, torch.bfloat16)
    assert load_prepared_sidecar(b, path) and b._prep is not None
    assert torch.equal(b(x.cuda()), y)
    f2 = dict(f); f2["bias"] = (f["bias"].float() + 1).bfloat16()
    c = build_module(shape, f2, torch.bfloat16)
    assert not load_prepared_sidecar(c, path)          # different parameters: refused, layer untouched
    assert c._prep is None
