"""Benchmark of the Tucker-MoE layer forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl ours|reference]

One "step" is one forward of the layer over one batch of synthetic tokens.  The default
workload is the prefill configuration (T=32768 tokens per GPU, d_in=1536, d_out=2304, E=64,
top-2, ranks (4,256,1024), bf16).  Tokens are sharded over the GPUs with the factor set
replicated; there is no collective on the data path, per-GPU work is fixed as N grows (weak
scaling) and `value` is tokens/s summed over all ranks, timed with CUDA events, max over ranks.

The JSON line also carries
  roofline      achieved TFLOP/s of the dominant kernel (algorithmic FLOPs / CUDA-event time)
                against the measured bf16 peak in MEASURED_PEAKS.json
  e2e           the same metric through the public call for host-resident activations
                (TuckerMoE.forward_host): pinned host -> device copy of x, the kernels and the
                device -> host copy of y are all inside the timed region, chunk-pipelined on 3 streams;
                with the copy rate of each direction alone, per rank
  strong        the workload's T tokens split over the N GPUs (T/N per GPU), same timing rules
  allgather     (N > 1) that split followed by the NCCL all-gather of y into a [T, d_out] buffer on every rank,
                unchunked and in 4 chunks overlapped with the kernels (sharding.py)
  parity        the run's output against the CPU oracle on a fixed token subset, outside the timed region
  cpu_baseline  the CPU restatement of the reference layer on this host (rank 0, N=1 only)
  gpu_eager_baseline  the same restatement as eager PyTorch on this GPU (rank 0, N=1 only)
  clocks        SM clock / throttle reasons sampled with nvidia-smi during the timed region

`--impl reference` times the reference algorithm's CPU path (the oracle restatement of
pure_torch_mlx/model.py:68-102, all host threads) on the same workload, each step a bounded
token sample.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (oracle shape key, tokens per GPU, description)
    "cfg2": ("cfg2", 32768, "prefill bf16 T=32768 d_in=1536 d_out=2304 E=64 top2 r=(4,256,1024)"),
    "cfg0": ("cfg0", 512, "fp32 T=512 d_in=1536 d_out=2304 E=8 top2 r=(4,256,1024)"),
    "cfg1": ("cfg1", 64, "decode bf16 T=64 d_in=1536 d_out=2304 E=8 top2 r=(4,256,1024)"),
    "cfg1_t8": ("cfg1", 8, "decode bf16 T=8 d_in=1536 d_out=2304 E=8 top2 r=(4,256,1024)"),
    "cfg1_t1": ("cfg1", 1, "decode bf16 T=1 d_in=1536 d_out=2304 E=8 top2 r=(4,256,1024)"),
    "cfg3": ("cfg3", 16384, "bf16 T=16384 E=64 top2"),
    "cfg4": ("cfg4", 131072, "skewed bf16 T=131072 d_in=3072 d_out=4608 E=256 top8 r=(8,512,2048), Zipf(1.2) router bias"),
}
for _e in (8, 64, 256, 1024):
    for _k in (2, 8):
        WORKLOADS[f"cfg3_e{_e}_k{_k}"] = (f"cfg3_e{_e}_k{_k}", 16384,
                                          f"sweep bf16 T=16384 d_in=1536 d_out=2304 E={_e} top{_k} r=(4,256,1024)")
for _n, _di, _do in (("x_up", 1536, 6144), ("out_proj", 768, 768), ("ffn_up", 768, 4608), ("ffn_down", 4608, 768)):
    WORKLOADS[f"shipped_{_n}"] = (f"shipped_{_n}", 16384,
                                  f"prefill bf16 T=16384 d_in={_di} d_out={_do} E=8 top2 r=(32,256,512): the reference model's shipped ranks")


def ncu_traffic(workload: str, kernel: str):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of `kernel` on `workload`, from the line
    `# traffic_bytes_per_launch <workload> <kernel> <bytes> commit <hash>` of a summary under profiles/ (None if absent)."""
    d = os.path.join(ROOT, "profiles")
    try:
        for name in sorted(os.listdir(d)):
            for line in open(os.path.join(d, name), errors="replace"):
                parts = line.split()
                if len(parts) >= 5 and parts[:2] == ["#", "traffic_bytes_per_launch"] and parts[2] == workload and parts[3] == kernel:
                    return {"bytes": int(parts[4]), "commit": parts[6] if len(parts) > 6 else None, "file": f"profiles/{name}"}
    except OSError:
        pass
    return None


N_INPUT_SETS = 4  # rotating x buffers so that no step re-reads the previous step's lines from L2


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle sampling in the background (read-only queries)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_info():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def cpu_reference_rate(workload: str, sample_tokens: int, reps: int):
    """tokens/s of the CPU restatement of the reference layer on `sample_tokens` tokens of the workload."""
    from oracle.tucker_moe_oracle import BENCH_SHAPES, layer_forward, make_factors, make_tokens
    shape, _, dtype, seed, rstd = BENCH_SHAPES[WORKLOADS[workload][0]]
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    f = make_factors(shape, seed, dtype, rstd)
    x = make_tokens(sample_tokens, shape.d_in, seed, dtype)
    layer_forward(x[:256], f, shape.top_k, shape.eps, chunk_tokens=64)  # warm-up
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        layer_forward(x, f, shape.top_k, shape.eps, chunk_tokens=64)
        times.append(time.perf_counter() - t0)
    dt = min(times)
    return sample_tokens / dt, threads, dt


def run_reference_arm(args):
    rank, world, _ = dist_info()
    if rank != 0:
        return
    shape_key, T, desc = WORKLOADS[args.workload]
    sample = min(T, 2048)
    times = []
    from oracle.tucker_moe_oracle import BENCH_SHAPES, layer_forward, make_factors, make_tokens
    shape, _, dtype, seed, rstd = BENCH_SHAPES[shape_key]
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    f = make_factors(shape, seed, dtype, rstd)
    x = make_tokens(sample, shape.d_in, seed, dtype)
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        layer_forward(x, f, shape.top_k, shape.eps, chunk_tokens=64)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    total = sum(times)
    value = sample * args.steps / total
    line = {
        "impl": "reference", "metric": "tucker_moe_layer_tokens_per_sec", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if dtype == torch.bfloat16 else "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {desc}", "tokens_per_step": sample,
                   "note": "reference algorithm (CPU restatement of pure_torch_mlx/model.py:68-102), "
                           f"each step a {sample}-token sample of the workload"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{sample} tokens per step, chunked 64"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_decode_step(args, dev):
    """The Tucker-MoE share of one decode step of the reference's language model (``pure_torch_mlx/model.py:390-397``,
    block pattern ``config.py:35-42``): 24 Mamba blocks x (x_up_proj 1536->6144; out_proj 768->768 behind its pre-norm,
    LayerScale + residual in the epilogue) and 6 transformer blocks x (ffn_gate, ffn_up 768->4608 on one normalised
    input with silu(gate)*up in the epilogue; ffn_down 4608->768 with the residual) = 66 layer calls per token, T = 1,
    the shipped ranks (r1, r2, r3) = (32, 512, 256), E = 8, top-2, every layer with its own factors (700 MB in all, so
    each call streams its factors from HBM).  The SSM / attention arithmetic between the calls is not part of this
    library: every layer gets a synthetic input of its shape.  The 66 calls are captured in one CUDA graph."""
    import mamba_tuckermoe_b200 as pkg
    from mamba_tuckermoe_b200 import _lib
    from mamba_tuckermoe_b200.synthetic import LayerShape, make_factors
    lib = _lib.load()
    dtype = torch.bfloat16

    def make(d_in, d_out, seed):
        shape = LayerShape(d_in, d_out, 8, 2, 32, 256, 512, 1e-5)
        m = pkg.TuckerMoE(d_in, d_out, pkg.TuckerMoEConfig(8, 2, 32, 512, 256, 1e-5))
        f = make_factors(shape, seed, torch.float32, 0.02)
        m.load_state_dict({"router.weight": f["router_w"], "U_in": f["U_in"], "inner_norm.weight": f["inner_norm_w"],
                           "U_expert": f["U_expert"], "core": f["core"], "U_out": f["U_out"], "bias": f["bias"]})
        return m.to(device=dev, dtype=dtype), shape

    blocks, factor_bytes, flops = [], 0, 0
    for b in range(30):
        if b % 5 < 4:
            layers = [make(1536, 6144, 5000 + 3 * b), make(768, 768, 5001 + 3 * b)]
        else:
            layers = [make(768, 4608, 5000 + 3 * b), make(768, 4608, 5001 + 3 * b), make(4608, 768, 5002 + 3 * b)]
        blocks.append([m for m, _ in layers])
        factor_bytes += sum(sh.factor_elems() * 2 for _, sh in layers)
        flops += sum(sh.flops_per_token() for _, sh in layers)
    n_calls = sum(len(b) for b in blocks)
    g = torch.Generator(device="cpu").manual_seed(77)
    x1536 = torch.randn(1, 1, 1536, generator=g).to(dev, dtype)
    x768 = torch.randn(1, 1, 768, generator=g).to(dev, dtype)
    norm_w = torch.ones(768, device=dev, dtype=dtype)
    gamma = torch.full((768,), 0.1, device=dev, dtype=dtype)

    def step():
        acc = x768
        for layers in blocks:
            if len(layers) == 2:
                layers[0](x1536)                                           # x_up_proj
                acc = pkg.fused_out_proj(layers[1], acc, (norm_w, 1e-5), gamma)   # norm -> out_proj -> residual
            else:
                acc = pkg.fused_ffn(layers[0], layers[1], layers[2], acc, (norm_w, 1e-5), gamma)
        return acc

    with torch.no_grad():
        for _ in range(3):
            y = step()
        torch.cuda.synchronize()
        launches0 = lib.tmoe_launch_count()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            y = step()
        ev1.record(); torch.cuda.synchronize()
        launches = lib.tmoe_launch_count() - launches0
        us_eager = ev0.elapsed_time(ev1) * 1e3 / args.steps
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                y = step()
            graph.replay(); side.synchronize()
            a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(side)
            for _ in range(args.steps):
                graph.replay()
            b2.record(side); side.synchronize()
            us_graph = a.elapsed_time(b2) * 1e3 / args.steps
        torch.cuda.current_stream().wait_stream(side)
    peaks = load_peaks()
    line = {
        "metric": "tucker_moe_decode_step_tokens_per_sec", "value": 1e6 / us_graph, "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": 3, "ms_per_step": us_graph / 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "decode_step: the 66 Tucker-MoE calls of one token of the reference LM (24 x {1536->6144, "
                               "768->768} + 6 x {768->4608, 768->4608, 4608->768}), T=1, E=8 top2 r=(32,256,512), one CUDA graph",
                   "layer_calls_per_token": n_calls, "l2": f"{factor_bytes / 1e6:.0f} MB of factors per token > 126 MB L2"},
        "us_per_token_graph": us_graph, "us_per_token_eager": us_eager, "us_per_layer_call_graph": us_graph / n_calls,
        "roofline": {"bound": "hbm", "kernel": "decode forward (one launch per layer call)", "achieved": factor_bytes / us_graph / 1e3,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": factor_bytes / us_graph / 1e3 / peaks["hbm_gbs"],
                     "traffic": None, "peak_source": f"{peaks['source']} (copy bandwidth)", "bytes_per_token": factor_bytes},
        "flops_per_token": flops, "gpu_launches": int(launches),
    }
    print(json.dumps(line), flush=True)


def run_ffn_pair(args, dev):
    """The feed-forward block of the reference's transformer block (``pure_torch_mlx/model.py:337-341``) at the shipped
    widths and ranks: x_res [T, 768] -> x_res + gamma * ffn_down(silu(ffn_gate(x_f)) * ffn_up(x_f)), x_f = RMSNorm(x_res),
    768 -> 4608 -> 768, E = 8 top-2, r = (32, 256, 512), T = 16384.  Times ``fused_ffn`` (gate and up in-projection / core
    stages in one launch: 5 launches) against the same three layers called one by one (6 launches)."""
    import mamba_tuckermoe_b200 as pkg
    from mamba_tuckermoe_b200 import _lib
    from mamba_tuckermoe_b200.synthetic import LayerShape, make_factors, make_tokens
    lib = _lib.load()
    dtype, T = torch.bfloat16, args.tokens if args.tokens > 0 else 16384

    def make(d_in, d_out, seed):
        shape = LayerShape(d_in, d_out, 8, 2, 32, 256, 512, 1e-5)
        m = pkg.TuckerMoE(d_in, d_out, pkg.TuckerMoEConfig(8, 2, 32, 512, 256, 1e-5))
        f = make_factors(shape, seed, torch.float32, 0.02)
        m.load_state_dict({"router.weight": f["router_w"], "U_in": f["U_in"], "inner_norm.weight": f["inner_norm_w"],
                           "U_expert": f["U_expert"], "core": f["core"], "U_out": f["U_out"], "bias": f["bias"]})
        return m.to(device=dev, dtype=dtype), shape

    (mg, sg), (mu, _), (md, sd) = make(768, 4608, 6001), make(768, 4608, 6002), make(4608, 768, 6003)
    xs = [make_tokens(T, 768, 6100 + i, dtype).to(dev) for i in range(N_INPUT_SETS)]
    nw = torch.ones(768, device=dev, dtype=dtype)
    gamma = torch.full((768,), 0.1, device=dev, dtype=dtype)

    def fused(x):
        return pkg.fused_ffn(mg, mu, md, x, (nw, 1e-5), gamma)

    def separate(x):
        gate = mg.forward_fused(x, pre_norm=(nw, 1e-5))
        act = mu.forward_fused(x, pre_norm=(nw, 1e-5), silu_gate=gate)
        return md.forward_fused(act, residual=x, layer_scale=gamma)

    res = {}
    with torch.no_grad():
        same = torch.equal(fused(xs[0]), separate(xs[0]))
        for name, fn in (("one_launch_gate_up", fused), ("separate_calls", separate)):
            for i in range(3):
                fn(xs[i % N_INPUT_SETS])
            torch.cuda.synchronize()
            n0 = lib.tmoe_launch_count()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(args.steps):
                fn(xs[i % N_INPUT_SETS])
            b.record(); torch.cuda.synchronize()
            res[name] = {"us_per_block": a.elapsed_time(b) * 1e3 / args.steps,
                         "launches_per_block": (lib.tmoe_launch_count() - n0) // args.steps}
    flops = T * (2 * sg.flops_per_token() + sd.flops_per_token())
    us = res["one_launch_gate_up"]["us_per_block"]
    peaks = load_peaks()
    print(json.dumps({
        "metric": "tucker_moe_ffn_block_tokens_per_sec", "value": T / (us * 1e-6), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": 3, "ms_per_step": us / 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"shipped_ffn_pair: FFN block 768 -> 4608 -> 768, E=8 top2 r=(32,256,512), T={T}, pre-norm, "
                               "silu(gate)*up and LayerScale residual fused"},
        "variants": res, "bit_identical": bool(same),
        "block_tflops": flops / us / 1e6, "block_frac_of_bf16_peak": flops / us / 1e6 / peaks["bf16_tflops"],
        "gpu_launches": int(res["one_launch_gate_up"]["launches_per_block"] * args.steps)}), flush=True)


def time_gathers(layer, xs, T, shape, dtype, dev, rank, world, steps, barrier, s_ms):
    """The T tokens split over the ranks (xs: this rank's inputs), forward + all-gather of y into a [T, d_out] buffer on
    every rank: NCCL in place per token chunk, and the copy-engine push into mapped peer buffers, 1 and 4 chunks each;
    then the two exchanges alone."""
    import torch.distributed as dist
    from mamba_tuckermoe_b200.sharding import PeerBuffers, sharded_forward
    Ts = T // world
    recv = (world - 1) * Ts * shape.d_out * xs[0].element_size()
    info = {"bytes_received_per_gpu": recv, "compute_only_ms": s_ms}

    def leg(name, fn):
        for i in range(2):
            fn(i)
        ms = timed_steps(fn, steps, barrier, dev, world) / steps
        info[name] = {"ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "ms_over_compute_only": ms - s_ms}

    y_all = torch.empty((T, shape.d_out), dtype=dtype, device=dev)
    for chunks in (1, 4):
        if T % (world * chunks) == 0:
            leg(f"nccl_chunks{chunks}", lambda i: sharded_forward(layer, xs[i % N_INPUT_SETS], n_tokens=T, gather=True,
                                                                  chunks=chunks, out=y_all))
    mine = y_all[rank * Ts:(rank + 1) * Ts]
    leg("nccl_alone", lambda i: dist.all_gather_into_tensor(y_all, mine))
    info["nccl_alone"]["gbs_received_per_gpu"] = recv / info["nccl_alone"]["ms_per_step"] / 1e6
    del y_all, mine
    try:
        peers = PeerBuffers(T, shape.d_out, dtype, dev)
    except RuntimeError as e:      # raised on every rank alike: the NCCL legs above stand, the peer-buffer legs are skipped
        info["peer_buffers"] = f"unavailable here: {e}"
        return info
    try:
        leg("in_kernel", lambda i: sharded_forward(layer, xs[i % N_INPUT_SETS], n_tokens=T, gather=True, peers=peers))
        for chunks in (1, 2, 4):
            leg(f"push_chunks{chunks}", lambda i: sharded_forward(layer, xs[i % N_INPUT_SETS], n_tokens=T, gather=True,
                                                                  chunks=chunks, peers=peers, in_kernel=False))
        lo = rank * Ts

        def push_alone(i):
            cur = torch.cuda.current_stream(dev)
            peers.push_stream.wait_stream(cur)
            peers.push(lo, lo + Ts)
            cur.wait_stream(peers.push_stream)
            peers.rendezvous(cur)
        leg("push_alone", push_alone)
        info["push_alone"]["gbs_received_per_gpu"] = recv / info["push_alone"]["ms_per_step"] / 1e6
    finally:
        peers.close()
    info["note"] = ("nccl_*: strong-sharded forward + in-place all_gather_into_tensor per token chunk on a side stream; push_*: "
                    "the same forward writing into a buffer that every peer has mapped, each finished chunk copied to all peers "
                    "by the copy engines (tmoe_peer_push), two one-element all-reduces as rendezvous; in_kernel: the out-projection GEMM "
                    "stores every output tile to its own and to all peers' buffers (tmoe_extras_t.peer_y), same rendezvous "
                    "(sharding.py)")
    return info


def run_strong_only(args, layer, shape, dtype, seed, T, rank, world, dev, zipf, desc):
    """The workload's T tokens split over the ranks: forward alone, then forward + NCCL all-gather of y (1 and 4 chunks)."""
    import torch.distributed as dist
    from mamba_tuckermoe_b200.sharding import sharded_forward
    from mamba_tuckermoe_b200.synthetic import make_tokens
    if T % world:
        raise SystemExit("--strong-only needs T divisible by the number of ranks")
    Ts = T // world
    xs = [make_tokens(Ts, shape.d_in, seed + 17 * rank + 1000 * i, dtype) for i in range(N_INPUT_SETS)]
    if zipf:
        for x in xs:
            x[:, 0] = 1.0
    xs = [x.to(dev) for x in xs]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    out = {}
    with torch.no_grad():
        for i in range(3):
            layer(xs[i % N_INPUT_SETS])
        s_ms = timed_steps(lambda i: layer(xs[i % N_INPUT_SETS]), args.steps, barrier, dev, world) / args.steps
        out["strong"] = {"tokens_per_gpu": Ts, "global_tokens": T, "ms_per_step": s_ms, "tokens_per_s": T / (s_ms * 1e-3)}
        if world > 1:
            out["allgather"] = time_gathers(layer, xs, T, shape, dtype, dev, rank, world, args.steps, barrier, s_ms)
    if rank == 0:
        v = out["strong"]["tokens_per_s"]
        print(json.dumps({"metric": "tucker_moe_layer_tokens_per_sec", "value": v, "unit": "tokens/s", "n_gpus": world,
                          "steps": args.steps, "warmup": 3, "ms_per_step": out["strong"]["ms_per_step"],
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                          "dtype": "bf16" if dtype == torch.bfloat16 else "f32", "data": "synthetic",
                          "config": {"workload": f"{args.workload}: {desc}", "global_tokens": T, "tokens_per_gpu": Ts,
                                     "sharding": f"{T} tokens split over {world} ranks, factors replicated"},
                          "layer_frac_of_bf16_peak": v * shape.flops_per_token() / 1e12 / world / load_peaks()["bf16_tflops"],
                          **out}), flush=True)
    if world > 1:
        dist.destroy_process_group()


SPIN_UP_STEPS = 3


def timed_steps(fn, steps, barrier, dev, world, detail=None):
    """CUDA-event time of `steps` calls of fn(i) bracketed by a barrier + synchronize on both sides; max over ranks (ms).
    SPIN_UP_STEPS untimed calls run between the opening barrier and the first event: the GPU leaves the barrier idle, and a
    region of a few milliseconds otherwise measures its way back to the working clocks (seen on 8 GPUs: 0.29 ms per step
    over 20 steps against 0.21 ms over 200).  `detail` (a dict) receives every rank's device time and the host time each
    rank spent enqueueing the steps."""
    import torch.distributed as dist
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    for i in range(SPIN_UP_STEPS):
        fn(steps - SPIN_UP_STEPS + i)
    ev0.record()
    h0 = time.perf_counter()
    for i in range(steps):
        fn(i)
    h1 = time.perf_counter()
    ev1.record()
    barrier()
    mine = torch.tensor([ev0.elapsed_time(ev1), (h1 - h0) * 1e3], dtype=torch.float64, device=dev)
    t_ms = mine[:1].clone()
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    if detail is not None:
        every = [torch.zeros_like(mine) for _ in range(world)] if world > 1 else [mine]
        if world > 1:
            dist.all_gather(every, mine)
        detail["device_ms_per_step_per_rank"] = [round(float(t[0]) / steps, 5) for t in every]
        detail["host_enqueue_ms_per_step_per_rank"] = [round(float(t[1]) / steps, 5) for t in every]
    return float(t_ms.item())


def copy_rates(x_host, y_host, x_dev, dev, world, reps=4):
    """Host<->device copy rates of this rank in GB/s, all ranks copying at the same time: [H2D alone, D2H alone, H2D and
    D2H while the other direction is busy too]."""
    import torch.distributed as dist
    y_dev = torch.empty(y_host.shape, dtype=y_host.dtype, device=dev)
    out = []
    for src, dst in ((x_host, x_dev), (y_dev, y_host)):
        dst.copy_(src, non_blocking=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            dst.copy_(src, non_blocking=True)
        b.record()
        torch.cuda.synchronize()
        out.append(src.numel() * src.element_size() * reps / (a.elapsed_time(b) * 1e-3) / 1e9)
    # both directions at once, on two streams: what a pipelined step actually gets from a full-duplex link
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev = []
    for st, src, dst in ((s_in, x_host, x_dev), (s_out, y_dev, y_host)):
        with torch.cuda.stream(st):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                dst.copy_(src, non_blocking=True)
            b.record()
            ev.append((a, b, src.numel() * src.element_size() * reps))
    torch.cuda.synchronize()
    out += [n / (a.elapsed_time(b) * 1e-3) / 1e9 for a, b, n in ev]
    rates = torch.tensor(out, dtype=torch.float64, device=dev)
    if world > 1:
        allr = [torch.zeros_like(rates) for _ in range(world)]
        dist.all_gather(allr, rates)
        return [[round(float(v), 2) for v in r] for r in allr]
    return [[round(float(v), 2) for v in rates]]


def parity_block(layer, shape, dtype, x_host0, f_typed, zipf):
    """The run's own output on a fixed token subset against the CPU oracle (outside every timed region)."""
    from oracle.parity import parity_report, subset_indices
    T = x_host0.shape[0]
    heavy = shape.r1 * shape.r3 * shape.r2 > 4 * 256 * 1024          # the largest layer costs 8x more per token on the CPU
    sub = subset_indices(T, 1024 if heavy else 4096, 1024 if heavy else 4096)
    with torch.no_grad():
        y, (idx, _, _) = layer.forward_with_routing(x_host0.to(layer.U_in.device))
    torch.cuda.synchronize()
    rep = parity_report(y[sub.to(y.device)], idx[sub.to(y.device)], x_host0[sub], f_typed, shape.top_k, shape.eps, dtype)
    rep["subset"] = f"first {min(T, 1024 if heavy else 4096)} + strided rest of one {T}-token step ({rep['tokens_checked']} tokens)"
    rep["reference"] = "CPU restatement of pure_torch_mlx/model.py:68-102 in the layer dtype; ties vs float64"
    return rep


def gpu_eager_rate(workload, dev, sample_tokens, reps=3):
    """tokens/s of the reference restatement run as eager PyTorch on this GPU (same box, no custom kernels), token-chunked
    so that the [chunk, r3, r2] intermediate of model.py:95 stays below 1 GiB."""
    from oracle.tucker_moe_oracle import BENCH_SHAPES, layer_forward, make_factors, make_tokens
    shape, _, dtype, seed, rstd = BENCH_SHAPES[WORKLOADS[workload][0]]
    f = {k: v.to(dev) for k, v in make_factors(shape, seed, dtype, rstd).items()}
    x = make_tokens(sample_tokens, shape.d_in, seed, dtype).to(dev)
    es = 2 if dtype == torch.bfloat16 else 4
    chunk = max(1, min(sample_tokens, (1 << 30) // (shape.r3 * shape.r2 * es)))
    with torch.no_grad():
        layer_forward(x, f, shape.top_k, shape.eps, chunk_tokens=chunk)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            layer_forward(x, f, shape.top_k, shape.eps, chunk_tokens=chunk)
        b.record()
        torch.cuda.synchronize()
    dt = a.elapsed_time(b) * 1e-3 / reps
    return {"value": sample_tokens / dt, "unit": "tokens/s", "kind": "reference restatement, eager PyTorch on this GPU",
            "dtype": "bf16" if dtype == torch.bfloat16 else "f32",
            "sample": f"{sample_tokens} tokens of the workload in chunks of {chunk}, mean of {reps} ({dt * 1e3:.1f} ms)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cfg2", choices=list(WORKLOADS) + ["decode_step", "shipped_ffn_pair"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=8)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--path", type=int, default=0, help="0 auto, 1 CUDA-core, 2 tensor-core")
    ap.add_argument("--allgather", type=int, default=-1,
                    help="time the strong-sharded forward followed by the NCCL all-gather of y (default: on when N > 1)")
    ap.add_argument("--profile", nargs="?", const="forward", default=None, choices=["forward", "router"],
                    help="short run for use under ncu: 'forward' = device-resident steps only (no per-kernel, e2e or CPU "
                         "legs); 'router' = the stand-alone router entry point (tmoe_router) on the workload's tokens")
    ap.add_argument("--tokens", type=int, default=0, help="override the workload's token count (profiling of small cases)")
    ap.add_argument("--strong-only", action="store_true",
                    help="N > 1: only the strong-sharded legs (the workload's T tokens split over the ranks, without and "
                         "with the all-gather of y); every rank generates just its own T/N tokens")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    rank, world, local = dist_info()
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    if args.workload == "decode_step":
        if rank == 0:
            run_decode_step(args, dev)
        return
    if args.workload == "shipped_ffn_pair":
        if rank == 0:
            run_ffn_pair(args, dev)
        return

    import mamba_tuckermoe_b200 as pkg
    from mamba_tuckermoe_b200 import _lib
    from mamba_tuckermoe_b200.synthetic import (BENCH_SHAPES, ZIPF_SHAPES, apply_zipf_router_bias, make_factors,
                                                make_tokens)

    shape_key, T, desc = WORKLOADS[args.workload]
    if args.tokens > 0:
        T = args.tokens
    shape, _, dtype, seed, rstd = BENCH_SHAPES[shape_key]
    peaks = load_peaks()
    lib = _lib.load()

    cfg = pkg.TuckerMoEConfig(shape.E, shape.top_k, shape.r1, shape.r2, shape.r3, shape.eps)
    layer = pkg.TuckerMoE(shape.d_in, shape.d_out, cfg)
    f = make_factors(shape, seed, torch.float32, rstd)
    zipf = shape_key in ZIPF_SHAPES
    if zipf:
        _, f = apply_zipf_router_bias(torch.zeros(1, shape.d_in), f, seed)
    layer.load_state_dict({"router.weight": f["router_w"], "U_in": f["U_in"], "inner_norm.weight": f["inner_norm_w"],
                           "U_expert": f["U_expert"], "core": f["core"], "U_out": f["U_out"], "bias": f["bias"]})
    layer = layer.to(device=dev, dtype=dtype)
    layer.path = args.path

    if args.strong_only:
        run_strong_only(args, layer, shape, dtype, seed, T, rank, world, dev, zipf, desc)
        return

    # this rank's token shard: seeded per rank; two of the host copies stay pinned for the end-to-end leg
    n_pinned = 2
    x_host = [make_tokens(T, shape.d_in, seed + 17 * rank + 1000 * i, dtype) for i in range(N_INPUT_SETS)]
    if zipf:
        for xh in x_host:
            xh[:, 0] = 1.0  # the constant input channel that carries the per-expert bias
    x_dev = [x.to(dev) for x in x_host]
    x_pin = [x_host[i].pin_memory() for i in range(n_pinned)]
    x_host = [x_host[0]]   # one pageable copy is kept for the parity subset
    y_host = torch.empty((T, shape.d_out), dtype=dtype).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    gather_info = strong = None
    if args.profile == "router":
        if rank == 0:
            profile_router(lib, _lib, layer, shape, dtype, x_dev, T, args.steps)
        return

    with torch.no_grad():
        for i in range(max(args.warmup, 3)):
            y = layer(x_dev[i % N_INPUT_SETS])
        torch.cuda.synchronize()
        st = pkg.read_device_status(dev)
        if st[0] != 0:
            raise RuntimeError(f"device status {st}")

        # ---------------- device-resident timing ----------------
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
            time.sleep(0.25)
        launches0 = lib.tmoe_launch_count()
        per_rank = {}
        ms_total = timed_steps(lambda i: layer(x_dev[i % N_INPUT_SETS]), args.steps, barrier, dev, world, detail=per_rank)
        # the counter also saw the untimed steps in front of the first event: every step makes the same launches
        launches = (lib.tmoe_launch_count() - launches0) * args.steps // (args.steps + SPIN_UP_STEPS)
        # the same steps replayed from a CUDA graph (one graph holds a step on each input set): what is left of a step
        # when the host's part -- Python, tensor-map encoding, four launches -- is taken out
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            layer(x_dev[0])
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for x in x_dev:
                    layer(x)
            graph.replay()
            side.synchronize()
            replays = max(1, -(-args.steps // N_INPUT_SETS))
            g_ms = timed_steps(lambda i: graph.replay(), replays, barrier, dev, world) / (replays * N_INPUT_SETS)
        torch.cuda.current_stream().wait_stream(side)
        per_rank["graph_replay"] = {"ms_per_step": g_ms, "tokens_per_s": world * T / (g_ms * 1e-3),
                                    "note": f"{replays} replays of a graph of {N_INPUT_SETS} steps, device-timed, max over ranks"}
        if rank == 0:
            time.sleep(0.15)
            clocks = sampler.stop()
        ms_step = ms_total / args.steps
        value = world * T * args.steps / (ms_total * 1e-3)

        if args.profile:
            if rank == 0:
                print(json.dumps({"profile_run": "forward", "tokens": T, "ms_per_step": ms_step, "tokens_per_s": value,
                                  "gpu_launches": int(launches)}), flush=True)
            if world > 1:
                dist.destroy_process_group()
            return

        # ---------------- strong sharding: the workload's T tokens split over the ranks ----------------
        if T % world == 0 and T // world >= 1:
            Ts = T // world
            if world == 1:
                strong = {"tokens_per_gpu": Ts, "global_tokens": T, "ms_per_step": ms_step, "tokens_per_s": value,
                          "note": "N = 1: identical to the line's own timing"}
            else:
                xs = [x[:Ts] for x in x_dev]
                for i in range(3):
                    layer(xs[i % N_INPUT_SETS])
                s_ms = timed_steps(lambda i: layer(xs[i % N_INPUT_SETS]), args.steps, barrier, dev, world) / args.steps
                strong = {"tokens_per_gpu": Ts, "global_tokens": T, "ms_per_step": s_ms, "tokens_per_s": T / (s_ms * 1e-3),
                          "note": "same T as at N = 1, T/N tokens per GPU, no collective; max over ranks"}
                # ---------------- ... followed by the all-gather of y ----------------
                want_gather = args.allgather != 0
                if want_gather:
                    gather_info = time_gathers(layer, xs, T, shape, dtype, dev, rank, world, max(5, args.steps // 4), barrier, s_ms)

        # ---------------- per-kernel timing of the two dominant kernels (stage API) ----------------
        kern = per_kernel_times(lib, _lib, layer, shape, dtype, x_dev[0], T, args.path)

        # ---------------- end to end with host buffers ----------------
        e2e_steps = max(2, min(args.e2e_steps, args.steps))
        for i in range(2):
            layer.forward_host(x_pin[i % n_pinned], out=y_host, pipelined=True)
        # the host inputs are ready before the loop and nothing reads y_host between steps: the copies of
        # consecutive steps may overlap; the closing event is recorded after the current stream has waited for the last copy out
        e_ms = timed_steps(lambda i: layer.forward_host(x_pin[i % n_pinned], out=y_host, pipelined=True), e2e_steps, barrier,
                           dev, world)
        e2e_value = world * T * e2e_steps / (e_ms * 1e-3)
        rates = copy_rates(x_pin[0], y_host, x_dev[0], dev, world)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    flops_tok = shape.flops_per_token()
    dom = kern["dominant"]
    peak_tf = peaks["bf16_tflops"]
    if dom is None:  # decode-shaped call: bound by streaming the factor set
        d = kern["decode"]
        roofline = {
            "bound": "hbm", "kernel": "small-T forward (decode kernels)" if d["resolved_path"] == 3 else "small-T forward (one tensor-core tile)", "achieved": d["gbs_cold"],
            "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": d["gbs_cold"] / peaks["hbm_gbs"], "traffic": None,
            "peak_source": f"{peaks['source']} (copy bandwidth)", "bytes_per_call": d["bytes"],
            "us_per_call_cold_l2": d["us_cold"], "us_per_call_warm": d["us_warm"], "us_per_call_graph": d["us_graph"], "us_per_call_graph_24_layers": d["us_graph_24_layers"],
        }
    else:
        tr = ncu_traffic(args.workload, dom["name"])
        roofline = {
            "bound": "tensor", "kernel": dom["name"], "achieved": dom["tflops"], "peak": peak_tf, "unit": "TFLOP/s",
            "frac": dom["tflops"] / peak_tf, "traffic": tr["bytes"] if tr else None,
            "traffic_source": (f"{tr['file']} (ncu dram read+write per launch, taken at commit {tr['commit']})" if tr else None),
            "peak_source": f"{peaks['source']} (burst bf16)",
            "flops_per_launch": dom["flops"], "us_per_launch": dom["us"],
        }
    line = {
        "metric": "tucker_moe_layer_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if dtype == torch.bfloat16 else "f32",
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: {desc}", "tokens_per_gpu": T, "global_tokens": T * world,
                   "sharding": f"tokens x{world}, factors replicated, no collective",
                   "l2": f"{N_INPUT_SETS} rotating input sets; x+z+y per step = "
                         f"{(T * (shape.d_in + 2 * shape.r2 + shape.d_out) * 2) / 1e6:.0f} MB > 126 MB L2",
                   "path": {0: "auto", 1: "cuda-core", 2: "tensor-core"}[args.path],
                   "timing": f"CUDA events around exactly {args.steps} steps; {SPIN_UP_STEPS} untimed steps run directly in front "
                             "of the first event, after the barrier"},
        "layer_tflops": value * flops_tok / 1e12 / world,
        "layer_frac_of_bf16_peak": value * flops_tok / 1e12 / world / peak_tf,
        "flops_per_token": flops_tok,
        "roofline": roofline,
        "kernels": kern["all"],
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": T * shape.d_in * x_pin[0].element_size(),
                "d2h_bytes_per_step": T * shape.d_out * y_host.element_size(), "steps": e2e_steps,
                "copy_gbs_per_rank_h2d_d2h": [r[:2] for r in rates],
                "copy_gbs_per_rank_h2d_d2h_both_at_once": [r[2:] for r in rates],
                "copy_gbs_all_ranks": [round(sum(r[0] for r in rates), 1), round(sum(r[1] for r in rates), 1)],
                "note": "copy_gbs: each direction alone / both at once, all ranks copying at once, pinned buffers"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "ranks": per_rank,
    }
    if strong:
        line["strong"] = strong
    if gather_info:
        line["allgather"] = gather_info
    if not args.no_parity:
        f_typed = {k: v.to(dtype) for k, v in f.items()}
        line["parity"] = parity_block(layer, shape, dtype, x_host[0], f_typed, zipf)
    if world == 1 and not args.no_cpu_baseline:
        rate, threads, dt = cpu_reference_rate(args.workload, min(T, 8192), 2)
        line["cpu_baseline"] = {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port",
                                "sample": f"{min(T, 8192)} tokens of the workload, best of 2 ({dt:.2f} s)"}
        if dtype == torch.bfloat16 or T <= 4096:
            line["gpu_eager_baseline"] = gpu_eager_rate(args.workload, dev, min(T, 8192))
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def profile_router(lib, _lib, layer, shape, dtype, x_dev, T, steps):
    """A few calls of the stand-alone router entry point (subsystem 1) for a profiler to capture."""
    L = _lib.layer_struct(shape, dtype)
    fd = {"router_w": layer.router.weight, "U_in": layer.U_in, "inner_norm_w": layer.inner_norm.weight,
          "U_expert": layer.U_expert, "core": layer.core, "U_out": layer.U_out, "bias": layer.bias}
    F = _lib.factors_struct(fd)
    ws = _lib.alloc_workspace(L, T, 1)
    dev = x_dev[0].device
    idx = torch.empty(T, shape.top_k, dtype=torch.int32, device=dev)
    gates = torch.empty(T, shape.top_k, dtype=torch.float32, device=dev)
    c = torch.empty(T, shape.r1, dtype=torch.float32, device=dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(steps + 1):
        if i == 1:
            a.record()
        rc = lib.tmoe_router(C.byref(L), C.byref(F), x_dev[i % len(x_dev)].data_ptr(), T, idx.data_ptr(), gates.data_ptr(),
                             c.data_ptr(), ws.data_ptr(), ws.numel(), _lib.current_stream_ptr())
        assert rc == 0, _lib.status_string(rc)
    b.record(); torch.cuda.synchronize()
    us = a.elapsed_time(b) * 1e3 / steps
    print(json.dumps({"profile_run": "router", "tokens": T, "us_per_call": us,
                      "gbs": T * shape.d_in * x_dev[0].element_size() / us / 1e3}), flush=True)


def decode_times(lib, _lib, layer, shape, dtype, x, T, reps=30):
    """Decode-shaped call (T <= 64): whole forward through tmoe_forward, CUDA events on the launching
    stream.  'cold': L2 flushed before every call, so the factors come from HBM; 'warm': back-to-back
    calls (factors L2-resident); 'graph': warm calls replayed from one CUDA graph of 20 forwards."""
    L = _lib.layer_struct(shape, dtype)
    fd = {"router_w": layer.router.weight, "U_in": layer.U_in, "inner_norm_w": layer.inner_norm.weight,
          "U_expert": layer.U_expert, "core": layer.core, "U_out": layer.U_out, "bias": layer.bias}
    F = _lib.factors_struct(fd)
    rpath = lib.tmoe_resolve_path(C.byref(L), T, 0)   # what a caller gets: decode-shaped kernels up to 8 tokens, one tensor-core tile above
    ws = _lib.alloc_workspace(L, T, rpath)
    prep = _lib.alloc_prepared(L, F)
    y = torch.empty(T, shape.d_out, dtype=dtype, device=x.device)
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=x.device)

    def call():
        rc = lib.tmoe_forward(C.byref(L), C.byref(F), prep.data_ptr(), x.data_ptr(), T, y.data_ptr(), None,
                              ws.data_ptr(), ws.numel(), rpath, _lib.current_stream_ptr())
        assert rc == 0, _lib.status_string(rc)

    for _ in range(3):
        call()
    torch.cuda.synchronize()
    cold = []
    for _ in range(reps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); call(); b.record()
        cold.append((a, b))
    torch.cuda.synchronize()
    us_cold = statistics.mean(a.elapsed_time(b) for a, b in cold) * 1e3
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        call()
    b.record(); torch.cuda.synchronize()
    us_warm = a.elapsed_time(b) * 1e3 / reps
    us_graph = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            call()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(20):
                    call()
            g.replay(); side.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(side)
            for _ in range(5):
                g.replay()
            b.record(side); side.synchronize()
            us_graph = a.elapsed_time(b) * 1e3 / 100
        torch.cuda.current_stream().wait_stream(side)
    except Exception as e:  # graph capture is a convenience measurement, not the product path
        us_graph = None
    # the same graph measurement with a different factor set per call, as in a decode step that walks through many
    # layers: 24 copies of the prepared buffer (> L2), so every call streams its factors from HBM
    us_graph_layers = None
    try:
        n_layers = 24
        preps = [prep.clone() for _ in range(n_layers)]
        wss = [_lib.alloc_workspace(L, T, rpath) for _ in range(n_layers)]

        def call_layer(i):
            rc = lib.tmoe_forward(C.byref(L), C.byref(F), preps[i].data_ptr(), x.data_ptr(), T, y.data_ptr(), None,
                                  wss[i].data_ptr(), wss[i].numel(), rpath, _lib.current_stream_ptr())
            assert rc == 0, _lib.status_string(rc)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            call_layer(0)
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, stream=side):
                for i in range(n_layers):
                    call_layer(i)
            g2.replay(); side.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(side)
            for _ in range(5):
                g2.replay()
            b.record(side); side.synchronize()
            us_graph_layers = a.elapsed_time(b) * 1e3 / (5 * n_layers)
        torch.cuda.current_stream().wait_stream(side)
    except Exception as e:
        us_graph_layers = None
    es = x.element_size()
    factor_bytes = shape.factor_elems() * es
    alg_bytes = factor_bytes + T * (shape.d_in + shape.d_out) * es
    return {"us_cold": us_cold, "us_warm": us_warm, "us_graph": us_graph, "us_graph_24_layers": us_graph_layers,
            "bytes": alg_bytes, "gbs_cold": alg_bytes / us_cold / 1e3, "resolved_path": int(rpath)}


def per_kernel_times(lib, _lib, layer, shape, dtype, x, T, path, reps=20):
    """CUDA-event time of each stage through the C-ABI stage entry points, on the current stream."""
    L = _lib.layer_struct(shape, dtype)
    rpath = lib.tmoe_resolve_path(C.byref(L), T, path)
    if rpath == 3 or T <= 64:   # small-T workloads: whole-forward timings (cold / warm / graph) through the path AUTO picks
        d = decode_times(lib, _lib, layer, shape, dtype, x, T)
        return {"all": {"decode_forward": d, "path": "decode" if d["resolved_path"] == 3 else "tensor-core"}, "dominant": None, "decode": d}
    fd = {"router_w": layer.router.weight, "U_in": layer.U_in, "inner_norm_w": layer.inner_norm.weight,
          "U_expert": layer.U_expert, "core": layer.core, "U_out": layer.U_out, "bias": layer.bias}
    F = _lib.factors_struct(fd)
    ws = _lib.alloc_workspace(L, T, rpath)
    ws_router = _lib.alloc_workspace(L, T, 1)  # the stand-alone router entry point uses the CUDA-core layout
    prep = _lib.alloc_prepared(L, F) if rpath == 2 else None
    if rpath == 1:
        path = 1
    pp = prep.data_ptr() if prep is not None else None
    zdt = torch.bfloat16 if rpath == 2 else torch.float32
    z = torch.empty(T, shape.r2, dtype=zdt, device=x.device)
    y = torch.empty(T, shape.d_out, dtype=dtype, device=x.device)
    idx = torch.empty(T, shape.top_k, dtype=torch.int32, device=x.device)
    gates = torch.empty(T, shape.top_k, dtype=torch.float32, device=x.device)
    c = torch.empty(T, shape.r1, dtype=torch.float32, device=x.device)
    st = _lib.current_stream_ptr()
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=x.device)

    def t(fn):
        fn(); torch.cuda.synchronize()
        evs = []
        for _ in range(reps):
            flush.zero_()  # evict L2 between launches
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); rc = fn(); b.record()
            assert rc == 0, _lib.status_string(rc)
            evs.append((a, b))
        torch.cuda.synchronize()
        return statistics.mean(a.elapsed_time(b) for a, b in evs) * 1e3  # us

    us_router = t(lambda: lib.tmoe_router(C.byref(L), C.byref(F), x.data_ptr(), T, idx.data_ptr(), gates.data_ptr(),
                                          c.data_ptr(), ws_router.data_ptr(), ws_router.numel(), st))
    us_incore = t(lambda: lib.tmoe_in_core(C.byref(L), C.byref(F), pp, x.data_ptr(), T, c.data_ptr(), z.data_ptr(),
                                           ws.data_ptr(), ws.numel(), rpath, st))
    us_out = t(lambda: lib.tmoe_out(C.byref(L), C.byref(F), pp, z.data_ptr(), T, y.data_ptr(), None, ws.data_ptr(),
                                    ws.numel(), rpath, st))
    f_in = T * (2 * shape.d_in * shape.r3 + 2 * shape.r3 * shape.r1 * shape.r2 + 2 * shape.r1 * shape.r2)
    f_out = T * 2 * shape.r2 * shape.d_out
    allk = {
        "router_standalone": {"us": us_router, "bytes": T * shape.d_in * x.element_size(),
                             "gbs": T * shape.d_in * x.element_size() / us_router / 1e3},
        "in_core": {"us": us_incore, "flops": f_in, "tflops": f_in / us_incore / 1e6},
        "out_gemm": {"us": us_out, "flops": f_out, "tflops": f_out / us_out / 1e6},
        "path": {1: "cuda-core", 2: "tensor-core"}[rpath],
    }
    name = "out_gemm" if us_out >= us_incore else "in_core"
    dom = dict(allk[name]); dom["name"] = ("tc_" if rpath == 2 else "simt_") + name
    return {"all": allk, "dominant": dom}


if __name__ == "__main__":
    main()
