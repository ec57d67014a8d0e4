"""Host-side pieces of bench.py that need no GPU: the reference arm's line, the traffic figures it reads from the profile
summaries, the peaks it divides by."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_reference_arm_prints_one_contract_line():
    """`bench.py --impl reference` times the CPU restatement of the reference layer on a bounded sample and prints the
    benchmark line with impl = reference, its own cpu_baseline block and an e2e block without copies."""
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "cfg0",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for k in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert k in line, k
    assert line["impl"] == "reference" and line["metric"] == "tucker_moe_layer_tokens_per_sec" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["dtype"] == "f32" and "workload" in line["config"]


def test_traffic_figures_come_from_the_profile_summaries():
    import bench
    for kernel in ("tc_out_gemm", "tc_in_core"):
        t = bench.ncu_traffic("cfg2", kernel)
        assert t is not None and t["bytes"] > 50_000_000 and t["file"].startswith("profiles/") and t["commit"]
        assert os.path.exists(os.path.join(ROOT, t["file"]))
    assert bench.ncu_traffic("cfg2", "no_such_kernel") is None
    peaks = bench.load_peaks()
    assert peaks["source"] in ("measured", "fallback") and 3000 < peaks["hbm_gbs"] < 9000 and 800 < peaks["bf16_tflops"] < 2500
    assert bench.SPIN_UP_STEPS >= 0 and "cfg2" in bench.WORKLOADS and "cfg4" in bench.WORKLOADS


def test_reference_arm_under_a_two_rank_launch_prints_once():
    """Launched the way the multi-GPU arm is (one process per rank), rank 0 alone times and prints; the others exit 0."""
    port = 29600 + os.getpid() % 300
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "bench.py"),
                          "--impl", "reference", "--gpus", "2", "--workload", "cfg0", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["value"] > 0
