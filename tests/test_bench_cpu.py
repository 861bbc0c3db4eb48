"""The benchmark driver's contract, checked on CPU (gloo ranks, tiny model): the baseline layout
(training TP != rollout TP with a reshard every step), the JSON line, and the wall-clock budget that
cuts warm-up and timed steps short without going below three of each."""
import json
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = ["--device", "cpu", "--model", "tiny_qwen2", "--prompts-per-gpu", "4", "--samples", "2", "--prompt-len", "16",
        "--min-response", "4", "--max-response", "12", "--pack-tokens", "128", "--fwd-pack-tokens", "256"]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _bench(n: int, *extra: str) -> dict:
    cmd = [sys.executable]
    if n > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
                "--master-port", str(_free_port())]
    cmd += [os.path.join(ROOT, "bench.py"), "--gpus", str(n), *TINY, *extra]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert res.returncode == 0 and len(lines) == 1, (res.stdout + res.stderr)[-3000:]
    return json.loads(lines[0])


def test_bench_baseline_layout_two_ranks():
    out = _bench(2, "--steps", "2", "--warmup", "1")
    assert out["n_gpus"] == 2 and out["steps"] == 2 and out["warmup"] == 1
    assert out["config"]["train_tp"] == 2 and out["config"]["rollout_tp"] == 1
    assert "rollout tp1 x dp2" in out["config"]["parallelism"]
    assert out["value"] > 0 and out["e2e"]["value"] > 0 and out["higher_is_better"] is True
    assert len(out["config"]["step_wall_s"]) == 2


def test_bench_budget_cuts_counts_but_keeps_three():
    out = _bench(1, "--steps", "6", "--warmup", "5", "--budget", "1")
    assert out["steps_requested"] == 6 and out["warmup_requested"] == 5
    assert out["steps"] == 3 and out["warmup"] == 3


def test_bench_reference_arm_reports_unavailable():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"],
                         capture_output=True, text=True, timeout=120, cwd=ROOT)
    out = json.loads(res.stdout.strip().splitlines()[-1])
    assert res.returncode == 0 and out["impl"] == "reference" and "unavailable" in out


def test_bench_baseline_layout_eight_ranks():
    """The headline layout of the 8-GPU run: training TP4 x DP2 resharded to rollout TP2 x DP4 every step."""
    out = _bench(8, "--steps", "1", "--warmup", "1", "--model-override", "num_query_groups=4")
    assert out["n_gpus"] == 8 and out["config"]["train_tp"] == 4 and out["config"]["rollout_tp"] == 2
    assert out["config"]["parallelism"].startswith("train tp4 x dp2") and out["value"] > 0


def test_bench_expert_parallel_model_with_rehomed_rollout():
    """An expert model through the benchmark driver: training EP2, rollout with every expert on each rank."""
    out = _bench(2, "--layout", "dp", "--steps", "1", "--warmup", "1", "--train-ep", "2", "--infer-ep", "1",
                 "--model-override", "num_experts=4", "--model-override", "moe_router_topk=2",
                 "--model-override", "moe_ffn_hidden_size=16")
    assert out["n_gpus"] == 2 and "experts ep2 -> rollout ep1" in out["config"]["parallelism"] and out["value"] > 0
