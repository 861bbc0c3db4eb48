#!/usr/bin/env python
"""Headline benchmark: end-to-end GRPO step throughput (rollout + reference log-probs + policy
update) of Qwen2.5-7B on synthetic prompts, weak scaling over the GPUs of one node.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Per GPU and step: 32 prompts of 1024 uniform random token ids, 8 samples each, response lengths
roughly uniform on [256, 2048] (EOS hazard in the sampler), rule reward "response contains token
7", group-normalised advantages, clip 0.2, KL 1e-3 against a frozen reference copy, AdamW.
Weights are random-init bf16; nothing is cached between steps.

``--layout baseline`` (default) is the co-located recipe of the reference's 7B GRPO config scaled to
the GPU count: 8 GPUs train TP4 x DP2 and roll out TP2 x DP4, 4 GPUs train TP4 and roll out
TP2 x DP2, 2 GPUs train TP2 and roll out TP1 x DP2, 1 GPU runs TP1; sequence parallelism and the
communication-fused TP linears are on whenever TP > 1, and the weights move between the two layouts
through the reshard copy-plan kernel every step.  ``--layout dp`` is pure data parallelism.

The timed region is K calls of the public trainer loop (``RayGRPOTrainer.fit`` advanced by one
iteration per call), bracketed by barrier + ``torch.cuda.synchronize()``; device time comes from
CUDA events, the maximum over ranks is reported.  One iteration takes most of a minute, so the
run also has a wall-clock budget (``--budget`` seconds from process start): it never runs more
than the requested counts, and once at least 3 warm-up steps are done it stops warming up or
timing when the next step would pass the budget (never fewer than 3 timed steps).  The counts that
actually ran are printed as ``steps`` / ``warmup`` beside ``steps_requested`` / ``warmup_requested``.
Rank 0 prints one JSON line, also when the process is told to terminate early.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import statistics
import subprocess
import sys
import tempfile
import time

T_PROCESS_START = time.time()
ROOT = os.path.dirname(os.path.abspath(__file__))

# GPUs -> (train TP, rollout TP); the remaining ranks are data parallel
BASELINE_LAYOUT = {1: (1, 1), 2: (2, 1), 4: (4, 2), 8: (4, 2)}
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen25_7b")
    ap.add_argument("--prompts-per-gpu", type=int, default=32)
    ap.add_argument("--samples", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--min-response", type=int, default=256)
    ap.add_argument("--max-response", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (development only)")
    ap.add_argument("--pack-tokens", type=int, default=8192, help="token budget of one training micro-batch per TP rank (multiplied by the training TP size)")
    ap.add_argument("--fwd-pack-tokens", type=int, default=32768,
                    help="token budget of one forward-only micro-batch (reference log-probs)")
    ap.add_argument("--eager", action="store_true", help="disable CUDA-graph decode")
    ap.add_argument("--keep-layers", type=int, default=28,
                    help="layers whose activations stay resident (the others are fully recomputed in the backward)")
    ap.add_argument("--layout", default="baseline", choices=["baseline", "dp"],
                    help="baseline: train TP4xDP2 -> rollout TP2xDP4 scaled to the GPU count; dp: data parallel only")
    ap.add_argument("--train-tp", type=int, default=None, help="override the training TP size")
    ap.add_argument("--infer-tp", type=int, default=None, help="override the rollout TP size")
    ap.add_argument("--train-ep", type=int, default=1, help="expert-parallel size of training (expert models)")
    ap.add_argument("--infer-ep", type=int, default=None,
                    help="expert-parallel size of the rollout (default: the training size; another value re-homes "
                         "the experts in the reshard plan)")
    ap.add_argument("--model-override", action="append", default=[], metavar="KEY=INT",
                    help="override an integer field of the model catalogue entry (development only)")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                    help="cpu runs the same loop on gloo ranks with fp32 weights (plumbing check only, not a benchmark)")
    ap.add_argument("--budget", type=float, default=780.0,
                    help="wall-clock seconds from process start after which no further step is started")
    return ap.parse_args()


def reference_arm(args) -> None:
    """The reference cannot run on this hardware: it is installed (``--no-deps``) under
    ``baseline/_ref`` but importing it needs tensordict / ray / torch_npu / megatron / vllm-ascend."""
    why = ("reference needs torch_npu+CANN/HCCL, megatron, mindspeed, vllm-ascend, ray and tensordict; "
           "none are installable offline (pip --no-deps install succeeded, import fails on tensordict)")
    print(json.dumps({"impl": "reference", "unavailable": why}))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = os.path.join(tempfile.gettempdir(), f"msrl_clocks_{os.getpid()}.csv")
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=self.fh, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    import torch
    import torch.distributed as dist

    from mindspeed_rl_b200 import ops
    from mindspeed_rl_b200.config import GenerateConfig, MegatronConfig, RLConfig, validate_rl_args
    from mindspeed_rl_b200.config.loader import load_model_catalogue
    from mindspeed_rl_b200.datasets.synthetic import SyntheticPromptLoader
    from mindspeed_rl_b200.obs import io_counter
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    from mindspeed_rl_b200.runtime.worker_group import SPMDWorkerGroup, spmd_init
    from mindspeed_rl_b200.trainer.grpo_trainer import RayGRPOTrainer
    from mindspeed_rl_b200.workers.integrated_worker import IntegratedWorker
    from mindspeed_rl_b200.workers.rule_reward import RuleReward

    local_rank = spmd_init()
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but the launcher started {world} process(es)")
    on_gpu = args.device == "cuda"
    dev = torch.device("cuda", local_rank) if on_gpu else torch.device("cpu")
    if args.layout == "dp":
        train_tp, infer_tp = 1, 1
    else:
        train_tp, infer_tp = BASELINE_LAYOUT.get(world, (min(world, 4), min(world, 2)))
    train_tp, infer_tp = args.train_tp or train_tp, args.infer_tp or infer_tp
    if world % train_tp or world % infer_tp:
        raise SystemExit(f"TP sizes {train_tp}/{infer_tp} do not divide {world} GPUs")
    initialize_model_parallel(train_tp, 1, 1, expert_model_parallel_size=args.train_ep,
                              moe_tp_extend_ep=bool(args.train_ep > 1 and train_tp > 1))
    parallelism = (f"train tp{train_tp} x dp{world // train_tp} (sequence parallel) -> "
                   f"rollout tp{infer_tp} x dp{world // infer_tp}") if train_tp > 1 else f"dp{world}"
    if args.train_ep > 1:
        parallelism += f", experts ep{args.train_ep} -> rollout ep{args.infer_ep or args.train_ep}"

    # micro-batches grow with the training TP size: the activations of a packed micro-batch are
    # sharded over the TP group, so per-GPU memory and per-GPU GEMM sizes stay those of TP1
    pack_tokens, fwd_pack_tokens = args.pack_tokens * train_tp, args.fwd_pack_tokens * train_tp
    n, gbs = args.samples, args.prompts_per_gpu * world
    max_len = args.prompt_len + args.max_response
    catalogue = load_model_catalogue([args.model])
    if args.layers:
        catalogue[args.model]["num_layers"] = args.layers
    for kv in args.model_override:
        key, val = kv.split("=")
        catalogue[args.model][key] = int(val)
    actor = MegatronConfig(dict(
        model=args.model, global_batch_size=gbs, micro_batch_size=8, seq_length=max_len, lr=1e-6,
        lr_decay_style="constant", weight_decay=0.01, clip_grad=1.0, adam_beta1=0.9, adam_beta2=0.95,
        stage="ray_grpo", train_iters=10 ** 6, seed=1234, bf16=True, use_distributed_optimizer=True,
        tensor_model_parallel_size=train_tp, sequence_parallel=train_tp > 1,
        expert_model_parallel_size=args.train_ep, moe_tp_extend_ep=bool(args.train_ep > 1 and train_tp > 1),
        moe_p2p_capacity_factor=2.0 if args.train_ep > 1 else 0.0,
        recompute_granularity="full", recompute_method="block" if args.keep_layers else None,
        recompute_num_layers=max(0, (args.layers or catalogue[args.model]["num_layers"]) - args.keep_layers)
        if args.keep_layers else None, recompute_activation_function=True,
        reset_attention_mask=True), catalogue)
    rl = RLConfig(dict(
        n_samples_per_prompt=n, mini_batch_size=gbs, epochs=1, clip_ratio=0.2, init_kl_coef=0.001,
        kl_penalty="low_var_kl", adv_estimator="group_norm", verifier_function=["contains_token_7"],
        verifier_weight=[1.0], actor_resource={"num_gpus": world}, use_remove_padding=True,
        use_dynamic_bsz=True, max_packing_token_size=pack_tokens,
        ref_max_packing_token_size=fwd_pack_tokens, log_max_throughput=False))
    gen = GenerateConfig(dict(
        infer_tensor_parallel_size=infer_tp, infer_expert_parallel_size=args.infer_ep or args.train_ep,
        max_num_seqs=args.prompts_per_gpu * n * infer_tp,
        max_model_len=max_len, max_num_batched_tokens=8192, kv_block_size=16, enable_prefix_caching=False,
        enforce_eager=bool(args.eager), gpu_memory_utilization=0.9, offload_train_grad=True,
        sampling_config=dict(max_tokens=args.max_response, temperature=1.0, top_k=-1, top_p=1.0, seed=None)))
    validate_rl_args(actor, actor, actor, rl, gen)
    eos = actor.padded_vocab_size - 1
    worker = IntegratedWorker(actor, rl, gen, eos_token_id=eos, pad_token_id=0, device=dev,
                              sampling_overrides=dict(eos_hazard=(args.min_response, args.max_response)))
    group = SPMDWorkerGroup(worker, num_gpus=world).initialize()
    reward = RuleReward(rl, None, actor)
    trainer = RayGRPOTrainer(group, reward_list=[reward], train_iters=0, save_interval=0,
                             adv_estimator="group_norm", kl_penalty="low_var_kl", init_kl_coef=0.001,
                             global_batch_size=gbs, n_samples_per_prompt=n, pad_token_id=0)
    loader = iter(SyntheticPromptLoader(gbs, args.prompt_len, actor.padded_vocab_size - 1, seed=1234))

    def run_step():
        trainer.train_iters = group.get_iteration() + 1
        return trainer.fit(loader)

    def fence():
        if world > 1:
            dist.barrier()
        if on_gpu:
            torch.cuda.synchronize()

    agree = torch.zeros(2, device=dev, dtype=torch.float64)

    def agreed(elapsed: float, last: float):
        """Every rank must take the same stop / go decision: use the maxima over ranks."""
        agree[0], agree[1] = elapsed, last
        if world > 1:
            dist.all_reduce(agree, op=dist.ReduceOp.MAX)
        return float(agree[0]), float(agree[1])

    def tokens_of(history):
        return sum((m["response_length/mean"] + m["prompt_length/mean"]) * gbs * n for m in history)

    state = {"history": [], "step_wall": [], "warmup": 0, "clocks": None, "done": False, "t0": None}

    def report(partial: bool, dev_ms=None, wall_ms=None, launches=None, io=(0, 0)):
        history, k = state["history"], len(state["history"])
        if rank != 0 or k == 0:
            return
        if wall_ms is None:
            wall_ms = sum(state["step_wall"][:k]) * 1e3
        if dev_ms is None:
            dev_ms = wall_ms
        tokens = tokens_of(history)
        value = tokens / (dev_ms / 1e3)
        mean = lambda key: sum(m.get(key, 0) or 0 for m in history) / k
        out = {
            "metric": "rl_e2e_tokens_per_sec (rollout+ref-logprob+update, all GPUs)", "value": value,
            "unit": "tokens/s", "n_gpus": world, "steps": k, "warmup": state["warmup"],
            "steps_requested": args.steps, "warmup_requested": args.warmup,
            "ms_per_step": dev_ms / k, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if on_gpu else "fp32 (cpu plumbing check)",
            "data": "synthetic: uniform random prompt ids, random-init weights, rule reward (token 7)",
            "config": {"model": "Qwen2.5-7B" if args.model == "qwen25_7b" and not args.layers and not args.model_override else
                       f"{args.model}(layers={args.layers})", "algorithm": "GRPO",
                       "global_batch": gbs, "n_samples_per_prompt": n, "seq_len": max_len,
                       "prompt_len": args.prompt_len, "response_len": f"uniform {args.min_response}-{args.max_response}",
                       "mean_response_len": mean("response_length/mean"), "parallelism": parallelism,
                       "layout": args.layout, "train_tp": train_tp, "rollout_tp": infer_tp,
                       "update_micro_batch_tokens": pack_tokens, "forward_micro_batch_tokens": fwd_pack_tokens,
                       "tokens_per_sec_per_gpu": value / world, "layers_not_recomputed": args.keep_layers,
                       "peak_device_memory_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1) if on_gpu else None,
                       "l2": "working set >> L2: every pass streams >= 3.8 GB of weights per GPU",
                       "budget_s": args.budget,
                       # the weight move alone: device time (CUDA events) of barrier + copy-plan kernel + barrier
                       "reshard_ms_per_step": mean("timing/resharding_device") * 1e3,
                       "kv_cache_alloc_ms_per_step": mean("timing/resharding_kv_cache") * 1e3,
                       "resharding_to_infer_host_ms_per_step": mean("timing/resharding_to_infer") * 1e3,
                       "step_wall_s": [round(t, 2) for t in state["step_wall"][:k]],
                       "timing_s": {key: round(mean(key), 3) for key in
                                    ("timing/rollout", "timing/reference_model", "timing/update",
                                     "timing/rule_reward", "timing/adv")}},
            "clocks": state["clocks"],
            "e2e": {"value": tokens / (wall_ms / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": io[0] // k, "d2h_bytes_per_step": io[1] // k},
            "gpu_launches": launches,
        }
        if partial:
            out["partial"] = "terminated before the requested steps finished; wall-clock times of the steps completed"
        print(json.dumps(out), flush=True)

    def on_term(signum, frame):
        if not state["done"]:
            state["done"] = True
            if state["clocks"] is None and state.get("sampler") is not None:
                state["clocks"] = state["sampler"].stop()
            report(partial=True)
        os._exit(0 if state["history"] else 143)

    signal.signal(signal.SIGTERM, on_term)

    # ---- warm-up: at least 3 steps when 3 or more were asked for; further ones only while all the
    # requested timed steps would still fit the budget
    last = 0.0
    while state["warmup"] < args.warmup:
        t = time.perf_counter()
        run_step()
        fence()
        state["warmup"] += 1
        elapsed, last = agreed(time.time() - T_PROCESS_START, time.perf_counter() - t)
        if rank == 0:
            print(f"[bench] warm-up step {state['warmup']}: {last:.1f} s (elapsed {elapsed:.0f} s)",
                  file=sys.stderr, flush=True)
        if state["warmup"] >= 3 and elapsed + (1 + args.steps) * last * 1.1 > args.budget:
            break
    fence()
    ops.reset_launch_count()
    io_counter.reset()
    state["sampler"] = sampler = ClockSampler(local_rank)
    if on_gpu:
        sampler.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fence()
    t_wall0 = time.perf_counter()
    if on_gpu:
        ev0.record()
    # ---- timed region
    while len(state["history"]) < args.steps:
        t = time.perf_counter()
        hist = run_step()
        dt = time.perf_counter() - t
        state["step_wall"].append(dt)
        if rank == 0:
            state["history"].extend(hist)
            print(f"[bench] timed step {len(state['history'])}: {dt:.1f} s, "
                  f"{tokens_of(hist) / dt:.0f} tokens/s", file=sys.stderr, flush=True)
        else:
            state["history"].append({})
        elapsed, last = agreed(time.time() - T_PROCESS_START, dt)
        if len(state["history"]) >= min(3, args.steps) and len(state["history"]) < args.steps \
                and elapsed + 1.15 * last > args.budget:
            break
    if on_gpu:
        ev1.record()
    fence()
    t_wall = time.perf_counter() - t_wall0
    state["done"] = True
    state["clocks"] = sampler.stop()
    dev_ms = ev0.elapsed_time(ev1) if on_gpu else t_wall * 1e3
    times = torch.tensor([dev_ms, t_wall * 1e3], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    report(False, float(times[0]), float(times[1]), ops.launch_count(), io_counter.counters())
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
