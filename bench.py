#!/usr/bin/env python
"""Headline benchmark: end-to-end GRPO step throughput (rollout + reference log-probs + policy
update) of Qwen2.5-7B on synthetic prompts, weak scaling over the GPUs of one node.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Per GPU and step: 32 prompts of 1024 uniform random token ids, 8 samples each, response lengths
roughly uniform on [256, 2048] (EOS hazard in the sampler), rule reward "response contains token
7", group-normalised advantages, clip 0.2, KL 1e-3 against a frozen reference copy, AdamW.
Weights are random-init bf16; nothing is cached between steps.  The timed region is K calls of
the public trainer loop (``RayGRPOTrainer.fit`` with ``train_iters`` advanced by one each call),
bracketed by barrier + ``torch.cuda.synchronize()``; device time comes from CUDA events, the
maximum over ranks is reported.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
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
    ap.add_argument("--pack-tokens", type=int, default=8192, help="token budget of one training micro-batch")
    ap.add_argument("--fwd-pack-tokens", type=int, default=32768,
                    help="token budget of one forward-only micro-batch (reference log-probs)")
    ap.add_argument("--eager", action="store_true", help="disable CUDA-graph decode")
    ap.add_argument("--keep-layers", type=int, default=28,
                    help="layers whose activations stay resident (the others are fully recomputed in the backward)")
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
    dev = torch.device("cuda", local_rank)
    initialize_model_parallel(1, 1, 1)           # data parallel over all GPUs (weak scaling)

    n, gbs = args.samples, args.prompts_per_gpu * world
    max_len = args.prompt_len + args.max_response
    catalogue = load_model_catalogue([args.model])
    if args.layers:
        catalogue[args.model]["num_layers"] = args.layers
    actor = MegatronConfig(dict(
        model=args.model, global_batch_size=gbs, micro_batch_size=8, seq_length=max_len, lr=1e-6,
        lr_decay_style="constant", weight_decay=0.01, clip_grad=1.0, adam_beta1=0.9, adam_beta2=0.95,
        stage="ray_grpo", train_iters=10 ** 6, seed=1234, bf16=True, use_distributed_optimizer=True,
        recompute_granularity="full", recompute_method="block" if args.keep_layers else None,
        recompute_num_layers=max(0, (args.layers or catalogue[args.model]["num_layers"]) - args.keep_layers)
        if args.keep_layers else None, recompute_activation_function=True,
        reset_attention_mask=True, sequence_parallel=False), catalogue)
    rl = RLConfig(dict(
        n_samples_per_prompt=n, mini_batch_size=gbs, epochs=1, clip_ratio=0.2, init_kl_coef=0.001,
        kl_penalty="low_var_kl", adv_estimator="group_norm", verifier_function=["contains_token_7"],
        verifier_weight=[1.0], actor_resource={"num_gpus": world}, use_remove_padding=True,
        use_dynamic_bsz=True, max_packing_token_size=args.pack_tokens,
        ref_max_packing_token_size=args.fwd_pack_tokens, log_max_throughput=False))
    gen = GenerateConfig(dict(
        infer_tensor_parallel_size=1, max_num_seqs=args.prompts_per_gpu * n, max_model_len=max_len,
        max_num_batched_tokens=8192, kv_block_size=16, enable_prefix_caching=False,
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

    def run_steps(k: int):
        trainer.train_iters = group.get_iteration() + k
        return trainer.fit(loader)

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    run_steps(args.warmup) if args.warmup > 0 else None
    fence()
    ops.reset_launch_count()
    io_counter.reset()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fence()
    t_wall0 = time.perf_counter()
    ev0.record()
    history = run_steps(args.steps)
    ev1.record()
    fence()
    t_wall = time.perf_counter() - t_wall0
    clocks = sampler.stop()
    dev_ms = ev0.elapsed_time(ev1)
    times = torch.tensor([dev_ms, t_wall * 1e3], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = float(times[0]), float(times[1])
    launches = ops.launch_count()
    h2d, d2h = io_counter.counters()
    if rank == 0:
        tokens = sum((m["response_length/mean"] + m["prompt_length/mean"]) * gbs * n for m in history)
        value = tokens / (dev_ms / 1e3)
        e2e = tokens / (wall_ms / 1e3)
        mean_resp = sum(m["response_length/mean"] for m in history) / max(len(history), 1)
        out = {
            "metric": "rl_e2e_tokens_per_sec (rollout+ref-logprob+update, all GPUs)", "value": value,
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / max(args.steps, 1), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: uniform random prompt ids, random-init weights, rule reward (token 7)",
            "config": {"model": "Qwen2.5-7B" if args.model == "qwen25_7b" and not args.layers else
                       f"{args.model}(layers={args.layers})", "algorithm": "GRPO",
                       "global_batch": gbs, "n_samples_per_prompt": n, "seq_len": max_len,
                       "prompt_len": args.prompt_len, "response_len": f"uniform {args.min_response}-{args.max_response}",
                       "mean_response_len": mean_resp, "parallelism": f"dp{world}",
                       "tokens_per_sec_per_gpu": value / world, "layers_not_recomputed": args.keep_layers,
                       "peak_device_memory_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
                       "l2": "working set >> L2: every pass streams >= 15 GB of weights",
                       "reshard_ms_per_step": sum(m.get("timing/resharding_to_infer", 0) for m in history)
                       / max(len(history), 1) * 1e3,
                       "timing_s": {k: history[-1].get(k) for k in
                                    ("timing/rollout", "timing/reference_model", "timing/update",
                                     "timing/rule_reward", "timing/adv")}},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d // max(args.steps, 1),
                    "d2h_bytes_per_step": d2h // max(args.steps, 1)},
            "gpu_launches": launches,
        }
        print(json.dumps(out))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
