"""Assembly of a complete RL run from a composed YAML config (shared by ``cli/train_*.py``).

Steps (reference: ``cli/train_grpo.py:42-224``): parse + validate the config sections, bring up
``torch.distributed`` and the parallel state, build the tokenizer, the co-located actor worker
group (actor + reference + rollout engine), optional critic / reward-model groups, the rule-reward
workers, the dataset and prompt loader (fast-forwarded to the checkpoint's consumed samples) and
finally the trainer, then ``fit``.

Launch with ``torchrun --nproc-per-node N cli/train_grpo.py --config-name <yaml>`` (one process
per GPU) or plain ``python`` for a single GPU / CPU run.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ..config import load_config, parse_training_config
from ..obs.loggers import Loggers
from ..parallel.state import initialize_model_parallel, set_parallel_state
from ..utils.tokenizer import get_tokenizer
from .placement import plan_placement
from .worker_group import SPMDWorkerGroup, spmd_init

logger = Loggers("launch")


def apply_runtime_env(path: Optional[str]) -> None:
    """Export the variables of ``configs/envs/runtime_env.yaml`` (``env_vars:`` mapping)."""
    if not path or not os.path.isfile(path):
        return
    import yaml

    env = (yaml.safe_load(open(path)) or {}).get("env_vars", {}) or {}
    for k, v in env.items():
        os.environ.setdefault(str(k), str(v))


def build_tokenizer(actor_config):
    ttype = actor_config.tokenizer_type or "PretrainedFromHF"
    if ttype in ("Identity", "IdentityTokenizer", "NullTokenizer"):
        return get_tokenizer("", "Identity", vocab_size=actor_config.padded_vocab_size)
    return get_tokenizer(actor_config.tokenizer_name_or_path, "HuggingFaceTokenizer", actor_config.prompt_type,
                         actor_config.prompt_type_path, use_fast=not actor_config.tokenizer_not_use_fast,
                         padding_side=actor_config.tokenizer_padding_side)


def build_data_iter(actor_config, rl_config, tokenizer, consumed_train_samples: int = 0, reiterable: bool = False):
    """Prompt loader over the packed dataset at ``data_path`` (or synthetic prompts when
    ``data_path`` is ``synthetic:<prompt_len>``)."""
    from ..datasets import InfiniteLoader, PromptDataLoader, PromptDataset, build_train_valid_test_datasets
    from ..datasets.synthetic import SyntheticPromptLoader

    gbs = actor_config.global_batch_size
    path = actor_config.data_path
    if isinstance(path, str) and path.startswith("synthetic"):
        plen = int(path.split(":")[1]) if ":" in path else rl_config.max_prompt_length
        loader = SyntheticPromptLoader(gbs, plen, actor_config.padded_vocab_size - 1, seed=actor_config.seed,
                                       with_labels="labels" in (actor_config.dataset_additional_keys or []))
        return loader if reiterable else iter(loader)
    samples = [(actor_config.train_iters or 1) * gbs, 0, 0]
    extra = type("DatasetArgs", (), dict(
        is_pairwise_dataset=actor_config.is_pairwise_dataset,
        dataset_additional_keys=actor_config.dataset_additional_keys,
        max_prompt_length=rl_config.max_prompt_length, prompt_type=actor_config.prompt_type,
        prompt_type_path=actor_config.prompt_type_path))()
    is_leader = not dist.is_initialized() or dist.get_rank() == 0
    barrier = dist.barrier if dist.is_initialized() and dist.get_world_size() > 1 else None
    train, _, _ = build_train_valid_test_datasets(
        path, actor_config.split or "100,0,0", rl_config.max_prompt_length, samples, PromptDataset, tokenizer,
        full_shuffle_instruction_dataset=actor_config.full_shuffle_instruction_dataset,
        no_shuffle=actor_config.no_shuffle, seed=actor_config.seed, extra_param=extra, is_leader=is_leader,
        barrier=barrier)
    loader = PromptDataLoader(train, gbs, actor_config.num_workers or 0, actor_config.seed,
                              actor_config.dataset_additional_keys, actor_config.no_shuffle,
                              consumed_samples=consumed_train_samples)
    return loader if reiterable else InfiniteLoader(loader)


def build_mm_data_iter(actor_config, rl_config, tokenizer):
    """Prompt iterator of a vision-language run (``datasets.multimodal_dataset``); only the driver reads it."""
    from ..datasets.image_processor import ImageProcessor
    from ..datasets.multimodal_dataset import MultiModalDataset, MultiModalPromptLoader

    proc = ImageProcessor(actor_config.patch_size, actor_config.spatial_merge_size)
    ds = MultiModalDataset(actor_config.data_path, tokenizer, proc, max_prompt_length=rl_config.max_prompt_length,
                           image_token_id=actor_config.image_token_id,
                           vision_start_token_id=actor_config.vision_start_token_id,
                           vision_end_token_id=actor_config.vision_end_token_id, truncation="left")
    return iter(MultiModalPromptLoader(ds, actor_config.global_batch_size, actor_config.seed or 0,
                                       shuffle=not actor_config.no_shuffle))


def role_parallel_state(mc, placement, role: str, rank: int):
    """Process groups of a role that owns a rank range of its own.  Collective over the whole job:
    every rank creates every group, the members keep them."""
    from ..parallel.state import ParallelState, RankLayout

    ranks = placement.of(role)
    layout = RankLayout(len(ranks), mc.tensor_model_parallel_size or 1, mc.pipeline_model_parallel_size or 1,
                        mc.context_parallel_size or 1, mc.expert_model_parallel_size or 1,
                        bool(mc.moe_tp_extend_ep), bool(mc.use_tp_pp_dp_mapping))
    return ParallelState(layout, rank - ranks[0], rank_offset=ranks[0])


def run_rl(config: Dict[str, Any], algorithm: str) -> Any:
    """``algorithm`` in {"grpo", "dapo", "ppo"}; returns the metric history of rank 0."""
    from ..trainer.dapo_trainer import RayDAPOTrainer
    from ..trainer.grpo_trainer import RayGRPOTrainer
    from ..trainer.ppo_trainer import RayPPOTrainer
    from ..workers.integrated_worker import IntegratedWorker
    from ..workers.model_workers import CriticWorker, ReferenceWorker, RewardWorker
    from ..workers.rule_reward import RuleReward

    cfg = parse_training_config(config, with_critic=(algorithm == "ppo"))
    actor_config, rl_config, generate_config = cfg["actor_config"], cfg["rl_config"], cfg["generate_config"]
    apply_runtime_env(rl_config.runtime_env_path)
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    spmd_init(actor_config.distributed_backend if torch.cuda.is_available() else "gloo")
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    # which ranks run which role: all on the actor's ranks (co-located) or on ranges of their own
    placement = plan_placement(world, rl_config, torch.cuda.device_count() or None)
    disjoint = placement.disjoint_roles()
    states = {"actor": initialize_model_parallel(
        actor_config.tensor_model_parallel_size, actor_config.pipeline_model_parallel_size,
        actor_config.context_parallel_size, actor_config.expert_model_parallel_size,
        actor_config.moe_tp_extend_ep, actor_config.use_tp_pp_dp_mapping,
        world_size=len(placement.of("actor")), rank=rank)}
    role_configs = {"reference": cfg["ref_config"], "reward": cfg.get("reward_config"),
                    "critic": cfg.get("critic_config")}
    for role, mc in role_configs.items():
        if role in placement.ranks and mc is not None:
            # every rank of the job takes part in creating the role's process groups
            states[role] = role_parallel_state(mc, placement, role, rank)
            if placement.contains(role, rank):
                set_parallel_state(states[role])      # model code on this rank sees its own role's groups
    tokenizer = build_tokenizer(actor_config)
    eos = tokenizer.eod if tokenizer.eod is not None else actor_config.padded_vocab_size - 1
    pad = tokenizer.pad if tokenizer.pad is not None else 0
    own_ref_ranks = "reference" in placement.ranks
    with_ref = algorithm != "dapo"
    worker = None
    if placement.contains("actor", rank):
        worker = IntegratedWorker(actor_config, rl_config, generate_config, eos_token_id=eos, pad_token_id=pad,
                                  ref_config=cfg["ref_config"], with_reference=with_ref and not own_ref_ranks,
                                  external_reference=with_ref and own_ref_ranks)
        worker._state = states["actor"]
    from ..obs.profiler import TensorDump, enable_range_markers, seed_all

    prof_cfg = (cfg.get("profiler_config") or {}).get("integrated")
    enable_range_markers(bool(getattr(prof_cfg, "mstx", False)))
    if worker is not None:
        worker.profiler_config = prof_cfg
        if cfg.get("msprobe_config") is not None and getattr(cfg["msprobe_config"], "msprobe", False):
            worker.tensor_dump = TensorDump(cfg["msprobe_config"])
            worker.tensor_dump.save_configs({"actor": actor_config, "rl": rl_config, "generate": generate_config})
    seed_all(actor_config.seed or 1234, deterministic=bool(getattr(actor_config, "npu_deterministic", False)
                                                             or getattr(actor_config, "use_deterministic", False)))
    actor_group = SPMDWorkerGroup(worker, ranks=placement.of("actor"), overlapping=disjoint).initialize()
    actor_group.rl_config, actor_group.megatron_config = rl_config, actor_config
    if worker is not None and rl_config.multi_turn_enable:
        worker.attach_tools(tokenizer)
    if worker is not None and actor_config.load:
        from ..checkpoint.mcore import load_checkpoint

        it, consumed = load_checkpoint(actor_config.load, worker.model.module, worker.optimizer, worker.scheduler,
                                       worker.parallel_state, actor_config)
        worker.iteration, worker.consumed_train_samples = it, consumed
        if worker.ref_model is not None:
            worker.ref_model.load_state_dict(worker.model.module.state_dict())

    def role_group(role: str, cls, mc, **kw):
        """Worker group of a stand-alone role: on the role's own ranks, or on the actor's."""
        def factory():
            w = cls(mc, rl_config, generate_config, pad_token_id=pad, **kw)
            w._state = states.get(role, states["actor"])
            w.profiler_config = prof_cfg
            if cfg.get("msprobe_config") is not None and getattr(cfg["msprobe_config"], "msprobe", False):
                w.tensor_dump = TensorDump(cfg["msprobe_config"])
            return w
        return SPMDWorkerGroup(factory=factory, ranks=placement.of(role), overlapping=disjoint).initialize()

    ref_group = role_group("reference", ReferenceWorker, cfg["ref_config"]) if (with_ref and own_ref_ranks) else None
    rewards = []
    if rl_config.reward_resource:
        rewards.append(role_group("reward", RewardWorker, cfg["reward_config"]))
    if rl_config.rule_reward:
        rewards.append(RuleReward(rl_config, tokenizer, actor_config))
    common = dict(
        train_iters=actor_config.train_iters, save_interval=actor_config.save_interval or 0,
        gamma=rl_config.gamma, lam=rl_config.lam, adv_estimator=rl_config.adv_estimator,
        kl_penalty=rl_config.kl_penalty, kl_ctrl_type=rl_config.kl_ctrl_type, kl_horizon=rl_config.kl_horizon,
        kl_target=rl_config.kl_target, init_kl_coef=rl_config.init_kl_coef,
        global_batch_size=actor_config.global_batch_size, micro_batch_size=actor_config.micro_batch_size,
        n_samples_per_prompt=rl_config.n_samples_per_prompt, tokenizer=tokenizer,
        dataset_additional_keys=actor_config.dataset_additional_keys, blocking=rl_config.blocking,
        guarantee_order=rl_config.guarantee_order, num_cpus_for_local_task=rl_config.num_cpus_for_local_task,
        partial_rollout_max_split=rl_config.partial_rollout_max_split, use_kl_in_reward=rl_config.use_kl_in_reward,
        use_tensorboard=rl_config.use_tensorboard, use_wandb=rl_config.use_wandb, use_swanlab=rl_config.use_swanlab,
        wandb_project=rl_config.wandb_project, wandb_exp_name=rl_config.wandb_exp_name,
        wandb_save_dir=rl_config.wandb_save_dir, swanlab_project=rl_config.swanlab_project,
        swanlab_exp_name=rl_config.swanlab_exp_name, swanlab_save_dir=rl_config.swanlab_save_dir,
        swanlab_mode=rl_config.swanlab_mode, pad_token_id=pad)
    consumed = actor_group.get_consumed_train_samples()
    vit_group = None
    if rl_config.is_multimodal:
        # vision-language run: the vision tower is a stage of its own (on the actor's ranks, or on
        # ``vit_resource``), the prompts come from the multimodal dataset
        from ..workers.vit_worker import VitWorker

        def vit_factory():
            w = VitWorker(cfg.get("vit_config"), rl_config, actor_config.hidden_size)
            w._state = states["actor"] if placement.colocated("vit", "actor") else None
            return w
        vit_group = SPMDWorkerGroup(factory=vit_factory, ranks=placement.of("vit"), overlapping=disjoint).initialize()
    if algorithm == "grpo":
        trainer = RayGRPOTrainer(actor_group, ref_worker=ref_group, reward_list=rewards, vit_worker=vit_group, **common)
        data = build_mm_data_iter(actor_config, rl_config, tokenizer) if rl_config.is_multimodal else \
            build_data_iter(actor_config, rl_config, tokenizer, consumed)
    elif algorithm == "dapo":
        trainer = RayDAPOTrainer(actor_group, reward_list=rewards, **common)
        data = build_data_iter(actor_config, rl_config, tokenizer, consumed, reiterable=True)
    elif algorithm == "ppo":
        critic_group = role_group("critic", CriticWorker, cfg["critic_config"],
                                  offload_between_stages=bool(generate_config.offload_train_param)
                                  and placement.colocated("critic", "actor"))
        trainer = RayPPOTrainer(actor_group, ref_worker=ref_group, reward_list=rewards, critic_worker=critic_group,
                                **common)
        data = build_data_iter(actor_config, rl_config, tokenizer, consumed)
    else:
        raise ValueError(f"unknown algorithm '{algorithm}'")
    history = trainer.fit(data)
    if dist.is_initialized():
        dist.barrier()
    return history


def main(algorithm: str, default_config: str, argv=None):
    config = load_config(argv, default_name=default_config)
    return run_rl(config, algorithm)
