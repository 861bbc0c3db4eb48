#!/usr/bin/env python
"""DPO training entry point (no rollout, plain ``torchrun`` SPMD).

    torchrun --nproc-per-node N cli/train_dpo.py --config-name dpo_qwen3_30b_a3b_b200

The YAML's ``megatron_training`` section holds model / parallel / optimiser / data options
(``is_pairwise_dataset: true``, ``dpo_loss_type``, ``ref_model``).  Reference: ``cli/train_dpo.py:69-145``.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

from mindspeed_rl_b200.checkpoint.mcore import load_checkpoint, save_checkpoint  # noqa: E402
from mindspeed_rl_b200.config import MegatronConfig, load_config  # noqa: E402
from mindspeed_rl_b200.datasets import InfiniteLoader, PromptDataLoader, PromptDataset, build_train_valid_test_datasets  # noqa: E402
from mindspeed_rl_b200.models.gpt import GPTModel  # noqa: E402
from mindspeed_rl_b200.models.transformer_config import TransformerConfig  # noqa: E402
from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer, OptimizerParamScheduler  # noqa: E402
from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel  # noqa: E402
from mindspeed_rl_b200.parallel.state import initialize_model_parallel  # noqa: E402
from mindspeed_rl_b200.parallel.tp_comm import TPComm  # noqa: E402
from mindspeed_rl_b200.runtime.launch import build_tokenizer  # noqa: E402
from mindspeed_rl_b200.runtime.worker_group import spmd_init  # noqa: E402
from mindspeed_rl_b200.trainer.dpo_trainer import DPOTrainer  # noqa: E402


def main(argv=None):
    config = load_config(argv, default_name="dpo_qwen3_30b_a3b_b200")
    mc = MegatronConfig(config.get("megatron_training"), config.get("model"))
    local_rank = spmd_init(mc.distributed_backend if torch.cuda.is_available() else "gloo")
    ps = initialize_model_parallel(mc.tensor_model_parallel_size, mc.pipeline_model_parallel_size,
                                   mc.context_parallel_size, mc.expert_model_parallel_size, mc.moe_tp_extend_ep)
    device = torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    comm = TPComm(ps.group("tp"), mc.sequence_parallel, world_size=ps.size("tp"), rank=ps.rank_in("tp"))
    tcfg = TransformerConfig.from_megatron(mc, params_dtype=dtype)
    core = GPTModel(tcfg, comm, device=device, seed=mc.seed)
    model = DistributedDataParallel(core, ps.group("dp_cp"), ps.size("dp_cp"))
    opt = DistributedOptimizer(model.buffers, lr=mc.lr or 5e-7, betas=(mc.adam_beta1, mc.adam_beta2),
                               weight_decay=mc.weight_decay, clip_grad=mc.clip_grad, dp_group=ps.group("dp_cp"),
                               dp_rank=ps.rank_in("dp_cp"), model_parallel_group=ps.group("mp"),
                               offload_to_host=bool(mc.swap_optimizer))
    iters = mc.train_iters or 1
    sch = OptimizerParamScheduler(opt, mc.lr or 5e-7, mc.min_lr or 0.0,
                                  int((mc.lr_warmup_fraction or 0) * iters * mc.global_batch_size),
                                  iters * mc.global_batch_size, mc.lr_decay_style or "constant")
    if mc.load:
        load_checkpoint(mc.load, core, opt, sch, ps, mc)
    ref = GPTModel(tcfg, comm, device=device, seed=mc.seed)
    ref.load_state_dict(core.state_dict())
    if mc.ref_model:
        load_checkpoint(mc.ref_model, ref, None, None, ps, mc, strict=False)
    for p in ref.parameters():
        p.requires_grad_(False)
    tokenizer = build_tokenizer(mc)
    extra = type("A", (), dict(is_pairwise_dataset=True, dataset_additional_keys=[], max_prompt_length=None))()
    train, _, _ = build_train_valid_test_datasets(mc.data_path, mc.split or "100,0,0", mc.seq_length,
                                                  [iters * mc.global_batch_size, 0, 0], PromptDataset, tokenizer,
                                                  no_shuffle=mc.no_shuffle, seed=mc.seed, extra_param=extra)
    # every rank draws the same global batches (same seed); the trainer keeps this replica's slice of the pairs
    loader = InfiniteLoader(PromptDataLoader(train, mc.global_batch_size, 0, mc.seed, no_shuffle=mc.no_shuffle,
                                             is_pairwise_dataset=True, tokenizer=getattr(tokenizer, "tokenizer", None)))
    trainer = DPOTrainer(model, ref, opt, sch, beta=mc.dpo_beta, loss_type=mc.dpo_loss_type, train_iters=iters, device=device,
                         pad_multiple=ps.size("tp") * ps.size("cp"), log_interval=mc.log_interval or 1,
                         dp_group=ps.group("dp_cp"), dp_rank=ps.rank_in("dp_cp"), dp_size=ps.size("dp_cp"),
                         save_fn=(lambda it: save_checkpoint(mc.save, it, core, opt, sch, ps, mc)) if mc.save else None,
                         save_interval=mc.save_interval or 0)
    hist = trainer.train(loader)
    if dist.is_initialized():
        dist.barrier()
    return hist


if __name__ == "__main__":
    main()
