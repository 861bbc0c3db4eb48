"""Co-located actor worker: training model + frozen reference + rollout engine on one GPU.

Stages (each loops "pull from the experience store -> compute -> write back" until the store
says the stage has consumed everything; reference: ``workers/actor_hybrid_worker.py:114-869``,
``workers/integrated_worker.py:27-287``):

* ``generate_sequences``      -- enter infer mode (reshard), rollout, exit infer mode
* ``compute_ref_log_prob``    -- frozen reference forward
* ``compute_log_prob``        -- actor forward (old log-probs)
* ``update``                  -- policy update
* ``save_checkpoint`` / ``get_iteration`` / ``get_consumed_train_samples``
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..models.gpt import GPTModel
from ..models.training_engine import TrainingEngine
from ..models.transformer_config import TransformerConfig
from ..optim.optimizer_config import OptimizerConfig
from ..parallel.ddp import DistributedDataParallel, expert_replica_groups
from ..parallel.state import get_parallel_state
from ..parallel.tp_comm import TPComm
from ..reshard.sharding_manager import ShardingManager
from ..rollout.engine import LLMEngine
from ..rollout.scheduler import SamplingParams
from .base_worker import BaseWorker, profiled_stage


def _now() -> float:
    return time.time()


class IntegratedWorker(BaseWorker):
    def __init__(self, actor_config, rl_config, generate_config, td=None, *, eos_token_id: int = -1,
                 pad_token_id: int = 0, device=None, ref_config=None, with_reference: bool = True,
                 sampling_overrides: Optional[dict] = None, seed: Optional[int] = None,
                 external_reference: bool = False):
        super().__init__(td, pad_token_id)
        self.actor_config, self.rl_config, self.generate_config = actor_config, rl_config, generate_config
        self.ref_config = ref_config or actor_config
        self.with_reference = with_reference
        # a reference worker on other ranks writes ``ref_log_prob``: the update consumes it although
        # this worker holds no reference model itself
        self.uses_ref_log_prob = with_reference or external_reference
        self.eos_token_id = eos_token_id
        self.device = torch.device(device if device is not None
                                   else ("cuda" if torch.cuda.is_available() else "cpu"))
        self.sampling_overrides = sampling_overrides or {}
        self.seed = actor_config.seed if seed is None else seed
        self.iteration = 0
        self.consumed_train_samples = 0
        self.initialized = False

    # ------------------------------------------------------------------------------------------
    def _maybe_init_arena(self, core, grads_fp32: bool) -> None:
        """Single-node multi-GPU jobs keep the flat parameter / gradient buffers in peer-mapped
        memory (``MSRL_SYMM=0`` falls back to NCCL collectives and gathered resharding)."""
        import os

        import torch.distributed as dist

        from ..parallel.symm import get_arena, init_arena

        team = self.parallel_state.layout.world_size        # the ranks of this role (the whole job when co-located)
        if (self.device.type != "cuda" or not dist.is_initialized() or team == 1
                or dist.get_world_size() > torch.cuda.device_count() or get_arena() is not None
                or os.environ.get("MSRL_SYMM", "1") != "1"):
            return
        n = sum(p.numel() for p in core.parameters())
        gc = self.generate_config
        # buffers that the rollout phase frees get peer-mapped segments of their own, not arena space
        per_elem = (0 if getattr(gc, "offload_train_param", False) else 2) + \
                   (0 if getattr(gc, "offload_train_grad", False) else (4 if grads_fp32 else 2))
        extra = 0
        m_local = self._fused_tp_rows()
        if m_local:
            tp = self.parallel_state.size("tp")
            extra = 2 * m_local * self.tcfg.hidden_size * 2 * (1 + tp) + (1 << 20)
        extra += self._moe_p2p_bytes()
        from ..parallel.symm import ArenaUnavailable
        try:
            init_arena(int(n * per_elem * 1.02) + (64 << 20) + extra,
                       group=self.parallel_state.group("all"), device=self.device)
        except ArenaUnavailable as e:
            # raised on every rank together: the job carries on with NCCL collectives and gathered resharding
            import logging
            logging.getLogger(__name__).warning("peer-mapped memory unavailable, using collectives: %s", e)
            self.tcfg.moe_p2p_dispatch_rows = 0

    def _moe_p2p_bytes(self) -> int:
        """Expert-parallel MoE models can move tokens between ranks through peer-mapped slabs
        (``moe_token_dispatcher_type: p2p`` or ``moe_p2p_capacity_factor`` > 0): size the slabs for
        ``factor`` times the average load of a rank (its own tokens x top-k) and reserve the arena
        bytes.  Sets ``tcfg.moe_p2p_dispatch_rows``; 0 keeps the all-to-all collectives."""
        ac, rl, c = self.actor_config, self.rl_config, self.tcfg
        ep = self.parallel_state.size("ep")
        factor = float(getattr(ac, "moe_p2p_capacity_factor", 0.0) or 0.0)
        if getattr(ac, "moe_token_dispatcher_type", None) == "p2p" and factor <= 0:
            factor = 2.0
        if not c.is_moe or ep <= 1 or factor <= 0:
            return 0
        from ..parallel.moe_dispatch import P2PDispatcher
        mbs = max(ac.micro_batch_size or 1, rl.actor_forward_micro_batch_size or 1,
                  rl.ref_forward_micro_batch_size or 1)
        tokens = max(rl.update_max_packing_token_size or 0, rl.actor_max_packing_token_size or 0,
                     rl.ref_max_packing_token_size or 0, mbs * (ac.seq_length or 0), 1)
        e_local = c.num_experts // ep
        rows = (int(factor * tokens * c.moe_router_topk) + e_local * 128 + 127) // 128 * 128
        c.moe_p2p_dispatch_rows = rows
        return P2PDispatcher.bytes_needed(ep, e_local, c.hidden_size, rows) + (1 << 20)

    def _fused_tp_rows(self) -> int:
        """Largest token shard (rows per TP rank, multiple of 256) a packed micro-batch can have,
        or 0 when the communication-fused TP linears do not apply (no TP / no sequence parallel /
        ``MSRL_FUSED_TP=0``)."""
        import os

        ac, rl = self.actor_config, self.rl_config
        tp = self.parallel_state.size("tp")
        if tp == 1 or not ac.sequence_parallel or os.environ.get("MSRL_FUSED_TP", "1") != "1":
            return 0
        mbs = max(ac.micro_batch_size or 1, rl.actor_forward_micro_batch_size or 1,
                  rl.ref_forward_micro_batch_size or 1)
        tokens = max(rl.update_max_packing_token_size or 0, rl.actor_max_packing_token_size or 0,
                     rl.ref_max_packing_token_size or 0, mbs * (ac.seq_length or 0))
        tokens += 256 * tp + mbs * tp * 2
        return (tokens // tp + 255) // 256 * 256

    def _maybe_attach_fused_tp(self) -> None:
        from ..parallel.symm import get_arena

        arena, m_local = get_arena(), self._fused_tp_rows()
        if arena is None or not m_local or self.device.type != "cuda":
            return
        from ..parallel.fused_tp import FusedTP

        ps = self.parallel_state
        need = 2 * m_local * self.tcfg.hidden_size * 2 * (1 + ps.size("tp")) + (1 << 19)
        if arena.free_bytes() < need:
            return
        self.comm.fused = FusedTP(arena, arena.team_ranks(ps.group("tp")), m_local, self.tcfg.hidden_size,
                                  self.tcfg.hidden_size)

    def initialize(self) -> None:
        ac, rl, gc = self.actor_config, self.rl_config, self.generate_config
        ps = self.parallel_state
        tp = ps.size("tp")
        self.comm = TPComm(ps.group("tp"), ac.sequence_parallel, world_size=tp, rank=ps.rank_in("tp"))
        dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        tcfg = TransformerConfig.from_megatron(ac, params_dtype=dtype)
        self.tcfg = tcfg
        # pipeline stage of this rank: embedding on the first, head on the last, a slice of layers each
        from ..parallel.pipeline import PipelineSchedule
        from ..reshard.planner import pipeline_layout

        pp, pp_rank = ps.size("pp"), ps.rank_in("pp")
        chunks = pipeline_layout(ac, pp)[pp_rank]          # this stage's model chunks (virtual stages)
        stage_kw = dict(pre_process=pp_rank == 0, post_process=pp_rank == pp - 1,
                        layer_numbers=sum(chunks, []), chunk_sizes=[len(c) for c in chunks])
        self.pipeline = None
        if pp > 1:
            self.pipeline = PipelineSchedule(
                ps.group("pp"), pp_rank, pp, ps.get_pipeline_model_parallel_prev_rank(),
                ps.get_pipeline_model_parallel_next_rank(), tcfg.hidden_size, dtype, self.device,
                seq_shard=tp if (ac.sequence_parallel and tp > 1) else 1, num_chunks=len(chunks),
                grad_group=ps.group("pp_grad"))
        core = GPTModel(tcfg, self.comm, device=self.device, seed=self.seed, **stage_kw)
        if tcfg.is_moe and gc.eplb_token_collects:
            # expert-load statistics of the rollout (input of cli/eplb_generate_map.py)
            for layer in core.decoder.layers:
                if hasattr(layer.mlp, "rollout_view"):
                    layer.mlp.collect_rollout_counts = True
        dp = ps.size("dp_cp")
        self._maybe_init_arena(core, bool(ac.accumulate_allreduce_grads_in_fp32))
        gc = self.generate_config
        self.model = DistributedDataParallel(core, ps.group("dp_cp"), dp,
                                             grad_in_fp32=bool(ac.accumulate_allreduce_grads_in_fp32),
                                             releasable_params=bool(getattr(gc, "offload_train_param", False)),
                                             releasable_grads=bool(getattr(gc, "offload_train_grad", False)),
                                             releasable_experts=ps.size("pp") == 1,
                                             frozen_buffer=tcfg.lora_r > 0,
                                             **expert_replica_groups(ps, tcfg))
        self._maybe_attach_fused_tp()
        self.model.attach_tensor_parallel(ps.group("tp"), tp, bool(ac.sequence_parallel))
        if getattr(ac, "overlap_grad_reduce", False) and dp > 1 and ps.size("pp") == 1 \
                and not int(getattr(tcfg, "moe_p2p_dispatch_rows", 0) or 0):
            # bucketed gradient reduction on a side stream while the backward continues (not with pipeline
            # schedules, and not beside the peer-memory expert dispatch, whose device barriers involve the
            # same pairs of ranks on the main stream)
            self.model.enable_grad_overlap()
        iters = ac.train_iters or 1
        n_updates = iters * max(1, (ac.global_batch_size * rl.n_samples_per_prompt) // max(rl.mini_batch_size, 1))
        samples = n_updates * rl.mini_batch_size            # the schedule is stepped in samples
        self.optimizer, self.scheduler = OptimizerConfig.from_training_config(ac).build(
            self.model.buffers, dp_group=ps.group("dp_cp"), dp_rank=ps.rank_in("dp_cp"),
            model_parallel_group=ps.group("mp"), tp_rank=ps.rank_in("tp"), total_steps=samples,
            warmup_steps=int((ac.lr_warmup_fraction or 0.0) * samples), default_lr=1e-6)
        loss_opts = dict(clip_ratio=rl.clip_ratio, kl_penalty=rl.kl_penalty, entropy_coeff=rl.entropy_coeff,
                         token_level_loss=rl.token_level_loss, clip_higher_enable=rl.clip_higher_enable,
                         clip_ratio_low=rl.clip_ratio_low, clip_ratio_high=rl.clip_ratio_high,
                         kl_ctrl=rl.init_kl_coef)
        pad_mult = tp * ps.size("cp") * (2 if (ps.size("cp") > 1 and ac.context_parallel_algo == "megatron_cp_algo") else 1)
        self.pad_multiple = pad_mult
        temperature = gc.sampling_config.get("temperature", 1.0) or 1.0
        common = dict(stage=ac.stage or "ray_grpo", temperature=temperature,
                      use_dynamic_bsz=rl.use_dynamic_bsz, pad_multiple=pad_mult,
                      dp_group=ps.group("dp_cp"), dp_size=dp, device=self.device,
                      dynamic_max_batch_size=rl.actor_dynamic_max_batch_size, pipeline=self.pipeline,
                      context_parallel=dict(group=ps.group("cp"), size=ps.size("cp"), rank=ps.rank_in("cp"),
                                            algo=ac.context_parallel_algo,
                                            ulysses_degree=getattr(ac, "ulysses_degree_in_cp", None) or 1)
                      if ps.size("cp") > 1 else None)
        self.actor = TrainingEngine(
            self.model, self.optimizer, self.scheduler, role="actor",
            micro_batch_size=ac.micro_batch_size or 1,
            forward_micro_batch_size=rl.actor_forward_micro_batch_size or ac.micro_batch_size or 1,
            mini_batch_size_per_dp=max(rl.mini_batch_size // dp, 1), epochs=rl.epochs,
            shuffle_mini_batch=rl.shuffle_mini_batch,
            max_packing_token_size=rl.update_max_packing_token_size,
            forward_max_packing_token_size=rl.actor_max_packing_token_size, **common, **loss_opts)
        self.ref_model = None
        self.reference = None
        if self.with_reference and tcfg.lora_r > 0:
            # LoRA: the frozen backbone without adapters *is* the reference policy (no second copy)
            self.reference = TrainingEngine(
                self.model, role="reference", disable_adapter=True,
                micro_batch_size=rl.ref_forward_micro_batch_size or self.ref_config.micro_batch_size or 1,
                max_packing_token_size=rl.ref_max_packing_token_size, **common)
        elif self.with_reference:
            rcfg = TransformerConfig.from_megatron(self.ref_config, params_dtype=dtype)
            self.ref_model = GPTModel(rcfg, self.comm, device=self.device, seed=self.seed, **stage_kw)
            self.ref_model.load_state_dict(core.state_dict())
            for p in self.ref_model.parameters():
                p.requires_grad_(False)
            self.reference = TrainingEngine(
                self.ref_model, role="reference",
                micro_batch_size=rl.ref_forward_micro_batch_size or self.ref_config.micro_batch_size or 1,
                max_packing_token_size=rl.ref_max_packing_token_size, **common)
        # rollout engine (infer TP == train TP here; other layouts go through reshard.planner)
        self.engine = LLMEngine(
            tcfg, self.device, max_num_seqs=gc.max_num_seqs, max_num_batched_tokens=gc.max_num_batched_tokens,
            max_model_len=gc.max_model_len, block_size=gc.kv_block_size,
            enable_prefix_caching=gc.enable_prefix_caching, enforce_eager=gc.enforce_eager,
            graph_batch_sizes=tuple(gc.graph_batch_sizes), eos_token_id=self.eos_token_id,
            pad_token_id=self.pad_token_id, comm=self.comm if tp > 1 else None, seed=self.seed,
            # expert-parallel replicas exchange tokens in every forward: their engines step together
            lockstep_group=ps.group("ep") if (tcfg.is_moe and ps.size("ep") > 1) else None)
        resharder = None
        from ..reshard.planner import wanted_infer_ep

        # the rollout needs its own copy of the weights when its layout differs from training's: another
        # TP size, pipeline stages to gather, another expert-parallel size or an expert placement map
        move = (gc.infer_tensor_parallel_size != tp or ps.size("pp") > 1
                or wanted_infer_ep(tcfg, ps.layout, gc) is not None
                or (tcfg.is_moe and bool(getattr(gc, "expert_map_path", None))))
        if not move and tp > 1:
            from ..parallel.symm import get_arena
            from ..reshard.planner import attach_peer_all_reduce

            attach_peer_all_reduce(self.comm, get_arena(), tcfg.hidden_size)   # rollout shares the training TP group
        if move:
            from ..reshard.planner import Resharder

            resharder = Resharder.for_worker(self, gc)
            self.engine = resharder.engine
        # rank layout of the rollout phase: context-parallel ranks hold identical weights and act
        # as independent rollout replicas, so dispatch follows a (rollout-TP x DP) layout
        self.rollout_state = resharder.infer_state if resharder is not None else None
        if self.rollout_state is None and ps.size("cp") > 1:
            from ..parallel.state import ParallelState, RankLayout

            self.rollout_state = ParallelState(RankLayout(ps.layout.world_size, tp=tp), ps.rank, backend=ps.backend,
                                               rank_offset=ps.rank_offset)
        self.sharding_manager = ShardingManager(
            self.model, self.engine, self.optimizer, offload_train_optimizer=gc.offload_train_optimizer,
            offload_train_grad=gc.offload_train_grad, offload_train_param=gc.offload_train_param,
            gpu_memory_utilization=gc.gpu_memory_utilization, resharder=resharder,
            # expert layers permute every token top-k times through several temporaries per forward
            headroom_bytes=(2 << 30) + (16 * gc.max_num_batched_tokens * tcfg.moe_router_topk * tcfg.hidden_size * 2
                                        if tcfg.is_moe else 0))
        self.sampling_params = SamplingParams.from_config(gc.sampling_config, n=rl.n_samples_per_prompt,
                                                          **self.sampling_overrides)
        self.initialized = True

    def init_transfer_dock(self, td, mm_td=None, sampling_transfer_dock=None) -> None:
        self.td = td
        self.mm_td = mm_td
        self.sampling_td = sampling_transfer_dock

    # vision-language runs: what the language model reads from the multimodal store per sample
    MM_COLUMNS = ("vit_embeds", "position_ids")

    def _mm_columns(self):
        return self.MM_COLUMNS if (getattr(self, "mm_td", None) is not None and self.rl_config.is_multimodal) else None

    def _with_image_token(self, batch):
        if batch is not None and "mm" in batch:
            batch["image_token_id"] = int(getattr(self.actor_config, "image_token_id", None) or 151655)
        return batch

    def get_iteration(self) -> int:
        return self.iteration

    def get_consumed_train_samples(self) -> int:
        return self.consumed_train_samples

    # ---- rollout -----------------------------------------------------------------------------------
    def enter_infer_mode(self) -> None:
        """Reshard into the rollout engine and keep it resident (DAPO re-sampling rounds)."""
        if self.sharding_manager.mode != "infer":
            self._t_enter = self.sharding_manager.enter_infer_mode()
            self._report_enter_infer()
            self._held_infer = True

    def _report_enter_infer(self) -> None:
        """``timing/resharding_enter_infer`` is the host time of the whole transition; the weight
        move alone (device time of barrier + copy-plan kernel + barrier) and the KV-cache
        allocation are logged beside it."""
        t = self.sharding_manager.last_timing
        self.update_metrics("timing/resharding_enter_infer", [self._t_enter])
        self.update_metrics("timing/resharding_device", [t.get("reshard_device", 0.0)])
        self.update_metrics("timing/resharding_kv_cache", [t.get("kv_cache_alloc", 0.0)])

    def exit_infer_mode(self) -> None:
        if self.sharding_manager.mode == "infer":
            t_exit = self.sharding_manager.exit_infer_mode()
            self.update_metrics("timing/resharding_exit_infer", [t_exit])
            self.update_metrics("timing/resharding_to_infer", [getattr(self, "_t_enter", 0.0) + t_exit])
            self._held_infer = False

    @profiled_stage("actor_generate")
    def generate_sequences(self) -> None:
        rl = self.rl_config
        held = getattr(self, "_held_infer", False)
        if not held:
            self._t_enter = self.sharding_manager.enter_infer_mode()
            self._report_enter_infer()
        main_td = self.td
        if getattr(self, "sampling_td", None) is not None:
            self.td = self.sampling_td          # rollouts of DAPO go to the sampling dock
        start = _now()
        n = rl.n_samples_per_prompt
        train_state = self._state
        if getattr(self, "rollout_state", None) is not None:
            # rollout replicas are (infer-TP)-sized: dispatch / write-back follow the rollout layout
            self._state = self.rollout_state
        partial = (rl.partial_rollout_max_split or 1) > 1
        columns = ["prompts", "prompt_length"] + (["responses", "response_length", "age"] if partial else [])
        try:
            while True:
                batch, idx, finished = self.dispatch_transfer_dock_data(
                    "actor_rollout", columns, rl.actor_rollout_dispatch_size, get_n_samples=not partial,
                    mm_columns=self._mm_columns())
                if finished:
                    break
                if batch is None:
                    time.sleep(0.002)
                    continue
                if partial:
                    self._generate_batch_partial(batch, idx)
                elif getattr(self, "multi_turn", None) is not None:
                    self._generate_batch_multi_turn(batch, idx, n)
                else:
                    self._generate_batch(batch, idx, n)
            end = _now()
            self.update_metrics("timing/rollout", [round(end, 4), round(start, 4)])
        finally:
            self.td = main_td
            self._state = train_state
        self._dump_expert_load()
        if not held:
            t_exit = self.sharding_manager.exit_infer_mode()
            self.update_metrics("timing/resharding_exit_infer", [t_exit])
            self.update_metrics("timing/resharding_to_infer", [self._t_enter + t_exit])

    def _dump_expert_load(self) -> None:
        """``generate_config.eplb_token_collects``: write the tokens every expert received during this
        rollout to ``eplb_token_save_path/eplb_token_collects_<rank>.json`` (one entry per MoE layer)."""
        gc = self.generate_config
        weights = getattr(self.engine.runner, "weights", None)
        if not (self.tcfg.is_moe and gc.eplb_token_collects and weights is not None):
            return
        import os

        os.makedirs(gc.eplb_token_save_path, exist_ok=True)
        rank = dist.get_rank() if dist.is_initialized() else 0
        for li, lw in enumerate(weights.layers):
            if lw.moe is not None and lw.moe.collect_counts:
                lw.moe.dump_counts(gc.eplb_token_save_path, li, rank)

    def _generate_batch(self, batch: Dict[str, torch.Tensor], idx: List[int], n: int) -> None:
        prompts, plen = batch["prompts"], batch["prompt_length"].reshape(-1)
        uniq = list(range(0, len(idx), n))                   # the store holds n copies per prompt
        prompt_lists = [prompts[i, :int(plen[i])].tolist() for i in uniq]
        mm = None
        if batch.get("mm") is not None:
            tok = int(getattr(self.actor_config, "image_token_id", None) or 151655)
            mm = [dict(batch["mm"][i] or {}, image_token_id=tok) for i in uniq]
        outs = self.engine.generate(prompt_lists, self.sampling_params, mm=mm)
        vocab = self.tcfg.vocab_size
        responses, input_ids, lengths = [], [], []
        for p, o in zip(prompt_lists, outs):
            for c in o.outputs:
                ids = [t if t < vocab else 0 for t in c.token_ids]
                responses.append(torch.tensor(ids, dtype=torch.int64))
                input_ids.append(torch.tensor(p + ids, dtype=torch.int64))
                lengths.append(torch.tensor([len(ids)], dtype=torch.int32))
        self.dump_key_data("actor_generate", "actor_infer_dump",
                           {"prompts": prompts, "prompt_length": plen, "responses": responses,
                            "response_length": lengths})
        self.collect_transfer_dock_data(
            {"responses": responses, "input_ids": input_ids, "response_length": lengths}, idx)

    # ---- partial rollout --------------------------------------------------------------------------------------
    def _generate_batch_partial(self, batch: Dict[str, torch.Tensor], idx: List[int]) -> None:
        """One round of partial rollout (reference: ``workers/actor_hybrid_worker.py:484-573``): every
        row continues from ``prompt + partial response`` for at most ``max_tokens / max_split`` new
        tokens; a row is complete on EOS, at ``max_tokens`` response tokens or at the context limit.
        Unfinished rows stay in the store (one round older) and are continued in a later iteration."""
        import dataclasses
        import math

        rl, base = self.rl_config, self.sampling_params
        self._partial_calls = getattr(self, "_partial_calls", 0) + 1
        max_tokens = base.max_tokens
        per_round = max(1, math.ceil(max_tokens / rl.partial_rollout_max_split))
        limit = self.engine.max_model_len
        rows = [i for i, ix in enumerate(idx) if ix >= 0]       # filler rows (index -2) are skipped
        prompts, plen = batch["prompts"], batch["prompt_length"].reshape(-1)
        resp, rlen = batch["responses"], batch["response_length"].reshape(-1)
        age = batch["age"].reshape(-1) if "age" in batch else torch.zeros(len(idx))
        ctxs, partials, params, rids = [], [], [], []
        for i in rows:
            p = prompts[i, :int(plen[i])].tolist()
            r = resp[i, :int(rlen[i])].tolist() if int(rlen[i]) > 0 else []
            budget = min(per_round, max_tokens - len(r), limit - len(p) - len(r))
            ctxs.append(p + r)
            partials.append((p, r))
            # every row is a request of its own here: with a fixed sampling seed all of them would draw the same
            # random numbers (the samples of one prompt would come out identical, round after round), so the seed
            # is spread over the row, the tokens it already has and the call
            seed = base.seed
            if seed is not None:
                seed = (((int(seed) * 1000003 + int(idx[i])) * 1000003 + len(r)) * 1000003 + self._partial_calls) \
                    & 0x7FFFFFFF
            params.append(dataclasses.replace(base, n=1, max_tokens=max(int(budget), 1), seed=seed))
            rids.append(f"pr_{idx[i]}_{int(age[i])}_{self.iteration}")
        outs = self.engine.generate(ctxs, params, request_ids=rids) \
            if (ctxs or self.engine.lockstep_group is not None) else []
        vocab = self.tcfg.vocab_size
        t = lambda v, dt=torch.int64: torch.tensor(v, dtype=dt)
        responses, input_ids, lengths, completed = [], [], [], []
        for (p, r), o in zip(partials, outs):
            c = o.outputs[0]
            new = [x if x < vocab else 0 for x in c.token_ids]
            full = r + new
            done = c.finish_reason == "stop" or len(full) >= max_tokens or len(p) + len(full) >= limit
            responses.append(t(full))
            input_ids.append(t(p + full))
            lengths.append(t([len(full)], torch.int32))
            completed.append(t([1 if done else 0], torch.int32))
        self.collect_transfer_dock_data(
            {"responses": responses, "input_ids": input_ids, "response_length": lengths,
             "rollout_completed": completed}, [idx[i] for i in rows])

    # ---- multi-turn tool use ----------------------------------------------------------------------------
    def attach_tools(self, tokenizer, tool_map=None) -> None:
        """Enable the multi-turn tool loop for rollouts (``rl_config.multi_turn_enable``)."""
        from ..tools.base import load_tool_map
        from ..tools.multi_turn import MultiTurnRollout

        rl = self.rl_config
        if tool_map is None:
            tool_map = load_tool_map(rl.tool_config_path) if rl.tool_config_path else {}
        comm = self.engine.comm

        def share(ids: List[int]) -> List[int]:
            # the rollout TP ranks run the engine in lock-step: rank 0's tool turn is the one all use
            if comm.world_size == 1:
                return ids
            import torch.distributed as dist

            box = [ids if comm.rank == 0 else None]
            dist.broadcast_object_list(box, src=dist.get_process_group_ranks(comm.group)[0], group=comm.group)
            return box[0]

        self.multi_turn = MultiTurnRollout(
            self.engine, tokenizer, tool_map, rl.tool_parser_format or "hermes", vocab_size=self.tcfg.vocab_size,
            max_total_response_length=rl.max_total_response_length or self.generate_config.max_model_len,
            max_tool_calls=rl.max_tool_calls or 1, max_parallel_calls=rl.max_parallel_calls or 1,
            max_tool_response_length=rl.max_tool_response_length or 256,
            tool_response_truncate_side=rl.tool_response_truncate_side or "middle", share_result=share)

    def _generate_batch_multi_turn(self, batch: Dict[str, torch.Tensor], idx: List[int], n: int) -> None:
        prompts, plen = batch["prompts"], batch["prompt_length"].reshape(-1)
        prompt_lists = [prompts[i, :int(plen[i])].tolist() for i in range(len(idx))]   # one request per sample
        res = self.multi_turn.generate(prompt_lists, self.sampling_params)
        t = lambda v, dt=torch.int64: torch.tensor(v, dtype=dt)
        self.collect_transfer_dock_data({
            "responses": [t(r["responses"]) for r in res], "input_ids": [t(r["input_ids"]) for r in res],
            "response_length": [t([r["response_length"]], torch.int32) for r in res],
            "response_mask": [t(r["response_mask"]) for r in res],
            "tool_call_num": [t([r["tool_call_num"]], torch.int32) for r in res]}, idx)

    # ---- forward-only stages ---------------------------------------------------------------------------
    def _logprob_stage(self, consumer: str, engine: TrainingEngine, out_column: str, dispatch_size: int,
                       timing_key: str) -> None:
        columns = ["input_ids", "responses", "response_length", "prompt_length"]
        start = _now()
        while True:
            batch, idx, finished = self.dispatch_transfer_dock_data(
                consumer, columns, dispatch_size, pad_multiple=1, get_n_samples=False,
                use_batch_seqlen_balance=self.rl_config.use_dp_batch_balance, mm_columns=self._mm_columns())
            if finished:
                break
            if batch is None:
                time.sleep(0.002)
                continue
            lp = engine.forward(self._with_image_token(batch))
            self.dump_key_data(consumer, "reference_dump" if out_column == "ref_log_prob" else "actor_train_dump",
                               {"input_ids": batch["input_ids"], "response_length": batch["response_length"],
                                out_column: lp})
            self.collect_transfer_dock_data({out_column: lp}, idx, lengths=batch["response_length"])
        self.update_metrics(timing_key, [round(_now(), 4), round(start, 4)])

    @profiled_stage("reference_compute_log_prob")
    def compute_ref_log_prob(self) -> None:
        if self.reference is None:
            raise RuntimeError("this worker was built without a reference model")
        self.sharding_manager.enter_forward_mode()
        self._logprob_stage("ref_log_prob", self.reference, "ref_log_prob",
                            self.rl_config.ref_dispatch_size, "timing/reference_model")
        self.update_metrics("end_time/reference", [round(_now(), 4)])
        self.sharding_manager.exit_forward_mode()

    @profiled_stage("actor_compute_log_prob")
    def compute_log_prob(self) -> None:
        self.sharding_manager.enter_forward_mode()
        self._logprob_stage("actor_log_prob", self.actor, "old_log_prob",
                            self.rl_config.actor_logprob_dispatch_size, "timing/old_log_p")
        self.update_metrics("end_time/old_log_p", [round(_now(), 4)])
        self.sharding_manager.exit_forward_mode()

    # ---- update ----------------------------------------------------------------------------------------
    @profiled_stage("actor_update")
    def update(self, kl_ctrl=None, skip_actor_log_prob: bool = False) -> None:
        rl = self.rl_config
        t_reshard = self.sharding_manager.enter_train_mode()
        self.update_metrics("timing/resharding_to_train", [t_reshard])
        columns = ["responses", "advantages", "input_ids", "response_length", "prompt_length"]
        if not skip_actor_log_prob:
            columns.append("old_log_prob")
        if self.uses_ref_log_prob and (self.actor_config.stage or "ray_grpo") != "ray_dapo":
            columns.append("ref_log_prob")
        if rl.multi_turn_enable:
            columns.append("response_mask")
        start = _now()
        while True:
            batch, idx, finished = self.dispatch_transfer_dock_data(
                "actor_train", columns, rl.actor_update_dispatch_size, get_n_samples=False,
                use_batch_seqlen_balance=rl.use_dp_batch_balance, mm_columns=self._mm_columns())
            if finished:
                break
            if batch is None:
                time.sleep(0.002)
                continue
            metrics = self.actor.update(self._with_image_token(batch), kl_ctrl)
            self.dump_key_data("actor_update", "actor_train_dump",
                               {**{k: batch[k] for k in ("responses", "advantages", "old_log_prob", "ref_log_prob")
                                   if k in batch},
                                **{k: (sum(v) / len(v) if isinstance(v, (list, tuple)) and v else v)
                                   for k, v in metrics.items() if k.startswith("actor/")}})
            self.consumed_train_samples += len(idx) * self.parallel_state.size("dp_cp")
            if self.is_writer():
                self.td.update_metrics("", value=metrics, cumulate=True)
        self.update_metrics("timing/update", [round(_now(), 4), round(start, 4)])
        self.iteration += 1
        self.sharding_manager.exit_train_mode()

    # ---- checkpoint ---------------------------------------------------------------------------------------
    def save_checkpoint(self, iteration: int) -> None:
        from ..checkpoint.mcore import save_checkpoint

        if not self.actor_config.save:
            return
        self.sharding_manager.enter_train_mode()
        save_checkpoint(self.actor_config.save, iteration, self.model.module, self.optimizer,
                        self.scheduler, self.parallel_state, self.actor_config,
                        consumed_train_samples=self.consumed_train_samples)
        self.sharding_manager.exit_train_mode()
