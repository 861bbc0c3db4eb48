"""Training / scoring engine shared by the actor, reference, critic and reward roles.

Flow (reference behaviour: ``mindspeed_rl/models/base/base_training_engine.py:125-537``):

``update``:  epochs x mini-batches (``mini_batch_size_per_dp`` rows) -> micro-batches (fixed
size, or token-budget bins when ``use_dynamic_bsz``) -> packed forward/backward with gradient
accumulation -> DP gradient reduction -> optimizer step -> LR scheduler step.
``forward``: the same micro-batching without gradients, results returned in input order.

What differs by design: every micro-batch is a *packed* token stream (remove-padding is not an
option but the only layout), labels/positions/gather indices are built vectorised on the host
and shipped once, the LM head never materialises logits, and the loss is a fused
forward+backward kernel over the response tokens.
"""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..obs.io_counter import to_device, to_host
from ..utils.device_status import check_device_status
from ..utils.seqlen_balancing import get_reverse_idx, rearrange_micro_batches
from .gpt import GPTModel, PackedMeta
from .loss.registry import BaseLossFunc, LossFuncFactory


def _unwrap(model):
    return model.module if hasattr(model, "module") and not isinstance(model, GPTModel) else model


class MicroBatch:
    """Packed view of some rows of a padded batch (host tensors until ``to``)."""

    def __init__(self, data: Dict[str, torch.Tensor], rows: Sequence[int], align: int, total_align: int = 1):
        """``align``: every sequence is padded to a multiple of it (TP x CP token sharding);
        ``total_align``: the last sequence takes extra padding so that the whole stream is a
        multiple of it (256 x TP lets the communication-fused GEMMs tile the token shards)."""
        rows_t = torch.as_tensor(list(rows), dtype=torch.int64)
        ids2d = data["input_ids"][rows_t].to(torch.int64)
        b, s = ids2d.shape
        p_len = data["prompt_length"][rows_t].reshape(-1).to(torch.int64)
        r_len = data["response_length"][rows_t].reshape(-1).to(torch.int64)
        lens = (p_len + r_len).clamp(max=s)
        padded = (lens + align - 1) // align * align
        if total_align > 1 and b:
            padded[-1] += (-int(padded.sum())) % total_align
        cu = torch.zeros(b + 1, dtype=torch.int64)
        cu[1:] = torch.cumsum(padded, 0)
        total = int(cu[-1])
        # the packed ids / next-token labels / positions are built by ``ops.packing.pack_tokens``: on
        # the device when the micro-batch is moved there (only the padded rows and three small
        # vectors cross PCIe), on the host the first time something asks for them
        ids2d = ids2d[:, :max(int(lens.max()) if b else 0, 1)].contiguous()      # columns no row uses stay behind
        self._ids2d, self._p_len, self._r_len = ids2d, p_len.to(torch.int32), r_len.to(torch.int32)
        self._packed = None
        width = data["responses"].shape[1]
        j = torch.arange(width).unsqueeze(0)
        self.resp_valid = j < r_len.unsqueeze(1)
        self.resp_index = (cu[:-1] + p_len - 1).unsqueeze(1) + j
        self.resp_index = torch.where(self.resp_valid, self.resp_index, torch.zeros_like(self.resp_index))
        self.last_index = cu[:-1] + lens - 1
        self.rows = rows_t
        self.cu = cu.to(torch.int32)
        self.cu_host = cu.clone()          # stays on the host (context-parallel index arithmetic)
        self.max_seqlen = int(padded.max()) if b else 0
        self.num_tokens = total
        self.data = {k: v[rows_t] for k, v in data.items() if torch.is_tensor(v) and v.shape[:1] == data["input_ids"].shape[:1]}
        # vision-language rows: ``data["mm"][r] = dict(vit_embeds [n_r, H], position_ids [P_r, 3])`` per sample
        self.image_index = self.image_embeds = self.pos3 = None
        self.image_token_id = data.get("image_token_id")
        mm = data.get("mm")
        if mm is not None:
            from ..datasets.mm_utils import extend_positions

            embeds, pos3, index = [], [], []
            for j, r in enumerate(rows_t.tolist()):
                item = mm[r] or {}
                n_tok = int(lens[j])
                row_ids = ids2d[j, :n_tok]
                where = torch.nonzero(row_ids == self.image_token_id).reshape(-1)
                e = item.get("vit_embeds")
                if e is not None and where.numel():
                    if e.shape[0] != where.numel():
                        raise ValueError(f"sample {r}: {where.numel()} image tokens but {e.shape[0]} embedding rows")
                    embeds.append(e)
                    index.append(where + int(cu[j]))
                pp = item.get("position_ids")
                pp = pp[:n_tok] if pp is not None else torch.arange(min(int(p_len[j]), n_tok)).unsqueeze(-1).expand(-1, 3)
                full = extend_positions(pp, max(n_tok - pp.shape[0], 0))
                pad = int(padded[j]) - n_tok
                pos3.append(torch.cat([full, full.new_zeros(pad, 3)]) if pad else full)
            self.pos3 = torch.cat(pos3) if pos3 else None
            if embeds:
                self.image_index, self.image_embeds = torch.cat(index), torch.cat(embeds)

    def _pack(self):
        if self._packed is None:
            from ..ops.packing import pack_tokens

            self._packed = pack_tokens(self._ids2d, self._p_len, self._r_len, self.cu, self.num_tokens)
        return self._packed

    ids = property(lambda self: self._pack()[0])
    labels = property(lambda self: self._pack()[1])
    positions = property(lambda self: self._pack()[2])

    def to(self, device) -> "MicroBatch":
        for k in ("cu", "resp_index", "resp_valid", "last_index", "_p_len", "_r_len"):
            t = getattr(self, k)
            setattr(self, k, to_device(t, t.dtype, device))
        ids2d = self._ids2d
        if torch.device(device).type == "cuda" and ids2d.numel() and int(ids2d.max()) < 2 ** 31:
            ids2d = ids2d.to(torch.int32)              # half the bytes over PCIe
        self._ids2d = to_device(ids2d, ids2d.dtype, device)
        self._packed = None
        for k in ("image_index", "image_embeds", "pos3"):
            t = getattr(self, k)
            if t is not None:
                setattr(self, k, to_device(t, t.dtype, device))
        return self

    def response_rows(self, per_token: torch.Tensor) -> torch.Tensor:
        """Per-token values of the packed stream ``[T]`` -> ``[b, R]`` response rows (zeros beyond each
        response).  Without autograd this is one gather kernel; with it, an index + mask that
        autograd knows how to invert."""
        if not (torch.is_grad_enabled() and per_token.requires_grad) and per_token.dim() == 1:
            from ..ops.packing import unpack_response

            return unpack_response(per_token, self.cu, self._p_len, self._r_len, self.resp_index.shape[1])
        return per_token[self.resp_index] * self.resp_valid

    def meta(self, rope_table_of=None) -> PackedMeta:
        """``rope_table_of(device)``: the model's one-axis rotary table, needed to build the per-token table
        of three-axis positions (vision-language rows only)."""
        if self.pos3 is None:
            return PackedMeta(self.cu, self.max_seqlen, self.positions)
        from ..datasets.mm_utils import mrope_table

        if getattr(self, "_rope_tab", None) is None:
            self._rope_tab = mrope_table(self.pos3, rope_table_of(self.pos3.device))
        order = torch.arange(self.num_tokens, dtype=torch.int32, device=self.pos3.device)
        return PackedMeta(self.cu, self.max_seqlen, order, image_index=self.image_index, image_embeds=self.image_embeds,
                          rope_table=self._rope_tab)


class TrainingEngine:
    def __init__(self, model, optimizer=None, opt_param_scheduler=None, *, stage: str = "ray_grpo",
                 role: str = "actor", micro_batch_size: int = 1, mini_batch_size_per_dp: int = 1,
                 epochs: int = 1, shuffle_mini_batch: bool = False, temperature: float = 1.0,
                 use_dynamic_bsz: bool = False, max_packing_token_size: Optional[int] = None,
                 forward_max_packing_token_size: Optional[int] = None,
                 dynamic_max_batch_size: Optional[int] = None, pad_multiple: int = 1, dp_group=None,
                 dp_size: int = 1, device=None, forward_micro_batch_size: Optional[int] = None,
                 want_entropy: Optional[bool] = None, forward_backward_func: Optional[Callable] = None,
                 pipeline=None, context_parallel: Optional[dict] = None, disable_adapter: bool = False,
                 **loss_options):
        self.model = model
        self.disable_adapter = disable_adapter   # LoRA: run the backbone without adapters (reference policy)
        self.pipeline = pipeline             # parallel.pipeline.PipelineSchedule when PP > 1
        cpi = context_parallel or {}         # {"group", "size", "rank", "algo"} when CP > 1
        self.cp_group, self.cp_size = cpi.get("group"), int(cpi.get("size", 1) or 1)
        self.cp_rank, self.cp_algo = int(cpi.get("rank", 0) or 0), cpi.get("algo")
        self.cp_ulysses = int(cpi.get("ulysses_degree", 1) or 1)
        self.core: GPTModel = _unwrap(model)
        self.optimizer, self.opt_param_scheduler = optimizer, opt_param_scheduler
        self.stage, self.role = stage, role
        self.micro_batch_size = micro_batch_size
        self.forward_micro_batch_size = forward_micro_batch_size or micro_batch_size
        self.mini_batch_size_per_dp = mini_batch_size_per_dp
        self.epochs, self.shuffle_mini_batch = epochs, shuffle_mini_batch
        self.temperature = temperature
        self.use_dynamic_bsz = use_dynamic_bsz
        self.max_packing_token_size = max_packing_token_size
        self.forward_max_packing_token_size = forward_max_packing_token_size or max_packing_token_size
        self.dynamic_max_batch_size = dynamic_max_batch_size
        self.pad_multiple = pad_multiple
        self.dp_group, self.dp_size = dp_group, dp_size
        self.device = device or next(self.core.parameters()).device
        self.forward_backward_func = forward_backward_func
        stage_key = "ray_grpo" if (stage == "ray_dapo" and role != "actor") else stage
        self.loss_func: BaseLossFunc = LossFuncFactory.get_instance(stage_key, role, **loss_options)
        c_ent = float(loss_options.get("entropy_coeff", 0.0) or 0.0)
        self.want_entropy = (role == "actor") if want_entropy is None else want_entropy
        self.entropy_needs_grad = c_ent != 0.0

    # ------------------------------------------------------------------------------------------
    def _total_align(self) -> int:
        """Token-count multiple of a packed stream: 256 per TP rank when the communication-fused
        linears are attached (their CTA pairs tile each rank's token shard in 256-row tiles)."""
        comm = self.core.comm
        if getattr(comm, "fused", None) is not None and comm.sequence_parallel:
            return 256 * comm.world_size
        return 1

    def _split(self, data: Dict[str, torch.Tensor], rows: List[int], update: bool) -> List[List[int]]:
        if not self.use_dynamic_bsz:
            mbs = self.micro_batch_size if update else self.forward_micro_batch_size
            return [rows[i:i + mbs] for i in range(0, len(rows), mbs)]
        lens = (data["prompt_length"].reshape(-1) + data["response_length"].reshape(-1))[rows].tolist()
        budget = self.max_packing_token_size if update else self.forward_max_packing_token_size
        parts = rearrange_micro_batches(lens, budget, self.dynamic_max_batch_size, self.dp_group)
        return [[rows[i] for i in p] for p in parts if p]

    def _run_model(self, mb: MicroBatch, want_entropy: bool, h_in: Optional[torch.Tensor] = None,
                   chunk: Optional[int] = None):
        """Returns the role's per-response-token outputs ``[b, R]`` (autograd-connected).
        ``h_in``: hidden states received from the previous pipeline stage (``None`` on the first)."""
        core = self.core
        x = mb.ids if h_in is None else h_in
        kw = {} if chunk is None else {"chunk": chunk}
        cp = self._context_parallel(mb)
        if cp is not None:
            # every CP rank runs its own tokens of every sequence; per-token outputs are gathered
            # back into packed order before the response positions are picked
            if h_in is None:
                x = cp.take_local(mb.ids)
            meta = PackedMeta(cp.cu_local, cp.max_local, cp.take_local(mb.positions), cp=cp)
            if self.loss_func.output_kind == "value":
                v = cp.gather_tokens(core.forward_values(x, meta, **kw))
                if self.role == "reward":
                    return v[mb.last_index].unsqueeze(-1), None
                return mb.response_rows(v), None
            logp, ent = core.forward_logprob(x, cp.take_local(mb.labels), meta, self.temperature, want_entropy, **kw)
            logp = cp.gather_tokens(logp)
            lp = mb.response_rows(logp)
            en = mb.response_rows(cp.gather_tokens(ent)) if want_entropy else None
            return lp, en
        if self.loss_func.output_kind == "value":
            v = core.forward_values(x, mb.meta(self._rope_table_of), **kw)
            if self.role == "reward":
                return v[mb.last_index].unsqueeze(-1), None
            return mb.response_rows(v), None
        logp, ent = core.forward_logprob(x, mb.labels, mb.meta(self._rope_table_of), self.temperature, want_entropy, **kw)
        lp = mb.response_rows(logp)
        en = mb.response_rows(ent) if want_entropy else None
        return lp, en

    def _stage_forward(self, mb: MicroBatch, h_in: Optional[torch.Tensor], want_entropy: bool,
                       chunk: Optional[int] = None):
        """One (virtual) pipeline stage: hidden states for inner stages, role outputs on the last one."""
        if not self.core.is_last_chunk(chunk):
            kw = {} if chunk is None else {"chunk": chunk}
            cp = self._context_parallel(mb)
            if cp is None:
                return self.core.hidden_states(mb.ids if h_in is None else h_in, mb.meta(self._rope_table_of), **kw)
            meta = PackedMeta(cp.cu_local, cp.max_local, cp.take_local(mb.positions), cp=cp)
            return self.core.hidden_states(cp.take_local(mb.ids) if h_in is None else h_in, meta, **kw)
        return self._run_model(mb, want_entropy, h_in, chunk)

    def _rope_table_of(self, device) -> torch.Tensor:
        return self.core.decoder.layers[0].rope_table(device)

    def _context_parallel(self, mb: MicroBatch):
        """Context-parallel helper of this micro-batch (cached on it), ``None`` without CP."""
        if self.cp_size <= 1:
            return None
        cp = getattr(mb, "_cp", None)
        if cp is None:
            from ..parallel.context_parallel import ContextParallel

            cp = ContextParallel(self.cp_group, self.cp_size, self.cp_rank, self.cp_algo, mb.cu_host, self.device,
                                 ulysses_degree=self.cp_ulysses)
            mb._cp = cp
        return cp

    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, data: Dict[str, torch.Tensor]) -> torch.Tensor:
        """Forward-only pass; returns ``[B, R]`` fp32 on the host in the order of ``data`` rows."""
        if self.disable_adapter:
            from .lora import adapter_disabled

            self.disable_adapter = False
            try:
                with adapter_disabled(self.core):
                    return self.forward(data)
            finally:
                self.disable_adapter = True
        self.model.eval()
        n = data["input_ids"].shape[0]
        width = 1 if self.role == "reward" else data["responses"].shape[1]
        out = torch.zeros(n, width, dtype=torch.float32)
        results = []
        if self.pipeline is not None:
            mbs = [MicroBatch(data, rows, self.pad_multiple, self._total_align()).to(self.device)
                   for rows in self._split(data, list(range(n)), update=False)]
            outs = self.pipeline.forward_only(mbs, lambda m: m.num_tokens // self.cp_size,
                                              lambda m, h, c=None: self._stage_forward(m, h, False, c))
            results = [(m.rows.tolist(), o[0].float()) for m, o in zip(mbs, outs)]
        else:
            for rows in self._split(data, list(range(n)), update=False):
                mb = MicroBatch(data, rows, self.pad_multiple, self._total_align()).to(self.device)
                vals, _ = self._run_model(mb, want_entropy=False)
                results.append((rows, vals.float()))
        for rows, vals in results:
            out[torch.as_tensor(rows)] = to_host(vals)
        return out

    # ------------------------------------------------------------------------------------------
    def update(self, data: Dict[str, torch.Tensor], kl_ctrl=None) -> Dict[str, List[float]]:
        """Run ``epochs`` passes of mini-batch updates over ``data``; returns metric lists."""
        self.model.train()
        if kl_ctrl is not None:
            self.loss_func.add_loss_meta_info({"kl_ctrl": getattr(kl_ctrl, "value", kl_ctrl)})
        n = data["input_ids"].shape[0]
        metrics: Dict[str, List[Any]] = {}
        lr_key = "critic/lr" if self.role == "critic" else "actor/lr"
        gn_key = "critic/grad_norm" if self.role == "critic" else "actor/grad_norm"
        for _ in range(self.epochs):
            order = torch.randperm(n).tolist() if self.shuffle_mini_batch else list(range(n))
            for s in range(0, n, self.mini_batch_size_per_dp):
                mini = order[s:s + self.mini_batch_size_per_dp]
                self._zero_grad()
                stats = self._forward_backward(data, mini)
                ok, grad_norm, _ = self._optimizer_step()
                if self.opt_param_scheduler is not None and ok:
                    self.opt_param_scheduler.step(increment=len(mini) * self.dp_size)
                for k, v in stats.items():
                    metrics.setdefault(k, []).append(v)
                metrics.setdefault(gn_key, []).append(grad_norm)
                if self.optimizer is not None:
                    metrics.setdefault(lr_key, []).append(self.optimizer.param_groups[0]["lr"])
        return {k: [float(x) for x in v] for k, v in metrics.items()}

    def _zero_grad(self) -> None:
        if hasattr(self.model, "zero_grad_buffer"):
            self.model.zero_grad_buffer()
        else:
            for p in self.core.parameters():
                p.grad = None
        if self.optimizer is not None and not hasattr(self.model, "zero_grad_buffer"):
            self.optimizer.zero_grad()

    def _pad_to_pipeline(self, parts: List[List[int]]) -> List[List[int]]:
        """The interleaved schedule walks groups of ``pp`` micro-batches: split the largest ones until the
        count is a multiple of the pipeline size (same decision on every rank of the replica)."""
        pp = self.pipeline.size
        parts = [list(p) for p in parts]
        while len(parts) % pp:
            big = max(range(len(parts)), key=lambda i: len(parts[i]))
            if len(parts[big]) < 2:
                raise ValueError(f"cannot form a multiple of {pp} micro-batches from {sum(map(len, parts))} samples; "
                                 f"raise the mini-batch size or lower the virtual pipeline size")
            half = len(parts[big]) // 2
            parts[big:big + 1] = [parts[big][:half], parts[big][half:]]
        return parts

    def _forward_backward(self, data, mini: List[int]) -> Dict[str, torch.Tensor]:
        parts = self._split(data, mini, update=True)
        if self.pipeline is not None and self.pipeline.num_chunks > 1:
            parts = self._pad_to_pipeline(parts)
        n_micro = len(parts)
        sums: Dict[str, torch.Tensor] = {}

        def loss_backward(mb: MicroBatch, outputs) -> None:
            out, ent = outputs
            scale = 1.0 / n_micro
            if self.use_dynamic_bsz:   # re-weight bins by their share of the mini-batch rows
                scale = len(mb.rows) / len(mini)
            batch_dev = {k: to_device(v, v.dtype, self.device) for k, v in mb.data.items()
                         if k not in ("input_ids", "prompts", "responses")}
            if not self.entropy_needs_grad and ent is not None:
                ent = ent.detach()
            grad, dent, stats = self.loss_func.compute(batch_dev, out.detach(), ent.detach() if ent is not None else None, scale)
            outs, grads = [out], [grad]
            if dent is not None and ent is not None and ent.requires_grad:
                outs.append(ent)
                grads.append(dent)
            torch.autograd.backward(outs, grads)
            for k, v in stats.items():
                v = v.detach() * scale
                sums[k] = v if k not in sums else sums[k] + v

        if self.pipeline is not None:
            mbs = [MicroBatch(data, rows, self.pad_multiple, self._total_align()).to(self.device) for rows in parts]
            self.pipeline.forward_backward(mbs, lambda m: m.num_tokens // self.cp_size,
                                           lambda m, h, c=None: self._stage_forward(m, h, self.want_entropy, c),
                                           loss_backward)
            return sums
        for i, rows in enumerate(parts):
            mb = MicroBatch(data, rows, self.pad_multiple, self._total_align()).to(self.device)
            if i == n_micro - 1 and hasattr(self.model, "begin_last_microbatch"):
                self.model.begin_last_microbatch()     # overlapped gradient reduction, when enabled
            loss_backward(mb, self._run_model(mb, want_entropy=self.want_entropy))
        return sums

    def _optimizer_step(self):
        if hasattr(self.model, "finish_grad_sync"):
            self.model.finish_grad_sync(to_shards=True)
        if self.optimizer is None:
            return True, 0.0, 0
        # a kernel whose bounded wait gave up (a late or absent peer) left incomplete gradients behind:
        # raise before they reach the weights (the optimizer step reads the gradient norm back anyway)
        if self.device.type == "cuda":
            check_device_status("gradients")
        result = self.optimizer.step()
        if getattr(self.core.cfg, "moe_router_enable_expert_bias", False):
            for layer in self.core.decoder.layers:
                if hasattr(layer.mlp, "update_expert_bias"):
                    layer.mlp.update_expert_bias(group=self.dp_group)
        fused = getattr(self.core.comm, "fused", None)
        if fused is not None:
            fused.invalidate_weights()       # cached transposed weights are stale now
        return result
