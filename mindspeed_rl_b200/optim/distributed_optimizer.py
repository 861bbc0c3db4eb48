"""AdamW over the flat parameter buffers, sharded across the data-parallel group (ZeRO-1), with
optional optimizer state in pinned host memory ("swap optimizer").

``step()`` = reduce-scatter-ed gradients -> global L2 norm (one tiny all-reduce) -> clip
coefficient computed on the device -> fused AdamW on this rank's shard (fp32 master + moments,
bf16 working copy written in the same pass) -> parameter all-gather.  It returns
``(update_successful, grad_norm, num_zeros_in_grad)`` like the Megatron optimizers the reference
drives (``mindspeed_rl/models/base/base_training_engine.py:523-531``).

Host mode keeps ``master / exp_avg / exp_avg_sq`` in pinned memory and streams them through two
device staging buffers in ``swap_optimizer_times`` chunks, overlapping H2D, the Adam kernel and
D2H on separate streams (reference feature: ``docs/zh/features/swap_optimizer.md:17-33``).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..parallel.ddp import ParamAndGradBuffer


class OptimizerParamScheduler:
    """Learning-rate schedule: linear warm-up then constant / linear / cosine decay."""

    def __init__(self, optimizer, max_lr: float, min_lr: float = 0.0, lr_warmup_steps: int = 0,
                 lr_decay_steps: int = 1, lr_decay_style: str = "constant"):
        self.optimizer = optimizer
        self.max_lr, self.min_lr = float(max_lr), float(min_lr)
        self.lr_warmup_steps, self.lr_decay_steps = lr_warmup_steps, max(lr_decay_steps, 1)
        self.lr_decay_style = lr_decay_style
        self.num_steps = 0
        self.step(0)

    def get_lr(self) -> float:
        n = self.num_steps
        if self.lr_warmup_steps > 0 and n <= self.lr_warmup_steps:
            return self.max_lr * n / self.lr_warmup_steps
        if self.lr_decay_style == "constant":
            return self.max_lr
        if n > self.lr_decay_steps:
            return self.min_lr
        ratio = (n - self.lr_warmup_steps) / max(self.lr_decay_steps - self.lr_warmup_steps, 1)
        delta = self.max_lr - self.min_lr
        if self.lr_decay_style == "linear":
            coeff = 1.0 - ratio
        elif self.lr_decay_style == "cosine":
            coeff = 0.5 * (math.cos(math.pi * ratio) + 1.0)
        else:
            raise ValueError(f"unknown lr_decay_style {self.lr_decay_style}")
        return self.min_lr + coeff * delta

    def step(self, increment: int = 1) -> None:
        self.num_steps += increment
        lr = self.get_lr()
        for g in self.optimizer.param_groups:
            g["lr"] = lr

    def state_dict(self):
        return dict(max_lr=self.max_lr, min_lr=self.min_lr, lr_warmup_steps=self.lr_warmup_steps,
                    lr_decay_steps=self.lr_decay_steps, lr_decay_style=self.lr_decay_style,
                    num_steps=self.num_steps)

    def load_state_dict(self, sd):
        self.num_steps = 0
        self.step(sd.get("num_steps", 0))


class DistributedOptimizer:
    def __init__(self, buffers: List[ParamAndGradBuffer], lr: float = 1e-6, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.01, clip_grad: float = 1.0,
                 dp_group=None, dp_rank: int = 0, model_parallel_group=None,
                 offload_to_host: bool = False, swap_chunks: int = 16,
                 norm_duplicate_filter=None, tp_rank: int = 0, reuse_fp32_param: bool = False,
                 overlap_param_gather: bool = False, gather_chunks: int = 8):
        self.buffers = buffers
        # update the shard chunk by chunk and fetch finished chunks from the peers meanwhile
        self.overlap_param_gather = bool(overlap_param_gather) and not offload_to_host
        self.gather_chunks = max(1, int(gather_chunks))
        self._gatherers: Dict[int, object] = {}
        # bf16 parameters double as the upper half of the fp32 master weights: only a 16-bit residual
        # is kept per element (2 bytes instead of 4; reference flag ``reuse_fp32_param``,
        # docs/zh/features/reuse_fp32_param.md in MindSpeed)
        self.reuse_fp32_param = bool(reuse_fp32_param) and not offload_to_host and \
            all(b.param_dtype == torch.bfloat16 for b in buffers)
        self.tp_rank = tp_rank
        self._rep_ranges = None
        self.param_groups = [dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)]
        self.clip_grad = clip_grad
        self.dp_group, self.dp_rank = dp_group, dp_rank
        self.mp_group = model_parallel_group
        self.offload_to_host = offload_to_host
        self.swap_chunks = max(1, swap_chunks)
        self.step_count = 0
        self.state: List[Dict[str, torch.Tensor]] = []
        self.norm_duplicate_filter = norm_duplicate_filter
        for buf in buffers:
            s, e = self._range(buf)
            shard = buf.param_data[s:e]
            if offload_to_host:
                pin = shard.is_cuda
                master = torch.empty(e - s, dtype=torch.float32, pin_memory=pin)
                master.copy_(shard.float())
                st = dict(master=master,
                          exp_avg=torch.zeros(e - s, dtype=torch.float32, pin_memory=pin),
                          exp_avg_sq=torch.zeros(e - s, dtype=torch.float32, pin_memory=pin))
            elif self.reuse_fp32_param:
                st = dict(master_lo=torch.zeros(e - s, dtype=torch.int16, device=shard.device),
                          exp_avg=torch.zeros(e - s, dtype=torch.float32, device=shard.device),
                          exp_avg_sq=torch.zeros(e - s, dtype=torch.float32, device=shard.device))
            else:
                st = dict(master=shard.float().clone(), exp_avg=torch.zeros(e - s, dtype=torch.float32,
                                                                            device=shard.device),
                          exp_avg_sq=torch.zeros(e - s, dtype=torch.float32, device=shard.device))
            self.state.append(st)
        dev = buffers[0].device
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._coef = torch.ones(1, dtype=torch.float32, device=dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self._streams = None

    # ------------------------------------------------------------------------------------------
    def zero_grad(self, set_to_none: bool = True) -> None:
        for b in self.buffers:
            b.zero_grad()

    _REPLICATED_SUFFIXES = ("layernorm.weight", "router.weight", "rm_head.weight", "rm_head.bias")

    def _replicated_ranges(self):
        """``(buffer index, lo, hi)`` element ranges of TP-replicated parameters inside this DP
        rank's shard (cached; the layout never changes)."""
        if self._rep_ranges is None:
            out = []
            for bi, buf in enumerate(self.buffers):
                s, e = self._range(buf)
                for p, slot in zip(buf.params, buf.slots):
                    if slot.name.endswith(self._REPLICATED_SUFFIXES) or getattr(p, "tp_replicated", False):
                        lo, hi = max(slot.start, s), min(slot.start + slot.numel, e)
                        if lo < hi:
                            out.append((bi, lo, hi))
            self._rep_ranges = out
        return self._rep_ranges

    def _range(self, buf: ParamAndGradBuffer) -> Tuple[int, int]:
        """This rank's shard of ``buf``: buffers that carry their own replica group (expert
        weights: expert-data-parallel ranks) are sharded over it, the others over ``dp_group``."""
        own = getattr(buf, "group", None) is not None or getattr(buf, "is_expert", False)
        return buf.shard_range(buf.dp_rank if own else self.dp_rank)

    def _grad_shard(self, buf: ParamAndGradBuffer) -> torch.Tensor:
        s, e = self._range(buf)
        return buf.grad_data[s:e]

    def compute_grad_norm(self) -> torch.Tensor:
        """Global L2 norm of the (already reduced) gradients; stays on the device."""
        self._sumsq.zero_()
        for buf in self.buffers:
            ops.sumsq_accumulate(self._grad_shard(buf), self._sumsq)
        if self.tp_rank > 0:
            # parameters replicated over TP must count once: the other TP ranks drop their copies
            dup = torch.zeros_like(self._sumsq)
            for bi, lo, hi in self._replicated_ranges():
                ops.sumsq_accumulate(self.buffers[bi].grad_data[lo:hi], dup)
            self._sumsq -= dup
        if dist.is_available() and dist.is_initialized():
            # every element of every shard (dense: one shard per DP rank; experts: one shard per
            # (EP, expert-DP) rank, all inside the DP group) is counted exactly once by this sum
            if self.dp_group is not None and dist.get_world_size(self.dp_group) > 1 and (
                    buffers_dp(self.buffers) > 1 or any(getattr(b, "is_expert", False) for b in self.buffers)):
                dist.all_reduce(self._sumsq, group=self.dp_group)
            if self.mp_group is not None and dist.get_world_size(self.mp_group) > 1:
                dist.all_reduce(self._sumsq, group=self.mp_group)
        return self._sumsq

    @torch.no_grad()
    def step(self) -> Tuple[bool, torch.Tensor, int]:
        self.step_count += 1
        g = self.param_groups[0]
        self.compute_grad_norm()
        ops.clip_coefficient(self._sumsq, float(self.clip_grad or 0.0), 1.0, self._coef, self._norm)
        for buf, st in zip(self.buffers, self.state):
            s, e = self._range(buf)
            grad = buf.grad_data[s:e]
            p16 = buf.param_data[s:e] if buf.param_dtype != torch.float32 else None
            if self.offload_to_host:
                self._step_host(st, grad, p16 if p16 is not None else buf.param_data[s:e], g,
                                p16 is None)
            elif self.reuse_fp32_param:
                self._step_reuse(st, grad, p16, g)
            elif self.overlap_param_gather and buf.dp_size > 1 and (buf.group is not None or self.dp_group is not None):
                self._step_pipelined(buf, st, grad, p16, g, s)
                continue
            else:
                ops.adamw_step(st["master"], st["exp_avg"], st["exp_avg_sq"], grad, p16, g["lr"],
                               g["betas"][0], g["betas"][1], g["eps"], g["weight_decay"],
                               self.step_count, self._coef)
                if p16 is None:
                    buf.param_data[s:e].copy_(st["master"])
            buf.gather_params(self.dp_group)
        return True, self._norm.clone(), 0

    def _step_pipelined(self, buf, st, grad, p16, g, s: int) -> None:
        """AdamW on the shard in chunks, each chunk's all-gather launched behind its update."""
        from ..parallel.ddp import ChunkedParamGather

        gatherer = self._gatherers.get(id(buf))
        if gatherer is None or gatherer.buf.param_data.data_ptr() != buf.param_data.data_ptr():
            gatherer = self._gatherers[id(buf)] = ChunkedParamGather(buf, self.dp_group, self.gather_chunks)
        for c, (lo, hi) in enumerate(gatherer.bounds):
            if self.reuse_fp32_param:
                self._step_reuse({k: (v[lo:hi] if torch.is_tensor(v) else v) for k, v in st.items()}, grad[lo:hi],
                                 p16[lo:hi], g)
            else:
                ops.adamw_step(st["master"][lo:hi], st["exp_avg"][lo:hi], st["exp_avg_sq"][lo:hi], grad[lo:hi],
                               p16[lo:hi] if p16 is not None else None, g["lr"], g["betas"][0], g["betas"][1],
                               g["eps"], g["weight_decay"], self.step_count, self._coef)
                if p16 is None:
                    buf.param_data[s + lo:s + hi].copy_(st["master"][lo:hi])
            gatherer.launch(c)
        gatherer.finish()

    # ---- fp32 master = (bf16 parameter, int16 residual) ------------------------------------------
    @staticmethod
    def compose_master(p16: torch.Tensor, lo: torch.Tensor) -> torch.Tensor:
        """fp32 bits = (bf16 bits << 16) + residual (signed)."""
        bits = (p16.view(torch.int16).to(torch.int32) << 16) + lo.to(torch.int32)
        return bits.view(torch.float32)

    @staticmethod
    def split_master(master: torch.Tensor, p16_out: torch.Tensor, lo_out: torch.Tensor) -> None:
        """bf16 = fp32 rounded half-up on the bit pattern, residual = fp32 bits - (bf16 bits << 16),
        which always fits 16 signed bits, so ``compose_master`` is exact."""
        bits = master.view(torch.int32)
        hi = (bits + 0x8000) >> 16
        p16_out.view(torch.int16).copy_(hi.to(torch.int16))
        lo_out.copy_((bits - (hi << 16)).to(torch.int16))

    def _step_reuse(self, st, grad, p16, g, chunk: int = 1 << 25) -> None:
        n = grad.numel()
        for s in range(0, n, chunk):
            e = min(n, s + chunk)
            master = self.compose_master(p16[s:e], st["master_lo"][s:e])
            ops.adamw_step(master, st["exp_avg"][s:e], st["exp_avg_sq"][s:e], grad[s:e], None, g["lr"],
                           g["betas"][0], g["betas"][1], g["eps"], g["weight_decay"], self.step_count, self._coef)
            self.split_master(master, p16[s:e], st["master_lo"][s:e])

    def _step_host(self, st, grad, p_out, g, fp32_params: bool) -> None:
        """Chunked H2D -> AdamW -> D2H with double buffering.  On a CPU tensor the same chunk loop runs without
        streams (the copies are then plain copies), which is how the chunk arithmetic is tested."""
        n = grad.numel()
        chunk = (n + self.swap_chunks - 1) // self.swap_chunks
        chunk = (chunk + 63) // 64 * 64
        dev = grad.device
        cuda = grad.is_cuda
        if self._streams is None:
            self._streams = (torch.cuda.Stream(), torch.cuda.Stream()) if cuda else (None, None)
            self._stage = [
                {k: torch.empty(chunk, dtype=torch.float32, device=dev) for k in ("master", "exp_avg", "exp_avg_sq")}
                for _ in range(2)]
        if self._stage[0]["master"].numel() < chunk:
            self._stage = [
                {k: torch.empty(chunk, dtype=torch.float32, device=dev) for k in ("master", "exp_avg", "exp_avg_sq")}
                for _ in range(2)]
        h2d, d2h = self._streams
        main = torch.cuda.current_stream() if cuda else None
        if cuda:
            h2d.wait_stream(main)
            d2h.wait_stream(main)
        done_events = [None, None]
        for i, s in enumerate(range(0, n, chunk)):
            e = min(n, s + chunk)
            k = i & 1
            stage = self._stage[k]
            if cuda:
                if done_events[k] is not None:
                    h2d.wait_event(done_events[k])     # staging buffer free again
                with torch.cuda.stream(h2d):
                    for key in ("master", "exp_avg", "exp_avg_sq"):
                        stage[key][:e - s].copy_(st[key][s:e], non_blocking=True)
                    ready = torch.cuda.Event()
                    ready.record(h2d)
                main.wait_event(ready)
            else:
                for key in ("master", "exp_avg", "exp_avg_sq"):
                    stage[key][:e - s].copy_(st[key][s:e])
            ops.adamw_step(stage["master"][:e - s], stage["exp_avg"][:e - s], stage["exp_avg_sq"][:e - s],
                           grad[s:e], None if fp32_params else p_out[s:e], g["lr"], g["betas"][0],
                           g["betas"][1], g["eps"], g["weight_decay"], self.step_count, self._coef)
            if fp32_params:
                p_out[s:e].copy_(stage["master"][:e - s])
            if cuda:
                computed = torch.cuda.Event()
                computed.record(main)
                d2h.wait_event(computed)
                with torch.cuda.stream(d2h):
                    for key in ("master", "exp_avg", "exp_avg_sq"):
                        st[key][s:e].copy_(stage[key][:e - s], non_blocking=True)
                    done = torch.cuda.Event()
                    done.record(d2h)
                done_events[k] = done
            else:
                for key in ("master", "exp_avg", "exp_avg_sq"):
                    st[key][s:e].copy_(stage[key][:e - s])
        if cuda:
            main.wait_stream(d2h)

    # ---- master <-> working copy ------------------------------------------------------------------
    def reload_model_params(self) -> None:
        """Refresh the fp32 master weights from the (externally modified) model parameters."""
        for buf, st in zip(self.buffers, self.state):
            s, e = self._range(buf)
            if "master_lo" in st:
                st["master_lo"].zero_()
            else:
                st["master"].copy_(buf.param_data[s:e].float())

    # ---- checkpoint ---------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        if self.offload_to_host and torch.cuda.is_available():
            torch.cuda.synchronize()        # the last step's device-to-host copies must have landed
        shards = []
        for buf, st in zip(self.buffers, self.state):
            d = {k: v.detach().cpu() for k, v in st.items() if k != "master_lo"}
            if "master_lo" in st:        # checkpoints always carry full fp32 master weights
                s, e = self._range(buf)
                d["master"] = self.compose_master(buf.param_data[s:e], st["master_lo"]).cpu()
            shards.append(d)
        return dict(step=self.step_count, param_groups=self.param_groups, shards=shards)

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = sd.get("step", 0)
        for buf, st, src in zip(self.buffers, self.state, sd["shards"]):
            for k in st:
                if k == "master_lo":
                    s, e = self._range(buf)
                    self.split_master(src["master"].to(st[k].device), buf.param_data[s:e], st[k])
                else:
                    st[k].copy_(src[k])

    # ---- memory choreography (offload between phases) --------------------------------------------
    def offload_state(self) -> None:
        """Move device-resident optimizer state to pinned host memory (rollout phase)."""
        if self.offload_to_host:
            return
        moved = False
        for st in self.state:
            for k, v in list(st.items()):
                if v.is_cuda:
                    host = torch.empty(v.shape, dtype=v.dtype, pin_memory=True)
                    host.copy_(v, non_blocking=True)
                    st[k] = host
                    moved = True
        if moved:
            torch.cuda.synchronize()
        self._state_offloaded = moved or getattr(self, "_state_offloaded", False)

    def onload_state(self) -> None:
        if not getattr(self, "_state_offloaded", False):
            return
        dev = self.buffers[0].device
        for st in self.state:
            for k, v in list(st.items()):
                st[k] = v.to(dev, non_blocking=True)
        self._state_offloaded = False


def buffers_dp(buffers: List[ParamAndGradBuffer]) -> int:
    return buffers[0].dp_size if buffers else 1
