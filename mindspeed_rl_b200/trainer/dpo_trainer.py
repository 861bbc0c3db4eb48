"""Direct preference optimisation (and plain SFT) trainer -- the non-RL ``torchrun`` path.

Batches are pairwise: the first half of the rows are the *chosen* sequences, the second half
the *rejected* ones, with ``labels == -100`` on prompt tokens.  The policy and a frozen reference
each produce per-sequence log-probabilities (sum over answer tokens, from the fused LM-head
kernel); the sigmoid DPO loss (``-log sigmoid(beta * ((pi_c - pi_r) - (ref_c - ref_r)))``, also
``hinge`` / ``ipo``) is evaluated in fp32 and its gradient w.r.t. the token log-probs is fed
straight into the model backward.  The reference implements this stage by delegating to an
external trainer (``cli/train_dpo.py:84,144-145``); here it is native.
"""
from __future__ import annotations

import time
from typing import Any, Dict, Iterator, List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..models.gpt import GPTModel, PackedMeta
from ..obs.io_counter import to_device
from ..obs.loggers import Loggers


def _pack_pairwise(batch: Dict[str, torch.Tensor], pad_multiple: int = 1):
    """Padded ``[2B, S]`` ids / labels / mask -> packed stream + per-token answer mask + row ids."""
    ids, labels, mask = batch["input_ids"], batch["labels"], batch["attention_mask"]
    lens = mask.sum(-1).to(torch.int64)
    b, s = ids.shape
    col = torch.arange(s).unsqueeze(0)
    valid = col < lens.unsqueeze(1)
    padded = (lens + pad_multiple - 1) // pad_multiple * pad_multiple
    cu = torch.zeros(b + 1, dtype=torch.int64)
    cu[1:] = torch.cumsum(padded, 0)
    total = int(cu[-1])
    dest = (cu[:-1].unsqueeze(1) + col)[valid]
    flat_ids = torch.zeros(total, dtype=torch.int64)
    flat_ids[dest] = ids[valid]
    # next-token targets; a position counts when its *target* is an answer token
    nxt = torch.cat([labels[:, 1:], torch.full((b, 1), -100, dtype=labels.dtype)], dim=1)
    flat_tgt = torch.full((total,), -100, dtype=torch.int64)
    flat_tgt[dest] = nxt[valid]
    row = torch.repeat_interleave(torch.arange(b), padded)
    pos = torch.arange(total) - torch.repeat_interleave(cu[:-1], padded)
    return flat_ids, flat_tgt, row, pos.to(torch.int32), cu.to(torch.int32), int(padded.max())


def sequence_logps(model: GPTModel, batch: Dict[str, torch.Tensor], device, pad_multiple: int = 1):
    ids, tgt, row, pos, cu, max_len = _pack_pairwise(batch, pad_multiple)
    answer = tgt != -100
    labels = torch.where(answer, tgt, torch.zeros_like(tgt))
    d = lambda t: to_device(t, t.dtype, device)
    logp, _ = model.forward_logprob(d(ids), d(labels), PackedMeta(d(cu), max_len, d(pos)))
    w = d(answer.float())
    seq = torch.zeros(batch["input_ids"].shape[0], device=logp.device, dtype=torch.float32)
    seq = seq.index_add(0, d(row), logp * w)
    return seq, w.sum()


def dpo_loss(pi_c, pi_r, ref_c, ref_r, beta: float, loss_type: str = "sigmoid", label_smoothing: float = 0.0):
    logits = (pi_c - pi_r) - (ref_c - ref_r)
    if loss_type == "sigmoid":
        loss = -F.logsigmoid(beta * logits) * (1 - label_smoothing) - F.logsigmoid(-beta * logits) * label_smoothing
    elif loss_type == "hinge":
        loss = torch.relu(1 - beta * logits)
    elif loss_type == "ipo":
        loss = (logits - 1 / (2 * beta)) ** 2
    else:
        raise ValueError(f"unknown dpo_loss_type '{loss_type}'")
    chosen_r = beta * (pi_c - ref_c).detach()
    rejected_r = beta * (pi_r - ref_r).detach()
    return loss.mean(), chosen_r, rejected_r


class DPOTrainer:
    def __init__(self, model, ref_model: Optional[GPTModel], optimizer, scheduler=None, *, beta: float = 0.1,
                 loss_type: str = "sigmoid", train_iters: int = 1, device=None, pad_multiple: int = 1,
                 dp_group=None, dp_rank: int = 0, dp_size: int = 1, log_interval: int = 1, save_fn=None,
                 save_interval: int = 0):
        """``dp_size`` > 1: every rank is handed the same global batch and trains on its own slice of the pairs
        (rows ``[rank * B / dp, (rank + 1) * B / dp)`` of the chosen and of the rejected half); the reported
        numbers are averaged over ``dp_group``."""
        self.model = model
        self.core = model.module if hasattr(model, "module") else model
        self.ref_model, self.optimizer, self.scheduler = ref_model, optimizer, scheduler
        self.beta, self.loss_type, self.train_iters = beta, loss_type, train_iters
        self.device = device or next(self.core.parameters()).device
        self.pad_multiple, self.dp_group = pad_multiple, dp_group
        self.dp_rank, self.dp_size = dp_rank, max(int(dp_size), 1)
        self.log_interval, self.save_fn, self.save_interval = log_interval, save_fn, save_interval
        self.logger = Loggers("DPOTrainer")
        self.iteration = 0

    def _my_pairs(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        if self.dp_size == 1:
            return batch
        half = batch["input_ids"].shape[0] // 2
        if half % self.dp_size:
            raise ValueError(f"{half} pairs per step do not divide over {self.dp_size} data-parallel ranks")
        per = half // self.dp_size
        rows = torch.arange(self.dp_rank * per, (self.dp_rank + 1) * per)
        rows = torch.cat([rows, half + rows])
        return {k: (v[rows] if torch.is_tensor(v) and v.dim() > 0 and v.shape[0] == 2 * half else v)
                for k, v in batch.items()}

    def _mean_over_replicas(self, values: Dict[str, float]) -> Dict[str, float]:
        if self.dp_size == 1 or not (dist.is_available() and dist.is_initialized()):
            return values
        keys = sorted(values)
        dev = self.device if dist.get_backend(self.dp_group) == "nccl" else "cpu"
        t = torch.tensor([values[k] for k in keys], dtype=torch.float64, device=dev)
        dist.all_reduce(t, group=self.dp_group)
        return {k: float(v) / self.dp_size for k, v in zip(keys, t.tolist())}

    def train_step(self, batch: Dict[str, torch.Tensor]) -> Dict[str, float]:
        batch = self._my_pairs(batch)
        half = batch["input_ids"].shape[0] // 2
        if hasattr(self.model, "zero_grad_buffer"):
            self.model.zero_grad_buffer()
        with torch.no_grad():
            if self.ref_model is not None:
                ref, _ = sequence_logps(self.ref_model, batch, self.device, self.pad_multiple)
            else:
                ref = torch.zeros(2 * half, device=self.device)
        seq, _ = sequence_logps(self.core, batch, self.device, self.pad_multiple)
        loss, cr, rr = dpo_loss(seq[:half], seq[half:], ref[:half], ref[half:], self.beta, self.loss_type)
        loss.backward()
        if hasattr(self.model, "finish_grad_sync"):
            self.model.finish_grad_sync(to_shards=True)
        _, grad_norm, _ = self.optimizer.step()
        if self.scheduler is not None:
            self.scheduler.step(increment=2 * half)
        out = self._mean_over_replicas({
            "dpo/loss": float(loss.detach()), "dpo/rewards_chosen": float(cr.mean()), "dpo/rewards_rejected": float(rr.mean()),
            "dpo/accuracy": float((cr > rr).float().mean()), "dpo/margin": float((cr - rr).mean())})
        out["grad_norm"] = float(grad_norm)
        out["lr"] = self.optimizer.param_groups[0]["lr"]
        out["pairs"] = half * self.dp_size
        return out

    def train(self, data_iter: Iterator[Dict[str, torch.Tensor]]) -> List[Dict[str, float]]:
        history = []
        while self.iteration < self.train_iters:
            t0 = time.time()
            m = self.train_step(next(data_iter))
            self.iteration += 1
            dt = time.time() - t0
            m["samples_per_sec"] = m.pop("pairs") / max(dt, 1e-9)
            m["time"] = dt
            history.append(m)
            if self.iteration % self.log_interval == 0:
                self.logger.info(m, self.iteration, self.train_iters)
            if self.save_fn and self.save_interval and self.iteration % self.save_interval == 0:
                self.save_fn(self.iteration)
        return history
