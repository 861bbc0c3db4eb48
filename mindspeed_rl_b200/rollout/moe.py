"""Expert layers of the rollout model runner.

``MoEWeights.forward`` routes the step's tokens (top-k, optional EPLB logical->physical expert
map), exchanges them over the expert-parallel group with an all-to-all (counts first, then
tokens), runs the local experts' ``w1 -> SwiGLU -> w2`` and combines the weighted results back
at the source rank.  Per-expert token counts can be accumulated for the expert-parallel load
balancer (reference: ``models/rollout/vllm_adapter/fused_moe.py:230-503``).
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..models.moe import route


_side_streams = {}


class MoEWeights:
    def __init__(self, cfg, router_w: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, ep_group=None,
                 ep_size: int = 1, ep_rank: int = 0, shared: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                 log2phy: Optional[torch.Tensor] = None, collect_counts: bool = False, p2p=None,
                 expert_bias: Optional[torch.Tensor] = None):
        """``w1 [H, E_local, 2F]``, ``w2 [E_local, F, H]`` (views are fine)."""
        self.cfg = cfg
        self.router_w, self.w1, self.w2 = router_w, w1, w2
        self.ep_group, self.ep_size, self.ep_rank = ep_group, ep_size, ep_rank
        self.num_local = w2.shape[0]
        self.shared = shared
        self.p2p = p2p                      # callable(x) -> peer-memory dispatcher of the EP group, or None
        self.log2phy = log2phy              # [E_logical, max_replicas] physical ids (-1 padded) or None
        self.collect_counts = collect_counts
        self.expert_bias = expert_bias      # selection bias of aux-loss-free balancing, or None
        self.counts = torch.zeros(cfg.num_experts, dtype=torch.int64)

    def _physical(self, top_idx: torch.Tensor) -> torch.Tensor:
        """EPLB: spread a logical expert's tokens round-robin over its physical replicas."""
        if self.log2phy is None:
            return top_idx
        table = self.log2phy.to(top_idx.device)
        n_rep = (table >= 0).sum(-1)
        slot = torch.arange(top_idx.numel(), device=top_idx.device).view_as(top_idx) % n_rep[top_idx]
        return table[top_idx, slot]

    @torch.no_grad()
    def forward(self, x: torch.Tensor, comm=None) -> torch.Tensor:
        cfg = self.cfg
        t, k = x.shape[0], cfg.moe_router_topk
        fork = self._fork_shared(x)
        logits = torch.matmul(x.float(), self.router_w.float().t())
        top_p, top_idx, _ = route(logits, cfg, self.expert_bias)
        if self.collect_counts:
            self.counts += torch.bincount(top_idx.reshape(-1).cpu(), minlength=cfg.num_experts)
        phys = self._physical(top_idx)
        n_phys = self.num_local * self.ep_size
        if self.ep_size == 1:
            # all experts here: plan + permute + grouped GEMMs + combine, no host round trip
            from ..ops import moe as K
            h, f = x.shape[1], self.w2.shape[1]
            plan = K.moe_plan(phys, n_phys)
            gu = K.grouped_gemm(K.moe_permute(x, plan), plan, self.w1.reshape(h, n_phys * 2 * f), True, 2 * f, 0, 2 * f)
            y = K.grouped_gemm(ops.swiglu_fwd(gu), plan, self.w2.reshape(n_phys * f, h), True, 0, f, h)
            out = K.moe_combine(y, plan, top_p)
            return self._add_shared(out, x, comm, fork)
        disp = self.p2p(x) if (self.p2p is not None and self.ep_size > 1) else None
        if disp is not None and disp.e_local == self.num_local:
            # tokens go straight into the expert slabs of their ranks and the outputs are pulled back:
            # no collective, no host round trip
            from ..ops import moe as K
            h, f = x.shape[1], self.w2.shape[1]
            e = self.num_local
            rt = disp.dispatch(x, phys)
            if rt is not None:       # None: some member's slab would overflow, all members use the collectives below
                # slab-sized intermediates come from grow-only scratch shared by all layers (and by all
                # captured decode graphs, which would otherwise each keep a private copy)
                from ..ops.elementwise import _workspace
                rows = disp.slab.shape[0]
                gu = _workspace("rollout_moe_gu", rows * 2 * f, x.device, x.dtype)[:rows * 2 * f].view(rows, 2 * f)
                act = _workspace("rollout_moe_act", rows * f, x.device, x.dtype)[:rows * f].view(rows, f)
                K.grouped_gemm(disp.slab, rt.plan, self.w1.reshape(h, e * 2 * f), True, 2 * f, 0, 2 * f, out=gu)
                K.grouped_gemm(ops.swiglu_fwd(gu, out=act), rt.plan, self.w2.reshape(e * f, h), True, 0, f, h,
                               out=disp.out_slab)
                out, _ = disp.combine(rt, top_p)
                return self._add_shared(out, x, comm, fork)
        flat = phys.reshape(-1)
        order = torch.argsort(flat, stable=True)
        token_of = order // k
        xp = x[token_of]
        counts = torch.bincount(flat, minlength=n_phys)
        if self.ep_size > 1:
            send = counts.view(self.ep_size, self.num_local)
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send.contiguous(), group=self.ep_group)
            send_rows, recv_rows = send.sum(1).tolist(), recv.sum(1).tolist()
            got = torch.empty(sum(recv_rows), x.shape[1], device=x.device, dtype=x.dtype)
            dist.all_to_all_single(got, xp.contiguous(), recv_rows, send_rows, group=self.ep_group)
            recv_l = recv.tolist()
            y_got = torch.empty_like(got)
            s = 0
            for r in range(self.ep_size):          # segments are (source rank, local expert)
                for j in range(self.num_local):
                    n = recv_l[r][j]
                    if n:
                        self._expert(got[s:s + n], j, y_got[s:s + n])
                    s += n
            y = torch.empty_like(xp)
            dist.all_to_all_single(y, y_got, send_rows, recv_rows, group=self.ep_group)
        else:
            y = torch.empty_like(xp)
            s = 0
            for j, n in enumerate(counts.tolist()):
                if n:
                    self._expert(xp[s:s + n], j, y[s:s + n])
                s += n
        w = top_p.reshape(-1)[order].to(x.dtype)
        out = torch.zeros(t, x.shape[1], device=x.device, dtype=torch.float32)
        out.index_add_(0, token_of, (y * w.unsqueeze(-1)).float())
        return self._add_shared(out.to(x.dtype), x, comm, fork)

    def _shared_mlp(self, x: torch.Tensor) -> torch.Tensor:
        from ..ops.gemm import linear_fwd

        fc1, fc2 = self.shared
        return linear_fwd(ops.swiglu_fwd(linear_fwd(x, fc1)), fc2)

    def _fork_shared(self, x: torch.Tensor):
        """Start the shared experts on a side stream, so that they run beside the routed experts' token
        exchange and grouped GEMMs (reference: the shared-expert stream of the fused MoE layer,
        ``models/rollout/vllm_adapter/fused_moe.py:230-373``).  Works inside a stream capture (the fork and
        the join become edges of the graph).  ``MSRL_MOE_SHARED_STREAM=0`` keeps everything on one stream."""
        if self.shared is None or not x.is_cuda or os.environ.get("MSRL_MOE_SHARED_STREAM", "1") != "1":
            return None
        side = _side_streams.get(x.device)
        if side is None:
            side = _side_streams[x.device] = torch.cuda.Stream(device=x.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            sh = self._shared_mlp(x)
        x.record_stream(side)
        return side, sh

    def _add_shared(self, out: torch.Tensor, x: torch.Tensor, comm, fork=None) -> torch.Tensor:
        if self.shared is None:
            return out
        if fork is not None:
            side, sh = fork
            torch.cuda.current_stream().wait_stream(side)
            sh.record_stream(torch.cuda.current_stream())
        else:
            sh = self._shared_mlp(x)
        return out + (comm.all_reduce(sh) if comm is not None else sh)

    def _expert(self, x: torch.Tensor, j: int, out: torch.Tensor) -> None:
        act = ops.swiglu_fwd(torch.matmul(x, self.w1[:, j]))
        torch.matmul(act, self.w2[j], out=out)

    def dump_counts(self, path: str, layer: int, rank: int) -> None:
        """Append this layer's ``{expert: count}`` to ``eplb_token_collects_{rank}.json``."""
        f = os.path.join(path, f"eplb_token_collects_{rank}.json")
        data = json.load(open(f)) if os.path.isfile(f) else {}
        data[str(layer)] = {str(i): int(c) for i, c in enumerate(self.counts.tolist())}
        with open(f, "w") as fh:
            json.dump(data, fh)
