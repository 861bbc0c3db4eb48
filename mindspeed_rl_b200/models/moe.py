"""Mixture-of-experts MLP block (Qwen3-MoE / DeepSeek style) with expert parallelism.

``tokens -> router (softmax | sigmoid, top-k, optional group-limited routing, renormalisation)
-> dispatch (permute by expert; all-to-all over the EP group) -> grouped expert GEMMs
(w1 -> SwiGLU -> w2) -> combine (weighted un-permute; all-to-all back) [+ shared experts]``

Parameter layout follows Megatron's ``GroupedMLP``: ``experts.weight1 [H, E_local * 2 * F]`` (per
expert ``[gate | up]`` columns), ``experts.weight2 [E_local * F, H]``, ``router.weight [E, H]``.
The experts' forward/backward is written by hand (like the dense layer); only the tiny router
graph ``[T, E]`` goes through autograd so that the load-balancing auxiliary loss and the
probability gradients need no hand derivation.

Three execution paths share the expert math (dispatch plan, permute / combine and the grouped
tcgen05 GEMM of ``ops/moe.py``, which read the stacked expert weights in place):
all experts on this rank (no host round trip in the forward); expert parallel with
``all_to_all_single`` over the EP group (counts on the host, any backend, also gloo);
expert parallel over peer-mapped memory (``parallel/moe_dispatch.py``: tokens are written straight
into the destination ranks' expert slabs and outputs are pulled back, chosen when
``moe_p2p_dispatch_rows`` > 0 and a symmetric arena exists).

Reference behaviour: flags ``moe_grouped_gemm``, ``moe_token_dispatcher_type: alltoall_seq``,
``moe_router_topk``, ``norm_topk_prob``, ``moe_aux_loss_coeff`` (``configs/model/qwen3_30b_a3b.yaml``)
and the rollout-side routing in ``models/rollout/vllm_adapter/fused_moe.py:230-503``.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..ops import gemm as _gemm
from ..parallel.state import get_parallel_state


def _normal(shape, std, dtype, device, gen):
    t = torch.empty(shape, dtype=torch.float32, device=device)
    t.normal_(0.0, std, generator=gen)
    return t.to(dtype)


class _W(nn.Module):
    def __init__(self, weight: torch.Tensor):
        super().__init__()
        self.weight = nn.Parameter(weight)


class _Experts(nn.Module):
    def __init__(self, w1: torch.Tensor, w2: torch.Tensor):
        super().__init__()
        self.weight1 = nn.Parameter(w1)
        self.weight2 = nn.Parameter(w2)


def route(logits: torch.Tensor, cfg, expert_bias: Optional[torch.Tensor] = None
          ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Router logits ``[T, E]`` (fp32) -> ``(top-k probabilities [T, k], expert ids [T, k], full
    score matrix [T, E])``; differentiable w.r.t. ``logits``.  ``expert_bias`` (load balancing without
    an auxiliary loss, ``moe_router_enable_expert_bias``) shifts the scores for the CHOICE of experts
    only; the combine weights stay the unbiased scores."""
    k = cfg.moe_router_topk
    if cfg.moe_router_score_function == "sigmoid":
        scores = torch.sigmoid(logits)
    else:
        scores = torch.softmax(logits, dim=-1)
    pick = scores if expert_bias is None else scores.detach() + expert_bias.to(scores.dtype)
    if cfg.moe_router_num_groups and cfg.moe_router_group_topk:
        t, e = scores.shape
        g = cfg.moe_router_num_groups
        grouped = scores.view(t, g, e // g)
        group_score = grouped.topk(min(2, e // g), dim=-1).values.sum(-1)
        keep = group_score.topk(cfg.moe_router_group_topk, dim=-1).indices
        mask = torch.zeros(t, g, dtype=torch.bool, device=scores.device).scatter_(1, keep, True)
        pick = scores.masked_fill(~mask.unsqueeze(-1).expand(t, g, e // g).reshape(t, e), float("-inf"))
    top_idx = pick.topk(k, dim=-1).indices
    top_p = scores.gather(-1, top_idx)
    if cfg.norm_topk_prob:
        top_p = top_p / (top_p.sum(-1, keepdim=True) + 1e-20)
    if cfg.moe_router_topk_scaling_factor:
        top_p = top_p * cfg.moe_router_topk_scaling_factor
    return top_p, top_idx, scores


def aux_loss(scores: torch.Tensor, top_idx: torch.Tensor, num_experts: int, topk: int, coeff: float) -> torch.Tensor:
    """Switch-style load balancing: ``coeff * E * sum_e f_e * P_e``."""
    t = scores.shape[0]
    counts = torch.zeros(num_experts, device=scores.device, dtype=scores.dtype)
    counts.scatter_add_(0, top_idx.reshape(-1), torch.ones(top_idx.numel(), device=scores.device, dtype=scores.dtype))
    f = counts / max(t * topk, 1)
    p = scores.mean(dim=0)
    return coeff * num_experts * (f * p).sum()


class MoELayer(nn.Module):
    def __init__(self, cfg, device, gen):
        super().__init__()
        self.cfg = cfg
        ps = get_parallel_state()
        self.ep_group = ps.group("ep")
        self.ep_size = ps.size("ep")
        self.ep_rank = ps.rank_in("ep")
        e, h, f = cfg.num_experts, cfg.hidden_size, cfg.moe_ffn_hidden_size
        if e % self.ep_size:
            raise ValueError("num_experts must be divisible by the expert-parallel size")
        self.num_local = e // self.ep_size
        layout = getattr(ps, "layout", None)
        tp = int(getattr(layout, "tp", 1) or 1)
        extend = bool(getattr(layout, "moe_tp_extend_ep", False))
        if tp > 1 and int(getattr(layout, "ep", 1) or 1) > 1 and not extend:
            raise ValueError("experts are never cut by tensor parallelism here: with tensor_model_parallel_size > 1 "
                             "and expert_model_parallel_size > 1 set moe_tp_extend_ep (experts spread over TP x EP)")
        if tp > 1 and extend and not cfg.sequence_parallel:
            raise ValueError("moe_tp_extend_ep with tensor parallelism needs sequence_parallel: every TP rank must "
                             "route its own tokens, or the experts would see every token tp times")
        # experts replicated over the TP group see only the local token shard under sequence parallelism:
        # their gradients are partial sums that the gradient sync adds up over TP (and counts once in the norm)
        self._experts_tp_partial = tp > 1 and not extend and bool(cfg.sequence_parallel)
        self._experts_tp_replicated = tp > 1 and not extend
        dt, std = cfg.params_dtype, cfg.init_method_std
        out_std = std / math.sqrt(2.0 * cfg.num_layers)
        self.router = _W(_normal((e, h), std, torch.float32, device, gen))
        if cfg.moe_router_enable_expert_bias:
            # not trained by gradients: nudged after every optimizer step towards an even load
            self.router.register_buffer("expert_bias", torch.zeros(e, dtype=torch.float32, device=device))
            self._load_since_update = torch.zeros(e, dtype=torch.float32, device=device)
        self.experts = _Experts(_normal((h, self.num_local * 2 * f), std, dt, device, gen),
                                _normal((self.num_local * f, h), out_std, dt, device, gen))
        for w in (self.experts.weight1, self.experts.weight2):
            w.tp_reduce_grad = self._experts_tp_partial
            w.tp_replicated = self._experts_tp_replicated
        self.shared_experts = None
        if cfg.n_shared_experts:
            from .gpt import MLP

            self.shared_experts = MLP(cfg, device, gen, ffn=f * cfg.n_shared_experts)
        self.last_aux_loss: Optional[torch.Tensor] = None
        self.token_counts: Optional[torch.Tensor] = None   # per-expert routed tokens (EPLB statistics)

    @torch.no_grad()
    def update_expert_bias(self, rate: float = 1e-3, group=None) -> None:
        """Auxiliary-loss-free balancing: after an optimizer step, raise the bias of experts that got
        fewer tokens than the mean since the last update and lower it for the others (all ranks of
        ``group`` see the same global load)."""
        if not self.cfg.moe_router_enable_expert_bias:
            return
        load = self._load_since_update
        if group is not None and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(load, group=group)
        self.router.expert_bias += rate * torch.sign(load.mean() - load)
        load.zero_()

    # ------------------------------------------------------------------------------------------
    def _w1(self) -> torch.Tensor:
        c = self.cfg
        return self.experts.weight1.view(c.hidden_size, self.num_local, 2 * c.moe_ffn_hidden_size)

    def _w2(self) -> torch.Tensor:
        c = self.cfg
        return self.experts.weight2.view(self.num_local, c.moe_ffn_hidden_size, c.hidden_size)

    def _exchange(self, x: torch.Tensor, send_counts: List[int], recv_counts: List[int]) -> torch.Tensor:
        out = torch.empty(sum(recv_counts), *x.shape[1:], device=x.device, dtype=x.dtype)
        dist.all_to_all_single(out, x.contiguous(), recv_counts, send_counts, group=self.ep_group)
        return out

    def _dispatch(self, x: torch.Tensor, top_idx: torch.Tensor):
        """Permute ``x`` rows into expert order (global experts), exchange over EP.

        Returns ``(xp_local, plan)`` where ``xp_local`` rows are grouped by local expert."""
        t, k = top_idx.shape
        e = self.cfg.num_experts
        flat = top_idx.reshape(-1)
        order = torch.argsort(flat, stable=True)                 # slots sorted by global expert
        token_of = order // k
        xp = x[token_of]
        counts = torch.bincount(flat, minlength=e)
        plan: Dict[str, Any] = dict(order=order, token_of=token_of, t=t, k=k)
        if self.ep_size == 1:
            plan["local_counts"] = counts.tolist()
            return xp, plan
        # counts exchange: row r of `recv` = tokens rank r sends to each of my local experts
        send = counts.view(self.ep_size, self.num_local)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send.contiguous(), group=self.ep_group)
        send_rows, recv_rows = send.sum(1).tolist(), recv.sum(1).tolist()
        got = self._exchange(xp, send_rows, recv_rows)          # grouped by (source rank, local expert)
        # regroup to (local expert, source rank)
        recv_l = recv.tolist()
        seg_starts, s = [], 0
        for r in range(self.ep_size):
            row = []
            for j in range(self.num_local):
                row.append(s)
                s += recv_l[r][j]
            seg_starts.append(row)
        idx = []
        for j in range(self.num_local):
            for r in range(self.ep_size):
                n = recv_l[r][j]
                if n:
                    idx.append(torch.arange(seg_starts[r][j], seg_starts[r][j] + n, device=x.device))
        perm = torch.cat(idx) if idx else torch.zeros(0, dtype=torch.long, device=x.device)
        plan.update(send_rows=send_rows, recv_rows=recv_rows, perm=perm,
                    local_counts=[sum(recv_l[r][j] for r in range(self.ep_size)) for j in range(self.num_local)])
        return got[perm], plan

    def _undispatch(self, y_local: torch.Tensor, plan) -> torch.Tensor:
        """Inverse of :meth:`_dispatch` for expert outputs (rows back in sorted-slot order)."""
        if self.ep_size == 1:
            return y_local
        back = torch.empty_like(y_local)
        back[plan["perm"]] = y_local
        return self._exchange(back, plan["recv_rows"], plan["send_rows"])

    def _redispatch(self, d_sorted: torch.Tensor, plan) -> torch.Tensor:
        """Send gradients w.r.t. expert outputs along the dispatch route."""
        if self.ep_size == 1:
            return d_sorted
        got = self._exchange(d_sorted, plan["send_rows"], plan["recv_rows"])
        return got[plan["perm"]]

    # ------------------------------------------------------------------------------------------
    def _experts_fwd(self, xp: torch.Tensor, counts: List[int], keep: bool):
        """Rows of ``xp`` are grouped by local expert (``counts`` rows each, known on the host after
        the count exchange).  They are re-laid into 128-row padded segments and run through the
        grouped GEMM kernels; the result comes back in the order of ``xp``."""
        from ..ops import moe as K

        c = self.cfg
        e, h, f = self.num_local, c.hidden_size, c.moe_ffn_hidden_size
        w1, w2 = self._w1().reshape(h, e * 2 * f), self._w2().reshape(e * f, h)
        ids = torch.repeat_interleave(torch.arange(e, device=xp.device),
                                      torch.tensor(counts, device=xp.device), output_size=xp.shape[0])
        plan = K.moe_plan(ids.view(-1, 1), e)
        xpp = K.moe_permute(xp, plan)
        gu = K.grouped_gemm(xpp, plan, w1, True, 2 * f, 0, 2 * f)
        act = ops.swiglu_fwd(gu)
        y = K.moe_combine(K.grouped_gemm(act, plan, w2, True, 0, f, h), plan)
        return y, ((plan, xpp, gu, act) if keep else None)

    def _experts_bwd(self, counts: List[int], ectx, dy: torch.Tensor) -> torch.Tensor:
        from ..ops import moe as K
        from .gpt import grad_buffer

        c = self.cfg
        e, h, f = self.num_local, c.hidden_size, c.moe_ffn_hidden_size
        w1, w2 = self._w1().reshape(h, e * 2 * f), self._w2().reshape(e * f, h)
        plan, xpp, gu, act = ectx
        dyp = K.moe_permute(dy, plan)
        dact = K.grouped_gemm(dyp, plan, w2, False, 0, f, f)
        dgu = ops.swiglu_bwd(gu, dact)
        dxp = K.moe_combine(K.grouped_gemm(dgu, plan, w1, False, 2 * f, 0, h), plan)
        if self.experts.weight1.requires_grad:
            g1 = grad_buffer(self.experts.weight1).view(h, e, 2 * f)
            g2 = grad_buffer(self.experts.weight2).view(e, f, h)
            start = 0                                   # padded segment starts follow from the host counts
            for j, n in enumerate(counts):
                if n:
                    r = slice(start, start + n)
                    g2[j].add_(torch.matmul(act[r].t(), dyp[r]).to(g2.dtype))
                    g1[:, j].add_(torch.matmul(xpp[r].t(), dgu[r]).to(g1.dtype))
                start += (n + K.PAD - 1) // K.PAD * K.PAD
        return dxp

    # ------------------------------------------------------------------------------------------
    def forward_tokens(self, x: torch.Tensor, comm, keep: bool):
        """``x [T, H]``: the tokens this rank owns (its sequence shard under sequence parallelism, all tokens
        otherwise) -> ``(out [T, H], ctx)``.  Routed experts are never cut by TP, so routing, dispatch and combine
        need no TP collective; only the shared experts (a tensor-parallel MLP) talk to the TP group."""
        cfg = self.cfg
        t = x.shape[0]
        with torch.enable_grad():
            xr = x.detach().float().requires_grad_(keep)
            logits = torch.matmul(xr, self.router.weight.t())
            top_p, top_idx, scores = route(logits, cfg, getattr(self.router, "expert_bias", None))
            aux = aux_loss(scores, top_idx, cfg.num_experts, cfg.moe_router_topk, cfg.moe_aux_loss_coeff) \
                if (keep and cfg.moe_aux_loss_coeff) else None
        self.last_aux_loss = aux.detach() if aux is not None else None
        self.token_counts = torch.bincount(top_idx.reshape(-1), minlength=cfg.num_experts)
        if cfg.moe_router_enable_expert_bias and keep:
            # ``keep`` marks the one pass per training step whose intermediates feed the backward (the recompute
            # pass under full recompute); forward-only passes (reference / old log-probs) do not count as load
            self._load_since_update += self.token_counts.float()
        if self.ep_size == 1:
            return self._forward_local(x, xr, top_p, top_idx, aux, comm, keep)
        disp = self._p2p_dispatcher(x)
        if disp is not None:
            done = self._forward_p2p(disp, x, xr, top_p, top_idx, aux, comm, keep)
            if done is not None:
                return done
            # the routing would overflow a member's slab: every member takes the all-to-all path below
        xp, plan = self._dispatch(x, top_idx)
        y_local, ectx = self._experts_fwd(xp, plan["local_counts"], keep)
        y_sorted = self._undispatch(y_local, plan)
        # combine: slot (token, k) weighted by its probability
        k = cfg.moe_router_topk
        w_sorted = top_p.detach().reshape(-1)[plan["order"]].to(x.dtype)
        out = torch.zeros(t, cfg.hidden_size, device=x.device, dtype=torch.float32)
        out.index_add_(0, plan["token_of"], (y_sorted * w_sorted.unsqueeze(-1)).float())
        out = out.to(x.dtype)
        shared_ctx = None
        if self.shared_experts is not None:
            sh, shared_ctx = self._shared_fwd(x, comm, keep)
            out = out + sh
        if not keep:
            return out, None
        ctx = dict(xr=xr, top_p=top_p, aux=aux, plan=plan, ectx=ectx, y_sorted=y_sorted,
                   w_sorted=w_sorted, shared=shared_ctx)
        return out, ctx

    # ---- all experts on this rank: dispatch plan + grouped GEMMs, no host round trip in the forward ----
    def _shared_fwd(self, x, comm, keep):
        """Shared experts are an ordinary tensor-parallel MLP over the tokens of this rank: tokens are gathered
        over TP under sequence parallelism (identity otherwise), the row-parallel output is reduce-scattered
        (all-reduced) back."""
        xg = comm.gather_seq(x)
        gu = _gemm.linear_fwd(xg, self.shared_experts.linear_fc1.weight)
        act = ops.swiglu_fwd(gu)
        y = comm.reduce_out(_gemm.linear_fwd(act, self.shared_experts.linear_fc2.weight))
        return y, ((xg, gu, act) if keep else None)

    def _shared_bwd(self, shared_ctx, dout, comm) -> torch.Tensor:
        from .gpt import accum_wgrad

        xg, gu, act = shared_ctx
        fc1, fc2 = self.shared_experts.linear_fc1.weight, self.shared_experts.linear_fc2.weight
        d_sh = comm.reduce_out_bwd(dout)
        dact = _gemm.linear_dgrad(d_sh, fc2)
        accum_wgrad(fc2, d_sh, act)
        dgu = ops.swiglu_bwd(gu, dact)
        accum_wgrad(fc1, dgu, xg)
        return comm.gather_seq_bwd(_gemm.linear_dgrad(dgu, fc1))

    def _forward_local(self, x, xr, top_p, top_idx, aux, comm, keep):
        from ..ops import moe as K

        c = self.cfg
        e, h, f = self.num_local, c.hidden_size, c.moe_ffn_hidden_size
        w1, w2 = self._w1().reshape(h, e * 2 * f), self._w2().reshape(e * f, h)
        plan = K.moe_plan(top_idx, e)
        xp = K.moe_permute(x, plan)
        gu = K.grouped_gemm(xp, plan, w1, True, 2 * f, 0, 2 * f)
        act = ops.swiglu_fwd(gu)
        y = K.grouped_gemm(act, plan, w2, True, 0, f, h)
        out = K.moe_combine(y, plan, top_p.detach())
        shared_ctx = None
        if self.shared_experts is not None:
            sh, shared_ctx = self._shared_fwd(x, comm, keep)
            out = out + sh
        if not keep:
            return out, None
        return out, dict(local=True, xr=xr, top_p=top_p, aux=aux, plan=plan, xp=xp, gu=gu, act=act, y=y,
                         shared=shared_ctx)

    # ---- expert parallel over peer-mapped memory: tokens are written into the destination ranks' slabs ----
    def _p2p_dispatcher(self, x: torch.Tensor):
        rows = int(getattr(self.cfg, "moe_p2p_dispatch_rows", 0) or 0)
        if rows <= 0 or not x.is_cuda:
            return None
        from ..parallel.moe_dispatch import dispatcher_for
        from ..parallel.symm import get_arena
        return dispatcher_for(get_arena(), self.ep_group, self.num_local, self.cfg.hidden_size, rows, x.dtype,
                              fallback=bool(getattr(self.cfg, "moe_p2p_overflow_fallback", True)))

    def _forward_p2p(self, disp, x, xr, top_p, top_idx, aux, comm, keep):
        from ..ops import moe as K

        c = self.cfg
        e, h, f = self.num_local, c.hidden_size, c.moe_ffn_hidden_size
        w1, w2 = self._w1().reshape(h, e * 2 * f), self._w2().reshape(e * f, h)
        route = disp.dispatch(x, top_idx)
        if route is None:
            return None
        gu = K.grouped_gemm(disp.slab, route.plan, w1, True, 2 * f, 0, 2 * f)
        act = ops.swiglu_fwd(gu)
        K.grouped_gemm(act, route.plan, w2, True, 0, f, h, out=disp.out_slab)
        xp = disp.slab.clone() if keep else None                  # the slab is reused by the next layer
        out, rows = disp.combine(route, top_p.detach(), keep_rows=keep)
        shared_ctx = None
        if self.shared_experts is not None:
            sh, shared_ctx = self._shared_fwd(x, comm, keep)
            out = out + sh
        if not keep:
            return out, None
        return out, dict(p2p=disp, xr=xr, top_p=top_p, top_idx=top_idx, aux=aux, route=route, xp=xp, gu=gu, act=act,
                         rows=rows, shared=shared_ctx)

    def _backward_p2p(self, ctx, x, dout, comm) -> torch.Tensor:
        from ..ops import moe as K
        from .gpt import grad_buffer

        c = self.cfg
        disp = ctx["p2p"]
        e, h, f = self.num_local, c.hidden_size, c.moe_ffn_hidden_size
        w1, w2 = self._w1().reshape(h, e * 2 * f), self._w2().reshape(e * f, h)
        top_p, top_idx = ctx["top_p"], ctx["top_idx"]
        t, k = top_idx.shape
        ident = K.MoePlan(None, None, torch.arange(t * k, dtype=torch.int32, device=x.device), None, t * k, t, k, 0)
        dprob = K.moe_slot_dot(dout, ctx["rows"], ident)                      # [T, k] fp32
        route = disp.dispatch(dout, top_idx, scale=top_p.detach())            # rows arrive scaled by their weight
        plan = route.plan
        dy = disp.slab
        dact = K.grouped_gemm(dy, plan, w2, False, 0, f, f)
        dgu = ops.swiglu_bwd(ctx["gu"], dact)
        if self.experts.weight1.requires_grad:
            self._expert_wgrads(plan, ctx["xp"], ctx["act"], dy, dgu)
        K.grouped_gemm(dgu, plan, w1, False, 2 * f, 0, h, out=disp.out_slab)
        dx, _ = disp.combine(route, None)
        return self._router_and_shared_bwd(ctx, x, dout, comm, dx.float(), dprob)

    def _backward_local(self, ctx, x, dout, comm) -> torch.Tensor:
        from ..ops import moe as K
        from .gpt import grad_buffer

        c = self.cfg
        e, h, f = self.num_local, c.hidden_size, c.moe_ffn_hidden_size
        w1, w2 = self._w1().reshape(h, e * 2 * f), self._w2().reshape(e * f, h)
        plan, top_p = ctx["plan"], ctx["top_p"]
        dy = K.moe_permute(dout, plan, top_p.detach())                    # rows scaled by their combine weight
        dprob = K.moe_slot_dot(dout, ctx["y"], plan)                      # [T, k] fp32
        dact = K.grouped_gemm(dy, plan, w2, False, 0, f, f)
        dgu = ops.swiglu_bwd(ctx["gu"], dact)
        dxp = K.grouped_gemm(dgu, plan, w1, False, 2 * f, 0, h)
        if self.experts.weight1.requires_grad:
            self._expert_wgrads(plan, ctx["xp"], ctx["act"], dy, dgu)
        dx = K.moe_combine(dxp, plan).float()
        return self._router_and_shared_bwd(ctx, x, dout, comm, dx, dprob)

    def _expert_wgrads(self, plan, xp, act, dy, dgu) -> None:
        """``dW2_e += act_e^T dy_e`` and ``dW1_e += x_e^T dgu_e`` for all local experts: two launches of the
        grouped weight-gradient GEMM that read the segment bounds on the device; the per-expert loop (which
        needs the counts on the host) remains for inputs that kernel does not cover."""
        from ..ops import moe as K
        from .gpt import grad_buffer

        c = self.cfg
        e, h, f = self.num_local, c.hidden_size, c.moe_ffn_hidden_size
        g1 = grad_buffer(self.experts.weight1).view(h, e, 2 * f)
        g2 = grad_buffer(self.experts.weight2).view(e, f, h)
        if K.grouped_wgrad_(g2, f * h, h, act, dy, plan) and K.grouped_wgrad_(g1, 2 * f, e * 2 * f, xp, dgu, plan):
            return
        counts, offsets = plan.counts.tolist(), plan.offsets.tolist()
        for j, n in enumerate(counts):
            if n == 0:
                continue
            r = slice(offsets[j], offsets[j] + n)
            g2[j].add_(torch.matmul(act[r].t(), dy[r]).to(g2.dtype))
            g1[:, j].add_(torch.matmul(xp[r].t(), dgu[r]).to(g1.dtype))

    def _router_and_shared_bwd(self, ctx, x, dout, comm, dx, dprob) -> torch.Tensor:
        """Probabilities (+ auxiliary loss) back to logits, x and the router weight; shared experts."""
        from .gpt import accum_wgrad, grad_buffer

        outs, grads = [ctx["top_p"]], [dprob]
        if ctx["aux"] is not None:
            outs.append(ctx["aux"])
            grads.append(torch.ones_like(ctx["aux"]))
        wants = [ctx["xr"]] + ([self.router.weight] if self.router.weight.requires_grad else [])
        got = torch.autograd.grad(outs, wants, grads, allow_unused=True)
        if got[0] is not None:
            dx += got[0]
        if len(got) > 1 and got[1] is not None:
            grad_buffer(self.router.weight).add_(got[1].to(grad_buffer(self.router.weight).dtype))
        if self.shared_experts is not None:
            dx += self._shared_bwd(ctx["shared"], dout, comm).float()
        return dx.to(x.dtype)

    def backward_tokens(self, ctx, x: torch.Tensor, dout: torch.Tensor, comm) -> torch.Tensor:
        from .gpt import accum_wgrad, grad_buffer

        if ctx.get("local"):
            return self._backward_local(ctx, x, dout, comm)
        if ctx.get("p2p") is not None:
            return self._backward_p2p(ctx, x, dout, comm)
        plan = ctx["plan"]
        d_tok = dout[plan["token_of"]]                                    # [T*k, H] in sorted-slot order
        dy_sorted = d_tok * ctx["w_sorted"].unsqueeze(-1)
        dw_sorted = (d_tok.float() * ctx["y_sorted"].float()).sum(-1)      # d loss / d prob per slot
        dy_local = self._redispatch(dy_sorted, plan)
        dxp_local = self._experts_bwd(plan["local_counts"], ctx["ectx"], dy_local)
        dxp_sorted = self._undispatch(dxp_local, plan)
        dx = torch.zeros_like(x, dtype=torch.float32)
        dx.index_add_(0, plan["token_of"], dxp_sorted.float())
        # router: probabilities (+ auxiliary loss) back to logits, x and the router weight
        dprob = torch.zeros(plan["t"] * plan["k"], device=x.device, dtype=torch.float32)
        dprob[plan["order"]] = dw_sorted
        outs, grads = [ctx["top_p"]], [dprob.view(plan["t"], plan["k"])]
        if ctx["aux"] is not None:
            outs.append(ctx["aux"])
            grads.append(torch.ones_like(ctx["aux"]))
        wants = [ctx["xr"]] + ([self.router.weight] if self.router.weight.requires_grad else [])
        got = torch.autograd.grad(outs, wants, grads, allow_unused=True)
        if got[0] is not None:
            dx += got[0]
        if len(got) > 1 and got[1] is not None:
            grad_buffer(self.router.weight).add_(got[1].to(grad_buffer(self.router.weight).dtype))
        if self.shared_experts is not None:
            dx += self._shared_bwd(ctx["shared"], dout, comm).float()
        return dx.to(x.dtype)

    # ------------------------------------------------------------------------------------------
    def rollout_view(self):
        """Weights as the rollout model runner consumes them (zero-copy)."""
        from ..rollout.moe import MoEWeights

        return MoEWeights(self.cfg, self.router.weight.data, self._w1().data, self._w2().data,
                          self.ep_group, self.ep_size, self.ep_rank, p2p=self._p2p_dispatcher,
                          expert_bias=getattr(self.router, "expert_bias", None),
                          collect_counts=bool(getattr(self, "collect_rollout_counts", False)),
                          shared=(self.shared_experts.linear_fc1.weight.data,
                                  self.shared_experts.linear_fc2.weight.data) if self.shared_experts else None)
