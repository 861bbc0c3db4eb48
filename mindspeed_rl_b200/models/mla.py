"""Multi-head latent attention (DeepSeek-V2/V3 style) for the training model and the rollout runner.

Queries and keys/values are produced through low-rank bottlenecks (reference switches:
``multi_latent_attention``, ``q_lora_rank``, ``kv_lora_rank``, ``qk_head_dim``,
``qk_pos_emb_head_dim``, ``v_head_dim`` -- ``mindspeed_rl/config_cls/megatron_config.py:237-238``;
parameter names as the reference re-assembles them for the rollout engine,
``mindspeed_rl/workers/resharding/weight_adaptor.py:244-324``):

    q      = W_uq  norm(W_dq x)                      -> per head [nope | rope]
    c, kr  = split(W_dkv x)                          -> latent [kv_lora], shared rotary key [rope]
    k_nope, v = split(W_ukv norm(c))                 -> per head
    k      = [k_nope | rope(kr) broadcast over heads],  q = [q_nope | rope(q_rope)]
    out    = W_o  softmax(q k^T * scale) v,   scale = mscale^2 / sqrt(nope + rope)

Tensor parallelism splits the heads: the up-projections are column parallel, the output projection
row parallel; the down-projections and the two norms are replicated and their gradients are summed
over the TP group (``tp_reduce_grad``).  The block is written with differentiable PyTorch operations
around the packed-sequence attention kernels (an autograd function over ``ops.attn_kv_fwd`` /
``attn_kv_bwd``); the transformer layer re-runs it in the backward (the block's activations are not
kept) and takes the gradients from autograd.  The attention kernels serve query/key and value heads
of one common size 64 or 128 (value heads are zero-padded up to the query size); other sizes (the
192 / 128 of the full-size DeepSeek models) run PyTorch's scaled-dot-product attention per sequence.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


def _normal(shape, std, dtype, device, gen):
    t = torch.empty(shape, dtype=torch.float32, device=device)
    t.normal_(0.0, std, generator=gen)
    return t.to(dtype)


class _W(nn.Module):
    def __init__(self, weight: torch.Tensor, replicated: bool = False):
        super().__init__()
        self.weight = nn.Parameter(weight)
        if replicated:       # same values on every TP rank; each rank sees only its heads' gradient
            self.weight.tp_reduce_grad = True
            self.weight.tp_replicated = True


def yarn_mscale(factor: float, mscale: float) -> float:
    return 1.0 if factor <= 1 else 0.1 * mscale * math.log(factor) + 1.0


def _rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope(x: torch.Tensor, cs: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE of ``x [T, heads, d]`` with ``cs [T, d] = [cos | sin]``."""
    d = x.shape[-1]
    cos, sin = cs[:, None, :d // 2], cs[:, None, d // 2:]
    xf = x.float()
    a, b = xf[..., :d // 2], xf[..., d // 2:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)


class _PackedAttention(torch.autograd.Function):
    """Causal attention over packed sequences through the framework's own kernels."""

    @staticmethod
    def forward(ctx, q, k, v, cu, max_len: int):
        out, lse = ops.attn_kv_fwd(q, k, v, cu, cu, max_len, True)
        ctx.save_for_backward(q, k, v, out, lse, cu)
        ctx.max_len = max_len
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu = ctx.saved_tensors
        dq, dk, dv = ops.attn_kv_bwd(dout.contiguous(), q, k, v, out, lse, cu, cu, ctx.max_len, ctx.max_len, True)
        return dq, dk, dv, None, None


def packed_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu: torch.Tensor, max_len: int,
                     scale: float) -> torch.Tensor:
    """``q, k [T, h, dq]``, ``v [T, h, dv]`` -> ``[T, h * dv]`` with the given soft-max scale."""
    t, h, dq = q.shape
    dv = v.shape[-1]
    kernel_ok = (not q.is_cuda) or (dq in (64, 128) and dv <= dq)
    if kernel_ok:
        # the kernels scale by 1/sqrt(dq); fold the rest of the requested scale into q
        qs = q * (scale * math.sqrt(dq)) if abs(scale * math.sqrt(dq) - 1.0) > 1e-12 else q
        vp = F.pad(v, (0, dq - dv)) if dv < dq else v
        out = _PackedAttention.apply(qs.contiguous(), k.contiguous(), vp.contiguous(), cu, max_len)
        return out.view(t, h, dq)[..., :dv].reshape(t, h * dv)
    outs = []
    bounds = cu.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e == s:
            continue
        o = F.scaled_dot_product_attention(q[s:e].transpose(0, 1).unsqueeze(0), k[s:e].transpose(0, 1).unsqueeze(0),
                                           v[s:e].transpose(0, 1).unsqueeze(0), is_causal=True, scale=scale)
        outs.append(o.squeeze(0).transpose(0, 1).reshape(e - s, h * dv))
    return torch.cat(outs, dim=0)


class MLASelfAttention(nn.Module):
    def __init__(self, cfg, device, gen):
        super().__init__()
        tp = cfg.tensor_model_parallel_size
        if cfg.num_attention_heads % tp:
            raise ValueError("attention heads must be divisible by the TP size")
        self.cfg = cfg
        self.nh = cfg.num_attention_heads // tp
        self.nope, self.rope, self.vd = cfg.qk_head_dim, cfg.qk_pos_emb_head_dim, cfg.v_head_dim
        self.qd = self.nope + self.rope
        h, dt, std = cfg.hidden_size, cfg.params_dtype, cfg.init_method_std
        out_std = std / math.sqrt(2.0 * cfg.num_layers)
        if cfg.q_lora_rank:
            self.linear_q_down_proj = _W(_normal((cfg.q_lora_rank, h), std, dt, device, gen), replicated=True)
            self.q_layernorm = _W(torch.ones(cfg.q_lora_rank, dtype=dt, device=device), replicated=True)
            self.linear_q_up_proj = _W(_normal((self.nh * self.qd, cfg.q_lora_rank), std, dt, device, gen))
            self.linear_q_proj = None
        else:
            self.linear_q_proj = _W(_normal((self.nh * self.qd, h), std, dt, device, gen))
            self.linear_q_down_proj = self.q_layernorm = self.linear_q_up_proj = None
        self.linear_kv_down_proj = _W(_normal((cfg.kv_lora_rank + self.rope, h), std, dt, device, gen), replicated=True)
        self.kv_layernorm = _W(torch.ones(cfg.kv_lora_rank, dtype=dt, device=device), replicated=True)
        self.linear_kv_up_proj = _W(_normal((self.nh * (self.nope + self.vd), cfg.kv_lora_rank), std, dt, device, gen))
        self.linear_proj = _W(_normal((h, self.nh * self.vd), out_std, dt, device, gen))
        sc = cfg.rope_scaling or {}
        m = yarn_mscale(float(sc.get("factor", 1.0)), float(sc.get("mscale_all_dim", 0.0) or 0.0)) if sc else 1.0
        self.softmax_scale = m * m / math.sqrt(self.qd)
        self._table = None

    @classmethod
    def from_tensors(cls, cfg, tp_size: int, tensors) -> "MLASelfAttention":
        """Forward-only block over existing tensors (the rollout's resharded copy of the weights): ``tensors`` maps
        the parameter names of this block (``linear_q_up_proj.weight`` ...) to tensors already cut for ``tp_size``
        ranks.  Nothing is allocated or initialised."""
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self.cfg = cfg
        self.nh = cfg.num_attention_heads // tp_size
        self.nope, self.rope, self.vd = cfg.qk_head_dim, cfg.qk_pos_emb_head_dim, cfg.v_head_dim
        self.qd = self.nope + self.rope

        class _View:                       # what ``qkv`` reads: an object with a ``weight``
            def __init__(self, w):
                self.weight = w

        for name in ("linear_q_down_proj", "q_layernorm", "linear_q_up_proj", "linear_q_proj",
                     "linear_kv_down_proj", "kv_layernorm", "linear_kv_up_proj", "linear_proj"):
            w = tensors.get(name + ".weight")
            object.__setattr__(self, name, _View(w) if w is not None else None)
        sc = cfg.rope_scaling or {}
        m = yarn_mscale(float(sc.get("factor", 1.0)), float(sc.get("mscale_all_dim", 0.0) or 0.0)) if sc else 1.0
        self.softmax_scale = m * m / math.sqrt(self.qd)
        self._table = None
        return self

    # ------------------------------------------------------------------------------------------
    def rope_table(self, device) -> torch.Tensor:
        if self._table is None or self._table.device != device:
            c = self.cfg
            self._table = ops.rope_table(c.max_position_embeddings, self.rope, c.rotary_base, device, c.rope_scaling)
        return self._table

    def qkv(self, x: torch.Tensor, positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """``x [T, H]`` (all tokens) -> ``q, k [T, nh, nope+rope]`` (rotary applied), ``v [T, nh, vd]``."""
        c, t = self.cfg, x.shape[0]
        eps = c.norm_epsilon
        if self.linear_q_proj is not None:
            q = F.linear(x, self.linear_q_proj.weight)
        else:
            q = F.linear(_rms(F.linear(x, self.linear_q_down_proj.weight), self.q_layernorm.weight, eps),
                         self.linear_q_up_proj.weight)
        q = q.view(t, self.nh, self.qd)
        ckv = F.linear(x, self.linear_kv_down_proj.weight)
        latent, k_rope = ckv[:, :c.kv_lora_rank], ckv[:, c.kv_lora_rank:]
        kv = F.linear(_rms(latent, self.kv_layernorm.weight, eps), self.linear_kv_up_proj.weight)
        kv = kv.view(t, self.nh, self.nope + self.vd)
        cs = self.rope_table(x.device)[positions.long()]
        q = torch.cat([q[..., :self.nope], _rope(q[..., self.nope:], cs)], dim=-1)
        k_rope = _rope(k_rope.unsqueeze(1), cs).expand(t, self.nh, self.rope)
        k = torch.cat([kv[..., :self.nope], k_rope], dim=-1)
        return q, k, kv[..., self.nope:]

    def forward(self, x: torch.Tensor, meta) -> torch.Tensor:
        """All tokens in, this rank's partial sum of the output projection out (``[T, H]``; the
        caller reduces over the TP group)."""
        q, k, v = self.qkv(x, meta.positions)
        attn = packed_attention(q, k, v, meta.cu_seqlens, meta.max_seqlen, self.softmax_scale)
        return F.linear(attn, self.linear_proj.weight)

    # ---- rollout -------------------------------------------------------------------------------------
    def rollout_supported(self) -> bool:
        """The paged-KV engine stores per-head keys and values of one common size."""
        return self.qd == self.vd and self.qd in (64, 128)

    @torch.no_grad()
    def rollout_qkv(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Per-head ``[q | k | v]`` groups (the interleaved layout of the rollout kernels, one KV head
        per query head), rotary applied and the soft-max scale folded into q."""
        q, k, v = self.qkv(x, positions)
        q = q * (self.softmax_scale * math.sqrt(self.qd))
        return torch.stack([q, k, v], dim=2).reshape(x.shape[0], self.nh * 3 * self.qd).contiguous()
