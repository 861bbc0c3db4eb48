"""Vision tower of the vision-language recipes (Qwen2-VL family shape).

``pixel_values [patches, C*T*P*P]`` -> patch embedding -> ``depth`` pre-norm transformer blocks with
full attention inside each image (two-axis rotary embedding over the patch grid) -> patch merger:
every ``merge x merge`` neighbourhood (consecutive rows, see ``datasets.image_processor``) is
concatenated and projected to the language model's hidden size.  The output rows replace the
embeddings of the image placeholder tokens of the prompt, in order.

The tower is small next to the language model and runs once per prompt, so it is written with
PyTorch modules (attention through ``scaled_dot_product_attention``, one call per image); it is
frozen during RL (the reference computes its embeddings in a forward-only stage,
``mindspeed_rl/workers/vit_worker.py:100-189``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class VisionConfig:
    patch_size: int = 14
    temporal_patch_size: int = 2
    in_channels: int = 3
    hidden_size: int = 1280
    depth: int = 32
    num_heads: int = 16
    intermediate_size: int = 3420
    spatial_merge_size: int = 2
    out_hidden_size: int = 3584          # hidden size of the language model
    norm_epsilon: float = 1e-6
    rotary_base: float = 10000.0

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size ** 2

    @classmethod
    def from_megatron(cls, cfg, llm_hidden: int) -> "VisionConfig":
        g = lambda k, d: getattr(cfg, k, None) or d
        return cls(patch_size=g("patch_size", 14), hidden_size=g("hidden_size", 1280), depth=g("num_layers", 32),
                   num_heads=g("num_attention_heads", 16), intermediate_size=g("ffn_hidden_size", 3420),
                   spatial_merge_size=g("spatial_merge_size", 2), out_hidden_size=llm_hidden)


class _RMSNorm(nn.Module):
    def __init__(self, n: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(n))
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def grid_positions(grid_thw: torch.Tensor, merge: int) -> torch.Tensor:
    """``(row, column)`` of every patch in the order the image processor emits them: ``[patches, 2]``."""
    out = []
    for t, h, w in grid_thw.tolist():
        hh = torch.arange(h).view(h // merge, 1, merge, 1).expand(h // merge, w // merge, merge, merge)
        ww = torch.arange(w).view(1, w // merge, 1, merge).expand(h // merge, w // merge, merge, merge)
        hw = torch.stack([hh.reshape(-1), ww.reshape(-1)], dim=-1)
        out.append(hw.repeat(t, 1))
    return torch.cat(out) if out else torch.zeros(0, 2, dtype=torch.long)


def _rotary_2d(x: torch.Tensor, pos: torch.Tensor, base: float) -> torch.Tensor:
    """``x [patches, heads, d]``: the first half of ``d`` rotates with the row index, the second half
    with the column index (rotate-half pairing inside each half)."""
    d = x.shape[-1] // 2
    inv = 1.0 / (base ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    out = []
    for axis in range(2):
        ang = pos[:, axis].float().unsqueeze(-1) * inv                    # [patches, d/2]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        part = x[..., axis * d:(axis + 1) * d].float()
        a, b = part[..., :d // 2], part[..., d // 2:]
        out.append(torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1))
    return torch.cat(out, dim=-1).to(x.dtype)


class _Block(nn.Module):
    def __init__(self, c: VisionConfig):
        super().__init__()
        self.c = c
        self.norm1, self.norm2 = _RMSNorm(c.hidden_size, c.norm_epsilon), _RMSNorm(c.hidden_size, c.norm_epsilon)
        self.qkv = nn.Linear(c.hidden_size, 3 * c.hidden_size)
        self.proj = nn.Linear(c.hidden_size, c.hidden_size)
        self.gate_up = nn.Linear(c.hidden_size, 2 * c.intermediate_size)
        self.down = nn.Linear(c.intermediate_size, c.hidden_size)

    def forward(self, x, pos, bounds: List[int]):
        c = self.c
        n, hd = x.shape[0], c.hidden_size // c.num_heads
        q, k, v = self.qkv(self.norm1(x)).view(n, 3, c.num_heads, hd).unbind(1)
        q, k = _rotary_2d(q, pos, c.rotary_base), _rotary_2d(k, pos, c.rotary_base)
        outs = []
        for s, e in zip(bounds[:-1], bounds[1:]):                         # attention stays inside an image
            o = F.scaled_dot_product_attention(q[s:e].transpose(0, 1).unsqueeze(0), k[s:e].transpose(0, 1).unsqueeze(0),
                                               v[s:e].transpose(0, 1).unsqueeze(0))
            outs.append(o.squeeze(0).transpose(0, 1).reshape(e - s, c.hidden_size))
        x = x + self.proj(torch.cat(outs) if outs else x[:0])
        g, u = self.gate_up(self.norm2(x)).chunk(2, dim=-1)
        return x + self.down(F.silu(g) * u)


class VisionTower(nn.Module):
    def __init__(self, cfg: VisionConfig, device=None, dtype=torch.float32, seed: int = 1234):
        super().__init__()
        self.cfg = cfg
        torch.manual_seed(seed)
        self.patch_embed = nn.Linear(cfg.patch_dim, cfg.hidden_size, bias=False)
        self.blocks = nn.ModuleList([_Block(cfg) for _ in range(cfg.depth)])
        m2 = cfg.spatial_merge_size ** 2
        self.merger_norm = _RMSNorm(cfg.hidden_size, cfg.norm_epsilon)
        self.merger = nn.Sequential(nn.Linear(cfg.hidden_size * m2, cfg.hidden_size * m2), nn.GELU(),
                                    nn.Linear(cfg.hidden_size * m2, cfg.out_hidden_size))
        self.to(device=device, dtype=dtype)

    @torch.no_grad()
    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """``[patches, patch_dim]``, ``[images, 3]`` -> ``[patches / merge^2, out_hidden]``."""
        c = self.cfg
        w = self.patch_embed.weight
        x = self.patch_embed(pixel_values.to(device=w.device, dtype=w.dtype))
        pos = grid_positions(grid_thw.cpu(), c.spatial_merge_size).to(x.device)
        sizes = (grid_thw[:, 0] * grid_thw[:, 1] * grid_thw[:, 2]).tolist()
        bounds = [0]
        for n in sizes:
            bounds.append(bounds[-1] + int(n))
        for blk in self.blocks:
            x = blk(x, pos, bounds)
        m2 = c.spatial_merge_size ** 2
        return self.merger(self.merger_norm(x).reshape(-1, c.hidden_size * m2))
