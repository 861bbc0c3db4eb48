"""Description of how q / k / v heads sit inside one row of the fused QKV projection output.

Two layouts exist in the framework:

* ``interleaved=True`` -- the training layout (Megatron mcore): per KV group
  ``[q_0 .. q_{rep-1}, k, v]`` repeated ``num_kv_heads`` times
  (reference: ``models/rollout/vllm_adapter/megatron_weight_loaders.py:154-172``);
* ``interleaved=False`` -- the rollout layout ``[all q | all k | all v]``.

Kernels never copy heads around: they receive a base offset plus
``(stride_t, group_stride, heads_per_group, head_stride)`` and compute
``offset(t, h) = t*stride_t + (h // hpg)*group_stride + (h % hpg)*head_stride``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch

HeadSpec = Tuple[int, Tuple[int, int, int, int]]  # (base offset, (stride_t, group_stride, hpg, head_stride))


@dataclass(frozen=True)
class QKVLayout:
    num_heads: int
    num_kv_heads: int
    head_dim: int
    interleaved: bool = True

    @property
    def rep(self) -> int:
        return self.num_heads // self.num_kv_heads

    @property
    def width(self) -> int:
        return (self.num_heads + 2 * self.num_kv_heads) * self.head_dim

    @property
    def q_width(self) -> int:
        return self.num_heads * self.head_dim

    def q(self) -> HeadSpec:
        if self.interleaved:
            return 0, (self.width, (self.rep + 2) * self.head_dim, self.rep, self.head_dim)
        return 0, (self.width, 0, self.num_heads, self.head_dim)

    def k(self) -> HeadSpec:
        if self.interleaved:
            return self.rep * self.head_dim, (self.width, (self.rep + 2) * self.head_dim, 1, self.head_dim)
        return self.num_heads * self.head_dim, (self.width, 0, self.num_kv_heads, self.head_dim)

    def v(self) -> HeadSpec:
        if self.interleaved:
            return (self.rep + 1) * self.head_dim, (self.width, (self.rep + 2) * self.head_dim, 1,
                                                    self.head_dim)
        return ((self.num_heads + self.num_kv_heads) * self.head_dim,
                (self.width, 0, self.num_kv_heads, self.head_dim))

    # ---- PyTorch views (reference path and tests) ------------------------------------------------
    def split(self, qkv: torch.Tensor):
        """``[T, width]`` -> q ``[T, nh, hd]``, k ``[T, nkv, hd]``, v ``[T, nkv, hd]`` (views/copies)."""
        t = qkv.shape[0]
        nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        if self.interleaved:
            g = qkv.view(t, nkv, self.rep + 2, hd)
            return (g[:, :, :self.rep].reshape(t, nh, hd), g[:, :, self.rep], g[:, :, self.rep + 1])
        q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)
        return q.view(t, nh, hd), k.view(t, nkv, hd), v.view(t, nkv, hd)

    def merge(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """Inverse of :meth:`split` (always materialises a new ``[T, width]`` tensor)."""
        t = q.shape[0]
        nkv, hd = self.num_kv_heads, self.head_dim
        if self.interleaved:
            g = torch.cat([q.reshape(t, nkv, self.rep, hd), k.reshape(t, nkv, 1, hd),
                           v.reshape(t, nkv, 1, hd)], dim=2)
            return g.reshape(t, self.width)
        return torch.cat([q.reshape(t, -1), k.reshape(t, -1), v.reshape(t, -1)], dim=-1)
