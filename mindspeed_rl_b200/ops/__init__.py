"""Python front-ends of the hand-written sm_100a kernels (sources in ``csrc/``).

Each op runs its CUDA kernel for CUDA tensors and a PyTorch fp32 formulation for CPU tensors;
on a GPU machine a missing kernel library is an error, never a silent fallback.
"""
from . import _lib
from ._lib import available as kernels_available, launch_count, reset_launch_count
from .layouts import QKVLayout
from .elementwise import (add, colsum_accumulate, embedding_grad_, headnorm_bwd_, headnorm_fwd_, rmsnorm_bwd,
                          rmsnorm_fwd, rope_, rope_table, swiglu_bwd, swiglu_fwd)
from .attention import attn_kv_bwd, attn_kv_fwd, attn_merge_, attn_varlen_bwd, attn_varlen_fwd
from .decode import (build_decode_groups, decode_group_max, decode_prefix_tile, kv_cache_gather, kv_cache_write,
                     paged_decode_attention, sample)
from .rl import (gae, group_norm_advantage, loss_weights, policy_loss_fwd_bwd,
                 policy_loss_reference, value_loss_fwd_bwd, value_loss_reference)
from .optim import adamw_step, cast_f32_to_bf16, clip_coefficient, sumsq_accumulate
from .lmhead import lmhead_logprob_bwd, lmhead_logprob_fwd

__all__ = [n for n in dir() if not n.startswith("_")]
