"""Decoder-only transformer (Qwen2 / Qwen3 dense and MoE families) for packed token streams.

Design notes
------------
* Activations are always packed ``[T, H]`` ("THD"); sequences are delimited by ``cu_seqlens``.
* Each transformer layer is **one autograd node** with a hand-written backward.  With
  ``recompute_granularity == "full"`` only the layer input is kept and the forward is re-run
  inside the backward; otherwise the intermediates are kept.  Parameter gradients are
  accumulated in place into ``param.main_grad`` (the contiguous DDP buffer) -- or ``param.grad``
  when the model is not wrapped -- so autograd never materialises a second copy.
* Parameter names and layouts follow Megatron-mcore (``decoder.layers.N.self_attention.linear_qkv``
  with the per-KV-group interleave, ``mlp.linear_fc1`` as ``[gate; up]`` per TP shard, ...), which is
  what the checkpoint format and the resharding planner expect
  (reference name map: ``mindspeed_rl/workers/resharding/weight_adaptor.py:54-65``).
* Tensor/sequence parallel communication goes through ``TPComm`` (NCCL baseline or fused kernels).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import QKVLayout
from ..parallel.tp_comm import NO_TP, TPComm
from . import lora
from .transformer_config import TransformerConfig


@dataclass
class PackedMeta:
    """Per micro-batch sequence metadata (device tensors are int32)."""
    cu_seqlens: torch.Tensor          # [B+1]
    max_seqlen: int
    positions: torch.Tensor           # [T]
    cp: Any = None                    # context-parallel helper (parallel.context_parallel), optional
    # vision-language inputs (optional): rows of the vision tower's output that replace the embeddings of
    # the image placeholder tokens at ``image_index`` (packed positions), and a per-token rotary table
    # ``[T, head_dim]`` built from three-axis position ids (then ``positions`` just numbers the tokens)
    image_index: Optional[torch.Tensor] = None
    image_embeds: Optional[torch.Tensor] = None
    rope_table: Optional[torch.Tensor] = None

    @classmethod
    def from_lengths(cls, lengths, device, align: int = 1) -> "PackedMeta":
        lens = torch.as_tensor(lengths, dtype=torch.int32)
        padded = (lens + (align - 1)) // align * align
        cu = torch.zeros(lens.numel() + 1, dtype=torch.int32)
        cu[1:] = torch.cumsum(padded, 0)
        pos = torch.cat([torch.arange(int(n), dtype=torch.int32) for n in padded.tolist()]) \
            if lens.numel() else torch.zeros(0, dtype=torch.int32)
        return cls(cu.to(device), int(padded.max()) if lens.numel() else 0, pos.to(device))


# ---------------------------------------------------------------------------------------------------
# gradient accumulation helpers
# ---------------------------------------------------------------------------------------------------
def grad_buffer(p: torch.Tensor) -> torch.Tensor:
    g = getattr(p, "main_grad", None)
    if g is None:
        if p.grad is None:
            p.grad = torch.zeros_like(p)
        g = p.grad
    return g


def accum_wgrad(p: torch.Tensor, dy: torch.Tensor, x: torch.Tensor) -> None:
    """``grad(p) += dy^T x`` for a weight ``p [out, in]``."""
    if not p.requires_grad:
        return
    from ..ops.gemm import linear_wgrad_

    linear_wgrad_(grad_buffer(p), dy, x)


def accum_vec(p: torch.Tensor, v: torch.Tensor) -> None:
    if p.requires_grad:
        grad_buffer(p).add_(v.to(grad_buffer(p).dtype))


class _Holder(nn.Module):
    """Parameter holder so that state-dict keys read ``<name>.weight`` / ``<name>.bias``."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        super().__init__()
        self.weight = nn.Parameter(weight)
        if bias is not None:
            self.bias = nn.Parameter(bias)
        else:
            self.bias = None


def _normal(shape, std, dtype, device, gen=None):
    t = torch.empty(shape, dtype=torch.float32, device=device)
    t.normal_(0.0, std, generator=gen)
    return t.to(dtype)


# ---------------------------------------------------------------------------------------------------
# Transformer layer
# ---------------------------------------------------------------------------------------------------
def _attach_lora(module: nn.Module, names, cfg: TransformerConfig, device, gen) -> None:
    """Adapters on the listed linears when the config asks for them (``models/lora.py``)."""
    if cfg.lora_r <= 0:
        return
    for name in names:
        if name in cfg.lora_target_modules:
            lora.attach(getattr(module, name), name, cfg, device, gen, cfg.sequence_parallel)


class SelfAttention(nn.Module):
    def __init__(self, cfg: TransformerConfig, device, gen):
        super().__init__()
        tp = cfg.tensor_model_parallel_size
        if cfg.num_attention_heads % tp or cfg.num_query_groups % tp:
            raise ValueError("attention heads and query groups must be divisible by the TP size")
        nh, nkv, hd = cfg.num_attention_heads // tp, cfg.num_query_groups // tp, cfg.head_dim
        self.layout = QKVLayout(nh, nkv, hd, interleaved=True)
        dt, std = cfg.params_dtype, cfg.init_method_std
        out_std = std / math.sqrt(2.0 * cfg.num_layers)
        bias = torch.zeros(self.layout.width, dtype=dt, device=device) if cfg.add_qkv_bias else None
        self.linear_qkv = _Holder(_normal((self.layout.width, cfg.hidden_size), std, dt, device, gen), bias)
        self.linear_proj = _Holder(_normal((cfg.hidden_size, nh * hd), out_std, dt, device, gen))
        if cfg.qk_layernorm:
            self.q_layernorm = _Holder(torch.ones(hd, dtype=dt, device=device))
            self.k_layernorm = _Holder(torch.ones(hd, dtype=dt, device=device))
        else:
            self.q_layernorm = self.k_layernorm = None
        _attach_lora(self, ("linear_qkv", "linear_proj"), cfg, device, gen)


class MLP(nn.Module):
    def __init__(self, cfg: TransformerConfig, device, gen, ffn: Optional[int] = None):
        super().__init__()
        tp = cfg.tensor_model_parallel_size
        f = (ffn or cfg.ffn_hidden_size) // tp
        dt, std = cfg.params_dtype, cfg.init_method_std
        out_std = std / math.sqrt(2.0 * cfg.num_layers)
        self.linear_fc1 = _Holder(_normal((2 * f, cfg.hidden_size), std, dt, device, gen))
        self.linear_fc2 = _Holder(_normal((cfg.hidden_size, f), out_std, dt, device, gen))
        _attach_lora(self, ("linear_fc1", "linear_fc2"), cfg, device, gen)


class TransformerLayer(nn.Module):
    def __init__(self, cfg: TransformerConfig, layer_number: int, device, gen, comm: TPComm):
        super().__init__()
        self.cfg = cfg
        self.layer_number = layer_number
        self.comm = comm
        dt = cfg.params_dtype
        self.input_layernorm = _Holder(torch.ones(cfg.hidden_size, dtype=dt, device=device))
        if cfg.multi_latent_attention:
            from .mla import MLASelfAttention

            self.self_attention = MLASelfAttention(cfg, device, gen)
        else:
            self.self_attention = SelfAttention(cfg, device, gen)
        self.pre_mlp_layernorm = _Holder(torch.ones(cfg.hidden_size, dtype=dt, device=device))
        if cfg.layer_is_moe(layer_number):
            from .moe import MoELayer

            self.mlp = MoELayer(cfg, device, gen)
        else:
            self.mlp = MLP(cfg, device, gen)
        self._rope_table = None

    # -- helpers ------------------------------------------------------------------------------------
    def rope_table(self, device) -> torch.Tensor:
        if self._rope_table is None or self._rope_table.device != device:
            c = self.cfg
            self._rope_table = ops.rope_table(c.max_position_embeddings, c.head_dim, c.rotary_base,
                                              device, c.rope_scaling)
        return self._rope_table

    def forward(self, h: torch.Tensor, meta: PackedMeta) -> torch.Tensor:
        if torch.is_grad_enabled() and (h.requires_grad or any(p.requires_grad for p in self.parameters())):
            return _LayerFn.apply(h, self, meta)
        out, _ = layer_forward(self, h, meta, keep=False)
        return out


def _attention_core_fwd(layer: TransformerLayer, qkv: torch.Tensor, meta: PackedMeta):
    """qk-norm -> rope -> attention.  Returns (attn_out, lse, saved_pre_norm, rstd_q, rstd_k)."""
    sa = layer.self_attention
    lay = sa.layout
    pre = rq = rk = None
    if sa.q_layernorm is not None:
        pre = qkv.clone()
        rq = ops.headnorm_fwd_(qkv, lay, "q", sa.q_layernorm.weight, layer.cfg.norm_epsilon)
        rk = ops.headnorm_fwd_(qkv, lay, "k", sa.k_layernorm.weight, layer.cfg.norm_epsilon)
    ops.rope_(qkv, lay, meta.positions, meta.rope_table if meta.rope_table is not None else layer.rope_table(qkv.device))
    if meta.cp is not None:
        attn, lse = meta.cp.attention_fwd(qkv, lay, meta)
    else:
        attn, lse = ops.attn_varlen_fwd(qkv, lay, meta.cu_seqlens, meta.max_seqlen, causal=True)
    return attn, lse, pre, rq, rk


def layer_forward(layer: TransformerLayer, h: torch.Tensor, meta: PackedMeta, keep: bool
                  ) -> Tuple[torch.Tensor, Optional[Dict[str, Any]]]:
    """Forward of one layer; ``keep`` returns the intermediates the backward needs."""
    cfg, comm, sa = layer.cfg, layer.comm, layer.self_attention
    eps = cfg.norm_epsilon
    x1, rstd1, _ = ops.rmsnorm_fwd(h, layer.input_layernorm.weight, eps, want_rstd=keep)
    lo: Dict[str, torch.Tensor] = {}      # adapter intermediates (only for adapted linears)
    qkv = attn = lse = pre = rq = rk = None
    if cfg.multi_latent_attention:
        # latent attention: one differentiable block, re-run in the backward (only its input is kept)
        x1g = comm.gather_seq(x1)
        with torch.no_grad():
            proj = comm.reduce_out(sa(x1g, meta))
    else:
        # column linears = (all-gather tokens ->) GEMM, row linears = GEMM (-> reduce-scatter tokens);
        # ``comm`` runs each pair as one fused kernel when it can
        qkv, x1g = comm.column_linear(x1, sa.linear_qkv.weight, sa.linear_qkv.bias)
        if lora.active(sa.linear_qkv):
            lo["qkv"] = lora.column_fwd(sa.linear_qkv, x1g, qkv)
        attn, lse, pre, rq, rk = _attention_core_fwd(layer, qkv, meta)
        proj = comm.row_linear(attn, sa.linear_proj.weight)
        if lora.active(sa.linear_proj):
            lo["proj"] = lora.row_fwd(sa.linear_proj, attn, proj, comm)[1]
    # residual add fused into the norm: one pass writes h1 = h + proj and its normalised form
    x2, rstd2, h1 = ops.rmsnorm_fwd(proj, layer.pre_mlp_layernorm.weight, eps, residual=h, want_rstd=keep)
    if isinstance(layer.mlp, MLP):
        gu, x2g = comm.column_linear(x2, layer.mlp.linear_fc1.weight)
        if lora.active(layer.mlp.linear_fc1):
            lo["fc1"] = lora.column_fwd(layer.mlp.linear_fc1, x2g, gu)
        y = ops.swiglu_fwd(gu)
        mlp_out = comm.row_linear(y, layer.mlp.linear_fc2.weight)
        if lora.active(layer.mlp.linear_fc2):
            lo["fc2"] = lora.row_fwd(layer.mlp.linear_fc2, y, mlp_out, comm)[1]
        # activation-function recompute: drop silu(g)*u and rebuild it from gu in the backward
        mlp_ctx = (gu, None if cfg.recompute_activation_function else y) if keep else None
    else:
        # expert layers work on the tokens this rank owns (under sequence parallelism every TP rank routes its
        # own shard); their shared experts gather / reduce inside
        x2g = x2
        mlp_out, mlp_ctx = layer.mlp.forward_tokens(x2, comm, keep)
    h2 = ops.add(h1, mlp_out)
    if not keep:
        return h2, None
    ctx = dict(h=h, rstd1=rstd1, x1g=x1g, qkv=qkv, attn=attn, lse=lse, pre=pre, rq=rq, rk=rk, h1=h1,
               rstd2=rstd2, x2g=x2g, mlp_ctx=mlp_ctx, lora=lo)
    return h2, ctx


def layer_backward(layer: TransformerLayer, ctx: Dict[str, Any], meta: PackedMeta, dh2: torch.Tensor
                   ) -> torch.Tensor:
    cfg, comm, sa = layer.cfg, layer.comm, layer.self_attention
    lay = getattr(sa, "layout", None)
    # ---- MLP ----
    if isinstance(layer.mlp, MLP):
        gu, y = ctx["mlp_ctx"]
        if y is None:
            y = ops.swiglu_fwd(gu)
        fc1, fc2 = layer.mlp.linear_fc1.weight, layer.mlp.linear_fc2.weight
        lo = ctx.get("lora") or {}
        dy, d_out = comm.row_linear_bwd(dh2, fc2)
        if "fc2" in lo:
            dy += lora.row_bwd(layer.mlp.linear_fc2, y, lo["fc2"], dh2, comm)
        accum_wgrad(fc2, d_out, y)
        dgu = ops.swiglu_bwd(gu, dy)
        accum_wgrad(fc1, dgu, ctx["x2g"])
        dx2 = comm.column_linear_bwd(dgu, fc1)
        if "fc1" in lo:
            dx2 = dx2 + lora.column_bwd(layer.mlp.linear_fc1, ctx["x2g"], lo["fc1"], dgu, comm)
    else:
        dx2 = layer.mlp.backward_tokens(ctx["mlp_ctx"], ctx["x2g"], dh2, comm)
    dh1 = ops.rmsnorm_bwd(dx2, ctx["h1"], layer.pre_mlp_layernorm.weight, ctx["rstd2"],
                          grad_buffer(layer.pre_mlp_layernorm.weight), dres=dh2)
    # ---- attention ----
    if cfg.multi_latent_attention:
        dx1 = _mla_backward(sa, ctx["x1g"], meta, comm, dh1)
        return ops.rmsnorm_bwd(dx1, ctx["h"], layer.input_layernorm.weight, ctx["rstd1"],
                               grad_buffer(layer.input_layernorm.weight), dres=dh1)
    lo = ctx.get("lora") or {}
    dattn, d_proj = comm.row_linear_bwd(dh1, sa.linear_proj.weight)
    if "proj" in lo:
        dattn += lora.row_bwd(sa.linear_proj, ctx["attn"], lo["proj"], dh1, comm)
    accum_wgrad(sa.linear_proj.weight, d_proj, ctx["attn"])
    if meta.cp is not None:
        dqkv = meta.cp.attention_bwd(dattn, ctx["qkv"], ctx["attn"], ctx["lse"], lay, meta)
    else:
        dqkv = ops.attn_varlen_bwd(dattn, ctx["qkv"], ctx["attn"], ctx["lse"], lay, meta.cu_seqlens,
                                   meta.max_seqlen, causal=True)
    ops.rope_(dqkv, lay, meta.positions, meta.rope_table if meta.rope_table is not None else layer.rope_table(dqkv.device),
              inverse=True)
    if sa.q_layernorm is not None:
        ops.headnorm_bwd_(dqkv, ctx["pre"], lay, "q", sa.q_layernorm.weight, ctx["rq"],
                          grad_buffer(sa.q_layernorm.weight))
        ops.headnorm_bwd_(dqkv, ctx["pre"], lay, "k", sa.k_layernorm.weight, ctx["rk"],
                          grad_buffer(sa.k_layernorm.weight))
    accum_wgrad(sa.linear_qkv.weight, dqkv, ctx["x1g"])
    if sa.linear_qkv.bias is not None and sa.linear_qkv.bias.requires_grad:
        ops.colsum_accumulate(dqkv, grad_buffer(sa.linear_qkv.bias))
    dx1 = comm.column_linear_bwd(dqkv, sa.linear_qkv.weight)
    if "qkv" in lo:
        dx1 = dx1 + lora.column_bwd(sa.linear_qkv, ctx["x1g"], lo["qkv"], dqkv, comm)
    dh = ops.rmsnorm_bwd(dx1, ctx["h"], layer.input_layernorm.weight, ctx["rstd1"],
                         grad_buffer(layer.input_layernorm.weight), dres=dh1)
    return dh


def _mla_backward(sa, x1g: torch.Tensor, meta: PackedMeta, comm: TPComm, dh1: torch.Tensor) -> torch.Tensor:
    """Backward of the latent-attention block: re-run it with autograd on, feed the gathered output
    gradient, add the parameter gradients to their buffers and return the input gradient (token
    shard under sequence parallelism)."""
    d_full = comm.reduce_out_bwd(dh1)
    params = [p for p in sa.parameters() if p.requires_grad]
    with torch.enable_grad():
        x = x1g.detach().requires_grad_(True)
        y = sa(x, meta)
        grads = torch.autograd.grad(y, [x] + params, d_full)
    for p, g in zip(params, grads[1:]):
        accum_vec(p, g)
    return comm.gather_seq_bwd(grads[0])


# Called with a layer right after its backward (one slot: the data-parallel wrapper installs itself while the
# last micro-batch of a step runs, so that bucketed gradient reduction overlaps the rest of the backward).
grads_ready_hook: List[Optional[Callable]] = [None]


class _LayerFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h: torch.Tensor, layer: TransformerLayer, meta: PackedMeta):
        # "full" keeps only the layer input and re-runs the forward in the backward; with
        # recompute_method "block" that applies to the first recompute_num_layers layers of the
        # stage only, the others keep their intermediates
        full_recompute = layer.cfg.recompute_granularity == "full" and getattr(layer, "recompute_full", True)
        out, saved = layer_forward(layer, h, meta, keep=not full_recompute)
        ctx.layer, ctx.meta, ctx.full = layer, meta, full_recompute
        ctx.swapped = False
        if full_recompute:
            ctx.save_for_backward(h)
        elif getattr(layer.cfg, "swap_attention", False):
            # kept activations wait for their backward in pinned host memory
            from .activation_swap import keys_of, swapper_for
            ctx.saved = swapper_for(h.device).offload(saved, keys_of(layer.cfg.swap_modules))
            ctx.swapped = True
        else:
            ctx.saved = saved
        return out

    @staticmethod
    def backward(ctx, dh2: torch.Tensor):
        layer, meta = ctx.layer, ctx.meta
        if ctx.full:
            (h,) = ctx.saved_tensors
            with torch.no_grad():
                _, saved = layer_forward(layer, h, meta, keep=True)
        else:
            saved = ctx.saved
            ctx.saved = None
            if ctx.swapped:
                from .activation_swap import swapper_for
                saved = swapper_for(dh2.device).restore(saved)
        with torch.no_grad():
            dh = layer_backward(layer, saved, meta, dh2.contiguous())
        hook = grads_ready_hook[0]
        if hook is not None:
            hook(layer)          # this layer's gradients are final for the micro-batch: their reduction may start
        return dh, None, None


# ---------------------------------------------------------------------------------------------------
# Embedding / output
# ---------------------------------------------------------------------------------------------------
def embedding_grad_accumulate(g: torch.Tensor, ids: torch.Tensor, d: torch.Tensor) -> None:
    """``g[ids[t]] += d[t]`` with the rows of one id summed in fp32 in token order: the result does not
    depend on the order in which atomics land (``index_add_`` into a bf16 buffer rounds after every
    addition, in a different order on every run)."""
    if ids.numel() == 0:
        return
    order = torch.argsort(ids, stable=True)
    uniq, counts = torch.unique_consecutive(ids[order], return_counts=True)
    if ops.embedding_grad_(g, d, order, uniq, counts):       # one block per id on the GPU
        return
    rows = torch.segment_reduce(d[order].float(), "sum", lengths=counts, axis=0, unsafe=True)
    g[uniq] = (g[uniq].float() + rows).to(g.dtype)


class _EmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weight: torch.Tensor, ids: torch.Tensor, comm: TPComm, vocab_start: int):
        v_local = weight.shape[0]
        if comm.world_size > 1:
            local = ids - vocab_start
            mine = (local >= 0) & (local < v_local)
            out = weight[local.clamp(0, v_local - 1)]
            out = out * mine.unsqueeze(-1).to(out.dtype)
            out = comm.reduce_out(out)
        else:
            local, mine = ids, None
            out = weight[ids]
        ctx.save_for_backward(local, mine if mine is not None else ids.new_empty(0))
        ctx.comm, ctx.weight = comm, weight
        return out

    @staticmethod
    def backward(ctx, dout: torch.Tensor):
        local, mine = ctx.saved_tensors
        comm, weight = ctx.comm, ctx.weight
        if weight.requires_grad:
            d = comm.reduce_out_bwd(dout.contiguous())
            g = grad_buffer(weight)
            if mine.numel():
                d = d * mine.unsqueeze(-1).to(d.dtype)
                local = local.clamp(0, weight.shape[0] - 1)
            embedding_grad_accumulate(g, local, d)
        return None, None, None, None


class _LogProbHeadFn(torch.autograd.Function):
    """final RMSNorm -> LM head -> (log p(label), entropy), logits never fully materialised."""

    @staticmethod
    def forward(ctx, h, model: "GPTModel", labels, inv_temp: float, want_entropy: bool):
        cfg, comm = model.cfg, model.comm
        x, rstd, _ = ops.rmsnorm_fwd(h, model.decoder.final_layernorm.weight, cfg.norm_epsilon)
        xg = comm.gather_seq(x)
        w = model.output_weight()
        logp, ent, lse = ops.lmhead_logprob_fwd(xg, w, labels, inv_temp, model.vocab_start, comm.group,
                                                want_entropy)
        ctx.model, ctx.inv_temp = model, inv_temp
        ctx.save_for_backward(h, rstd, labels, lse, ent if ent is not None else lse.new_empty(0))
        if ent is None:
            ent = torch.zeros_like(logp)
            ctx.mark_non_differentiable(ent)
        return logp, ent

    @staticmethod
    def backward(ctx, dlogp, dent):
        model = ctx.model
        cfg, comm = model.cfg, model.comm
        h, rstd, labels, lse, ent = ctx.saved_tensors
        with torch.no_grad():
            x, _, _ = ops.rmsnorm_fwd(h, model.decoder.final_layernorm.weight, cfg.norm_epsilon,
                                      want_rstd=False)
            xg = comm.gather_seq(x)
            w = model.output_weight()
            has_ent = ent.numel() > 0 and dent is not None
            dxg = ops.lmhead_logprob_bwd(xg, w, labels, lse, ent if has_ent else None, dlogp,
                                         dent if has_ent else None,
                                         grad_buffer(w) if w.requires_grad else None, ctx.inv_temp,
                                         model.vocab_start)
            dx = comm.gather_seq_bwd(dxg)
            dh = ops.rmsnorm_bwd(dx, h, model.decoder.final_layernorm.weight, rstd,
                                 grad_buffer(model.decoder.final_layernorm.weight))
        return dh, None, None, None, None


class _Decoder(nn.Module):
    def __init__(self, cfg, layer_numbers: List[int], device, gen, comm, post_process: bool):
        super().__init__()
        self.layers = nn.ModuleList([TransformerLayer(cfg, n, device, gen, comm) for n in layer_numbers])
        block = cfg.recompute_method == "block" and cfg.recompute_num_layers is not None
        for i, layer in enumerate(self.layers):
            layer.recompute_full = (i < cfg.recompute_num_layers) if block else True
        if post_process:
            self.final_layernorm = _Holder(torch.ones(cfg.hidden_size, dtype=cfg.params_dtype,
                                                      device=device))
        else:
            self.final_layernorm = None


class _Embedding(nn.Module):
    def __init__(self, cfg, device, gen):
        super().__init__()
        v = cfg.vocab_size // cfg.tensor_model_parallel_size
        self.word_embeddings = _Holder(_normal((v, cfg.hidden_size), cfg.init_method_std,
                                               cfg.params_dtype, device, gen))


class GPTModel(nn.Module):
    """One pipeline stage (or the whole model) of the decoder.

    ``pre_process`` owns the embedding, ``post_process`` the final norm, the LM head and the
    optional scalar value head (``rm_head`` -- critic / outcome reward model; reference:
    ``mindspeed_rl/models/orm/orm_model.py:87-184``).
    """

    def __init__(self, cfg: TransformerConfig, comm: Optional[TPComm] = None, pre_process: bool = True,
                 post_process: bool = True, layer_numbers: Optional[List[int]] = None, device=None,
                 seed: int = 1234, chunk_sizes: Optional[List[int]] = None):
        """``chunk_sizes``: with an interleaved (virtual) pipeline the rank's layers form several
        chunks that are run separately (``hidden_states(..., chunk=c)``); ``layer_numbers`` lists the
        layers of all chunks in order.  The embedding belongs to chunk 0 of the first rank, the head to
        the last chunk of the last rank."""
        super().__init__()
        self.cfg = cfg
        self.comm = comm or NO_TP
        self.pre_process, self.post_process = pre_process, post_process
        device = torch.device(device if device is not None else "cpu")
        gen = torch.Generator(device=device).manual_seed(seed + 7919 * self.comm.rank)
        layer_numbers = list(range(cfg.num_layers)) if layer_numbers is None else layer_numbers
        self.layer_numbers = layer_numbers
        sizes = list(chunk_sizes) if chunk_sizes else [len(layer_numbers)]
        if sum(sizes) != len(layer_numbers):
            raise ValueError("chunk sizes do not add up to the number of layers of this stage")
        self.chunk_bounds = [0]
        for n_ in sizes:
            self.chunk_bounds.append(self.chunk_bounds[-1] + n_)
        self.num_chunks = len(sizes)
        if cfg.vocab_size % cfg.tensor_model_parallel_size:
            raise ValueError("vocab size must be divisible by the TP size")
        self.vocab_start = self.comm.rank * (cfg.vocab_size // cfg.tensor_model_parallel_size)
        self.embedding = _Embedding(cfg, device, gen) if pre_process else None
        self.decoder = _Decoder(cfg, layer_numbers, device, gen, self.comm, post_process)
        self.output_layer = None
        self.rm_head = None
        if post_process:
            if cfg.untie_embeddings_and_output_weights or not pre_process:
                v = cfg.vocab_size // cfg.tensor_model_parallel_size
                self.output_layer = _Holder(_normal((v, cfg.hidden_size), cfg.init_method_std,
                                                    cfg.params_dtype, device, gen))
            if cfg.value_head:
                self.rm_head = nn.Linear(cfg.hidden_size, 1, bias=True, device=device,
                                         dtype=torch.float32)
        if cfg.lora_r > 0:
            lora.freeze_base(self)          # only the adapters (and nothing else) are trained

    # -----------------------------------------------------------------------------------------------
    def output_weight(self) -> torch.Tensor:
        if self.output_layer is not None:
            return self.output_layer.weight
        return self.embedding.word_embeddings.weight

    def embed(self, ids: torch.Tensor) -> torch.Tensor:
        return _EmbedFn.apply(self.embedding.word_embeddings.weight, ids, self.comm, self.vocab_start)

    def _place_image_embeds(self, h: torch.Tensor, meta: PackedMeta) -> torch.Tensor:
        """Replace the embeddings of the image placeholder tokens by the vision tower's rows (constants:
        the tower is frozen).  Under sequence parallelism ``h`` holds this rank's token shard."""
        idx, rows = meta.image_index.long(), meta.image_embeds.to(h.dtype)
        if self.comm.sequence_parallel:
            per = h.shape[0]
            lo = self.comm.rank * per
            keep = (idx >= lo) & (idx < lo + per)
            idx, rows = idx[keep] - lo, rows[keep]
        return h.index_copy(0, idx, rows) if idx.numel() else h

    def run_layers(self, h: torch.Tensor, meta: PackedMeta, chunk: Optional[int] = None) -> torch.Tensor:
        layers = self.decoder.layers if chunk is None else \
            list(self.decoder.layers)[self.chunk_bounds[chunk]:self.chunk_bounds[chunk + 1]]
        for layer in layers:
            h = layer(h, meta)
        return h

    def is_first_chunk(self, chunk: Optional[int]) -> bool:
        return self.pre_process and (chunk is None or chunk == 0)

    def is_last_chunk(self, chunk: Optional[int]) -> bool:
        return self.post_process and (chunk is None or chunk == self.num_chunks - 1)

    def hidden_states(self, ids_or_h: torch.Tensor, meta: PackedMeta, chunk: Optional[int] = None) -> torch.Tensor:
        h = self.embed(ids_or_h) if self.is_first_chunk(chunk) else ids_or_h
        if self.is_first_chunk(chunk) and meta.image_index is not None and meta.image_index.numel():
            h = self._place_image_embeds(h, meta)
        if torch.is_grad_enabled() and not h.requires_grad and \
                any(p.requires_grad for p in self.decoder.parameters()):
            # layer nodes only run their backward when an input requires grad
            h = h.detach().requires_grad_(True)
        return self.run_layers(h, meta, chunk)

    def forward_logprob(self, ids_or_h: torch.Tensor, labels: torch.Tensor, meta: PackedMeta,
                        temperature: float = 1.0, want_entropy: bool = False, chunk: Optional[int] = None
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
        """Packed ids (or the previous stage's hidden states) -> per-token ``(logp, entropy)``."""
        h = self.hidden_states(ids_or_h, meta, chunk)
        if not self.is_last_chunk(chunk):
            return h, None
        return _LogProbHeadFn.apply(h, self, labels, 1.0 / temperature, want_entropy)

    def forward_values(self, ids_or_h: torch.Tensor, meta: PackedMeta, chunk: Optional[int] = None) -> torch.Tensor:
        """Per-token scalar from the value head (fp32), ``[T]``."""
        h = self.hidden_states(ids_or_h, meta, chunk)
        if not self.is_last_chunk(chunk):
            return h
        x = _NormFn.apply(h, self.decoder.final_layernorm.weight, self.cfg.norm_epsilon)
        xg = self.comm.gather_seq(x) if not torch.is_grad_enabled() else _GatherSeq.apply(x, self.comm)
        return self.rm_head(xg.float()).squeeze(-1)

    def forward_logits(self, ids: torch.Tensor, meta: PackedMeta) -> torch.Tensor:
        """Full (local-vocab) logits ``[T, V/tp]`` -- evaluation / tests only."""
        h = self.hidden_states(ids, meta)
        x, _, _ = ops.rmsnorm_fwd(h, self.decoder.final_layernorm.weight, self.cfg.norm_epsilon,
                                  want_rstd=False)
        from ..ops.gemm import linear_fwd

        return linear_fwd(self.comm.gather_seq(x), self.output_weight())


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, eps):
        y, rstd, _ = ops.rmsnorm_fwd(h, w, eps)
        ctx.save_for_backward(h, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        h, w, rstd = ctx.saved_tensors
        dx = ops.rmsnorm_bwd(dy.contiguous(), h, w, rstd, grad_buffer(w))
        return dx, None, None


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return comm.gather_seq(x)

    @staticmethod
    def backward(ctx, d):
        return ctx.comm.gather_seq_bwd(d.contiguous()), None


def count_parameters(model: nn.Module) -> int:
    return sum(p.numel() for p in model.parameters())
