"""Activation offload to pinned host memory between a layer's forward and its backward.

Reference feature: ``swap_attention`` (MindSpeed ``docs/features/swap_attention.md``; flag in
``mindspeed_rl/config_cls/megatron_config.py``): instead of recomputing a layer, its saved
activations leave the device on a side stream right after the forward and come back, one layer
ahead of use, during the backward.  Here it applies to the layers that keep their intermediates
(``recompute_method: block`` leaves ``num_layers - recompute_num_layers`` of them per stage, all
layers without recompute).

Every large tensor of a layer's saved context is copied device->host on the swap stream (which
first waits for the forward that produced it); the device copy is released as soon as that copy is
done.  The backward of layer i waits for its own host->device copies and immediately issues those
of the layer saved before it, so the transfer of layer i-1 overlaps the backward math of layer i.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

MIN_BYTES = 1 << 20          # smaller tensors (row statistics, log-sum-exp) stay on the device

# entries of a layer's saved context by the part of the layer that produced them (``swap_modules`` names
# the parts that take part; the rest stays on the device)
MODULE_KEYS = {
    "input_norm": ("h", "x1g"),
    "self_attention": ("qkv", "attn", "pre", "lora"),
    "post_attention_norm": ("h1", "x2g"),
    "mlp": ("mlp_ctx",),
}


def keys_of(modules) -> Optional[frozenset]:
    """Context entries covered by the named layer parts; unknown names are an error."""
    out = set()
    for m in modules:
        if m not in MODULE_KEYS:
            raise ValueError(f"swap_modules: unknown part {m!r}; known: {sorted(MODULE_KEYS)}")
        out.update(MODULE_KEYS[m])
    return frozenset(out)


class _Swapped:
    """A tensor that currently lives in host memory."""
    __slots__ = ("host", "dev", "ready")

    def __init__(self, host: torch.Tensor):
        self.host = host
        self.dev: Optional[torch.Tensor] = None
        self.ready = None


class SwapHandle:
    def __init__(self, saved: Dict[str, Any], prev: Optional["SwapHandle"]):
        self.saved = saved
        self.prev = prev
        self.prefetched = False
        self.restored = False


class ActivationSwapper:
    def __init__(self, device, min_bytes: int = MIN_BYTES):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.min_bytes = min_bytes
        self.last: Optional[SwapHandle] = None
        self.bytes_out = 0
        self.bytes_in = 0

    # ---- forward side ---------------------------------------------------------------------------
    def _out(self, t):
        if not torch.is_tensor(t) or t.numel() * t.element_size() < self.min_bytes:
            return t
        self.bytes_out += t.numel() * t.element_size()
        if not self.cuda:
            return _Swapped(t.clone())
        host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        host.copy_(t, non_blocking=True)
        t.record_stream(self.stream)           # the allocator may reuse t only after the copy
        return _Swapped(host)

    def offload(self, saved: Dict[str, Any], keys: Optional[frozenset] = None) -> SwapHandle:
        """Move the large tensors of ``saved`` (of its entries ``keys`` when given) to the host; returns
        the handle the backward restores."""
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
        out: Dict[str, Any] = {}
        ctx = torch.cuda.stream(self.stream) if self.cuda else _Null()
        seen: Dict[int, Any] = {}

        def conv(v):
            if torch.is_tensor(v):
                key = v.data_ptr()
                if key not in seen:            # the same tensor may sit under two names
                    seen[key] = self._out(v)
                return seen[key]
            if isinstance(v, tuple):
                return tuple(conv(x) for x in v)
            if isinstance(v, dict):
                return {k: conv(x) for k, x in v.items()}
            return v
        with ctx:
            for k, v in saved.items():
                out[k] = conv(v) if (keys is None or k in keys) else v
        handle = SwapHandle(out, self.last if (self.last is not None and not self.last.restored) else None)
        self.last = handle
        return handle

    # ---- backward side --------------------------------------------------------------------------
    def _each(self, saved):
        for v in saved.values():
            if isinstance(v, _Swapped):
                yield v
            elif isinstance(v, (tuple, dict)):
                for x in (v.values() if isinstance(v, dict) else v):
                    if isinstance(x, _Swapped):
                        yield x

    def prefetch(self, handle: Optional[SwapHandle]) -> None:
        if handle is None or handle.prefetched or handle.restored:
            return
        handle.prefetched = True
        done = set()
        if self.cuda:
            with torch.cuda.stream(self.stream):
                for s in self._each(handle.saved):
                    if id(s) in done:
                        continue
                    done.add(id(s))
                    s.dev = torch.empty(s.host.shape, dtype=s.host.dtype, device=self.device)
                    s.dev.copy_(s.host, non_blocking=True)
                    self.bytes_in += s.host.numel() * s.host.element_size()
                ev = torch.cuda.Event()
                ev.record(self.stream)
            for s in self._each(handle.saved):
                s.ready = ev
        else:
            for s in self._each(handle.saved):
                if s.dev is None:
                    s.dev = s.host
                    self.bytes_in += s.host.numel() * s.host.element_size()

    def restore(self, handle: SwapHandle) -> Dict[str, Any]:
        """Device tensors of ``handle`` (waits for their copies), and starts the copies of the
        context saved before it."""
        self.prefetch(handle)
        main = torch.cuda.current_stream(self.device) if self.cuda else None

        def conv(v):
            if isinstance(v, _Swapped):
                if self.cuda:
                    main.wait_event(v.ready)
                    v.dev.record_stream(main)
                return v.dev
            if isinstance(v, tuple):
                return tuple(conv(x) for x in v)
            if isinstance(v, dict):
                return {k: conv(x) for k, x in v.items()}
            return v
        out = {k: conv(v) for k, v in handle.saved.items()}
        handle.restored = True
        handle.saved = {}
        if self.last is handle:
            self.last = None
        self.prefetch(handle.prev)
        return out


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_swappers: Dict[Any, ActivationSwapper] = {}


def swapper_for(device) -> ActivationSwapper:
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = str(device)
    if key not in _swappers:
        _swappers[key] = ActivationSwapper(device)
    return _swappers[key]
