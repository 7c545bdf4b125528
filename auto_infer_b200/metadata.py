"""Per-step attention metadata.  The reference passes two host lists
(cumulative query lengths, per-sequence kv lengths) to its vendor op on every
layer (auto_infer/layers/attention/gqa.py:91-92).  Here they are turned into
device-side work lists once per step and cached on the context object, so all
layers of the step share one plan and one host-to-device copy."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import ops

_ATTR = "_b200_step_meta"


class StepMetadata:
    """Plans for one (step, head geometry): the split-KV decode plan covers the
    sequences whose q_len * group fits one 16-row MMA tile; wider sequences
    (prefill chunks) are listed for the prefill kernel.

    With ``capacity_seqs`` the decode plan keeps its buffers and is refilled by
    ``rebuild()``: no allocation per step, and launches recorded into a CUDA graph
    stay valid."""

    def __init__(self, cu_seqlens_q: Sequence[int], seqlens_kv: Sequence[int], num_q_heads: int,
                 num_kv_heads: int, head_dim: int, device, causal_base: Optional[Sequence[int]] = None,
                 num_ctas: Optional[int] = None, capacity_seqs: Optional[int] = None):
        self.num_q_heads, self.num_kv_heads, self.head_dim = num_q_heads, num_kv_heads, head_dim
        self.device = device
        self._scan(cu_seqlens_q, seqlens_kv)
        self.decode = ops.DecodePlan(self.cu_seqlens_q, self.seqlens_kv, num_q_heads, num_kv_heads,
                                     device, head_dim=head_dim, num_ctas=num_ctas,
                                     causal_base=causal_base, capacity_seqs=capacity_seqs)
        self._plan_prefill(causal_base)

    def _scan(self, cu_seqlens_q, seqlens_kv) -> None:
        self.cu_seqlens_q = [int(c) for c in cu_seqlens_q]
        self.seqlens_kv = [int(k) for k in seqlens_kv]
        if len(self.cu_seqlens_q) != len(self.seqlens_kv):
            raise ValueError("cu_seqlens_q and seqlens_kv must have one entry per sequence")
        self.num_tokens = self.cu_seqlens_q[-1] if self.cu_seqlens_q else 0
        group = self.num_q_heads // self.num_kv_heads
        prev = 0
        self.prefill_seqs = []
        for b, end in enumerate(self.cu_seqlens_q):
            if (end - prev) * group > 16:
                self.prefill_seqs.append(b)
            prev = end

    def _plan_prefill(self, causal_base) -> None:
        assert self.decode.skipped_seqs == len(self.prefill_seqs)
        prefill = getattr(self, "prefill", None)
        if prefill is not None and prefill.replayable and \
                self.num_tokens <= prefill.capacity_tokens and len(self.cu_seqlens_q) <= prefill.capacity_seqs:
            # refilled in place, also with a step that has no wide rows: a launch recorded
            # against this plan then finds an empty item list
            prefill.refill(self.cu_seqlens_q, self.seqlens_kv, causal_base)
            return
        self.prefill = None
        if self.prefill_seqs:
            replay = self.decode.replayable
            self.prefill = ops.PrefillPlan(self.cu_seqlens_q, self.seqlens_kv, self.num_q_heads,
                                           self.num_kv_heads, self.device, min_rows=16,
                                           causal_base=causal_base,
                                           capacity_tokens=self.num_tokens if replay else None,
                                           capacity_seqs=self.decode.capacity_seqs if replay else None)

    @property
    def capacity_seqs(self) -> int:
        return self.decode.capacity_seqs if self.decode.replayable else 0

    def rebuild(self, cu_seqlens_q: Sequence[int], seqlens_kv: Sequence[int],
                causal_base: Optional[Sequence[int]] = None) -> "StepMetadata":
        """Plan another step in place (decode plan refilled at its fixed address)."""
        self._scan(cu_seqlens_q, seqlens_kv)
        self.decode.refill(self.cu_seqlens_q, self.seqlens_kv, causal_base)
        self._plan_prefill(causal_base)
        return self


def cached_step_metadata(ctx, num_q_heads: int, num_kv_heads: int, head_dim: int, device):
    """The metadata already attached to ``ctx`` for this head geometry, or None."""
    cache = getattr(ctx, _ATTR, None)
    if cache is None:
        return None
    return cache.get((num_q_heads, num_kv_heads, head_dim, str(device)))


def step_metadata(ctx, num_q_heads: int, num_kv_heads: int, head_dim: int, device,
                  causal_base: Optional[Sequence[int]] = None, pool: Optional[dict] = None) -> StepMetadata:
    """Fetch (or build and attach) the metadata of ``ctx`` for this head
    geometry.  The context is a plain mutable dataclass in the reference
    (auto_infer/forward_context.py:9), which already carries per-step extras
    such as the rope tables the same way (auto_infer/models/base.py:75).

    ``pool`` (a dict the backend owns) keeps one refillable metadata object per
    geometry: a new context then costs host planning and one small copy, not a set
    of allocations.  A pooled plan serves one step at a time: contexts of steps
    that overlap on the GPU must run on one stream."""
    cache = getattr(ctx, _ATTR, None)
    if cache is None:
        cache = {}
        setattr(ctx, _ATTR, cache)
    key = (num_q_heads, num_kv_heads, head_dim, str(device))
    meta = cache.get(key)
    if meta is None:
        pooled = pool.get(key) if pool is not None else None
        if pooled is not None and pooled.capacity_seqs >= len(ctx.cu_seqlens_q):
            meta = pooled.rebuild(ctx.cu_seqlens_q, ctx.seqlens_kv, causal_base)
        else:
            capacity = None
            if pool is not None:
                capacity = max(16, 1 << (max(len(ctx.cu_seqlens_q), 1) - 1).bit_length())
            meta = StepMetadata(ctx.cu_seqlens_q, ctx.seqlens_kv, num_q_heads, num_kv_heads, head_dim,
                                device, causal_base=causal_base, capacity_seqs=capacity)
            if pool is not None:
                pool[key] = meta
        cache[key] = meta
    return meta
