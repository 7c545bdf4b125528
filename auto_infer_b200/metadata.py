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


# A mixed step (decode rows + prefill chunks) may run its two kernels side by side on disjoint
# SMs: the decode kernel is bound by memory bandwidth, the wide-query kernel by the tensor pipe
# and shared memory.  Cost model, measured on the part: a decode CTA streaming beside the
# wide-query kernel moves about 53 GB/s (all of them together at most the copy bandwidth); one
# 128 x 128 tile of the wide-query kernel takes about 1.26 us on one SM.
_HBM_GBS = 6450.0
_DECODE_GBS_PER_SM = 53.0
_PREFILL_US_PER_TILE = 1.26
_DECODE_FIXED_US, _PREFILL_FIXED_US = 6.0, 4.0


def mixed_split(decode_bytes: int, prefill_tiles: int, sms: int, prefill_items: int = 0,
                longest_item_tiles: int = 0) -> int:
    """SMs to give the wide-query kernel in a mixed step (a multiple of 8), or 0 when running the
    two kernels one after the other on all SMs is expected to be as fast (within 7 %).  The
    wide-query kernel's work comes in items of 128 query rows (``prefill_items`` of them, the
    longest ``longest_item_tiles`` tiles): with few items per SM the longest ones set its time."""
    if decode_bytes <= 0 or prefill_tiles <= 0 or sms < 32:
        return 0

    def t_dec(n):
        return decode_bytes / (min(_HBM_GBS, n * _DECODE_GBS_PER_SM) * 1e3) + _DECODE_FIXED_US

    def t_pre(n):
        tiles = prefill_tiles / n
        if prefill_items and longest_item_tiles:
            rounds = -(-prefill_items // n)
            if rounds <= 2:                       # whole items, longest first: the last round sets the time
                tiles = max(tiles, longest_item_tiles * rounds)
            else:
                tiles += longest_item_tiles / 2
        return tiles * _PREFILL_US_PER_TILE + _PREFILL_FIXED_US

    one_after_the_other = t_dec(sms) + t_pre(sms)
    best_n, best_t = 0, one_after_the_other
    for n in range(8, sms - 7, 8):
        t = max(t_dec(sms - n), t_pre(n))
        if t < best_t:
            best_n, best_t = n, t
    return best_n if best_t < 0.93 * one_after_the_other else 0


def scan_step(cu_seqlens_q, seqlens_kv, num_q_heads: int, num_kv_heads: int, head_dim: int,
              causal_base=None):
    """(indices of the sequences for the wide-query kernel, KV bytes the decode kernel reads,
    128 x 128 tiles the wide-query kernel computes, its items, the longest item's tiles) of a step."""
    group = num_q_heads // num_kv_heads
    prefill_seqs, decode_bytes, prefill_tiles, prefill_items, longest = [], 0, 0, 0, 0
    prev = 0
    for b, end in enumerate(cu_seqlens_q):
        q_len, kv = int(end) - prev, int(seqlens_kv[b])
        prev = int(end)
        if q_len * group > 16:
            prefill_seqs.append(b)
            base = int(causal_base[b]) if causal_base is not None else kv - q_len
            tokens_per_item = max(1, 128 // group)
            for first in range(0, q_len, tokens_per_item):
                last_key = min(base + min(first + tokens_per_item, q_len) - 1, kv - 1)
                tiles = last_key // 128 + 1 if last_key >= 0 else 0
                prefill_tiles += tiles * num_kv_heads
                prefill_items += num_kv_heads
                longest = max(longest, tiles)
        elif q_len > 0:
            decode_bytes += kv * 2 * num_kv_heads * head_dim * 2
    return prefill_seqs, decode_bytes, prefill_tiles, prefill_items, longest


class StepMetadata:
    """Plans for one (step, head geometry): the split-KV decode plan covers the
    sequences whose q_len * group fits one 16-row MMA tile; wider sequences
    (prefill chunks) are listed for the prefill kernel.

    With ``capacity_seqs`` the decode plan keeps its buffers and is refilled by
    ``rebuild()``: no allocation per step, and launches recorded into a CUDA graph
    stay valid."""

    def __init__(self, cu_seqlens_q: Sequence[int], seqlens_kv: Sequence[int], num_q_heads: int,
                 num_kv_heads: int, head_dim: int, device, causal_base: Optional[Sequence[int]] = None,
                 num_ctas: Optional[int] = None, capacity_seqs: Optional[int] = None,
                 prefill_ctas: int = 0):
        """``prefill_ctas`` > 0: the step's two kernels are meant to run side by side, the
        wide-query kernel on that many SMs and the decode kernel (planned here for the rest) on
        the others; see ``mixed_split``."""
        self.num_q_heads, self.num_kv_heads, self.head_dim = num_q_heads, num_kv_heads, head_dim
        self.device = device
        self.prefill_ctas = int(prefill_ctas)
        if self.prefill_ctas:
            num_ctas = (int(num_ctas) if num_ctas else ops.sm_count(torch.device(device))) - self.prefill_ctas
            if num_ctas < 1:
                raise ValueError("prefill_ctas leaves no SM to the decode kernel")
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
                  causal_base: Optional[Sequence[int]] = None, pool: Optional[dict] = None,
                  split_mixed: bool = False) -> StepMetadata:
    """Fetch (or build and attach) the metadata of ``ctx`` for this head
    geometry.  The context is a plain mutable dataclass in the reference
    (auto_infer/forward_context.py:9), which already carries per-step extras
    such as the rope tables the same way (auto_infer/models/base.py:75).

    ``pool`` (a dict the backend owns) keeps one refillable metadata object per
    geometry: a new context then costs host planning and one small copy, not a set
    of allocations.  A pooled plan serves one step at a time: contexts of steps
    that overlap on the GPU must run on one stream.

    ``split_mixed``: a step with both decode rows and prefill chunks is planned for running its
    two kernels side by side when ``mixed_split`` expects a gain (``meta.prefill_ctas`` > 0)."""
    cache = getattr(ctx, _ATTR, None)
    if cache is None:
        cache = {}
        setattr(ctx, _ATTR, cache)
    key = (num_q_heads, num_kv_heads, head_dim, str(device))
    meta = cache.get(key)
    if meta is None:
        prefill_ctas = 0
        if split_mixed and torch.device(device).type == "cuda":
            _, decode_bytes, prefill_tiles, items, longest = scan_step(
                ctx.cu_seqlens_q, ctx.seqlens_kv, num_q_heads, num_kv_heads, head_dim, causal_base)
            prefill_ctas = mixed_split(decode_bytes, prefill_tiles, ops.sm_count(torch.device(device)),
                                       items, longest)
        pool_key = key + (prefill_ctas,)           # a plan is built for one share of the SMs
        pooled = pool.get(pool_key) if pool is not None else None
        if pooled is not None and pooled.capacity_seqs >= len(ctx.cu_seqlens_q):
            meta = pooled.rebuild(ctx.cu_seqlens_q, ctx.seqlens_kv, causal_base)
        else:
            capacity = None
            if pool is not None:
                capacity = max(16, 1 << (max(len(ctx.cu_seqlens_q), 1) - 1).bit_length())
            meta = StepMetadata(ctx.cu_seqlens_q, ctx.seqlens_kv, num_q_heads, num_kv_heads, head_dim,
                                device, causal_base=causal_base, capacity_seqs=capacity,
                                prefill_ctas=prefill_ctas)
            if pool is not None:
                pool[pool_key] = meta
        cache[key] = meta
    return meta
