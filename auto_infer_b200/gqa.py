"""GQA attention backend for B200: the same q/k/v projection, optional QK
RMSNorm, NeoX RoPE and o_proj wrapper as auto-infer's GQA family
(auto_infer/layers/attention/gqa.py:27-49), with the two vendor operators of
``GqaFIABackend`` (gqa.py:76-94) replaced by calls into the CUDA library."""
from __future__ import annotations

import torch

from contextlib import nullcontext
from dataclasses import dataclass

from . import ops
from .base import AttentionBackend, _lin
from .metadata import StepMetadata, cached_step_metadata, step_metadata


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last axis in fp32 (device-agnostic stand-in for the
    vendor op behind auto_infer/layers/norm.py:5-9)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


class B200GqaBackend(AttentionBackend):
    """Paged GQA attention on sm_100a.  Constructor arguments and cache shape
    match ``GqaFIABackend`` (gqa.py:56-74), so the registry builder can pass the
    same keyword set."""

    _one_launch_step = True           # paged_attention may fold the slot write into the attention launch
    _overlap_mixed = True             # a mixed step may run its two kernels side by side on disjoint SMs

    def __init__(self, n_q_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                 num_layers: int, device, dtype, w: dict = None, layer_prefix=None, rms_eps=None,
                 tp_group=None):
        if n_q_heads % n_kv_heads:
            raise ValueError("n_q_heads must be a multiple of n_kv_heads")
        self.n_q_heads = n_q_heads
        self.n_kv_heads = n_kv_heads
        self.head_dim = head_dim
        self.scale = scale
        self.num_layers = num_layers
        self.device = torch.device(device)
        self.dtype = dtype
        self.w = w
        self.layer_prefix = layer_prefix or (lambda i: f"model.layers.{i}.")
        self.rms_eps = rms_eps
        self.tp_group = tp_group
        self._meta_pool: dict = {}        # refillable per-step plans, one per head geometry
        self._side_stream = None          # second stream of a mixed step run side by side

    # -- cache ------------------------------------------------------------
    def alloc_kv_caches(self, num_blocks: int, block_size: int) -> list:
        """Per-layer (2, num_blocks, block_size, n_kv, head_dim) zeros, the shape
        of gqa.py:69-74.  A (block, kv head) K tile is block_size rows of
        head_dim*2 bytes at stride n_kv*head_dim*2: one 4-D TMA box."""
        if self.dtype != torch.bfloat16:
            raise NotImplementedError("the B200 kernels are built for bf16 caches")
        shape = (2, num_blocks, block_size, self.n_kv_heads, self.head_dim)
        return [torch.zeros(shape, device=self.device, dtype=self.dtype)
                for _ in range(self.num_layers)]

    # -- whole sub-block ----------------------------------------------------
    def attention(self, layer_idx: int, x: torch.Tensor, ctx) -> torch.Tensor:
        """The sub-block of auto_infer/layers/attention/gqa.py:27-49 (its wiring is the plug-in
        contract): packed QKV projection, optional QK RMSNorm, NeoX RoPE, slot write, paged
        attention, o_proj, tensor-parallel all-reduce.  Everything between the two GEMMs
        runs in two launches here: the fused prologue (norm + RoPE + slot write) and the
        attention kernel."""
        t = x.shape[0]
        n_q, n_kv, hd = self.n_q_heads, self.n_kv_heads, self.head_dim
        w = self.w
        p = self.layer_prefix(layer_idx) + "self_attn."
        qkv = _lin(x, w[p + "qkv_proj.weight"], w.get(p + "qkv_proj.bias"))
        q, k, v = qkv.split((n_q * hd, n_kv * hd, n_kv * hd), dim=-1)
        cache = ctx.kv_caches[layer_idx]
        qn = w.get(p + "q_norm.weight")
        q = ops.gqa_rope_cache(q.view(t, n_q, hd), k.view(t, n_kv, hd), v.view(t, n_kv, hd), ctx.cos, ctx.sin,
                               cache[0], cache[1], ctx.slot_mapping, q_norm_weight=qn,
                               k_norm_weight=w[p + "k_norm.weight"] if qn is not None else None,
                               eps=self.rms_eps if self.rms_eps is not None else 1e-6)
        o = self._attn(layer_idx, q, None, None, ctx).reshape(t, n_q * hd)
        out = _lin(o, w[p + "o_proj.weight"])
        if self.tp_group is not None and torch.distributed.get_world_size(self.tp_group) > 1:
            torch.distributed.all_reduce(out, group=self.tp_group)
        return out

    # -- the op pair that differs per execution mode (gqa.py:76-94) ---------
    def _write_kv(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor, ctx) -> None:
        cache = ctx.kv_caches[layer_idx]
        ops.reshape_and_cache(k, v, cache[0], cache[1], ctx.slot_mapping)

    def _attn(self, layer_idx: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              ctx) -> torch.Tensor:
        cache = ctx.kv_caches[layer_idx]
        meta = step_metadata(ctx, self.n_q_heads, self.n_kv_heads, self.head_dim, q.device,
                             pool=self._meta_pool, split_mixed=self._overlap_mixed)
        out = torch.empty(q.shape[0], self.n_q_heads, self.head_dim, dtype=q.dtype, device=q.device)
        if meta.prefill is not None and meta.prefill_ctas and meta.decode.info.num_items:
            # A mixed step, side by side: the wide-query kernel (tensor pipe, shared memory) on
            # its share of the SMs from a second stream, the decode kernel (memory bandwidth) on
            # the rest from this one; they write disjoint rows of `out` and join before returning.
            cur = torch.cuda.current_stream(q.device)
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(q.device)
            fork, join = torch.cuda.Event(), torch.cuda.Event()
            fork.record(cur)
            self._side_stream.wait_event(fork)
            with torch.cuda.stream(self._side_stream):
                ops.paged_prefill_gqa(q, cache[0], cache[1], ctx.block_table, meta.prefill, self.scale,
                                      out=out, max_ctas=meta.prefill_ctas)
                join.record(self._side_stream)
            ops.paged_decode_gqa(q, cache[0], cache[1], ctx.block_table, meta.decode, self.scale, out=out)
            cur.wait_event(join)
            return out
        if meta.decode.info.num_items:
            ops.paged_decode_gqa(q, cache[0], cache[1], ctx.block_table, meta.decode, self.scale,
                                 out=out)
        if meta.prefill is not None:
            ops.paged_prefill_gqa(q, cache[0], cache[1], ctx.block_table, meta.prefill, self.scale,
                                  out=out)
        return out

    def paged_attention(self, layer_idx: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                        ctx) -> torch.Tensor:
        """Cache write followed by attention for already projected and rotated
        q/k/v: the part of ``attention`` this package accelerates.  A step of decode-shaped
        rows only (no chunk for the wide-query kernel) is one launch: the attention kernel
        stores the new rows itself."""
        cache = ctx.kv_caches[layer_idx]
        meta = step_metadata(ctx, self.n_q_heads, self.n_kv_heads, self.head_dim, q.device,
                             pool=self._meta_pool, split_mixed=self._overlap_mixed)
        if meta.prefill is None and meta.decode.info.num_items and self._one_launch_step:
            return ops.paged_decode_gqa_write(q, k, v, ctx.slot_mapping, cache[0], cache[1], ctx.block_table,
                                              meta.decode, self.scale)
        self._write_kv(layer_idx, k, v, ctx)
        return self._attn(layer_idx, q, k, v, ctx)


@dataclass(frozen=True)
class _GraphRegistration:
    """One captured attention call: the refillable plan its launch reads and the static
    tensors it was recorded against (the counterpart of ``_FiaRegistration``,
    auto_infer/layers/attention/graph_fia.py:6-14)."""
    meta: StepMetadata
    layer_idx: int
    query: torch.Tensor
    output: torch.Tensor
    block_size: int


class B200GraphGqaBackend(B200GqaBackend):
    """Graph-capturable variant, the counterpart of ``GraphGqaBackend`` +
    ``GraphFiaLifecycle`` (auto_infer/layers/attention/gqa.py:134-226,
    graph_fia.py:17-104) with the attributes the graph runners touch: ``capturing``,
    ``reg``, ``begin_capture() / end_capture()``, ``update() / update_registrations() /
    update_many()``, ``supports_prefill_graph``.

    The reference re-issues every layer's attention task on the host before each replay,
    because its vendor op takes the step's length lists as host arguments.  Here a captured
    launch reads lengths and work list from a plan at a fixed device address, so an update
    is ONE refill of that plan (host planning + one small copy) for all layers of the graph.

    Capture protocol (what the reference's runners do, worker/graph_decode_runner.py
    ``_capture``): run the step once eagerly with the context the capture will use
    (``capturing`` False) - that is when the plan's buffers are allocated - then
    ``begin_capture()``, record the step with the same context object, ``end_capture()``.
    The plan the capture used is taken out of the backend's pool and belongs to the graph
    from then on (``gear.reg = backend.reg``)."""

    supports_prefill_graph = True       # the wide-query launch is replayable too (gears of a fixed token count)

    _one_launch_step = False          # the recorded launches go through _write_kv / _attn
    _overlap_mixed = False            # a recorded gear keeps its launches on one stream

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.capturing = False
        self.reg: list = []

    def alloc_kv_caches(self, num_blocks: int, block_size: int) -> list:
        """Per layer TWO tensors (k, v), each (num_blocks, block_size, n_kv, head_dim), as
        gqa.py:192-200 (the runner passes num_blocks + its scratch blocks)."""
        if self.dtype != torch.bfloat16:
            raise NotImplementedError("the B200 kernels are built for bf16 caches")
        shape = (num_blocks, block_size, self.n_kv_heads, self.head_dim)
        return [(torch.zeros(shape, device=self.device, dtype=self.dtype),
                 torch.zeros(shape, device=self.device, dtype=self.dtype))
                for _ in range(self.num_layers)]

    # -- lifecycle (graph_fia.py:63-68) --------------------------------------
    def begin_capture(self) -> None:
        self.capturing = True
        self.reg = []

    def end_capture(self) -> None:
        self.capturing = False

    def _attn(self, layer_idx: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              ctx) -> torch.Tensor:
        if not self.capturing:
            return super()._attn(layer_idx, q, k, v, ctx)
        meta = cached_step_metadata(ctx, self.n_q_heads, self.n_kv_heads, self.head_dim, q.device)
        if meta is None or not meta.decode.replayable:
            raise RuntimeError(
                "capture needs one eager step with the same context first (capturing False): the "
                "plan's buffers cannot be allocated while the stream is being captured")
        if meta.prefill is not None and not meta.prefill.replayable:
            raise RuntimeError("the context's prefill plan was not built for replay")
        for key, pooled in list(self._meta_pool.items()):
            if pooled is meta:                      # the plan now belongs to this capture
                del self._meta_pool[key]
        cache = ctx.kv_caches[layer_idx]
        out = torch.empty(q.shape[0], self.n_q_heads, self.head_dim, dtype=q.dtype, device=q.device)
        ops.paged_decode_gqa(q, cache[0], cache[1], ctx.block_table, meta.decode, self.scale, out=out)
        if meta.prefill is not None:                # a prefill gear: both launches are recorded
            ops.paged_prefill_gqa(q, cache[0], cache[1], ctx.block_table, meta.prefill, self.scale, out=out)
        self.reg.append(_GraphRegistration(meta, layer_idx, q, out, cache[0].shape[1]))
        return out

    # -- per-step update (graph_fia.py:87-104) --------------------------------
    @staticmethod
    def _refill(meta: StepMetadata, ctx, stream) -> None:
        captured_prefill = meta.prefill
        with (torch.cuda.stream(stream) if stream is not None else nullcontext()):
            meta.rebuild(ctx.cu_seqlens_q, ctx.seqlens_kv)
        if meta.prefill is not captured_prefill:
            if captured_prefill is None:
                raise ValueError("this graph was captured on a step without wide query blocks: a step with "
                                 "prefill chunks needs a prefill gear (capture it with such a step)")
            raise ValueError("the step exceeds the token or sequence count the prefill gear was captured with")

    def update(self, ctx, stream=None) -> None:
        self.update_registrations(self.reg, ctx, stream)

    def update_registrations(self, registrations, ctx, stream=None) -> None:
        seen = set()
        for registration in registrations:
            if id(registration.meta) not in seen:
                seen.add(id(registration.meta))
                self._refill(registration.meta, ctx, stream)

    def update_many(self, contexts, stream=None) -> None:
        if len(contexts) != len(self.reg):
            raise ValueError("graph-task contexts must match registrations")
        seen = set()
        for ctx, registration in zip(contexts, self.reg):
            if id(registration.meta) not in seen:
                seen.add(id(registration.meta))
                self._refill(registration.meta, ctx, stream)
