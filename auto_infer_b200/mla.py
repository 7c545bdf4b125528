"""MLA attention backends for B200 (DeepSeek-V2/V3, Moonlight): the absorbed latent form
(``B200MlaBackend``) and the non-absorbed per-head form (``B200MlaPagedBackend``).

The absorbed form:

Same sub-block as auto-infer's ``mla_paged_absorbed``
(auto_infer/layers/attention/mla.py:76-122): q projection (optionally through the
q-LoRA), latent ``ckv = rms_norm(kv_a(x)[:kvl])`` plus the decoupled RoPE key,
the query folded into latent space with W_UK, attention of all heads over ONE
latent head of width kvl + rope, the first kvl output columns folded back with
W_UV, then o_proj.  The two vendor calls in it (cache write, paged attention) go
to the CUDA library; the latent is cached once per token instead of twice."""
from __future__ import annotations

from contextlib import nullcontext
from dataclasses import dataclass

import torch

from . import ops
from .base import AttentionBackend
from .gqa import rms_norm


def build_absorb_weights(kv_b_weight, num_heads, qk_nope, v_head_dim, kv_lora_rank):
    """kv_b_proj (H*(nope+vd), kvl) -> W_UK (H, nope, kvl), W_UV (H, vd, kvl)
    (auto_infer/layers/attention/mla.py:67-73)."""
    w = kv_b_weight.view(num_heads, qk_nope + v_head_dim, kv_lora_rank)
    w_uk, w_uv = w.split([qk_nope, v_head_dim], dim=1)
    return w_uk.contiguous(), w_uv.contiguous()


class B200MlaBackend(AttentionBackend):
    """Constructor keywords follow ``MlaFIABackend`` (mla.py:190-211).  Only the
    absorbed form is built (``absorb`` must stay True): it is the one whose cache
    is 9x smaller and whose attention is a single dense contraction.  ``num_heads`` is
    the number of heads THIS rank holds.  The kernel takes up to 16 heads at a time (one
    16-row MMA tile per sequence): a rank with more heads runs it once per slice of
    ``heads_per_launch`` heads, each slice streaming the latent cache again, so DeepSeek-V3's
    128 heads want a head-parallel degree of 8 (MLA has no all-reduce inside attention,
    auto_infer/layers/attention/mla.py:282-285) and merely work without it."""

    MAX_HEADS_PER_LAUNCH = 16

    def __init__(self, w: dict, *, num_heads: int, qk_nope: int, qk_rope: int, v_head_dim: int,
                 kv_lora_rank: int, q_lora_rank, rms_eps: float, softmax_scale: float,
                 num_layers: int, device, dtype, absorb: bool = True, layer_prefix=None):
        if not absorb:
            raise NotImplementedError("the B200 MLA backend implements the absorbed latent form only")
        if num_heads <= 0:
            raise ValueError("num_heads must be positive")
        # equal slices: the largest divisor of num_heads that fits one launch
        self.heads_per_launch = max(h for h in range(1, self.MAX_HEADS_PER_LAUNCH + 1) if num_heads % h == 0)
        self.w = w
        self.num_heads = num_heads
        self.qk_nope = qk_nope
        self.qk_rope = qk_rope
        self.v_head_dim = v_head_dim
        self.kv_lora_rank = kv_lora_rank
        self.q_lora_rank = q_lora_rank
        self.rms_eps = rms_eps
        self.softmax_scale = softmax_scale
        self.num_layers = num_layers
        self.device = torch.device(device)
        self.dtype = dtype
        self.absorb = True
        self.layer_prefix = layer_prefix or (lambda i: f"model.layers.{i}.")
        self._absorb_w: dict = {}

    def alloc_kv_caches(self, num_blocks: int, block_size: int) -> list:
        """Per layer ONE latent tensor (num_blocks, block_size, 1, kvl + rope),
        returned as both members of the (k_cache, v_cache) pair the reference's
        callers unpack (mla.py:214-219 allocates two)."""
        shape = (num_blocks, block_size, 1, self.kv_lora_rank + self.qk_rope)
        caches = []
        for _ in range(self.num_layers):
            latent = torch.zeros(shape, device=self.device, dtype=self.dtype)
            caches.append((latent, latent))
        return caches

    def _weights(self, layer_idx: int):
        if layer_idx not in self._absorb_w:
            prefix = self.layer_prefix(layer_idx)
            self._absorb_w[layer_idx] = build_absorb_weights(
                self.w[prefix + "self_attn.kv_b_proj.weight"], self.num_heads, self.qk_nope,
                self.v_head_dim, self.kv_lora_rank)
        return self._absorb_w[layer_idx]

    def attention(self, layer_idx: int, x: torch.Tensor, ctx) -> torch.Tensor:
        """The sub-block of ``mla_paged_absorbed`` (auto_infer/layers/attention/mla.py:76-122;
        its wiring is the plug-in contract, so the steps and their names follow it): q
        projection (optionally through the q-LoRA), kv_a projection, then ONE fused launch
        for the latent RMSNorm, both interleaved rotary embeddings and the latent slot
        write, the absorbed query, latent attention, W_UV, o_proj."""
        w, prefix = self.w, self.layer_prefix(layer_idx)
        t = x.shape[0]
        nh, nope, rope, vd, kvl = (self.num_heads, self.qk_nope, self.qk_rope, self.v_head_dim,
                                   self.kv_lora_rank)
        if self.q_lora_rank is None:
            q = x @ w[prefix + "self_attn.q_proj.weight"].t()
        else:
            q = rms_norm(x @ w[prefix + "self_attn.q_a_proj.weight"].t(),
                         w[prefix + "self_attn.q_a_layernorm.weight"], self.rms_eps)
            q = q @ w[prefix + "self_attn.q_b_proj.weight"].t()
        q = q.view(t, nh, nope + rope)
        q_nope, q_pe = q.split([nope, rope], dim=-1)
        ckv_full = x @ w[prefix + "self_attn.kv_a_proj_with_mqa.weight"].t()
        w_uk, w_uv = self._weights(layer_idx)
        q_latent = torch.empty(t, nh, kvl + rope, dtype=x.dtype, device=x.device)
        q_latent[..., :kvl] = torch.einsum("tnp,npl->tnl", q_nope, w_uk)
        latent_cache = ctx.kv_caches[layer_idx][0]
        ops.mla_rope_norm_cache(ckv_full, w[prefix + "self_attn.kv_a_layernorm.weight"], self.rms_eps, q_pe,
                                q_latent[..., kvl:], ctx.cos, ctx.sin, latent_cache, ctx.slot_mapping,
                                kv_lora_rank=kvl)
        o_latent = self._latent_attn(layer_idx, q_latent, ctx)
        o = torch.einsum("tnl,nvl->tnv", o_latent, w_uv)
        return o.reshape(t, nh * vd) @ w[prefix + "self_attn.o_proj.weight"].t()

    # -- the accelerated part: latent write + latent attention --------------
    def latent_attention(self, layer_idx: int, q_latent: torch.Tensor, k_latent: torch.Tensor,
                         ctx) -> torch.Tensor:
        """Latent slot write followed by latent attention for rows that are already normed and
        rotated."""
        latent_cache = ctx.kv_caches[layer_idx][0]
        ops.reshape_and_cache(k_latent, None, latent_cache, None, ctx.slot_mapping)
        return self._latent_attn(layer_idx, q_latent, ctx)

    def _latent_attn(self, layer_idx: int, q_latent: torch.Tensor, ctx) -> torch.Tensor:
        latent_cache = ctx.kv_caches[layer_idx][0]
        plan, block_table = self._plan(ctx, q_latent.device)
        return self._run_slices(q_latent, latent_cache, block_table, plan)

    def _run_slices(self, q_latent: torch.Tensor, latent_cache: torch.Tensor, block_table: torch.Tensor,
                    plan) -> torch.Tensor:
        """The kernel once per slice of ``heads_per_launch`` heads (one launch when the rank holds
        at most 16): a slice is a strided view of q_latent, its rows go to their columns of out."""
        h = self.heads_per_launch
        if h == self.num_heads:
            return ops.mla_decode_absorbed(q_latent, latent_cache, block_table, plan,
                                           self.softmax_scale, kv_lora_rank=self.kv_lora_rank)
        out = torch.empty(q_latent.shape[0], self.num_heads, self.kv_lora_rank, dtype=q_latent.dtype,
                          device=q_latent.device)
        for first in range(0, self.num_heads, h):
            part = ops.mla_decode_absorbed(q_latent[:, first:first + h], latent_cache, block_table, plan,
                                           self.softmax_scale, kv_lora_rank=self.kv_lora_rank)
            out[:, first:first + h].copy_(part)
        return out

    def _plan(self, ctx, device):
        """One plan per step.  The kernel takes q_len * heads <= 16 rows per
        sequence; a longer query block (prefill chunk) is planned as q_len
        single-token sequences that share the block-table row and end at
        kv_len - q_len + 1 + i keys, which is the same bottom-right causal mask."""
        cached = getattr(ctx, "_b200_mla_plan", None)
        if cached is not None and cached[0] == (self.heads_per_launch, str(device)):
            return cached[1], cached[2]
        cu, kv = list(ctx.cu_seqlens_q), list(ctx.seqlens_kv)
        block_table = ctx.block_table
        max_q = max(1, 16 // self.heads_per_launch)
        prev, wide = 0, False
        for end in cu:
            wide |= (end - prev) > max_q
            prev = end
        if wide:
            new_cu, new_kv, rows = [], [], []
            prev = acc = 0
            for b, end in enumerate(cu):
                q_len = end - prev
                prev = end
                for i in range(q_len):
                    acc += 1
                    new_cu.append(acc)
                    new_kv.append(kv[b] - q_len + 1 + i)
                    rows.append(b)
            cu, kv = new_cu, new_kv
            block_table = block_table.index_select(
                0, torch.tensor(rows, dtype=torch.long, device=block_table.device))
        plan = self._make_plan(cu, kv, device, wide)
        assert plan.skipped_seqs == 0
        setattr(ctx, "_b200_mla_plan", ((self.heads_per_launch, str(device)), plan, block_table))
        return plan, block_table

    def _make_plan(self, cu, kv, device, wide: bool):
        return ops.MlaDecodePlan(cu, kv, self.heads_per_launch, device, kv_lora_rank=self.kv_lora_rank)


@dataclass(frozen=True)
class _GraphMlaRegistration:
    """One captured latent-attention call: the refillable plan its launch reads and the static
    tensors it was recorded against (the counterpart of ``_FiaRegistration``,
    auto_infer/layers/attention/graph_fia.py:6-14)."""
    plan: object
    layer_idx: int
    query: torch.Tensor
    output: torch.Tensor


class B200GraphMlaBackend(B200MlaBackend):
    """Graph-capturable absorbed MLA: the lifecycle surface of ``GraphFiaLifecycle``
    (auto_infer/layers/attention/graph_fia.py:17-104: ``capturing``, ``reg``,
    ``begin_capture() / end_capture()``, ``update() / update_registrations() /
    update_many()``) that the graph runners drive on ``GraphMlaBackend``
    (auto_infer/layers/attention/mla.py:258-366), over the latent kernel.  The reference's
    graph flavour of MLA is the non-absorbed one, because its vendor op cannot take the
    576-wide head; here the captured launch is the absorbed kernel reading lengths and work
    list from a plan at a fixed device address, and an update is one refill of that plan for
    all layers.  Decode gears only (``supports_prefill_graph`` False): a prefill chunk is
    planned as one single-token sequence per query row, whose count changes with the step.

    Capture protocol as for ``B200GraphGqaBackend``: one eager step with the context the
    capture will use (that allocates the plan), ``begin_capture()``, the same step recorded
    with the same context object, ``end_capture()``, ``gear.reg = backend.reg``."""

    supports_prefill_graph = False

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.capturing = False
        self.reg: list = []
        self._plan_pool: dict = {}        # refillable plans by batch size

    def begin_capture(self) -> None:
        self.capturing = True
        self.reg = []

    def end_capture(self) -> None:
        self.capturing = False

    def _make_plan(self, cu, kv, device, wide: bool):
        if wide:        # per-row expansion: not replayable, and never recorded
            return ops.MlaDecodePlan(cu, kv, self.heads_per_launch, device, kv_lora_rank=self.kv_lora_rank)
        key = (len(cu), str(device))
        plan = self._plan_pool.get(key)
        if plan is None:
            if self.capturing:
                raise RuntimeError(
                    "capture needs one eager step with the same context first (capturing False): the "
                    "plan's buffers cannot be allocated while the stream is being captured")
            plan = ops.MlaDecodePlan(cu, kv, self.heads_per_launch, device, kv_lora_rank=self.kv_lora_rank,
                                     capacity_seqs=len(cu))
            self._plan_pool[key] = plan
        else:
            plan.refill(cu, kv)
        return plan

    def _latent_attn(self, layer_idx: int, q_latent: torch.Tensor, ctx) -> torch.Tensor:
        if not self.capturing:
            return super()._latent_attn(layer_idx, q_latent, ctx)
        cached = getattr(ctx, "_b200_mla_plan", None)
        if cached is None or cached[0] != (self.heads_per_launch, str(q_latent.device)) or not cached[1].replayable:
            raise RuntimeError(
                "capture needs one eager step with the same context first (capturing False), and a "
                "decode-shaped step: a prefill chunk cannot be recorded")
        plan, block_table = cached[1], cached[2]
        for key, pooled in list(self._plan_pool.items()):
            if pooled is plan:                      # the plan now belongs to this capture
                del self._plan_pool[key]
        latent_cache = ctx.kv_caches[layer_idx][0]
        out = self._run_slices(q_latent, latent_cache, block_table, plan)
        self.reg.append(_GraphMlaRegistration(plan, layer_idx, q_latent, out))
        return out

    # -- per-step update (graph_fia.py:87-104) --------------------------------
    def _refill(self, plan, ctx, stream) -> None:
        cu, kv = list(ctx.cu_seqlens_q), list(ctx.seqlens_kv)
        max_q = max(1, 16 // self.heads_per_launch)
        prev = 0
        for end in cu:
            if end - prev > max_q:
                raise ValueError("this graph was captured on a decode-shaped step: a step with wider query "
                                 "blocks runs eagerly")
            prev = end
        with (torch.cuda.stream(stream) if stream is not None else nullcontext()):
            plan.refill(cu, kv)

    def update(self, ctx, stream=None) -> None:
        self.update_registrations(self.reg, ctx, stream)

    def update_registrations(self, registrations, ctx, stream=None) -> None:
        seen = set()
        for registration in registrations:
            if id(registration.plan) not in seen:
                seen.add(id(registration.plan))
                self._refill(registration.plan, ctx, stream)

    def update_many(self, contexts, stream=None) -> None:
        if len(contexts) != len(self.reg):
            raise ValueError("graph-task contexts must match registrations")
        seen = set()
        for ctx, registration in zip(contexts, self.reg):
            if id(registration.plan) not in seen:
                seen.add(id(registration.plan))
                self._refill(registration.plan, ctx, stream)


def ds_rope_interleave(x: torch.Tensor) -> torch.Tensor:
    """DeepSeek's interleaved rotary layout -> the half-split one ``rotate_half`` expects
    (auto_infer/layers/rotary_embedding/__init__.py:15-23): even dims first, then odd."""
    *lead, d = x.shape
    return x.view(*lead, d // 2, 2).transpose(-1, -2).reshape(*lead, d)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """(auto_infer/layers/rotary_embedding/__init__.py:10-12)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


class B200MlaPagedBackend(AttentionBackend):
    """The non-absorbed MLA sub-block of ``MlaFIABackend(absorb=False)``
    (auto_infer/layers/attention/mla.py:134-164, 167-255): per-head decompressed
    K = [k_nope | k_pe] (192 wide) and V (128 wide) in caches of the reference's own shapes
    (mla.py:214-216), attention as multi-head attention with one kv head per query head.  The
    projections and the rotary embedding are the reference's torch chain, op for op; the two
    vendor calls (``write_kv``, ``paged_fia``) go to the CUDA library.  It exists for engines
    that keep the reference's default cache layout; the absorbed backend reads 9x fewer bytes
    per token and is the form to prefer on this hardware.  No tensor-parallel all-reduce, as in
    the reference (mla.py:282-285)."""

    def __init__(self, w: dict, *, num_heads: int, qk_nope: int, qk_rope: int, v_head_dim: int,
                 kv_lora_rank: int, q_lora_rank, rms_eps: float, softmax_scale: float,
                 num_layers: int, device, dtype, absorb: bool = False, layer_prefix=None):
        if absorb:
            raise ValueError("absorb=True is B200MlaBackend")
        if qk_nope + qk_rope != 192 or v_head_dim != 128:
            raise NotImplementedError(
                f"the multi-head kernel is built for K 192 / V 128 per head, not {qk_nope + qk_rope} / {v_head_dim}")
        self.w = w
        self.num_heads = num_heads
        self.qk_nope = qk_nope
        self.qk_rope = qk_rope
        self.v_head_dim = v_head_dim
        self.kv_lora_rank = kv_lora_rank
        self.q_lora_rank = q_lora_rank
        self.rms_eps = rms_eps
        self.softmax_scale = softmax_scale
        self.num_layers = num_layers
        self.device = torch.device(device)
        self.dtype = dtype
        self.absorb = False
        self.layer_prefix = layer_prefix or (lambda i: f"model.layers.{i}.")

    def alloc_kv_caches(self, num_blocks: int, block_size: int) -> list:
        """Per layer (k_cache, v_cache) with the shapes of mla.py:214-216."""
        kshape = (num_blocks, block_size, self.num_heads, self.qk_nope + self.qk_rope)
        vshape = (num_blocks, block_size, self.num_heads, self.v_head_dim)
        return [(torch.zeros(kshape, device=self.device, dtype=self.dtype),
                 torch.zeros(vshape, device=self.device, dtype=self.dtype))
                for _ in range(self.num_layers)]

    def attention(self, layer_idx: int, x: torch.Tensor, ctx) -> torch.Tensor:
        """``_MlaProjMixin.attention`` (mla.py:134-164): q projection (optionally through the
        q-LoRA), kv_a projection, latent RMSNorm, kv_b decompression, interleaved rotary
        embedding of q_pe and of the shared k_pe, per-head K = [k_nope | k_pe], slot write,
        attention, o_proj."""
        w, p = self.w, self.layer_prefix(layer_idx)
        t = x.shape[0]
        nh, nope, rope, vd = self.num_heads, self.qk_nope, self.qk_rope, self.v_head_dim
        cos1, sin1 = ctx.cos, ctx.sin
        if self.q_lora_rank is None:
            q = x @ w[p + "self_attn.q_proj.weight"].t()
        else:
            q = rms_norm(x @ w[p + "self_attn.q_a_proj.weight"].t(),
                         w[p + "self_attn.q_a_layernorm.weight"], self.rms_eps)
            q = q @ w[p + "self_attn.q_b_proj.weight"].t()
        q = q.view(t, nh, nope + rope)
        q_nope, q_pe = q.split([nope, rope], dim=-1)
        ckv = x @ w[p + "self_attn.kv_a_proj_with_mqa.weight"].t()
        ckv, k_pe = ckv.split([self.kv_lora_rank, rope], dim=-1)
        k_pe = k_pe.view(t, 1, rope)
        kv = rms_norm(ckv, w[p + "self_attn.kv_a_layernorm.weight"], self.rms_eps)
        kv = (kv @ w[p + "self_attn.kv_b_proj.weight"].t()).view(t, nh, nope + vd)
        k_nope, v = kv.split([nope, vd], dim=-1)
        q_pe = ds_rope_interleave(q_pe)
        k_pe = ds_rope_interleave(k_pe)
        q_pe = q_pe * cos1 + rotate_half(q_pe) * sin1
        k_pe = k_pe * cos1 + rotate_half(k_pe) * sin1
        q = torch.cat([q_nope, q_pe], dim=-1)
        k = torch.cat([k_nope, k_pe.expand(t, nh, rope)], dim=-1).contiguous()
        v = v.contiguous()
        o = self.paged_attention(layer_idx, q, k, v, ctx).reshape(t, nh * vd)
        return o @ w[p + "self_attn.o_proj.weight"].t()

    # -- the accelerated part: write_kv + paged_fia (mla.py:238-254) ---------
    def _write_kv(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor, ctx) -> None:
        kc, vc = ctx.kv_caches[layer_idx]
        ops.reshape_and_cache(k, v, kc, vc, ctx.slot_mapping)

    def _attn(self, layer_idx: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ctx) -> torch.Tensor:
        kc, vc = ctx.kv_caches[layer_idx]
        return ops.paged_mha(q, kc, vc, ctx.block_table, self._plan(ctx, q.device), self.softmax_scale)

    def paged_attention(self, layer_idx: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                        ctx) -> torch.Tensor:
        self._write_kv(layer_idx, k, v, ctx)
        return self._attn(layer_idx, q, k, v, ctx)

    def _plan(self, ctx, device):
        """One plan per step, shared by the layers (kept on the context object)."""
        key = (self.num_heads, str(device))
        cached = getattr(ctx, "_b200_mha_plan", None)
        if cached is not None and cached[0] == key:
            return cached[1]
        plan = ops.MhaPlan(list(ctx.cu_seqlens_q), list(ctx.seqlens_kv), self.num_heads, device)
        setattr(ctx, "_b200_mha_plan", (key, plan))
        return plan
