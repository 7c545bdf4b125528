"""GQA attention backend for B200: the same q/k/v projection, optional QK
RMSNorm, NeoX RoPE and o_proj wrapper as auto-infer's GQA family
(auto_infer/layers/attention/gqa.py:27-49), with the two vendor operators of
``GqaFIABackend`` (gqa.py:76-94) replaced by calls into the CUDA library."""
from __future__ import annotations

import torch

from . import ops
from .base import AttentionBackend, _lin
from .metadata import step_metadata


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """NeoX rotation (auto_infer/layers/rotary_embedding/__init__.py:10-12)."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last axis in fp32 (device-agnostic stand-in for the
    vendor op behind auto_infer/layers/norm.py:5-9)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


class B200GqaBackend(AttentionBackend):
    """Paged GQA attention on sm_100a.  Constructor arguments and cache shape
    match ``GqaFIABackend`` (gqa.py:56-74), so the registry builder can pass the
    same keyword set."""

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
        t = x.shape[0]
        n_q, n_kv, hd = self.n_q_heads, self.n_kv_heads, self.head_dim
        w = self.w
        p = self.layer_prefix(layer_idx) + "self_attn."
        qkv = _lin(x, w[p + "qkv_proj.weight"], w.get(p + "qkv_proj.bias"))
        q, k, v = qkv.split((n_q * hd, n_kv * hd, n_kv * hd), dim=-1)
        q = q.view(t, n_q, hd)
        k = k.view(t, n_kv, hd)
        v = v.view(t, n_kv, hd)
        qn = w.get(p + "q_norm.weight")
        if qn is not None:
            q = rms_norm(q, qn, self.rms_eps)
            k = rms_norm(k, w[p + "k_norm.weight"], self.rms_eps)
        q = q * ctx.cos + rotate_half(q) * ctx.sin
        k = k * ctx.cos + rotate_half(k) * ctx.sin
        self._write_kv(layer_idx, k, v, ctx)
        o = self._attn(layer_idx, q, k, v, ctx).reshape(t, n_q * hd)
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
                             pool=self._meta_pool)
        out = torch.empty(q.shape[0], self.n_q_heads, self.head_dim, dtype=q.dtype, device=q.device)
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
        q/k/v: the part of ``attention`` this package accelerates."""
        self._write_kv(layer_idx, k, v, ctx)
        return self._attn(layer_idx, q, k, v, ctx)
