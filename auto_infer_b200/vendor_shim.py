"""CUDA stand-in for the vendor module auto-infer calls (``torch_npu``), for running the
reference's own, unmodified backends and model code on a B200.

auto-infer reaches its device runtime in three places only: ``auto_infer/platform.py:5-15``
(``npu_device``), the ``torch.npu`` stream / event / graph classes the runners use, and the
functions of ``torch_npu`` it imports inside its layers:

    _npu_reshape_and_cache            auto_infer/layers/attention/base.py:41-45
    npu_fused_infer_attention_score   auto_infer/layers/attention/base.py:48-61
    npu_rms_norm / npu_add_rms_norm   auto_infer/layers/norm.py:5-17
    npu_swiglu                        auto_infer/layers/mlp.py:16-20, models/qwen2.py:110

``install()`` registers this module as ``torch_npu``, aliases ``torch.npu`` to ``torch.cuda``
and points ``auto_infer.platform.npu_device`` at a CUDA device.  With that, the reference's
``GqaFIABackend`` and ``MlaFIABackend`` (mode "paged"; MLA in its default non-absorbed form)
run on the kernels of this package through the very calls they already make: the two paged operators go to the C-ABI library, the three small
elementwise operators to plain torch (they are outside the attention path and not what
this package accelerates).  The families registered by ``install_into_auto_infer()`` are the
faster way in (one plan per step instead of one per layer call, fused prologue); the shim is
for bring-up and for the reference's own parity gates (``tools/parity.py``).

Call signatures and return arities follow the reference's call sites, keyword for keyword."""
from __future__ import annotations

import sys
from typing import Optional, Sequence

import torch

from . import ops
from .metadata import StepMetadata

_MODULE_NAME = "torch_npu"
_plan_cache: dict = {}


def _npu_reshape_and_cache(key, value, key_cache, value_cache, slot_indices) -> None:
    """``cache[slot] = row`` for the step's K and V (base.py:41-45)."""
    ops.reshape_and_cache(key, value, key_cache, value_cache, slot_indices)


def _step_plan(actual_seq_q: Sequence[int], actual_seq_kv: Sequence[int], num_heads: int,
               num_kv_heads: int, head_dim: int, device) -> StepMetadata:
    """The reference hands the same two host lists to every layer's call: plan once per
    distinct (lists, geometry) and keep the last few."""
    key = (tuple(int(c) for c in actual_seq_q), tuple(int(k) for k in actual_seq_kv), num_heads,
           num_kv_heads, head_dim, str(device))
    meta = _plan_cache.get(key)
    if meta is None:
        if len(_plan_cache) >= 8:
            _plan_cache.pop(next(iter(_plan_cache)))
        meta = StepMetadata(key[0], key[1], num_heads, num_kv_heads, head_dim, device)
        _plan_cache[key] = meta
    return meta


def _mha_plan(actual_seq_q: Sequence[int], actual_seq_kv: Sequence[int], num_heads: int, device):
    """As ``_step_plan``, for the K-192 / V-128 multi-head kernel."""
    key = ("mha", tuple(int(c) for c in actual_seq_q), tuple(int(k) for k in actual_seq_kv), num_heads, str(device))
    plan = _plan_cache.get(key)
    if plan is None:
        if len(_plan_cache) >= 8:
            _plan_cache.pop(next(iter(_plan_cache)))
        plan = ops.MhaPlan(key[1], key[2], num_heads, device)
        _plan_cache[key] = plan
    return plan


def npu_fused_infer_attention_score(query, key, value, *, block_table, input_layout="TND", block_size,
                                    actual_seq_lengths, actual_seq_lengths_kv, num_key_value_heads,
                                    num_heads, scale, atten_mask=None, sparse_mode=3):
    """Paged attention with the call contract of base.py:48-61: query (T, num_heads, D) packed
    TND, key / value 3-D cache views (num_blocks, block_size, num_kv_heads * D),
    ``actual_seq_lengths`` cumulative, ``actual_seq_lengths_kv`` per sequence, bottom-right
    causal mask (``sparse_mode`` 3; the 2048 x 2048 ``atten_mask`` template is an artefact of
    the vendor op and is ignored).  Returns ``(out, None)`` like the vendor op's
    ``(attention_out, softmax_lse)`` pair, whose second member the reference drops."""
    if input_layout != "TND" or sparse_mode != 3:
        raise NotImplementedError("only the layout and mask mode auto-infer uses: TND, sparse_mode 3")
    t, n_q, d = query.shape
    num_blocks = key.shape[0]
    if key.shape[1] != block_size or key.shape[2] != num_key_value_heads * d:
        raise ValueError("key must be the (num_blocks, block_size, num_kv_heads * head_dim) cache view")
    if value.shape[2] != num_key_value_heads * d:
        # the non-absorbed MLA call of MlaFIABackend._attn (auto_infer/layers/attention/mla.py:247-255):
        # one kv head per query head, K rows 192 wide, V rows 128 wide
        dv = value.shape[2] // num_key_value_heads
        if num_key_value_heads != num_heads or (d, dv) != (192, 128) or value.shape[2] != num_heads * dv:
            raise NotImplementedError("unequal K / V widths are served for the non-absorbed MLA shape only "
                                      "(one kv head per query head, K 192 / V 128)")
        plan = _mha_plan(actual_seq_lengths, actual_seq_lengths_kv, num_heads, query.device)
        out = ops.paged_mha(query, key.view(num_blocks, block_size, num_heads, d),
                            value.view(num_blocks, block_size, num_heads, dv), block_table, plan, scale)
        return out, None
    k4 = key.view(num_blocks, block_size, num_key_value_heads, d)
    v4 = value.view(num_blocks, block_size, num_key_value_heads, d)
    meta = _step_plan(actual_seq_lengths, actual_seq_lengths_kv, num_heads, num_key_value_heads, d,
                      query.device)
    out = torch.empty(t, n_q, d, dtype=query.dtype, device=query.device)
    if meta.decode.info.num_items:
        ops.paged_decode_gqa(query, k4, v4, block_table, meta.decode, scale, out=out)
    if meta.prefill is not None:
        ops.paged_prefill_gqa(query, k4, v4, block_table, meta.prefill, scale, out=out)
    return out, None


def rms_norm_reference(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last axis in fp32, rounded, then scaled by the weight."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


def npu_rms_norm(x, weight, eps):
    """``(normed, rstd)`` as norm.py:5-9 unpacks it (the second member is unused there)."""
    return rms_norm_reference(x, weight, eps), None


def npu_add_rms_norm(x, residual, weight, eps):
    """``(normed, rstd, residual + x)`` as norm.py:12-17 unpacks it."""
    new_residual = residual + x
    return rms_norm_reference(new_residual, weight, eps), None, new_residual


def npu_swiglu(gate_up):
    """``silu(gate) * up`` on the packed ``[gate | up]`` projection (mlp.py:16-20)."""
    gate, up = gate_up.chunk(2, dim=-1)
    return torch.nn.functional.silu(gate) * up


def cuda_device(index: int = 0) -> torch.device:
    """Replacement of ``auto_infer.platform.npu_device`` (platform.py:5-15)."""
    if not torch.cuda.is_available():
        raise RuntimeError("the B200 backend needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(index)
    return torch.device("cuda", index)


def install(patch_platform: bool = True) -> list:
    """Make ``import torch_npu`` resolve to this module (unless a real one is importable),
    alias ``torch.npu`` to ``torch.cuda`` and, when auto-infer is importable, point its
    ``platform.npu_device`` here.  Returns what was installed."""
    done = []
    if _MODULE_NAME not in sys.modules:
        try:
            __import__(_MODULE_NAME)
        except ImportError:
            sys.modules[_MODULE_NAME] = sys.modules[__name__]
            done.append("torch_npu")
    if not hasattr(torch, "npu"):
        torch.npu = torch.cuda
        if not hasattr(torch.cuda, "NPUGraph"):
            torch.cuda.NPUGraph = torch.cuda.CUDAGraph        # worker/graph_decode_runner.py:387
        done.append("torch.npu")
    if patch_platform:
        try:
            from auto_infer import platform as ref_platform
        except ImportError:
            ref_platform = None
        if ref_platform is not None and ref_platform.npu_device is not cuda_device:
            ref_platform.npu_device = cuda_device
            done.append("auto_infer.platform.npu_device")
    return done
