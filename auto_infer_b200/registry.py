"""Attention-family registry with the interface of
auto_infer/layers/attention/registry.py:11-157: families are registered by name,
``build_attention_backend(model, mode, num_blocks, block_size)`` looks the
model's ``ATTENTION_FAMILY`` up and returns ``(backend, kv_caches)``.  The
families registered here build the B200 backends; ``install_into_auto_infer``
adds them to the reference's own registry under new names."""
from __future__ import annotations

from typing import Callable

AttentionBuilder = Callable[[object, str], object]
MtpAttentionBuilder = Callable[[object, str, str], object]
_FAMILIES: dict = {}
_MTP_FAMILIES: dict = {}
_MODES = {"dense", "paged", "graph"}


def register_attention_family(name: str, builder: AttentionBuilder) -> None:
    if not name:
        raise ValueError("attention family name must not be empty")
    if name in _FAMILIES:
        raise ValueError(f"attention family already registered: {name}")
    _FAMILIES[name] = builder


def register_mtp_attention_family(name: str, builder: MtpAttentionBuilder) -> None:
    if not name:
        raise ValueError("MTP attention family name must not be empty")
    if name in _MTP_FAMILIES:
        raise ValueError(f"MTP attention family already registered: {name}")
    _MTP_FAMILIES[name] = builder


def _dense_unavailable(family: str):
    raise NotImplementedError(
        f"{family}: mode 'dense' is auto-infer's eager torch bring-up path; use the reference's "
        "DenseBackend / MlaDenseBackend for it (install_into_auto_infer() routes it there)")


def _gqa(model, mode: str):
    from .gqa import B200GqaBackend, B200GraphGqaBackend
    if mode == "dense":
        _dense_unavailable("gqa")
    cfg = model.cfg
    # "graph": the same kernels behind the lifecycle surface the graph runners drive
    # (auto_infer/layers/attention/gqa.py:134-226); lengths are read from a refillable plan
    # in device memory, so a replay needs one plan refill instead of a per-layer re-issue.
    cls = B200GraphGqaBackend if mode == "graph" else B200GqaBackend
    return cls(
        n_q_heads=model.n_q_local, n_kv_heads=model.n_kv_local, head_dim=cfg.head_dim,
        scale=cfg.head_dim ** -0.5, num_layers=cfg.num_layers, device=model.device,
        dtype=model.dtype, w=model.w, layer_prefix=model.layer_prefix, rms_eps=cfg.rms_eps)


def _gqa_mtp(model, mode: str, prefix: str):
    from .gqa import B200GqaBackend, B200GraphGqaBackend
    cfg = model.cfg
    cls = B200GraphGqaBackend if mode == "graph" else B200GqaBackend
    return cls(
        n_q_heads=model.n_q_local, n_kv_heads=model.n_kv_local, head_dim=cfg.head_dim,
        scale=cfg.head_dim ** -0.5, num_layers=1, device=model.device, dtype=model.dtype,
        w=model.w, layer_prefix=lambda _: prefix, rms_eps=cfg.rms_eps)


def _mla(model, mode: str):
    from .mla import B200GraphMlaBackend, B200MlaBackend, B200MlaPagedBackend
    if mode == "dense":
        _dense_unavailable("mla")
    cfg = model.cfg
    # The reference keeps the absorbed form off by default because its vendor op rejects a
    # 576-wide head (auto_infer/models/deepseek_v2.py:62-64); here it is the default.  A model
    # that sets ``_mla_b200_absorb = False`` keeps the reference's per-head K 192 / V 128
    # caches (auto_infer/layers/attention/registry.py:80-85 reads ``_mla_absorb`` the same way).
    absorb = getattr(model, "_mla_b200_absorb", True)
    if mode == "graph":
        if not absorb:
            raise NotImplementedError("mla: mode 'graph' is built for the absorbed form only")
        cls = B200GraphMlaBackend
    else:
        cls = B200MlaBackend if absorb else B200MlaPagedBackend
    return cls(
        model.w, num_heads=cfg.num_heads, qk_nope=cfg.qk_nope, qk_rope=cfg.qk_rope,
        v_head_dim=cfg.v_head_dim, kv_lora_rank=cfg.kv_lora_rank, q_lora_rank=cfg.q_lora_rank,
        rms_eps=cfg.rms_eps, softmax_scale=model._softmax_scale, num_layers=cfg.num_layers,
        device=model.device, dtype=model.dtype, absorb=absorb, layer_prefix=model.layer_prefix)


register_attention_family("gqa", _gqa)
register_attention_family("mla", _mla)
register_mtp_attention_family("gqa", _gqa_mtp)


def build_attention_backend(model, mode: str, num_blocks: int = 0, block_size: int = 0):
    if mode not in _MODES:
        raise ValueError(f"unsupported attention mode: {mode}")
    family = model.ATTENTION_FAMILY
    try:
        builder = _FAMILIES[family]
    except KeyError:
        choices = ", ".join(sorted(_FAMILIES))
        raise KeyError(
            f"unregistered attention family: {family}; registered families: {choices}") from None
    backend = builder(model, mode)
    return backend, backend.alloc_kv_caches(num_blocks, block_size)


def build_mtp_attention_backend(model, mode: str, prefix: str, num_blocks: int = 0,
                                block_size: int = 0):
    if mode not in {"paged", "graph"}:
        raise ValueError(f"unsupported MTP attention mode: {mode}")
    family = model.ATTENTION_FAMILY
    try:
        builder = _MTP_FAMILIES[family]
    except KeyError:
        raise NotImplementedError(f"{family} MTP attention does not support {mode} mode") from None
    backend = builder(model, mode, prefix)
    return backend, backend.alloc_kv_caches(num_blocks, block_size)


def install_into_auto_infer(suffix: str = "_b200") -> list:
    """Register the B200 families in auto-infer's own registry (names
    ``gqa_b200`` / ``mla_b200``; a model opts in by setting
    ``ATTENTION_FAMILY``).  Mode 'dense' is handed to the reference's eager
    backends.  Returns the names registered.  Raises ImportError when auto-infer
    is not importable."""
    from auto_infer.layers.attention import registry as ref

    names = []
    for name, builder in list(_FAMILIES.items()):
        ref_dense = ref._FAMILIES.get(name)

        def wrapped(model, mode, _builder=builder, _dense=ref_dense):
            if mode == "dense" and _dense is not None:
                return _dense(model, mode)
            return _builder(model, mode)

        ref.register_attention_family(name + suffix, wrapped)
        names.append(name + suffix)
    for name, builder in list(_MTP_FAMILIES.items()):
        ref.register_mtp_attention_family(name + suffix, builder)
    return names
