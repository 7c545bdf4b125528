"""Host-side surface of the plug-in: the registry and the backend classes keep the
names, arguments and error behaviour of auto-infer's attention registry
(auto_infer/layers/attention/registry.py, tests/test_attention_backend.py there)."""
from types import SimpleNamespace

import pytest
import torch

from auto_infer_b200 import registry
from auto_infer_b200.base import AttentionBackend
from auto_infer_b200.forward_context import ForwardContext
from auto_infer_b200.gqa import B200GqaBackend
from auto_infer_b200.mla import B200MlaBackend, build_absorb_weights
from auto_infer_b200.token_layout import slot_mapping


def _gqa_model(family="gqa"):
    cfg = SimpleNamespace(head_dim=128, num_layers=3, rms_eps=1e-6)
    return SimpleNamespace(cfg=cfg, n_q_local=8, n_kv_local=2, w={}, layer_prefix=lambda i: f"model.layers.{i}.",
                           device="cpu", dtype=torch.bfloat16, ATTENTION_FAMILY=family)


def _mla_model():
    cfg = SimpleNamespace(num_heads=16, qk_nope=128, qk_rope=64, v_head_dim=128, kv_lora_rank=512,
                          q_lora_rank=None, rms_eps=1e-6, num_layers=2)
    return SimpleNamespace(cfg=cfg, w={}, layer_prefix=lambda i: f"model.layers.{i}.", device="cpu",
                           dtype=torch.bfloat16, _softmax_scale=192 ** -0.5, _mla_absorb=False,
                           ATTENTION_FAMILY="mla")


def test_backend_interface_is_abstract_and_minimal():
    with pytest.raises(TypeError):
        AttentionBackend()
    assert AttentionBackend.__abstractmethods__ == {"alloc_kv_caches", "attention"}


def test_gqa_family_builds_paged_and_graph_backends_with_reference_cache_shape():
    for mode in ("paged", "graph"):
        backend, caches = registry.build_attention_backend(_gqa_model(), mode, num_blocks=5, block_size=128)
        assert isinstance(backend, B200GqaBackend)
        assert len(caches) == 3
        assert caches[0].shape == (2, 5, 128, 2, 128) and caches[0].dtype == torch.bfloat16
        assert float(caches[0].abs().sum()) == 0.0
        assert backend.scale == 128 ** -0.5


def test_mla_family_caches_the_latent_once():
    backend, caches = registry.build_attention_backend(_mla_model(), "paged", num_blocks=4, block_size=128)
    assert isinstance(backend, B200MlaBackend)
    k_cache, v_cache = caches[1]
    assert k_cache is v_cache and k_cache.shape == (4, 128, 1, 576)


def test_registry_errors_match_the_reference():
    with pytest.raises(ValueError, match="unsupported attention mode"):
        registry.build_attention_backend(_gqa_model(), "eager")
    with pytest.raises(KeyError, match="unregistered attention family: nope; registered families"):
        registry.build_attention_backend(_gqa_model("nope"), "paged")
    with pytest.raises(ValueError, match="already registered"):
        registry.register_attention_family("gqa", lambda m, mode: None)
    with pytest.raises(ValueError, match="must not be empty"):
        registry.register_attention_family("", lambda m, mode: None)
    with pytest.raises(NotImplementedError):
        registry.build_attention_backend(_gqa_model(), "dense")


def test_new_family_needs_no_dispatcher_branch():
    seen = []

    class Fake(AttentionBackend):
        def alloc_kv_caches(self, num_blocks, block_size):
            seen.append((num_blocks, block_size))
            return ["cache"]

        def attention(self, layer_idx, x, ctx):
            return x

    registry.register_attention_family("fake_family_for_test", lambda model, mode: Fake())
    try:
        backend, caches = registry.build_attention_backend(_gqa_model("fake_family_for_test"), "paged", 7, 16)
        assert isinstance(backend, Fake) and caches == ["cache"] and seen == [(7, 16)]
    finally:
        registry._FAMILIES.pop("fake_family_for_test")


def test_mtp_capability_is_registered_separately():
    backend, caches = registry.build_mtp_attention_backend(_gqa_model(), "paged", "model.mtp_layers.0.", 3, 128)
    assert backend.num_layers == 1 and backend.layer_prefix(5) == "model.mtp_layers.0."
    assert len(caches) == 1
    with pytest.raises(NotImplementedError, match="mla MTP attention does not support paged mode"):
        registry.build_mtp_attention_backend(_mla_model(), "paged", "x.")
    with pytest.raises(ValueError, match="unsupported MTP attention mode"):
        registry.build_mtp_attention_backend(_gqa_model(), "dense", "x.")


def test_forward_context_fields_are_the_reference_set():
    import dataclasses
    names = [f.name for f in dataclasses.fields(ForwardContext)]
    assert names == ["token_ids", "positions", "slot_mapping", "block_table", "cu_seqlens_q",
                     "seqlens_kv", "attn_mask", "attn_backend", "kv_caches", "is_decode", "cos", "sin",
                     "active_token_mask"]


def test_slot_mapping_and_absorb_split():
    import numpy as np
    assert slot_mapping(np.asarray([7, 8, 9]), np.asarray([5, 6]), 4).tolist() == [33, 34]
    w = torch.arange(2 * (3 + 2) * 4, dtype=torch.float32).view(2 * 5, 4)
    w_uk, w_uv = build_absorb_weights(w, 2, 3, 2, 4)
    assert w_uk.shape == (2, 3, 4) and w_uv.shape == (2, 2, 4)
    assert torch.equal(w_uk[1], w[5:8]) and torch.equal(w_uv[0], w[3:5])


def test_backends_refuse_to_run_without_cuda_tensors():
    backend, caches = registry.build_attention_backend(_gqa_model(), "paged", 2, 128)
    ctx = ForwardContext(None, None, torch.zeros(1, dtype=torch.int32), torch.zeros(1, 1, dtype=torch.int32),
                         [1], [1], None, backend, caches, True)
    q = torch.zeros(1, 8, 128, dtype=torch.bfloat16)
    k = torch.zeros(1, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        backend.paged_attention(0, q, k, k, ctx)
