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
    backend, caches = registry.build_attention_backend(_gqa_model(), "paged", num_blocks=5, block_size=128)
    assert isinstance(backend, B200GqaBackend)
    assert len(caches) == 3
    assert caches[0].shape == (2, 5, 128, 2, 128) and caches[0].dtype == torch.bfloat16
    assert float(caches[0].abs().sum()) == 0.0
    assert backend.scale == 128 ** -0.5


def test_graph_mode_has_the_lifecycle_surface_the_graph_runners_drive():
    """Attributes read by auto_infer/worker/graph_decode_runner.py:231,281,389-400,432-449
    and the two-tensor cache of auto_infer/layers/attention/gqa.py:192-200."""
    from auto_infer_b200.gqa import B200GraphGqaBackend
    backend, caches = registry.build_attention_backend(_gqa_model(), "graph", num_blocks=5, block_size=16)
    assert isinstance(backend, B200GraphGqaBackend) and isinstance(backend, B200GqaBackend)
    assert len(caches) == 3 and len(caches[0]) == 2
    assert caches[0][0].shape == caches[0][1].shape == (5, 16, 2, 128)
    assert caches[0][0].data_ptr() != caches[0][1].data_ptr()
    assert backend.capturing is False and backend.reg == []
    assert backend.supports_prefill_graph is True
    backend.begin_capture()
    assert backend.capturing is True and backend.reg == []
    backend.end_capture()
    assert backend.capturing is False
    for name in ("update", "update_registrations", "update_many"):
        assert callable(getattr(backend, name))
    with pytest.raises(ValueError, match="graph-task contexts must match registrations"):
        backend.update_many([object()])
    mtp, _ = registry.build_mtp_attention_backend(_gqa_model(), "graph", "model.mtp_layers.0.", 2, 16)
    assert isinstance(mtp, B200GraphGqaBackend) and mtp.num_layers == 1


def test_mla_family_caches_the_latent_once():
    backend, caches = registry.build_attention_backend(_mla_model(), "paged", num_blocks=4, block_size=128)
    assert isinstance(backend, B200MlaBackend)
    k_cache, v_cache = caches[1]
    assert k_cache is v_cache and k_cache.shape == (4, 128, 1, 576)


def test_mla_family_keeps_the_reference_per_head_caches_on_request():
    """``_mla_b200_absorb = False``: the non-absorbed form with the cache shapes of
    auto_infer/layers/attention/mla.py:214-216."""
    from auto_infer_b200.mla import B200MlaPagedBackend
    model = _mla_model()
    model._mla_b200_absorb = False
    backend, caches = registry.build_attention_backend(model, "paged", num_blocks=4, block_size=16)
    assert isinstance(backend, B200MlaPagedBackend) and not backend.absorb
    k_cache, v_cache = caches[0]
    assert k_cache.shape == (4, 16, 16, 192) and v_cache.shape == (4, 16, 16, 128)
    with pytest.raises(NotImplementedError):
        B200MlaPagedBackend({}, num_heads=4, qk_nope=64, qk_rope=32, v_head_dim=64, kv_lora_rank=64,
                            q_lora_rank=None, rms_eps=1e-6, softmax_scale=1.0, num_layers=1, device="cpu",
                            dtype=torch.bfloat16)


def test_mla_graph_mode_has_the_lifecycle_surface():
    """Mode "graph" of the MLA family: the attributes the graph runners touch
    (auto_infer/layers/attention/graph_fia.py:17-104)."""
    from auto_infer_b200.mla import B200GraphMlaBackend
    backend, caches = registry.build_attention_backend(_mla_model(), "graph", num_blocks=4, block_size=128)
    assert isinstance(backend, B200GraphMlaBackend) and caches[0][0].shape == (4, 128, 1, 576)
    assert backend.capturing is False and backend.reg == [] and backend.supports_prefill_graph is False
    backend.begin_capture()
    assert backend.capturing and backend.reg == []
    backend.end_capture()
    assert not backend.capturing
    for name in ("update", "update_registrations", "update_many"):
        assert callable(getattr(backend, name))
    with pytest.raises(ValueError):
        backend.update_many([object()])
    model = _mla_model()
    model._mla_b200_absorb = False
    with pytest.raises(NotImplementedError):
        registry.build_attention_backend(model, "graph", num_blocks=4, block_size=128)


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


# --------------------------------------------------------------------------- #
# the documented integration step, against the reference's own registry
# --------------------------------------------------------------------------- #
def _reference_registry():
    """auto-infer's registry module, or skip: the reference tree is only present on
    the build machine (``PYTHONPATH`` or the sibling checkout)."""
    import importlib
    import os
    import sys
    try:
        return importlib.import_module("auto_infer.layers.attention.registry")
    except ImportError:
        pass
    sibling = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                           "reference")
    if os.path.isdir(os.path.join(sibling, "auto_infer")):
        sys.path.insert(0, sibling)
        try:
            return importlib.import_module("auto_infer.layers.attention.registry")
        except ImportError:
            sys.path.remove(sibling)
    pytest.skip("auto_infer (the reference runtime) is not importable here")


def test_install_into_auto_infer_serves_the_reference_builders():
    """After ``install_into_auto_infer()`` the REFERENCE's ``build_attention_backend`` /
    ``build_mtp_attention_backend`` (auto_infer/layers/attention/registry.py:119-157) build
    the B200 backends for models that opt in by family name, and hand mode 'dense' to the
    reference's own eager backends."""
    ref = _reference_registry()
    if "gqa_b200" not in ref._FAMILIES:
        names = registry.install_into_auto_infer()
        assert set(names) == {"gqa_b200", "mla_b200"}
    with pytest.raises(ValueError, match="already registered"):
        registry.install_into_auto_infer()

    backend, caches = ref.build_attention_backend(_gqa_model("gqa_b200"), "paged", num_blocks=3, block_size=128)
    assert isinstance(backend, B200GqaBackend)
    assert len(caches) == 3 and caches[0].shape == (2, 3, 128, 2, 128)
    backend, caches = ref.build_attention_backend(_gqa_model("gqa_b200"), "graph", num_blocks=3, block_size=128)
    assert isinstance(backend, B200GqaBackend) and hasattr(backend, "update_many") and len(caches[0]) == 2

    from auto_infer.layers.attention.gqa import DenseBackend
    from auto_infer.layers.attention.mla import MlaDenseBackend
    dense, caches = ref.build_attention_backend(_gqa_model("gqa_b200"), "dense")
    assert isinstance(dense, DenseBackend) and caches == []
    mla_model = _mla_model()
    mla_model.ATTENTION_FAMILY = "mla_b200"
    dense, _ = ref.build_attention_backend(mla_model, "dense")
    assert isinstance(dense, MlaDenseBackend)
    backend, caches = ref.build_attention_backend(mla_model, "paged", num_blocks=2, block_size=128)
    assert isinstance(backend, B200MlaBackend) and caches[0][0].shape == (2, 128, 1, 576)

    mtp, caches = ref.build_mtp_attention_backend(_gqa_model("gqa_b200"), "paged", "model.mtp_layers.0.",
                                                  num_blocks=2, block_size=128)
    assert isinstance(mtp, B200GqaBackend) and mtp.num_layers == 1
    assert mtp.layer_prefix(0) == "model.mtp_layers.0." and len(caches) == 1
    with pytest.raises(ValueError, match="unsupported MTP attention mode"):
        ref.build_mtp_attention_backend(_gqa_model("gqa_b200"), "dense", "model.mtp_layers.0.")


def test_mla_backend_slices_heads_beyond_one_launch():
    """More than 16 heads on one rank (DeepSeek-V3's 128 without head parallelism) run as equal
    slices of at most 16 heads per launch; the slice is the largest divisor that fits."""
    def heads(n):
        return B200MlaBackend({}, num_heads=n, qk_nope=128, qk_rope=64, v_head_dim=128, kv_lora_rank=512,
                              q_lora_rank=None, rms_eps=1e-6, softmax_scale=192 ** -0.5, num_layers=1,
                              device="cpu", dtype=torch.bfloat16).heads_per_launch
    assert heads(16) == 16 and heads(128) == 16 and heads(8) == 8
    assert heads(24) == 12 and heads(20) == 10 and heads(17) == 1
    with pytest.raises(ValueError):
        heads(0)


def test_mixed_step_split_model():
    """The SM split of a mixed step: none when one side is missing or too small to matter, a
    multiple of 8 otherwise, larger for more prefill work; and the scan that feeds it."""
    from auto_infer_b200.metadata import mixed_split, scan_step
    assert mixed_split(0, 1000, 148) == 0 and mixed_split(10 ** 9, 0, 148) == 0
    assert mixed_split(10 ** 9, 3, 148) == 0                  # a sliver of prefill work: not worth a split
    n = mixed_split(1_060_000_000, 8448, 148)                 # the mixed benchmark configuration
    assert n % 8 == 0 and 40 <= n <= 72
    assert mixed_split(1_060_000_000, 12000, 148) > n > mixed_split(1_060_000_000, 5000, 148) > 0
    # 32 q / 8 kv heads: a 512-token chunk over a 1 024-token prefix and two decode rows
    seqs, dec_bytes, tiles, items, longest = scan_step([1, 513, 514], [100, 1536, 7], 32, 8, 128)
    assert seqs == [1] and dec_bytes == (100 + 7) * 2 * 8 * 128 * 2
    # items of 32 tokens (128 rows / group 4): item i sees keys up to 1024 + 32 i + 31
    assert tiles == sum(((1024 + 32 * i + 31) // 128 + 1) for i in range(16)) * 8
    assert items == 16 * 8 and longest == (1024 + 511) // 128 + 1
    # few long items: a share of the SMs that needs a second round of items is not worth it
    # (16 decode rows of 2 600 tokens beside ONE 512-token chunk over an 8 192-token prefix)
    _, db, pt, it, lg = scan_step(list(range(1, 17)) + [16 + 512], [2600] * 16 + [8192 + 512], 32, 8, 128)
    assert it == 128 and mixed_split(db, pt, 148, it, lg) == 0 and mixed_split(db, pt, 148) > 0
