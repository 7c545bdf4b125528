"""Self-check of the parity comparators (CPU): on references of the size the long-context
configurations produce, the stated absolute tolerance accepts a wrong output and the
scale-free comparison rejects it.  Guards the GPU parity tests against going blind."""
import pytest
import torch

from oracle import paged_attention_oracle as orc
from tests.parity import TOL, assert_scale_free, scale_free_violations


def _long_gqa_reference():
    """One config-5-length sequence (131 072 keys, group of 8 query heads on one kv head)."""
    from auto_infer_b200 import synth
    b = synth.build_gqa_batch("c5_like", [(1, 131072)], 8, 1, 128, 1024, 5)
    return orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                               b.seqlens_kv, b.scale)


def _mla_reference():
    """Two config-3-length latent rows (8 192 and 3 000 keys, 16 heads, 512 value columns)."""
    from auto_infer_b200 import synth
    b = synth.build_mla_batch("c3_like", [(1, 8192), (1, 3000)], 16, 96, 3)
    return orc.mla_latent_attention(b.q, b.kv_cache, b.block_table, b.cu_seqlens_q, b.seqlens_kv,
                                    b.scale, 512)


@pytest.fixture(scope="module", params=["gqa_131072", "mla_8192"])
def reference(request):
    torch.set_num_threads(max(torch.get_num_threads(), 4))
    return _long_gqa_reference() if request.param == "gqa_131072" else _mla_reference()


def _passes_stated_tolerance(out, ref) -> bool:
    try:
        torch.testing.assert_close(out.float(), ref.float(), **TOL)
        return True
    except AssertionError:
        return False


def test_absolute_tolerance_is_blind_at_long_context(reference):
    """Why the extra comparison exists: zeros pass rtol 2e-2 / atol 2e-2 here."""
    assert _passes_stated_tolerance(torch.zeros_like(reference), reference) or \
        _passes_stated_tolerance(0.9 * reference.float(), reference)


def test_scale_free_comparison_accepts_the_reference_and_its_bf16_neighbours(reference):
    assert_scale_free(reference, reference)
    # the same values rounded from a slightly different fp32 result (one ulp of slack)
    jitter = (reference.float() * (1 + 2.0 ** -9)).to(torch.bfloat16)
    assert_scale_free(jitter, reference)


@pytest.mark.parametrize("wrong", ["zeros", "scaled_0.9", "dropped_half", "one_row_swapped"])
def test_scale_free_comparison_rejects_wrong_outputs(reference, wrong):
    ref = reference
    if wrong == "zeros":
        out = torch.zeros_like(ref)
    elif wrong == "scaled_0.9":
        out = (0.9 * ref.float()).to(ref.dtype)
    elif wrong == "dropped_half":               # as if half of the keys had been skipped
        g = torch.Generator().manual_seed(1)
        out = (ref.float() + ref.float().std() * torch.randn(ref.shape, generator=g)).to(ref.dtype)
    else:
        out = ref.clone()
        out[0, 0], out[0, 1] = ref[0, 1], ref[0, 0]
    assert scale_free_violations(out, ref)
    with pytest.raises(AssertionError):
        assert_scale_free(out, ref)
