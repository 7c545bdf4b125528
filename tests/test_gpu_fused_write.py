"""The one-launch form of a decode step (slot write + attention, b200_paged_decode_gqa_write)
against the two-launch form and the oracle: outputs bit-equal to write-then-attend, caches
bit-exact against the oracle's write (auto_infer/layers/attention/base.py:41-61)."""
import pytest
import torch

from oracle import paged_attention_oracle as orc
from tests.parity import assert_attention_close

pytestmark = pytest.mark.gpu


def _both_ways(b, num_ctas=None, capacity_seqs=None):
    """Runs the step both ways on copies of the same cache; returns (fused out, fused cache,
    two-launch out, two-launch cache, fused lse)."""
    from auto_infer_b200 import ops
    d1, d2 = b.to("cuda"), b.to("cuda")
    plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, "cuda", num_ctas=num_ctas,
                          capacity_seqs=capacity_seqs)
    lse = torch.empty(b.num_tokens, b.n_q, dtype=torch.float32, device="cuda")
    fused = ops.paged_decode_gqa_write(d1.q, d1.k_new, d1.v_new, d1.slot_mapping, d1.kv_cache[0], d1.kv_cache[1],
                                       d1.block_table, plan, b.scale, lse_out=lse)
    ops.reshape_and_cache(d2.k_new, d2.v_new, d2.kv_cache[0], d2.kv_cache[1], d2.slot_mapping)
    plain = ops.paged_decode_gqa(d2.q, d2.kv_cache[0], d2.kv_cache[1], d2.block_table, plan, b.scale)
    torch.cuda.synchronize()
    assert ops.read_status("cuda") == 0
    return fused.cpu(), d1.kv_cache.cpu(), plain.cpu(), d2.kv_cache.cpu(), lse.cpu()


def _check(b, **kw):
    fused, cache1, plain, cache2, lse = _both_ways(b, **kw)
    orc.write_kv(b.k_new, b.v_new, b.kv_cache[0], b.kv_cache[1], b.slot_mapping.tolist())
    assert torch.equal(cache1, b.kv_cache), "fused write: cache differs from the oracle's write"
    assert torch.equal(cache2, b.kv_cache)
    assert torch.equal(fused, plain), "fused step differs from write-then-attend"
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                                       b.seqlens_kv, b.scale, return_lse=True)
    assert_attention_close(fused, ref, lse, ref_lse, what=b.name)


@pytest.mark.parametrize("block_size", [16, 128])
@pytest.mark.parametrize("heads", [(8, 2), (16, 8), (32, 4)])
def test_single_token_rows_at_every_tile_position(block_size, heads):
    """New row first in a tile (kv_len = 64k + 1), last in a tile, alone in the sequence."""
    from auto_infer_b200 import synth
    n_q, n_kv = heads
    seqs = [(1, 1), (1, 2), (1, 64), (1, 65), (1, 128), (1, 129), (1, 777), (1, 1024), (1, 1025), (1, 3000)]
    pool = sum((kv + block_size - 1) // block_size for _, kv in seqs) + 2
    b = synth.build_gqa_batch("one-token rows", seqs, n_q, n_kv, 128, pool, 31 + block_size + n_q,
                              block_size=block_size)
    for num_ctas in (None, 2):
        _check(b, num_ctas=num_ctas)


def test_multi_token_rows_straddling_a_tile_and_a_page():
    """MTP-verify rows: the new keys cross a 64-token tile edge (and a 16-token page edge)."""
    from auto_infer_b200 import synth
    seqs = [(2, 65), (2, 64), (2, 2), (2, 129), (2, 3), (2, 500)]
    b = synth.build_gqa_batch("two-token rows", seqs, 16, 2, 128, 80, 77, block_size=16)
    _check(b)
    seqs = [(4, 66), (4, 67), (4, 4), (3, 3), (4, 258)]
    b = synth.build_gqa_batch("four-token rows", seqs, 8, 2, 128, 12, 78, block_size=128)
    for num_ctas in (None, 1, 5):
        _check(b, num_ctas=num_ctas)


def test_long_pairs_cut_over_many_ctas():
    """The pair's last piece (the one holding the new row) sits on another CTA than its first."""
    from auto_infer_b200 import ops, synth
    b = synth.build_gqa_batch("cut pairs", [(1, 40000), (1, 12345)], 8, 2, 128, 420, 5)
    plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, "cuda")
    assert plan.info.num_partials > 0
    _check(b)


def test_replayable_plan_refilled_between_steps():
    from auto_infer_b200 import ops, synth
    steps = [[(1, 100), (1, 900), (1, 64)], [(1, 101), (1, 901), (1, 65)], [(2, 300), (1, 17), (2, 129)]]
    plan = None
    for i, seqs in enumerate(steps):
        b = synth.build_gqa_batch("replay", seqs, 16, 8, 128, 40, 200 + i)
        d = b.to("cuda")
        if plan is None:
            plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, "cuda", capacity_seqs=3)
            assert plan.replayable
        else:
            plan.refill(b.cu_seqlens_q, b.seqlens_kv)
        out = ops.paged_decode_gqa_write(d.q, d.k_new, d.v_new, d.slot_mapping, d.kv_cache[0], d.kv_cache[1],
                                         d.block_table, plan, b.scale)
        orc.write_kv(b.k_new, b.v_new, b.kv_cache[0], b.kv_cache[1], b.slot_mapping.tolist())
        ref = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                                  b.seqlens_kv, b.scale)
        assert torch.equal(d.kv_cache.cpu(), b.kv_cache)
        assert_attention_close(out.cpu(), ref, what=f"replay step {i}")
        assert ops.read_status("cuda") == 0


def test_padding_rows_and_bad_slots():
    """A negative slot is not stored (the row still takes part in its own attention); a slot
    past the pool sets the status bit and is not stored either."""
    from auto_infer_b200 import _lib, ops, synth
    b = synth.build_gqa_batch("padding", [(1, 70), (1, 33), (1, 200)], 8, 2, 128, 8, 13)
    d = b.to("cuda")
    before = d.kv_cache.clone()
    slots = d.slot_mapping.clone()
    slots[1] = -1
    plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, "cuda")
    out = ops.paged_decode_gqa_write(d.q, d.k_new, d.v_new, slots, d.kv_cache[0], d.kv_cache[1], d.block_table,
                                     plan, b.scale)
    assert ops.read_status("cuda") == 0
    orc.write_kv(b.k_new, b.v_new, b.kv_cache[0], b.kv_cache[1], b.slot_mapping.tolist())
    ref = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q, b.seqlens_kv,
                              b.scale)
    assert_attention_close(out.cpu(), ref, what="padding row")
    skipped = int(b.slot_mapping[1])
    flat = d.kv_cache.view(2, -1, b.n_kv, 128)
    assert torch.equal(flat[:, skipped], before.view(2, -1, b.n_kv, 128)[:, skipped])
    for t in (0, 2):
        s = int(b.slot_mapping[t])
        assert torch.equal(flat[0, s].cpu(), b.k_new[t]) and torch.equal(flat[1, s].cpu(), b.v_new[t])

    slots[1] = d.kv_cache.shape[1] * d.kv_cache.shape[2] + 5
    snapshot = d.kv_cache.clone()
    ops.paged_decode_gqa_write(d.q, d.k_new, d.v_new, slots, d.kv_cache[0], d.kv_cache[1], d.block_table,
                               plan, b.scale)
    assert ops.read_status("cuda") & _lib.STATUS_BAD_SLOT
    assert torch.equal(d.kv_cache, snapshot)          # rows 0 and 2 rewritten with the same bytes


def test_refuses_plans_that_leave_rows_to_the_wide_query_kernel():
    from auto_infer_b200 import _lib, ops, synth
    b = synth.build_gqa_batch("mixed", [(1, 70), (40, 200)], 8, 2, 128, 8, 14).to("cuda")
    plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, "cuda")
    assert plan.info.skipped_seqs == 1
    with pytest.raises(ValueError):
        ops.paged_decode_gqa_write(b.q, b.k_new, b.v_new, b.slot_mapping, b.kv_cache[0], b.kv_cache[1],
                                   b.block_table, plan, b.scale)
    import ctypes
    lib = _lib.load()
    out = torch.empty_like(b.q)
    rc = lib.b200_paged_decode_gqa_write(
        b.q.data_ptr(), b.q.stride(0), b.k_new.data_ptr(), b.k_new.stride(0), b.v_new.data_ptr(),
        b.v_new.stride(0), b.slot_mapping.data_ptr(), b.kv_cache[0].data_ptr(), b.kv_cache[1].data_ptr(),
        b.kv_cache.shape[1], b.block_size, b.block_table.data_ptr(), b.block_table.stride(0),
        plan.dev.data_ptr(), ctypes.byref(plan.info), plan.num_ctas, b.n_q, b.n_kv, 128, float(b.scale),
        plan.workspace.data_ptr(), plan.workspace.numel(), out.data_ptr(), 0, None, None, None)
    assert rc == -2      # B200_EUNSUPPORTED


@pytest.mark.parametrize("cfg", ["c1", "c4"])
def test_full_size_configs(cfg):
    from auto_infer_b200 import synth
    _check(synth.CONFIGS[cfg]())
