"""Parity of the split-KV paged GQA decode / MTP-verify kernel with the oracle
(and with the reference's own outputs in the golden fixtures), through the C ABI.
Tolerance for bf16 outputs: rtol 2e-2 / atol 2e-2."""
import pytest
import torch

from oracle import paged_attention_oracle as orc
from tests.parity import assert_attention_close, assert_scale_free

pytestmark = pytest.mark.gpu


def _decode(q, kc, vc, bt, cu, kv, scale, n_q, n_kv, num_ctas=None, want_lse=False, f32=False):
    from auto_infer_b200 import ops
    plan = ops.DecodePlan(cu, kv, n_q, n_kv, "cuda", num_ctas=num_ctas)
    lse = torch.empty(q.shape[0], n_q, dtype=torch.float32, device="cuda") if want_lse else None
    out = ops.paged_decode_gqa(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), plan, scale,
                               out_f32=f32, lse_out=lse)
    torch.cuda.synchronize()
    assert ops.read_status("cuda") == 0
    return (out.cpu(), lse.cpu()) if want_lse else out.cpu()


@pytest.mark.parametrize("name", ["decode_bs16", "decode_bs128", "mtp_verify_bs128",
                                  "drafter_ragged_bs16"])
def test_golden_reference_outputs(golden_paged, name):
    case = next(c for c in golden_paged["paged"] if c["name"] == name)
    for num_ctas in (None, 1, 3):
        out = _decode(case["q"], case["k_cache"], case["v_cache"], case["block_table"], case["cu"],
                      case["kv_lens"], case["scale"], case["n_q"], case["n_kv"], num_ctas=num_ctas)
        assert_attention_close(out, case["out"], what=f"{name} ctas={num_ctas}")


def test_lse_and_fp32_partial_output(golden_paged):
    case = next(c for c in golden_paged["paged"] if c["name"] == "mtp_verify_bs128")
    ref, ref_lse = orc.paged_attention(case["q"], case["k_cache"], case["v_cache"], case["block_table"],
                                       case["cu"], case["kv_lens"], case["scale"], return_lse=True)
    for num_ctas in (2, 148):
        out, lse = _decode(case["q"], case["k_cache"], case["v_cache"], case["block_table"], case["cu"],
                           case["kv_lens"], case["scale"], case["n_q"], case["n_kv"], num_ctas=num_ctas,
                           want_lse=True, f32=True)
        assert out.dtype == torch.float32
        assert_attention_close(out, ref, lse, ref_lse)


@pytest.mark.parametrize("ctx", [1, 63, 64, 65, 127, 128, 129, 1000])
def test_page_boundary_contexts(ctx):
    from auto_infer_b200 import synth
    b = synth.build_gqa_batch("edge", [(1, ctx), (2, ctx + 1)], 8, 2, 128, 24, 100 + ctx)
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                                       b.seqlens_kv, b.scale, return_lse=True)
    out, lse = _decode(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q, b.seqlens_kv,
                       b.scale, b.n_q, b.n_kv, want_lse=True)
    assert_attention_close(out, ref, lse, ref_lse)


def test_strided_block_table_and_query_views():
    """The runner hands a column-sliced view of a larger block-table buffer and
    the backend hands q as a slice of the packed projection."""
    from auto_infer_b200 import ops, synth
    b = synth.build_gqa_batch("views", [(1, 300), (1, 45), (1, 129)], 8, 2, 128, 16, 77)
    ref = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                              b.seqlens_kv, b.scale)
    big_bt = torch.full((8, 32), -7, dtype=torch.int32)
    big_bt[:3, :b.block_table.shape[1]] = b.block_table
    packed = torch.zeros(3, 8 * 128 + 512, dtype=torch.bfloat16)
    packed[:, :8 * 128] = b.q.reshape(3, -1)
    packed_d = packed.cuda()
    q_view = packed_d[:, :8 * 128].view(3, 8, 128)
    plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, 8, 2, "cuda")
    cache = b.kv_cache.cuda()
    out = ops.paged_decode_gqa(q_view, cache[0], cache[1], big_bt.cuda()[:3, :b.block_table.shape[1]],
                               plan, b.scale)
    assert_attention_close(out.cpu(), ref)


def test_empty_batch_and_zero_length_rows():
    from auto_infer_b200 import ops, synth
    plan = ops.DecodePlan([], [], 8, 2, "cuda")
    assert plan.info.num_items == 0
    b = synth.build_gqa_batch("ragged", [(1, 70), (1, 200)], 8, 2, 128, 8, 5)
    # a middle sequence with no query tokens this step
    cu = [1, 1, 2]
    kv = [70, 55, 200]
    bt = torch.zeros(3, b.block_table.shape[1], dtype=torch.int32)
    bt[0], bt[2] = b.block_table[0], b.block_table[1]
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], bt, cu, kv, b.scale, return_lse=True)
    out, lse = _decode(b.q, b.kv_cache[0], b.kv_cache[1], bt, cu, kv, b.scale, 8, 2, want_lse=True)
    assert_attention_close(out, ref, lse, ref_lse)


def test_shared_prefix_blocks_alias():
    from auto_infer_b200 import synth
    seqs = [(1, 400), (1, 300), (2, 513)]
    b = synth.build_gqa_batch("alias", seqs, 16, 8, 128, 16, 9, shared_prefix_tokens=[256, 256, 256])
    assert b.block_table[0, 0] == b.block_table[1, 0] == b.block_table[2, 0]
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                                       b.seqlens_kv, b.scale, return_lse=True)
    out, lse = _decode(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q, b.seqlens_kv,
                       b.scale, b.n_q, b.n_kv, want_lse=True)
    assert_attention_close(out, ref, lse, ref_lse)


@pytest.mark.parametrize("cfg", ["c1", "c4"])
def test_full_size_configs_write_then_attend(cfg):
    """Configs 1 and 4 at full size: slot write of the step's tokens (bit-exact)
    followed by attention, against the oracle doing the same."""
    from auto_infer_b200 import ops, synth
    b = synth.CONFIGS[cfg]()
    d = b.to("cuda")
    ops.reshape_and_cache(d.k_new, d.v_new, d.kv_cache[0], d.kv_cache[1], d.slot_mapping)
    orc.write_kv(b.k_new, b.v_new, b.kv_cache[0], b.kv_cache[1], b.slot_mapping.tolist())
    assert torch.equal(d.kv_cache.cpu(), b.kv_cache)
    plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, "cuda")
    assert plan.skipped_seqs == 0
    lse = torch.empty(b.num_tokens, b.n_q, dtype=torch.float32, device="cuda")
    out = ops.paged_decode_gqa(d.q, d.kv_cache[0], d.kv_cache[1], d.block_table, plan, b.scale, lse_out=lse)
    out32 = ops.paged_decode_gqa(d.q, d.kv_cache[0], d.kv_cache[1], d.block_table, plan, b.scale, out_f32=True)
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                                       b.seqlens_kv, b.scale, return_lse=True)
    assert_attention_close(out.cpu(), ref, lse.cpu(), ref_lse, what=cfg)
    assert_attention_close(out32.cpu(), ref, what=cfg + " fp32 rows")
    assert ops.read_status("cuda") == 0


def test_long_context_sampled_against_oracle_and_split_invariance():
    """Config-5-shaped sequences (64 q / 8 kv heads, 131072 tokens) generated on
    the device: one sequence is pulled back and checked against the oracle (bf16
    rows, fp32 rows and the log-sum-exp; the outputs are ~0.005 in size, so the
    comparison that counts is the one relative to the row's own rms), and the
    result must not depend on how the tiles were cut across CTAs."""
    from auto_infer_b200 import ops, synth
    b = synth.config5("cuda", batch=2)
    plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, "cuda")
    lse = torch.empty(b.num_tokens, b.n_q, dtype=torch.float32, device="cuda")
    out = ops.paged_decode_gqa(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, plan, b.scale, lse_out=lse)
    out32 = ops.paged_decode_gqa(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, plan, b.scale,
                                 out_f32=True)
    plan2 = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, "cuda", num_ctas=37)
    lse2 = torch.empty_like(lse)
    out2 = ops.paged_decode_gqa(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, plan2, b.scale,
                                out_f32=True, lse_out=lse2)
    assert_scale_free(out2, out32, "37-CTA cut against 148-CTA cut", atol_rms=1e-2, rtol=1e-3, rel_l2=5e-3)
    torch.testing.assert_close(lse2, lse, atol=1e-4, rtol=1e-5)
    seq = 1
    ids = b.block_table[seq].long()
    kc = b.kv_cache[0][ids].cpu()
    vc = b.kv_cache[1][ids].cpu()
    bt = torch.arange(ids.numel(), dtype=torch.int32)[None]
    ref, ref_lse = orc.paged_attention(b.q[seq:seq + 1].cpu(), kc, vc, bt, [1], [b.seqlens_kv[seq]],
                                       b.scale, return_lse=True)
    assert_attention_close(out[seq:seq + 1].cpu(), ref, lse[seq:seq + 1].cpu(), ref_lse, "bf16 rows")
    assert_attention_close(out32[seq:seq + 1].cpu(), ref, what="fp32 rows")
    assert ops.read_status("cuda") == 0


def test_out_of_pool_block_id_is_flagged_not_fatal():
    from auto_infer_b200 import ops, synth
    b = synth.build_gqa_batch("badblock", [(1, 200)], 8, 2, 128, 4, 3).to("cuda")
    bt = b.block_table.clone()
    bt[0, 1] = 9999
    plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, 8, 2, "cuda")
    out = ops.paged_decode_gqa(b.q, b.kv_cache[0], b.kv_cache[1], bt, plan, b.scale)
    torch.cuda.synchronize()
    assert ops.read_status("cuda") & 2
    assert torch.isfinite(out.float()).all()


def test_unwritten_cache_slots_may_hold_anything():
    """Slots of a sequence's last page past kv_len are never written by the engine: with NaN / Inf
    bit patterns there (a pool from torch.empty), the rows must still come out finite and right -
    their weight is 0, but 0 x NaN would poison the row if the bytes reached the MMA."""
    from auto_infer_b200 import ops, synth
    seqs = [(1, 70), (2, 129), (1, 64), (1, 5)]
    b = synth.build_gqa_batch("poison", seqs, 8, 2, 128, 8, 314)
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                                       b.seqlens_kv, b.scale, return_lse=True)
    cache = b.kv_cache.clone()
    for row, (_, kv_len) in zip(b.block_table.tolist(), seqs):
        last = (kv_len - 1) // 128
        tail = kv_len - last * 128
        cache[0, row[last], tail:] = float("nan")
        cache[1, row[last], tail:] = float("nan")
        cache[1, row[last], tail::2] = float("inf")
    out, lse = _decode(b.q, cache[0], cache[1], b.block_table, b.cu_seqlens_q, b.seqlens_kv, b.scale,
                       b.n_q, b.n_kv, want_lse=True)
    assert torch.isfinite(out.float()).all()
    assert_attention_close(out, ref, lse, ref_lse, "poisoned tails")
