"""Parity of the wide-query (chunked prefill / multi-token verify) attention
kernel with the oracle and the reference's golden outputs, through the C ABI.
Tolerance for bf16 outputs: rtol 2e-2 / atol 2e-2."""
import pytest
import torch

from oracle import paged_attention_oracle as orc
from tests.parity import assert_attention_close, assert_scale_free

pytestmark = pytest.mark.gpu


def _prefill(q, kc, vc, bt, cu, kv, scale, n_q, n_kv, min_rows=0, want_lse=False):
    from auto_infer_b200 import ops
    plan = ops.PrefillPlan(cu, kv, n_q, n_kv, "cuda", min_rows=min_rows)
    lse = torch.empty(q.shape[0], n_q, dtype=torch.float32, device="cuda") if want_lse else None
    out = torch.zeros(q.shape, dtype=torch.bfloat16, device="cuda")
    qd, kd, vd, btd = q.cuda(), kc.cuda(), vc.cuda(), bt.cuda()
    ops.paged_prefill_gqa(qd, kd, vd, btd, plan, scale, out=out, lse_out=lse)
    # the same plan serves every layer of a step: a second launch must find the
    # work queue reset and reproduce the result bit for bit
    again = torch.zeros_like(out)
    ops.paged_prefill_gqa(qd, kd, vd, btd, plan, scale, out=again)
    torch.cuda.synchronize()
    assert torch.equal(out, again)
    assert ops.read_status("cuda") == 0
    return (out.cpu(), lse.cpu()) if want_lse else out.cpu()


@pytest.mark.parametrize("name", ["chunk_prefill_bs128", "decode_bs16", "mtp_verify_bs128",
                                  "drafter_ragged_bs16"])
def test_golden_reference_outputs(golden_paged, name):
    """Every golden case, decode-shaped ones included: the kernel handles any q_len."""
    case = next(c for c in golden_paged["paged"] if c["name"] == name)
    out = _prefill(case["q"], case["k_cache"], case["v_cache"], case["block_table"], case["cu"],
                   case["kv_lens"], case["scale"], case["n_q"], case["n_kv"])
    assert_attention_close(out, case["out"], what=name)


@pytest.mark.parametrize("q_len,prefix", [(1, 0), (33, 0), (128, 0), (129, 64), (200, 1000), (512, 300)])
def test_chunk_over_prefix_shapes(q_len, prefix):
    from auto_infer_b200 import synth
    b = synth.build_gqa_batch("chunk", [(q_len, prefix + q_len), (7, 77)], 8, 2, 128, 24, 300 + q_len)
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table,
                                       b.cu_seqlens_q, b.seqlens_kv, b.scale, return_lse=True)
    out, lse = _prefill(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                        b.seqlens_kv, b.scale, b.n_q, b.n_kv, want_lse=True)
    assert_attention_close(out, ref, lse, ref_lse)


@pytest.mark.parametrize("n_q,n_kv", [(4, 4), (16, 2), (6, 2), (12, 2)])
def test_group_sizes(n_q, n_kv):
    """Groups that divide 128 take the Q tile as one TMA box (1, 8), the others
    (3, 6) copy it row by row; ragged tails in both."""
    from auto_infer_b200 import synth
    b = synth.build_gqa_batch("groups", [(150, 150 + 200), (45, 45), (3, 130)], n_q, n_kv, 128, 24, 911 + n_q)
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table,
                                       b.cu_seqlens_q, b.seqlens_kv, b.scale, return_lse=True)
    out, lse = _prefill(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                        b.seqlens_kv, b.scale, b.n_q, b.n_kv, want_lse=True)
    assert_attention_close(out, ref, lse, ref_lse)


def test_many_ragged_items_per_cta():
    """Forty-eight sequences of random query and prefix lengths: more work items than
    CTAs, items of one to eight KV tiles, ragged last row tiles - every CTA goes through
    several item hand-overs (mailbox, accumulator release, row-sum exchange)."""
    from auto_infer_b200 import synth
    g = torch.Generator().manual_seed(77)
    q_lens = torch.randint(5, 301, (48,), generator=g).tolist()
    prefixes = torch.randint(0, 701, (48,), generator=g).tolist()
    seqs = [(q, q + p) for q, p in zip(q_lens, prefixes)]
    blocks = sum((kv + 127) // 128 for _, kv in seqs) + 4
    b = synth.build_gqa_batch("ragged", seqs, 8, 2, 128, blocks, 78)
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table,
                                       b.cu_seqlens_q, b.seqlens_kv, b.scale, return_lse=True)
    out, lse = _prefill(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                        b.seqlens_kv, b.scale, b.n_q, b.n_kv, want_lse=True)
    assert_attention_close(out, ref, lse, ref_lse)


def test_context_parallel_slice_with_rows_that_see_no_key():
    """The keys [128, 200) of a 200-token prompt as one context-parallel rank holds them
    (local block table, local length, causal base in local coordinates): the first 128
    query positions see none of them, so their work items have no KV tile at all and must
    come out as zeros with lse = -inf; the others are partial sums for the merge."""
    from auto_infer_b200 import ops, synth
    b = synth.build_gqa_batch("cp_slice", [(200, 200)], 8, 2, 128, 8, 4242)
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                                       b.seqlens_kv, b.scale, return_lse=True, kv_ranges=[(128, 200)])
    plan = ops.PrefillPlan(b.cu_seqlens_q, [72], b.n_q, b.n_kv, "cuda", min_rows=0, causal_base=[-128])
    out = torch.full(b.q.shape, 7.0, dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros(b.q.shape[0], b.n_q, dtype=torch.float32, device="cuda")
    local_bt = b.block_table[:, 1:].contiguous().cuda()
    ops.paged_prefill_gqa(b.q.cuda(), b.kv_cache[0].cuda(), b.kv_cache[1].cuda(), local_bt, plan, b.scale,
                          out=out, lse_out=lse)
    torch.cuda.synchronize()
    assert ops.read_status("cuda") == 0
    assert torch.equal(out[:128].cpu(), torch.zeros_like(out[:128].cpu()))
    assert torch.isinf(lse[:128]).all() and (lse[:128] < 0).all()
    assert_attention_close(out.cpu(), ref, lse[128:].cpu(), ref_lse[128:])


def test_two_kernels_agree_on_a_long_context():
    """Size-independent check at config-5 scale: a decode row is a one-row chunk, so the
    wide-query kernel (tcgen05, rotated tile order, 1 024 KV tiles per item) and the
    split-KV decode kernel (mma.sync, tiles cut across CTAs) must give the same rows
    and the same log-sum-exp for a 131 072-token context."""
    from auto_infer_b200 import ops, synth
    b = synth.config5("cuda", batch=2)
    dplan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, "cuda")
    lse_d = torch.empty(b.q.shape[0], b.n_q, dtype=torch.float32, device="cuda")
    out_d = ops.paged_decode_gqa(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, dplan, b.scale,
                                 lse_out=lse_d)
    pplan = ops.PrefillPlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, "cuda", min_rows=0)
    lse_p = torch.empty_like(lse_d)
    out_p = torch.zeros(b.q.shape, dtype=torch.bfloat16, device="cuda")
    ops.paged_prefill_gqa(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, pplan, b.scale,
                          out=out_p, lse_out=lse_p)
    torch.cuda.synchronize()
    assert ops.read_status("cuda") == 0
    torch.testing.assert_close(lse_p, lse_d, atol=2e-3, rtol=2e-3)
    # both outputs are bf16 roundings of values ~0.005 in size: compare relative to the row's rms
    assert_scale_free(out_p, out_d, "wide-query kernel against split-KV decode kernel")
    # and one sequence against the oracle (rows and log-sum-exp)
    seq = 0
    ids = b.block_table[seq].long()
    bt = torch.arange(ids.numel(), dtype=torch.int32)[None]
    ref, ref_lse = orc.paged_attention(b.q[seq:seq + 1].cpu(), b.kv_cache[0][ids].cpu(), b.kv_cache[1][ids].cpu(),
                                       bt, [1], [b.seqlens_kv[seq]], b.scale, return_lse=True)
    assert_attention_close(out_p[seq:seq + 1].cpu(), ref, lse_p[seq:seq + 1].cpu(), ref_lse, "wide-query kernel")


def test_mixed_batch_through_the_backend():
    """Decode rows and prefill chunks in one step, as the scheduler orders them
    (decode first): the backend sends each row to the kernel built for it and the
    slot write comes first."""
    from auto_infer_b200 import ops, synth
    from auto_infer_b200.forward_context import ForwardContext
    from auto_infer_b200.gqa import B200GqaBackend
    seqs = [(1, 700), (1, 64), (2, 333), (96, 96 + 256), (40, 40)]
    b = synth.build_gqa_batch("mixed", seqs, 16, 4, 128, 32, 55, shared_prefix_tokens=[0, 0, 0, 256, 0])
    d = b.to("cuda")
    backend = B200GqaBackend(b.n_q, b.n_kv, b.head_dim, b.scale, 1, "cuda", torch.bfloat16)
    ctx = ForwardContext(None, None, d.slot_mapping, d.block_table, b.cu_seqlens_q, b.seqlens_kv,
                         None, backend, [d.kv_cache], False)
    out = backend.paged_attention(0, d.q, d.k_new, d.v_new, ctx)
    orc.write_kv(b.k_new, b.v_new, b.kv_cache[0], b.kv_cache[1], b.slot_mapping.tolist())
    assert torch.equal(d.kv_cache.cpu(), b.kv_cache)
    ref = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                              b.seqlens_kv, b.scale)
    assert_attention_close(out.cpu(), ref)
    assert ops.read_status("cuda") == 0


def test_config2_full_size_mixed_batch():
    """Config 2: 60 decode rows + four 512-token chunks over nested shared
    prefixes of 0/1024/2048/4096 tokens (aliased physical blocks)."""
    from auto_infer_b200 import ops, synth
    from auto_infer_b200.forward_context import ForwardContext
    from auto_infer_b200.gqa import B200GqaBackend
    d = synth.config2("cuda")            # 2 GiB pool: generated on the device, copied back for the oracle
    b = d.to("cpu")
    assert b.block_table[61, 0] == b.block_table[62, 0] == b.block_table[63, 0]
    backend = B200GqaBackend(b.n_q, b.n_kv, b.head_dim, b.scale, 1, "cuda", torch.bfloat16)
    ctx = ForwardContext(None, None, d.slot_mapping, d.block_table, b.cu_seqlens_q, b.seqlens_kv,
                         None, backend, [d.kv_cache], False)
    out = backend.paged_attention(0, d.q, d.k_new, d.v_new, ctx).cpu()
    # shared prefix blocks are written by several requests in this synthetic step only where
    # their new tokens land, which is never inside the shared (full, read-only) blocks
    orc.write_kv(b.k_new, b.v_new, b.kv_cache[0], b.kv_cache[1], b.slot_mapping.tolist())
    assert torch.equal(d.kv_cache.cpu(), b.kv_cache)
    torch.set_num_threads(max(torch.get_num_threads(), 8))
    ref = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                              b.seqlens_kv, b.scale, literal_max_kv=0)
    assert_attention_close(out, ref, what="config 2 (60 decode rows + 4 chunks)")
    assert ops.read_status("cuda") == 0
    # this step is one the backend runs side by side (wide-query kernel on its share of the SMs,
    # decode kernel on the rest); one after the other on all SMs gives the same rows, up to the
    # order in which a cut pair's pieces are summed (the decode plan is another one)
    from auto_infer_b200.metadata import cached_step_metadata
    meta = cached_step_metadata(ctx, b.n_q, b.n_kv, b.head_dim, d.q.device)
    assert meta.prefill_ctas > 0 and meta.decode.num_ctas == ops.sm_count("cuda") - meta.prefill_ctas
    plain = B200GqaBackend(b.n_q, b.n_kv, b.head_dim, b.scale, 1, "cuda", torch.bfloat16)
    plain._overlap_mixed = False
    ctx2 = ForwardContext(None, None, d.slot_mapping, d.block_table, b.cu_seqlens_q, b.seqlens_kv,
                          None, plain, [d.kv_cache], False)
    out2 = plain.paged_attention(0, d.q, d.k_new, d.v_new, ctx2).cpu()
    assert cached_step_metadata(ctx2, b.n_q, b.n_kv, b.head_dim, d.q.device).prefill_ctas == 0
    chunk_rows = slice(60, None)                      # the chunks' rows come from the same plan: same bits
    assert torch.equal(out[chunk_rows], out2[chunk_rows])
    assert_attention_close(out2, ref, what="config 2, one kernel after the other")
    for _ in range(3):                                # repeated side by side steps on the pooled plans
        again = backend.paged_attention(0, d.q, d.k_new, d.v_new, ForwardContext(
            None, None, d.slot_mapping, d.block_table, b.cu_seqlens_q, b.seqlens_kv, None, backend,
            [d.kv_cache], False)).cpu()
        assert torch.equal(again, out)
    assert ops.read_status("cuda") == 0
