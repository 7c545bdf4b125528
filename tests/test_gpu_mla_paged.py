"""Parity of the K-192 / V-128 multi-head paged kernel (the non-absorbed MLA form,
auto_infer/layers/attention/mla.py:23-64, 134-164, 167-255) with the reference's own outputs
(golden fixtures) and with the oracle, through the C ABI.  Tolerance for bf16 outputs:
rtol 2e-2 / atol 2e-2 plus the row-relative checks of tests/parity.py."""
import pytest
import torch

from oracle import paged_attention_oracle as orc
from tests.paging import page_out
from tests.parity import TOL, assert_attention_close, assert_scale_free

pytestmark = pytest.mark.gpu


def _run(q, k_cache, v_cache, table, cu, kv, scale, num_ctas=None, f32=False, causal_base=None):
    from auto_infer_b200 import ops
    nh = q.shape[1]
    plan = ops.MhaPlan(cu, kv, nh, "cuda", num_ctas=num_ctas, causal_base=causal_base)
    lse = torch.empty(q.shape[0], nh, dtype=torch.float32, device="cuda")
    out = ops.paged_mha(q.cuda(), k_cache.cuda(), v_cache.cuda(), table.cuda(), plan, scale, out_f32=f32,
                        lse_out=lse)
    torch.cuda.synchronize()
    assert ops.read_status("cuda") == 0
    return out.cpu(), lse.cpu(), plan


def _random_batch(seqs, nh, block_size, seed, fill=0.0):
    """seqs: (q_len, kv_len) per sequence.  Returns q, caches, table, cu, kv lens."""
    g = torch.Generator().manual_seed(seed)
    lens = [kv for _, kv in seqs]
    k = torch.randn(sum(lens), nh, 192, generator=g).to(torch.bfloat16)
    v = torch.randn(sum(lens), nh, 128, generator=g).to(torch.bfloat16)
    q = torch.randn(sum(ql for ql, _ in seqs), nh, 192, generator=g).to(torch.bfloat16)
    k_cache, v_cache, table, _ = page_out(k, v, lens, block_size, seed + 1, fill=fill)
    cu, acc = [], 0
    for ql, _ in seqs:
        acc += ql
        cu.append(acc)
    return q, k_cache, v_cache, table, cu, lens


def test_prefill_rows_against_reference_core(golden_mla_paged):
    for name in ("plain_q", "q_lora"):
        case = golden_mla_paged[name]
        for block_size in (16, 128):
            k_cache, v_cache, table, _ = page_out(case["k"], case["v"], case["lens"], block_size, 3)
            for num_ctas in (None, 2):
                out, _, _ = _run(case["q"], k_cache, v_cache, table, case["cu"], case["lens"], case["scale"],
                                 num_ctas=num_ctas)
                assert_attention_close(out, case["core_out"], what=f"{name} bs={block_size}")


def test_decode_and_verify_rows_against_reference_core(golden_mla_paged):
    rows = golden_mla_paged["decode_rows"]
    for i, r in enumerate(rows["rows"]):
        k_cache, v_cache, table, _ = page_out(r["k"], r["v"], [r["kv_len"]], 16, 40 + i)
        for num_ctas in (None, 1, 600):
            out, _, plan = _run(r["q"], k_cache, v_cache, table, [r["q_len"]], [r["kv_len"]], rows["scale"],
                                num_ctas=num_ctas)
            assert_attention_close(out, r["o"], what=f"rows {i} ctas={num_ctas} splits={plan.info.num_splits}")


@pytest.mark.parametrize("block_size", [16, 128])
def test_mixed_steps_against_oracle(block_size):
    """Decode rows, verify rows, chunks over a prefix and whole prompts in one step, contexts at
    every tile edge, with and without key splits; lse pins QK^T, the mask and the sums."""
    seqs = [(1, 1), (1, 63), (1, 64), (1, 65), (2, 129), (1, 700), (5, 5), (70, 70), (64, 200), (130, 1000),
            (1, 2500)]
    q, kc, vc, table, cu, kv = _random_batch(seqs, 4, block_size, 11)
    ref, ref_lse = orc.paged_attention(q, kc, vc, table, cu, kv, 192 ** -0.5, return_lse=True)
    for num_ctas in (None, 1, 2000):
        out, lse, plan = _run(q, kc, vc, table, cu, kv, 192 ** -0.5, num_ctas=num_ctas)
        assert_attention_close(out, ref, lse, ref_lse, what=f"ctas={num_ctas} splits={plan.info.num_splits}")
    out32, _, _ = _run(q, kc, vc, table, cu, kv, 192 ** -0.5, f32=True)
    assert out32.dtype == torch.float32
    assert_attention_close(out32, ref, what="fp32 rows")


def test_key_splits_are_used_and_merged():
    """A decode batch of few sequences: the plan cuts the keys so that the SMs fill up."""
    seqs = [(1, 5000), (1, 3000), (2, 8191)]
    q, kc, vc, table, cu, kv = _random_batch(seqs, 16, 128, 21)
    ref, ref_lse = orc.paged_attention(q, kc, vc, table, cu, kv, 192 ** -0.5, return_lse=True)
    out, lse, plan = _run(q, kc, vc, table, cu, kv, 192 ** -0.5)
    assert plan.info.num_splits > 1
    assert_attention_close(out, ref, lse, ref_lse, what=f"splits={plan.info.num_splits}")


def test_unwritten_cache_tails_may_hold_anything():
    """Slots past kv_len in a sequence's last page (and whole spare pages) are NaN."""
    seqs = [(1, 70), (3, 130), (40, 100), (1, 64)]
    q, kc, vc, table, cu, kv = _random_batch(seqs, 4, 16, 31, fill=float("nan"))
    clean_k, clean_v = torch.nan_to_num(kc, nan=0.0), torch.nan_to_num(vc, nan=0.0)
    ref, ref_lse = orc.paged_attention(q, clean_k, clean_v, table, cu, kv, 192 ** -0.5, return_lse=True)
    out, lse, _ = _run(q, kc, vc, table, cu, kv, 192 ** -0.5)
    assert torch.isfinite(out.float()).all()
    assert_attention_close(out, ref, lse, ref_lse, what="NaN tails")


def test_shifted_causal_base_and_empty_rows():
    """A causal base below kv_len - q_len (rows that see fewer keys, down to none)."""
    seqs = [(4, 100), (3, 50)]
    q, kc, vc, table, cu, kv = _random_batch(seqs, 4, 16, 41)
    base = [60, -2]                 # sequence 1: rows 0 and 1 see nothing, row 2 sees key 0
    out, lse, _ = _run(q, kc, vc, table, cu, kv, 192 ** -0.5, causal_base=base)
    # the same thing through the oracle: each row as a one-token sequence ending at base + i + 1
    new_cu, new_kv, rows = [], [], []
    for b, (ql, _) in enumerate(seqs):
        for i in range(ql):
            new_cu.append(len(new_cu) + 1)
            new_kv.append(max(base[b] + i + 1, 0))
            rows.append(b)
    live = [i for i, n in enumerate(new_kv) if n > 0]
    ref, ref_lse = orc.paged_attention(q[live], kc, vc, table[[rows[i] for i in live]],
                                       list(range(1, len(live) + 1)), [new_kv[i] for i in live], 192 ** -0.5,
                                       return_lse=True)
    assert_attention_close(out[live], ref, lse[live], ref_lse, what="shifted base")
    dead = [i for i, n in enumerate(new_kv) if n == 0]
    assert dead and (out[dead] == 0).all() and torch.isinf(lse[dead]).all()


def test_empty_step_and_argument_checks():
    from auto_infer_b200 import ops
    plan = ops.MhaPlan([], [], 4, "cuda")
    assert plan.info.num_items == 0
    q, kc, vc, table, cu, kv = _random_batch([(1, 70)], 4, 16, 51)
    plan = ops.MhaPlan(cu, kv, 4, "cuda")
    with pytest.raises(RuntimeError):
        ops.paged_mha(q.cuda()[..., :128].contiguous(), kc.cuda()[..., :128].contiguous(), vc.cuda(), table.cuda(),
                      plan, 1.0)
    bad = table.clone()
    bad[0, 0] = 10_000
    ops.paged_mha(q.cuda(), kc.cuda(), vc.cuda(), bad.cuda(), plan, 1.0)
    assert ops.read_status("cuda") & 2


def test_backend_sub_block_against_reference(golden_mla_paged):
    """B200MlaPagedBackend.attention on the reference's own prefill inputs, then one decode
    step per sequence against the oracle's restatement continuing from the same caches."""
    from auto_infer_b200.forward_context import ForwardContext
    from auto_infer_b200.mla import B200MlaPagedBackend
    for name in ("plain_q", "q_lora"):
        case = golden_mla_paged[name]
        nh, lens, bs = case["nh"], case["lens"], 16
        w = {k: v.cuda() for k, v in case["w"].items()}
        backend = B200MlaPagedBackend(w, num_heads=nh, qk_nope=case["nope"], qk_rope=case["rope"],
                                      v_head_dim=case["vd"], kv_lora_rank=case["kvl"], q_lora_rank=case["q_lora"],
                                      rms_eps=1e-6, softmax_scale=case["scale"], num_layers=1, device="cuda",
                                      dtype=torch.bfloat16)
        # room for one more token per sequence
        _, _, table, slots = page_out(torch.zeros(sum(lens) + 3, 1, 1, dtype=torch.bfloat16),
                                      torch.zeros(sum(lens) + 3, 1, 1, dtype=torch.bfloat16),
                                      [n + 1 for n in lens], bs, 9)
        pre_slots, dec_slots, at = [], [], 0
        for n in lens:
            pre_slots += slots[at:at + n]
            dec_slots.append(slots[at + n])
            at += n + 1
        caches = backend.alloc_kv_caches(int(table.max()) + 1, bs)
        ctx = ForwardContext(None, None, torch.tensor(pre_slots, dtype=torch.int32).cuda(), table.cuda(),
                             case["cu"], lens, None, backend, caches, False, cos=case["cos"].cuda(),
                             sin=case["sin"].cuda())
        out = backend.attention(0, case["x"].cuda(), ctx).cpu()
        assert_scale_free(out, case["block_out"], f"{name} prefill block", atol_rms=5e-2, rtol=2e-2, rel_l2=2e-2)
        torch.testing.assert_close(out.float(), case["block_out"].float(), **TOL)

        # oracle on CPU caches brought to the same state, then a decode step on both
        k_cpu, v_cpu = torch.zeros_like(caches[0][0]).cpu(), torch.zeros_like(caches[0][1]).cpu()
        common = dict(num_heads=nh, qk_nope=case["nope"], qk_rope=case["rope"], v_head_dim=case["vd"],
                      kv_lora_rank=case["kvl"], q_lora_rank=case["q_lora"], rms_eps=1e-6, softmax_scale=case["scale"])
        orc.mla_paged_block(case["x"], case["w"], "model.layers.0.", cos=case["cos"], sin=case["sin"], k_cache=k_cpu,
                            v_cache=v_cpu, slots=pre_slots, block_table=table, cu_seqlens_q=case["cu"],
                            seqlens_kv=lens, **common)
        # the projections are bf16 GEMMs of two libraries: rows agree to rounding, not bit for bit
        torch.testing.assert_close(caches[0][0].cpu().float(), k_cpu.float(), **TOL)
        torch.testing.assert_close(caches[0][1].cpu().float(), v_cpu.float(), **TOL)
        k_cpu, v_cpu = caches[0][0].cpu(), caches[0][1].cpu()       # continue from the device's own rows
        g = torch.Generator().manual_seed(77)
        x1 = torch.randn(len(lens), case["hidden"], generator=g).to(torch.bfloat16)
        pick = torch.tensor([n - 1 for n in lens])          # any rows of the tables will do as positions
        cos1, sin1 = case["cos"][pick], case["sin"][pick]
        cu1, kv1 = list(range(1, len(lens) + 1)), [n + 1 for n in lens]
        ref1 = orc.mla_paged_block(x1, case["w"], "model.layers.0.", cos=cos1, sin=sin1, k_cache=k_cpu,
                                   v_cache=v_cpu, slots=dec_slots, block_table=table, cu_seqlens_q=cu1,
                                   seqlens_kv=kv1, **common)
        ctx1 = ForwardContext(None, None, torch.tensor(dec_slots, dtype=torch.int32).cuda(), table.cuda(),
                              cu1, kv1, None, backend, caches, True, cos=cos1.cuda(), sin=sin1.cuda())
        out1 = backend.attention(0, x1.cuda(), ctx1).cpu()
        torch.testing.assert_close(caches[0][0].cpu().float(), k_cpu.float(), **TOL)
        torch.testing.assert_close(caches[0][1].cpu().float(), v_cpu.float(), **TOL)
        assert_scale_free(out1, ref1, f"{name} decode block", atol_rms=5e-2, rtol=2e-2, rel_l2=2e-2)


@pytest.mark.parametrize("batch", [4, 16])
def test_decode_at_config3_lengths(batch):
    """16 heads, contexts 1 024-8 192 as in the MLA decode configuration, per-head caches."""
    g = torch.Generator().manual_seed(60 + batch)
    seqs = [(1, int(n)) for n in torch.randint(1024, 8193, (batch,), generator=g)]
    q, kc, vc, table, cu, kv = _random_batch(seqs, 16, 128, 61)
    ref, ref_lse = orc.paged_attention(q, kc, vc, table, cu, kv, 192 ** -0.5, return_lse=True)
    out, lse, _ = _run(q, kc, vc, table, cu, kv, 192 ** -0.5)
    assert_attention_close(out, ref, lse, ref_lse, what=f"batch {batch}")
