"""The oracle's non-absorbed MLA restatement against outputs of the reference's own
``MlaDenseBackend`` (auto_infer/layers/attention/mla.py:134-164, 369-399), K 192 / V 128."""
import torch

from oracle import paged_attention_oracle as orc
from tests.paging import page_out
from tests.parity import TOL, assert_scale_free


def _block(case, block_size, seed):
    nh, lens = case["nh"], case["lens"]
    total = sum(lens)
    need = sum((n + block_size - 1) // block_size for n in lens) + 2
    k_cache = torch.zeros(need, block_size, nh, case["nope"] + case["rope"], dtype=torch.bfloat16)
    v_cache = torch.zeros(need, block_size, nh, case["vd"], dtype=torch.bfloat16)
    # pages dealt in a shuffled order
    _, _, table, slots = page_out(torch.zeros(total, 1, 1, dtype=torch.bfloat16),
                                  torch.zeros(total, 1, 1, dtype=torch.bfloat16), lens, block_size, seed,
                                  spare_blocks=2)
    return orc.mla_paged_block(
        case["x"], case["w"], "model.layers.0.", num_heads=nh, qk_nope=case["nope"], qk_rope=case["rope"],
        v_head_dim=case["vd"], kv_lora_rank=case["kvl"], q_lora_rank=case["q_lora"], rms_eps=1e-6,
        cos=case["cos"], sin=case["sin"], k_cache=k_cache, v_cache=v_cache, slots=slots, block_table=table,
        cu_seqlens_q=case["cu"], seqlens_kv=lens, softmax_scale=case["scale"], return_qkv=True)


def test_sub_block_against_reference_outputs(golden_mla_paged):
    for name in ("plain_q", "q_lora"):
        case = golden_mla_paged[name]
        for block_size in (16, 128):
            out, q, k, v, o = _block(case, block_size, 5)
            assert torch.equal(q, case["q"]) and torch.equal(k, case["k"]) and torch.equal(v, case["v"]), name
            torch.testing.assert_close(o.float(), case["core_out"].float(), **TOL)
            assert_scale_free(o, case["core_out"], f"{name} core rows")
            assert_scale_free(out, case["block_out"], f"{name} after o_proj", atol_rms=5e-2, rtol=2e-2, rel_l2=2e-2)


def test_decode_and_verify_rows_against_reference_core(golden_mla_paged):
    rows = golden_mla_paged["decode_rows"]
    for i, r in enumerate(rows["rows"]):
        k_cache, v_cache, table, _ = page_out(r["k"], r["v"], [r["kv_len"]], 16, 40 + i)
        out = orc.paged_attention(r["q"], k_cache, v_cache, table, [r["q_len"]], [r["kv_len"]], rows["scale"])
        torch.testing.assert_close(out.float(), r["o"].float(), **TOL)
        assert_scale_free(out, r["o"], f"rows {i}")
