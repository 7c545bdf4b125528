"""The CPU oracle against outputs of the reference's own functions (committed
fixtures from tests/golden/make_golden.py) and against the integer known-answer
vectors of the reference's stager tests."""
import numpy as np
import torch

from oracle import paged_attention_oracle as orc


def test_dense_core_matches_reference_outputs(golden_small):
    """q_len == kv_len packed segments, fp32: the oracle core must reproduce
    dense_causal_attention bit for bit."""
    for case in golden_small["dense"]:
        q, k, v = case["q"], case["k"], case["v"]
        group = case["n_q"] // case["n_kv"]
        outs, start = [], 0
        for end in case["cu"]:
            o, _ = orc._core_literal(q[start:end], k[start:end].repeat_interleave(group, 1),
                                     v[start:end].repeat_interleave(group, 1), case["hd"] ** -0.5)
            outs.append(o)
            start = end
        assert torch.equal(torch.cat(outs), case["out"]), case["seed"]


def test_paged_attention_matches_reference_outputs(golden_paged):
    """Decode, MTP-verify, ragged drafter and chunked-prefill rows over paged
    caches equal the reference function's rows bit for bit."""
    for case in golden_paged["paged"]:
        out = orc.paged_attention(case["q"], case["k_cache"], case["v_cache"], case["block_table"],
                                  case["cu"], case["kv_lens"], case["scale"])
        assert torch.equal(out, case["out"]), case["name"]


def test_grouped_long_context_form_agrees_with_literal(golden_paged):
    for case in golden_paged["paged"]:
        out = orc.paged_attention(case["q"], case["k_cache"], case["v_cache"], case["block_table"],
                                  case["cu"], case["kv_lens"], case["scale"], literal_max_kv=0)
        torch.testing.assert_close(out.float(), case["out"].float(), atol=8e-3, rtol=8e-3)


def test_slot_mapping_known_answers(golden_small):
    s = golden_small["slots"]
    bt = np.asarray([7, 8, 9])
    assert orc.slot_mapping(bt, np.arange(10), 4).tolist() == s["slots_bs4_pos0_9"]
    assert orc.slot_mapping(np.asarray([5, 0, 3]), np.asarray([0, 127, 128, 129, 300, 383]),
                            128).tolist() == s["slots_bs128"]
    # literal vectors from the reference's stager tests (block_size 4):
    # request a at position 5 on blocks [7,8,9], request b at position 1 on [3]
    assert int(orc.slot_mapping(np.asarray([7, 8, 9]), 5, 4)) == 33
    assert int(orc.slot_mapping(np.asarray([3]), 1, 4)) == 13
    # MTP verify width 2 -> slots [33,34] and [13,14]
    assert orc.slot_mapping(np.asarray([7, 8, 9]), np.asarray([5, 6]), 4).tolist() == [33, 34]
    assert orc.slot_mapping(np.asarray([3]), np.asarray([1, 2]), 4).tolist() == [13, 14]
    # mixed prefill: a = 4 tokens on block 5, b = 2 tokens from position 1 on block 7
    assert orc.slot_mapping(np.asarray([5]), np.arange(4), 4).tolist() == [20, 21, 22, 23]
    assert orc.slot_mapping(np.asarray([7]), np.asarray([1, 2]), 4).tolist() == [29, 30]
    # prefix-cache hit: request b shares a's two full blocks and writes only new slots
    assert s["kvm_b_blocks"][:2] == s["kvm_shared"] == s["kvm_a_blocks"][:2]
    assert orc.slot_mapping(np.asarray(s["kvm_b_blocks"]), np.arange(8, 10), 4).tolist() \
        == s["kvm_b_new_slots"]


def test_write_kv_is_a_slot_scatter():
    g = torch.Generator().manual_seed(5)
    kc = torch.zeros(6, 4, 2, 8, dtype=torch.bfloat16)
    vc = torch.zeros(6, 4, 2, 8, dtype=torch.bfloat16)
    k = torch.randn(5, 2, 8, generator=g).to(torch.bfloat16)
    v = torch.randn(5, 2, 8, generator=g).to(torch.bfloat16)
    slots = [20, 21, 3, 0, 23]
    orc.write_kv(k, v, kc, vc, slots)
    for t, s in enumerate(slots):
        assert torch.equal(kc[s // 4, s % 4], k[t]) and torch.equal(vc[s // 4, s % 4], v[t])
    assert kc.float().abs().sum() == k.float().abs().sum()


def test_absorb_weights_and_absorbed_algebra(golden_small):
    m = golden_small["mla"]
    w_uk, w_uv = orc.build_absorb_weights(m["kv_b"], m["nh"], m["nope"], m["vd"], m["kvl"])
    assert torch.equal(w_uk, m["w_uk"]) and torch.equal(w_uv, m["w_uv"])
    # full sequences written into pages, absorbed path vs the reference's
    # non-absorbed dense answer (tolerance of scripts/verify_mla_absorb.py)
    bs = 8
    lens = np.diff([0] + m["cu"]).tolist()
    n_blocks = sum((l + bs - 1) // bs for l in lens)
    cache = torch.zeros(n_blocks, bs, 1, m["kvl"] + m["rope"], dtype=torch.bfloat16)
    bt = torch.zeros(len(lens), max((l + bs - 1) // bs for l in lens), dtype=torch.int32)
    cur, start = 0, 0
    for b, l in enumerate(lens):
        nb = (l + bs - 1) // bs
        bt[b, :nb] = torch.arange(cur, cur + nb)
        slots = orc.slot_mapping(bt[b].numpy().astype(np.int64), np.arange(l), bs)
        orc.write_kv(m["latent"][start:start + l, None, :], None, cache, None, slots)
        cur += nb
        start += l
    out = orc.mla_absorbed_attention(m["q_nope"], m["q_pe"], cache, bt, m["cu"], lens,
                                     m["scale"], w_uk, w_uv)
    torch.testing.assert_close(out.float(), m["out_nonabsorbed"].float(), atol=2e-2, rtol=2e-2)
    mine = orc.mla_nonabsorbed_attention(m["q_nope"], m["q_pe"], m["latent"], m["kv_b"], m["nh"],
                                         m["nope"], m["vd"], m["cu"], m["scale"])
    assert torch.equal(mine, m["out_nonabsorbed"])


def test_latent_576_decode_rows(golden_small):
    lat = golden_small["mla"]["lat576"]
    bs = 128
    for kv_len, tokens, q, o in zip(lat["seqs"], lat["latent"], lat["q"], lat["o"]):
        nb = (kv_len + bs - 1) // bs
        cache = torch.zeros(nb, bs, 1, 576, dtype=torch.bfloat16)
        cache.view(-1, 1, 576)[:kv_len] = tokens
        bt = torch.arange(nb, dtype=torch.int32)[None]
        got = orc.mla_latent_attention(q, cache, bt, [1], [kv_len], lat["scale"], 512)
        # the reference ran its bf16 P @ V on stride-0 expanded heads and padded
        # rows; a different GEMM shape may round the last bf16 bit differently
        torch.testing.assert_close(got.float(), o.float(), atol=4e-3, rtol=8e-3)


def test_wrapper_matches_reference_dense_backend(golden_small):
    c = golden_small["wrapper"]
    bs = 16
    nb = (c["t"] + bs - 1) // bs
    cache = torch.zeros(2, nb + 2, bs, c["n_kv"], c["hd"], dtype=torch.bfloat16)
    blocks = np.asarray([4, 1, 0][:nb])
    bt = torch.tensor(blocks, dtype=torch.int32)[None]
    slots = orc.slot_mapping(blocks, np.arange(c["t"]), bs)
    out = orc.gqa_attention_block(c["x"], c["w"], "model.layers.0.", c["n_q"], c["n_kv"], c["hd"],
                                  c["hd"] ** -0.5, c["cos"], c["sin"], cache, slots, bt,
                                  [c["t"]], [c["t"]])
    assert torch.equal(out, c["out"])


def test_split_and_merge_equals_unsplit(golden_paged):
    """Context-parallel convention: contiguous key ranges per rank merged by
    log-sum-exp equal the unsplit answer."""
    case = golden_paged["paged"][4]           # chunked prefill: masks cross the split points
    full, lse_full = orc.paged_attention(case["q"], case["k_cache"], case["v_cache"],
                                         case["block_table"], case["cu"], case["kv_lens"],
                                         case["scale"], return_lse=True)
    for ranks in (2, 3):
        parts, lses = [], []
        for r in range(ranks):
            ranges = [((kv * r) // ranks, (kv * (r + 1)) // ranks) for kv in case["kv_lens"]]
            o, l = orc.paged_attention(case["q"], case["k_cache"], case["v_cache"],
                                       case["block_table"], case["cu"], case["kv_lens"],
                                       case["scale"], return_lse=True, kv_ranges=ranges)
            parts.append(o.float().reshape(-1, case["hd"]))
            lses.append(l.reshape(-1))
        o, lse = orc.lse_combine(torch.stack(parts), torch.stack(lses))
        torch.testing.assert_close(o.float().view_as(full), full.float(), atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(lse.view_as(lse_full), lse_full, atol=1e-4, rtol=1e-4)
