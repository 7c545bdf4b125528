"""Parity of the absorbed-MLA decode kernel (576-wide latent, stored once) with
the oracle and with the reference's golden outputs, through the C ABI.
Tolerance: rtol 2e-2 / atol 2e-2 (the tolerance of scripts/verify_mla_absorb.py)."""
import pytest
import torch

from oracle import paged_attention_oracle as orc
from tests.parity import TOL, assert_attention_close, assert_scale_free

pytestmark = pytest.mark.gpu


def _mla(q_latent, cache, bt, cu, kv, scale, heads, num_ctas=None, want_lse=False):
    from auto_infer_b200 import ops
    plan = ops.MlaDecodePlan(cu, kv, heads, "cuda", num_ctas=num_ctas)
    lse = torch.empty(q_latent.shape[0], heads, dtype=torch.float32, device="cuda") if want_lse else None
    out = ops.mla_decode_absorbed(q_latent.cuda(), cache.cuda(), bt.cuda(), plan, scale, lse_out=lse)
    torch.cuda.synchronize()
    assert ops.read_status("cuda") == 0
    return (out.cpu(), lse.cpu()) if want_lse else out.cpu()


def test_golden_latent_rows_from_the_reference_core(golden_small):
    lat = golden_small["mla"]["lat576"]
    for kv_len, tokens, q, o in zip(lat["seqs"], lat["latent"], lat["q"], lat["o"]):
        nb = (kv_len + 127) // 128
        cache = torch.zeros(nb, 128, 1, 576, dtype=torch.bfloat16)
        cache.view(-1, 1, 576)[:kv_len] = tokens
        bt = torch.arange(nb, dtype=torch.int32)[None]
        for num_ctas in (None, 1, 3):
            got = _mla(q, cache, bt, [1], [kv_len], lat["scale"], 16, num_ctas=num_ctas)
            assert_attention_close(got, o, what=f"golden latent row kv_len={kv_len} ctas={num_ctas}")


@pytest.mark.parametrize("ctx,bs", [(1, 128), (31, 128), (32, 128), (33, 128), (128, 128), (129, 128),
                                    (1000, 16), (257, 32)])
def test_page_and_tile_boundaries(ctx, bs):
    from auto_infer_b200 import synth
    b = synth.build_mla_batch("edge", [(1, ctx), (1, ctx + 40)], 16, 160 if bs < 128 else 24,
                              500 + ctx, block_size=bs)
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache, b.kv_cache, b.block_table, b.cu_seqlens_q,
                                       b.seqlens_kv, b.scale, return_lse=True)
    out, lse = _mla(b.q, b.kv_cache, b.block_table, b.cu_seqlens_q, b.seqlens_kv, b.scale, 16,
                    want_lse=True)
    assert_attention_close(out, ref[..., :512], lse, ref_lse)


def test_fewer_heads_and_two_query_rows():
    """8 heads x 2 query rows fill the 16 MMA rows (multi-token verify shape)."""
    from auto_infer_b200 import synth
    b = synth.build_mla_batch("mtp", [(2, 300), (1, 77), (2, 2)], 8, 16, 91)
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache, b.kv_cache, b.block_table, b.cu_seqlens_q,
                                       b.seqlens_kv, b.scale, return_lse=True)
    out, lse = _mla(b.q, b.kv_cache, b.block_table, b.cu_seqlens_q, b.seqlens_kv, b.scale, 8, want_lse=True)
    assert_attention_close(out, ref[..., :512], lse, ref_lse)


@pytest.mark.parametrize("batch", [4, 16, 64])
def test_config3_full_size_with_absorbed_projections(batch):
    """Config 3: latent write (bit-exact), latent attention, then the absorbed
    value projection; compared on the final (T, 16, 128) output."""
    from auto_infer_b200 import ops, synth
    d = synth.config3(batch, "cuda")            # 4096-page latent pool generated on the device
    b = d.to("cpu")
    ops.reshape_and_cache(d.k_new, None, d.kv_cache, None, d.slot_mapping)
    orc.write_kv(b.k_new, None, b.kv_cache, None, b.slot_mapping.tolist())
    assert torch.equal(d.kv_cache.cpu(), b.kv_cache)
    plan = ops.MlaDecodePlan(b.cu_seqlens_q, b.seqlens_kv, 16, "cuda")
    lse = torch.empty(b.num_tokens, 16, dtype=torch.float32, device="cuda")
    o_latent = ops.mla_decode_absorbed(d.q, d.kv_cache, d.block_table, plan, b.scale, lse_out=lse)
    o_latent32 = ops.mla_decode_absorbed(d.q, d.kv_cache, d.block_table, plan, b.scale, out_f32=True)
    out = torch.einsum("tnl,nvl->tnv", o_latent, d.extra["w_uv"]).cpu()
    ref = orc.mla_absorbed_attention(b.extra["q_nope"], b.extra["q_pe"], b.kv_cache, b.block_table,
                                     b.cu_seqlens_q, b.seqlens_kv, b.scale, b.extra["w_uk"],
                                     b.extra["w_uv"])
    # the final rows pass through one more bf16 contraction (W_UV) on each side: the stated
    # tolerance plus a row-relative L2 bound; the kernel's own output is held to the full check
    torch.testing.assert_close(out.float(), ref.float(), **TOL)
    assert_scale_free(out, ref, "rows after W_UV", atol_rms=5e-2, rtol=2e-2, rel_l2=2e-2)
    full, ref_lse = orc.paged_attention(b.q, b.kv_cache, b.kv_cache, b.block_table, b.cu_seqlens_q,
                                        b.seqlens_kv, b.scale, return_lse=True)
    assert_attention_close(o_latent.cpu(), full[..., :512], lse.cpu(), ref_lse, "latent rows (bf16)")
    assert_attention_close(o_latent32.cpu(), full[..., :512], what="latent rows (fp32)")
    assert ops.read_status("cuda") == 0


def test_backend_block_decode_and_prefill_rows():
    """The whole sub-block (projections, latent norm, interleaved RoPE, write,
    attention, W_UV, o_proj) through B200MlaBackend against the oracle's
    restatement; a 5-token prefill row exercises the per-token expansion."""
    from auto_infer_b200 import ops
    from auto_infer_b200.forward_context import ForwardContext
    from auto_infer_b200.mla import B200MlaBackend
    from auto_infer_b200 import synth
    g = torch.Generator().manual_seed(77)
    hidden, nh, nope, rope, vd, kvl, qlr = 256, 16, 128, 64, 128, 512, 96
    p = "model.layers.0.self_attn."

    def rnd(*shape, s=0.05):
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)

    w = {p + "q_a_proj.weight": rnd(qlr, hidden), p + "q_a_layernorm.weight": rnd(qlr, s=1.0).abs(),
         p + "q_b_proj.weight": rnd(nh * (nope + rope), qlr, s=0.2),
         p + "kv_a_proj_with_mqa.weight": rnd(kvl + rope, hidden, s=0.2),
         p + "kv_a_layernorm.weight": rnd(kvl, s=1.0).abs(),
         p + "kv_b_proj.weight": rnd(nh * (nope + vd), kvl), p + "o_proj.weight": rnd(hidden, nh * vd)}
    seqs = [(1, 200), (5, 5 + 130), (1, 1)]
    t = sum(q for q, _ in seqs)
    table, rows = synth.deal_block_tables(seqs, 128, 8, g)
    slots, cu, kv, acc = [], [], [], 0
    for (q_len, kv_len), row in zip(seqs, rows):
        slots += [row[pos // 128] * 128 + pos % 128 for pos in range(kv_len - q_len, kv_len)]
        acc += q_len
        cu.append(acc)
        kv.append(kv_len)
    x = rnd(t, hidden, s=1.0)
    cache = rnd(8, 128, 1, kvl + rope, s=1.0)
    ang = torch.randn(t, 1, rope, generator=g)
    cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
    scale = (nope + rope) ** -0.5
    ref_cache = cache.clone()
    ref = orc.mla_absorbed_block(x, w, "model.layers.0.", num_heads=nh, qk_nope=nope, qk_rope=rope,
                                 v_head_dim=vd, kv_lora_rank=kvl, q_lora_rank=qlr, rms_eps=1e-6,
                                 cos=cos, sin=sin, latent_cache=ref_cache, slots=slots,
                                 block_table=table, cu_seqlens_q=cu, seqlens_kv=kv, softmax_scale=scale)
    wd = {k: v.cuda() for k, v in w.items()}
    backend = B200MlaBackend(wd, num_heads=nh, qk_nope=nope, qk_rope=rope, v_head_dim=vd,
                             kv_lora_rank=kvl, q_lora_rank=qlr, rms_eps=1e-6, softmax_scale=scale,
                             num_layers=1, device="cuda", dtype=torch.bfloat16)
    caches = backend.alloc_kv_caches(8, 128)
    assert caches[0][0] is caches[0][1] and caches[0][0].shape == (8, 128, 1, 576)
    caches[0][0].copy_(cache)
    ctx = ForwardContext(None, None, torch.tensor(slots, dtype=torch.int32).cuda(), table.cuda(), cu, kv,
                         None, backend, caches, False, cos=cos.cuda(), sin=sin.cuda())
    out = backend.attention(0, x.cuda(), ctx)
    # projections run in cuBLAS here and in CPU GEMMs there: the new latent rows can differ by an ulp
    torch.testing.assert_close(caches[0][0].cpu().float(), ref_cache.float(), atol=4e-2, rtol=2e-2)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=3e-2, rtol=3e-2)
    assert ops.read_status("cuda") == 0


def test_more_heads_than_one_launch_holds_run_as_slices():
    """40 heads on one rank: four launches of 10 heads each over the same latent cache and plan (the
    two-token sequence exceeds 16 rows per launch and takes the per-row expansion)."""
    from auto_infer_b200 import ops, synth
    from auto_infer_b200.forward_context import ForwardContext
    from auto_infer_b200.mla import B200MlaBackend
    heads = 40
    b = synth.build_mla_batch("sliced heads", [(1, 70), (1, 600), (2, 129), (1, 1)], heads, 12, 91)
    d = b.to("cuda")
    backend = B200MlaBackend({}, num_heads=heads, qk_nope=128, qk_rope=64, v_head_dim=128, kv_lora_rank=512,
                             q_lora_rank=None, rms_eps=1e-6, softmax_scale=b.scale, num_layers=1, device="cuda",
                             dtype=torch.bfloat16)
    assert backend.heads_per_launch == 10
    ctx = ForwardContext(None, None, d.slot_mapping, d.block_table, b.cu_seqlens_q, b.seqlens_kv, None, backend,
                         [(d.kv_cache, d.kv_cache)], True)
    out = backend.latent_attention(0, d.q, d.k_new, ctx).cpu()
    orc.write_kv(b.k_new, None, b.kv_cache, None, b.slot_mapping.tolist())
    assert torch.equal(d.kv_cache.cpu(), b.kv_cache)
    ref = orc.paged_attention(b.q, b.kv_cache, b.kv_cache, b.block_table, b.cu_seqlens_q, b.seqlens_kv, b.scale)
    assert_attention_close(out, ref[..., :512], what="40 heads in slices of 10")
    assert ops.read_status("cuda") == 0
