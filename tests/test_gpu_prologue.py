"""The fused prologue kernels (QK RMSNorm + NeoX RoPE + slot write for GQA; latent RMSNorm +
interleaved RoPE + latent write for MLA) against the eager chain of bf16 tensor ops they
replace (auto_infer/layers/attention/gqa.py:40-47, mla.py:96-113, restated in the oracle).
Without a norm the kernels round exactly where the chain does: bit-exact.  With a norm the
fp32 sum of squares is taken in another order, which can move a value by one bf16 step."""
import pytest
import torch

from oracle import paged_attention_oracle as orc

pytestmark = pytest.mark.gpu


def _ulp_close(got, want, ulps):
    """|got - want| <= ulps bf16 steps of the larger magnitude."""
    g, w = got.float(), want.float()
    step = torch.maximum(g.abs(), w.abs()) * 2.0 ** -7        # one bf16 step is at most 2^-7 relative
    bad = (g - w).abs() > ulps * step + 1e-30
    assert not bad.any(), f"{int(bad.sum())} values differ by more than {ulps} bf16 steps"


def _rope_tables(positions, dim, g):
    inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    ang = torch.tensor(positions, dtype=torch.float32)[:, None] * inv[None]
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos()[:, None, :].to(torch.bfloat16), ang.sin()[:, None, :].to(torch.bfloat16)


@pytest.mark.parametrize("qk_norm", [False, True])
@pytest.mark.parametrize("n_q,n_kv", [(8, 2), (16, 8), (5, 1)])
def test_gqa_prologue_matches_the_eager_chain(qk_norm, n_q, n_kv):
    from auto_infer_b200 import ops
    g = torch.Generator().manual_seed(31 + n_q)
    t, hd, bs, nb = 37, 128, 16, 9
    qkv = (torch.randn(t, (n_q + 2 * n_kv) * hd, generator=g) * 1.5).to(torch.bfloat16)
    q, k, v = qkv.split((n_q * hd, n_kv * hd, n_kv * hd), dim=-1)
    q, k, v = q.view(t, n_q, hd), k.view(t, n_kv, hd), v.view(t, n_kv, hd)
    cos, sin = _rope_tables(list(range(100, 100 + t)), hd, g)
    qn = (torch.rand(hd, generator=g) + 0.5).to(torch.bfloat16) if qk_norm else None
    kn = (torch.rand(hd, generator=g) + 0.5).to(torch.bfloat16) if qk_norm else None
    slots = torch.randperm(nb * bs, generator=g)[:t].to(torch.int32)
    slots[5] = -1                                              # a padding row: not written
    cache = torch.randn(2, nb, bs, n_kv, hd, generator=g).to(torch.bfloat16)

    # the eager chain, on the CPU
    qe, ke = q, k
    if qk_norm:
        qe, ke = orc.rms_norm(q, qn, 1e-6), orc.rms_norm(k, kn, 1e-6)
    qe = qe * cos + orc.rotate_half(qe) * sin
    ke = ke * cos + orc.rotate_half(ke) * sin
    want_cache = cache.clone()
    keep = slots >= 0
    orc.write_kv(ke[keep], v[keep], want_cache[0], want_cache[1], slots[keep].tolist())

    qkv_d = qkv.cuda()
    qd, kd, vd = qkv_d.split((n_q * hd, n_kv * hd, n_kv * hd), dim=-1)
    cache_d = cache.cuda()
    q_out, k_out = ops.gqa_rope_cache(qd.view(t, n_q, hd), kd.view(t, n_kv, hd), vd.view(t, n_kv, hd),
                                      cos.cuda(), sin.cuda(), cache_d[0], cache_d[1], slots.cuda(),
                                      q_norm_weight=qn.cuda() if qk_norm else None,
                                      k_norm_weight=kn.cuda() if qk_norm else None, eps=1e-6, want_k=True)
    torch.cuda.synchronize()
    assert ops.read_status("cuda") == 0
    assert torch.equal(cache_d[1].cpu(), want_cache[1])        # values: a plain copy, always bit-exact
    if qk_norm:
        _ulp_close(q_out.cpu(), qe, 1)
        _ulp_close(k_out.cpu(), ke, 1)
        _ulp_close(cache_d[0].cpu(), want_cache[0], 1)
    else:
        assert torch.equal(q_out.cpu(), qe)
        assert torch.equal(k_out.cpu(), ke)
        assert torch.equal(cache_d[0].cpu(), want_cache[0])
    # the cache holds exactly the rotated keys the kernel returned
    got_rows = cache_d[0].view(-1, n_kv, hd)[slots[keep].long().cuda()]
    assert torch.equal(got_rows, k_out[keep.cuda()])


def test_mla_prologue_matches_the_eager_chain():
    from auto_infer_b200 import ops
    g = torch.Generator().manual_seed(77)
    t, nh, nope, rope, kvl, bs, nb = 21, 16, 128, 64, 512, 16, 6
    q = (torch.randn(t, nh, nope + rope, generator=g)).to(torch.bfloat16)
    ckv_full = (torch.randn(t, kvl + rope, generator=g) * 2).to(torch.bfloat16)
    norm_w = (torch.rand(kvl, generator=g) + 0.5).to(torch.bfloat16)
    ang = torch.randn(t, 1, rope, generator=g)
    cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
    slots = torch.randperm(nb * bs, generator=g)[:t].to(torch.int32)
    cache = torch.randn(nb, bs, 1, kvl + rope, generator=g).to(torch.bfloat16)

    # eager chain (auto_infer/layers/attention/mla.py:96-113)
    q_pe = q[..., nope:]
    ckv, k_pe = ckv_full.split([kvl, rope], dim=-1)
    ckv = orc.rms_norm(ckv, norm_w, 1e-6)
    k_pe = orc.ds_rope_interleave(k_pe.view(t, 1, rope))
    q_pe_e = orc.ds_rope_interleave(q_pe)
    q_pe_e = q_pe_e * cos + orc.rotate_half(q_pe_e) * sin
    k_pe = k_pe * cos + orc.rotate_half(k_pe) * sin
    k_latent = torch.cat([ckv.unsqueeze(1), k_pe], dim=-1).contiguous()
    want_cache = cache.clone()
    orc.write_kv(k_latent, None, want_cache, None, slots.tolist())

    qd = q.cuda()
    q_latent = torch.zeros(t, nh, kvl + rope, dtype=torch.bfloat16, device="cuda")
    cache_d = cache.cuda()
    got_k = ops.mla_rope_norm_cache(ckv_full.cuda(), norm_w.cuda(), 1e-6, qd[..., nope:], q_latent[..., kvl:],
                                    cos.cuda(), sin.cuda(), cache_d, slots.cuda(), kv_lora_rank=kvl,
                                    want_k_latent=True)
    torch.cuda.synchronize()
    assert ops.read_status("cuda") == 0
    assert torch.equal(q_latent[..., kvl:].cpu(), q_pe_e)      # rotary only: bit-exact
    assert float(q_latent[..., :kvl].abs().sum()) == 0.0       # the other columns are not touched
    assert torch.equal(got_k[..., kvl:].cpu(), k_pe)
    _ulp_close(got_k[..., :kvl].cpu(), k_latent[..., :kvl], 1)
    _ulp_close(cache_d.cpu(), want_cache, 1)
    assert torch.equal(cache_d.view(-1, 1, kvl + rope)[slots.long().cuda()], got_k)


def test_copy_blocks_moves_pages_bit_exactly():
    """Block transfer with the contract of auto_infer/pd/connector.py:30-51: both cache layouts
    (dense (2, blocks, ...) tensor and (k, v) tuple), same ids on both sides; plus the
    remapped form."""
    from auto_infer_b200 import ops
    g = torch.Generator().manual_seed(9)
    shape = (12, 16, 2, 128)
    def rnd(*s):
        return torch.randn(*s, generator=g).to(torch.bfloat16)
    src = [rnd(2, *shape), (rnd(*shape), rnd(*shape))]
    dst = [rnd(2, *shape), (rnd(*shape), rnd(*shape))]
    ids = [7, 0, 11, 3]
    want = [dst[0].clone(), (dst[1][0].clone(), dst[1][1].clone())]
    for b in ids:
        want[0][:, b] = src[0][:, b]
        want[1][0][b] = src[1][0][b]
        want[1][1][b] = src[1][1][b]
    src_d = [src[0].cuda(), (src[1][0].cuda(), src[1][1].cuda())]
    dst_d = [dst[0].cuda(), (dst[1][0].cuda(), dst[1][1].cuda())]
    ops.copy_blocks(src_d, dst_d, ids)
    torch.cuda.synchronize()
    assert torch.equal(dst_d[0].cpu(), want[0])
    assert torch.equal(dst_d[1][0].cpu(), want[1][0]) and torch.equal(dst_d[1][1].cpu(), want[1][1])
    # remapped: pages land on other ids of a larger pool
    big = [torch.zeros(2, 20, *shape[1:], dtype=torch.bfloat16, device="cuda")]
    ops.copy_blocks(src_d[:1], big, ids, target_block_ids=[19, 18, 1, 2])
    torch.cuda.synchronize()
    for s_id, d_id in zip(ids, [19, 18, 1, 2]):
        assert torch.equal(big[0][:, d_id].cpu(), src[0][:, s_id])
    assert float(big[0][:, 5].abs().sum()) == 0.0
    with pytest.raises(ValueError, match="layer counts must match"):
        ops.copy_blocks(src_d, dst_d[:1], ids)
    assert ops.read_status("cuda") == 0
