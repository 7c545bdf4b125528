"""The whole GQA attention sub-block through ``B200GqaBackend.attention()`` on the GPU
(packed QKV projection with bias, optional per-head QK RMSNorm, NeoX RoPE, slot write,
paged attention, o_proj) against the reference's own output for it (golden ``wrapper``
case, produced by DenseBackend.attention of auto_infer/layers/attention/gqa.py:27-49,120-131)
and against the oracle's restatement of the same wiring."""
import numpy as np
import pytest
import torch

from oracle import paged_attention_oracle as orc
from tests.parity import assert_scale_free

pytestmark = pytest.mark.gpu
# projections run in cuBLAS here and in CPU GEMMs there, with one more bf16 rounding per stage
BLOCK_TOL = dict(atol=3e-2, rtol=3e-2)


def _ctx(backend, caches, slots, bt, cu, kv, cos, sin):
    from auto_infer_b200.forward_context import ForwardContext
    return ForwardContext(None, None, torch.as_tensor(slots, dtype=torch.int32).cuda(), bt.cuda(), cu, kv,
                          None, backend, caches, False, cos=cos.cuda(), sin=sin.cuda())


def test_reference_wrapper_case_prefill(golden_small):
    """One 37-token prompt: the reference's dense output for the sub-block is the target."""
    from auto_infer_b200 import ops
    from auto_infer_b200.gqa import B200GqaBackend
    c = golden_small["wrapper"]
    bs, t = 16, c["t"]
    nb = (t + bs - 1) // bs
    blocks = np.asarray([4, 1, 0][:nb])
    bt = torch.tensor(blocks, dtype=torch.int32)[None]
    slots = orc.slot_mapping(blocks, np.arange(t), bs)
    w = {k: v.cuda() for k, v in c["w"].items()}
    backend = B200GqaBackend(c["n_q"], c["n_kv"], c["hd"], c["hd"] ** -0.5, 1, "cuda", torch.bfloat16, w=w)
    caches = backend.alloc_kv_caches(nb + 2, bs)
    out = backend.attention(0, c["x"].cuda(), _ctx(backend, caches, slots, bt, [t], [t], c["cos"], c["sin"]))
    torch.testing.assert_close(out.cpu().float(), c["out"].float(), **BLOCK_TOL)
    assert_scale_free(out.cpu(), c["out"], "sub-block output", atol_rms=5e-2, rtol=2e-2, rel_l2=2e-2)
    # the cache now holds the rotated keys and the values at the reference's slots
    ref_cache = torch.zeros(2, nb + 2, bs, c["n_kv"], c["hd"], dtype=torch.bfloat16)
    orc.gqa_attention_block(c["x"], c["w"], "model.layers.0.", c["n_q"], c["n_kv"], c["hd"], c["hd"] ** -0.5,
                            c["cos"], c["sin"], ref_cache, slots, bt, [t], [t])
    torch.testing.assert_close(caches[0].cpu().float(), ref_cache.float(), atol=4e-2, rtol=2e-2)
    assert ops.read_status("cuda") == 0


@pytest.mark.parametrize("qk_norm", [False, True])
def test_mixed_step_with_qk_norm_and_bias(qk_norm):
    """A decode row, an MTP-verify pair and a short chunk over cached prefixes in one step,
    Qwen3-style per-head QK RMSNorm on or off, against the oracle's restatement."""
    from auto_infer_b200 import ops, synth
    from auto_infer_b200.gqa import B200GqaBackend
    g = torch.Generator().manual_seed(11 + qk_norm)
    hidden, n_q, n_kv, hd, bs = 128, 8, 2, 128, 128
    p = "model.layers.0.self_attn."

    def rnd(*shape, s=0.1):
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)

    w = {p + "qkv_proj.weight": rnd((n_q + 2 * n_kv) * hd, hidden), p + "qkv_proj.bias": rnd((n_q + 2 * n_kv) * hd),
         p + "o_proj.weight": rnd(hidden, n_q * hd)}
    if qk_norm:
        w[p + "q_norm.weight"] = rnd(hd, s=1.0).abs() + 0.5
        w[p + "k_norm.weight"] = rnd(hd, s=1.0).abs() + 0.5
    seqs = [(1, 300), (2, 131), (40, 40 + 200), (1, 1)]
    t = sum(q for q, _ in seqs)
    table, rows = synth.deal_block_tables(seqs, bs, 12, g)
    slots, cu, kv, acc, pos = [], [], [], 0, []
    for (q_len, kv_len), row in zip(seqs, rows):
        for x in range(kv_len - q_len, kv_len):
            slots.append(row[x // bs] * bs + x % bs)
            pos.append(x)
        acc += q_len
        cu.append(acc)
        kv.append(kv_len)
    x = rnd(t, hidden, s=1.0)
    cache = rnd(2, 12, bs, n_kv, hd, s=1.0)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    ang = torch.tensor(pos, dtype=torch.float32)[:, None] * inv[None]
    ang = torch.cat([ang, ang], dim=-1)
    cos, sin = ang.cos()[:, None, :].to(torch.bfloat16), ang.sin()[:, None, :].to(torch.bfloat16)
    ref_cache = cache.clone()
    ref = orc.gqa_attention_block(x, w, "model.layers.0.", n_q, n_kv, hd, hd ** -0.5, cos, sin, ref_cache, slots,
                                  table, cu, kv, rms_eps=1e-6)
    backend = B200GqaBackend(n_q, n_kv, hd, hd ** -0.5, 1, "cuda", torch.bfloat16,
                             w={k: v.cuda() for k, v in w.items()}, rms_eps=1e-6)
    caches = backend.alloc_kv_caches(12, bs)
    caches[0].copy_(cache)
    out = backend.attention(0, x.cuda(), _ctx(backend, caches, slots, table, cu, kv, cos, sin))
    torch.testing.assert_close(caches[0].cpu().float(), ref_cache.float(), atol=4e-2, rtol=2e-2)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **BLOCK_TOL)
    assert_scale_free(out.cpu(), ref, "sub-block output", atol_rms=5e-2, rtol=2e-2, rel_l2=2e-2)
    assert ops.read_status("cuda") == 0
