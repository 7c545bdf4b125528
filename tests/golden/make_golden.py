"""Generate the committed golden fixtures by running the reference's own code.

Run once, in a container that has the auto-infer sources importable:

    PYTHONPATH=<auto-infer checkout> python tests/golden/make_golden.py

Every output below is produced by a function imported from auto-infer itself
(``dense_causal_attention``, ``DenseBackend``, ``MlaDenseBackend``,
``build_absorb_weights``, ``slot_mapping``, ``KVCacheManager``,
``pack_qwen2_projections``); nothing from this repository is involved.  The
fixtures hold inputs and outputs so the tests do not depend on RNG stability.

Paged / decode shapes (q_len < kv_len) are obtained from the reference function,
which only handles q_len == kv_len, by zero-padding the query to the full
sequence length and keeping the last q_len rows: rows of a causal softmax are
independent, so those rows are exactly the bottom-right-causal answer.
"""
import os
import sys

import numpy as np
import torch

from auto_infer.engine.kv_cache_manager import KVCacheManager
from auto_infer.engine.token_layout import slot_mapping
from auto_infer.layers.attention.base import dense_causal_attention
from auto_infer.layers.attention.gqa import DenseBackend
from auto_infer.layers.attention.mla import MlaDenseBackend, build_absorb_weights
from auto_infer.models.qwen2 import pack_qwen2_projections

HERE = os.path.dirname(os.path.abspath(__file__))


class _Ctx:
    pass


def _ref_paged_rows(q, k_full, v_full, n_q, n_kv, scale):
    """Reference answer for the last q_len rows of one sequence."""
    kv_len, q_len = k_full.shape[0], q.shape[0]
    q_pad = torch.zeros(kv_len, n_q, q.shape[-1], dtype=q.dtype)
    q_pad[kv_len - q_len:] = q
    backend = DenseBackend(n_q_heads=n_q, n_kv_heads=n_kv, head_dim=q.shape[-1], scale=scale)
    ctx = _Ctx()
    ctx.cu_seqlens_q = [kv_len]
    out = backend._attn(0, q_pad, k_full, v_full, ctx)
    return out[kv_len - q_len:]


def dense_cases():
    """Tiny fp32 cases shaped like the reference's own unit tests
    (tests/test_attention_backend.py:46-140, seeds 0, 1, 2, 4)."""
    cases = []
    for seed, (t_list, n_q, n_kv, hd) in {0: ([4], 1, 1, 8), 1: ([5], 4, 2, 4),
                                          2: ([3, 4], 2, 2, 4), 4: ([2, 5, 1], 4, 1, 8)}.items():
        torch.manual_seed(seed)
        total = sum(t_list)
        q = torch.randn(total, n_q, hd)
        k = torch.randn(total, n_kv, hd)
        v = torch.randn(total, n_kv, hd)
        backend = DenseBackend(n_q_heads=n_q, n_kv_heads=n_kv, head_dim=hd, scale=hd ** -0.5)
        ctx = _Ctx()
        ctx.cu_seqlens_q = list(np.cumsum(t_list))
        out = backend._attn(0, q, k, v, ctx)
        cases.append(dict(seed=seed, q=q, k=k, v=v, cu=[int(c) for c in ctx.cu_seqlens_q],
                          n_q=n_q, n_kv=n_kv, hd=hd, out=out))
    return cases


def paged_cases():
    """bf16 paged cases: decode (q_len 1), MTP verify (q_len 2), a drafter-like
    ragged batch (q_len 1..2), chunked prefill over a cached prefix, block sizes
    16 and 128, contexts on both sides of page boundaries."""
    specs = [
        dict(name="decode_bs16", seed=11, bs=16, n_q=8, n_kv=2, hd=128,
             seqs=[(1, 1), (1, 16), (1, 17), (1, 300), (1, 129)]),
        dict(name="decode_bs128", seed=12, bs=128, n_q=4, n_kv=2, hd=128,
             seqs=[(1, 127), (1, 128), (1, 129), (1, 515)]),
        dict(name="mtp_verify_bs128", seed=13, bs=128, n_q=8, n_kv=2, hd=128,
             seqs=[(2, 2), (2, 130), (2, 257), (2, 384)]),
        dict(name="drafter_ragged_bs16", seed=14, bs=16, n_q=4, n_kv=1, hd=128,
             seqs=[(1, 11), (2, 22), (1, 31), (2, 42), (2, 2)]),
        dict(name="chunk_prefill_bs128", seed=15, bs=128, n_q=4, n_kv=2, hd=128,
             seqs=[(40, 40), (33, 161), (64, 320), (1, 77)]),
    ]
    cases = []
    for s in specs:
        g = torch.Generator().manual_seed(s["seed"])
        bs, n_q, n_kv, hd = s["bs"], s["n_q"], s["n_kv"], s["hd"]
        scale = hd ** -0.5
        need = sum((kv + bs - 1) // bs for _, kv in s["seqs"])
        pool = need + 3
        perm = torch.randperm(pool, generator=g).tolist()
        k_cache = torch.zeros(pool, bs, n_kv, hd, dtype=torch.bfloat16)
        v_cache = torch.zeros(pool, bs, n_kv, hd, dtype=torch.bfloat16)
        max_blocks = max((kv + bs - 1) // bs for _, kv in s["seqs"])
        block_table = torch.zeros(len(s["seqs"]), max_blocks, dtype=torch.int32)
        qs, outs, cu, kv_lens = [], [], [], []
        acc, cursor = 0, 0
        for b, (q_len, kv_len) in enumerate(s["seqs"]):
            nb = (kv_len + bs - 1) // bs
            blocks = perm[cursor:cursor + nb]
            cursor += nb
            block_table[b, :nb] = torch.tensor(blocks, dtype=torch.int32)
            k_full = torch.randn(kv_len, n_kv, hd, generator=g).to(torch.bfloat16)
            v_full = torch.randn(kv_len, n_kv, hd, generator=g).to(torch.bfloat16)
            q = torch.randn(q_len, n_q, hd, generator=g).to(torch.bfloat16)
            slots = slot_mapping(np.asarray(blocks, dtype=np.int64), np.arange(kv_len), bs)
            k_cache.view(-1, n_kv, hd)[torch.from_numpy(slots)] = k_full
            v_cache.view(-1, n_kv, hd)[torch.from_numpy(slots)] = v_full
            outs.append(_ref_paged_rows(q, k_full, v_full, n_q, n_kv, scale))
            qs.append(q)
            acc += q_len
            cu.append(acc)
            kv_lens.append(kv_len)
        cases.append(dict(name=s["name"], bs=bs, n_q=n_q, n_kv=n_kv, hd=hd, scale=scale,
                          q=torch.cat(qs), k_cache=k_cache, v_cache=v_cache,
                          block_table=block_table, cu=cu, kv_lens=kv_lens, out=torch.cat(outs)))
    return cases


def slot_cases():
    """Integer known answers from the reference's slot arithmetic and block
    allocator, including a prefix-cache hit that makes two requests share
    physical blocks."""
    out = {}
    bt = np.asarray([7, 8, 9], dtype=np.int64)
    out["slots_bs4_pos0_9"] = slot_mapping(bt, np.arange(10), 4).tolist()
    out["slots_bs128"] = slot_mapping(np.asarray([5, 0, 3], dtype=np.int64),
                                      np.asarray([0, 127, 128, 129, 300, 383]), 128).tolist()
    kvm = KVCacheManager(num_blocks=16, block_size=4)
    prompt = list(range(100, 111))                      # 11 tokens -> 2 full blocks + partial
    a_blocks = kvm.allocate(11)
    kvm.register_prefix(prompt, a_blocks)
    hit = kvm.match_prefix(prompt[:10])                 # request b shares the two full blocks
    b_blocks = hit + kvm.allocate(10 - len(hit) * 4)
    out["kvm_a_blocks"] = [int(x) for x in a_blocks]
    out["kvm_b_blocks"] = [int(x) for x in b_blocks]
    out["kvm_shared"] = [int(x) for x in hit]
    out["kvm_b_new_slots"] = slot_mapping(np.asarray(b_blocks, dtype=np.int64),
                                          np.arange(8, 10), 4).tolist()
    return out


def mla_cases():
    """Absorbed-MLA fixtures: the reference's weight split, the reference's
    non-absorbed dense attention on full sequences (the form
    scripts/verify_mla_absorb.py compares the absorbed path against), and the
    latent MQA attention itself for decode rows through the reference core."""
    g = torch.Generator().manual_seed(21)
    nh, nope, rope, vd, kvl = 4, 32, 16, 32, 64
    scale = (nope + rope) ** -0.5
    kv_b = (torch.randn(nh * (nope + vd), kvl, generator=g) * 0.05).to(torch.bfloat16)
    w_uk, w_uv = build_absorb_weights(kv_b, nh, nope, vd, kvl)
    lens = [9, 20]
    total = sum(lens)
    latent = torch.randn(total, kvl + rope, generator=g).to(torch.bfloat16)
    q_nope = torch.randn(total, nh, nope, generator=g).to(torch.bfloat16)
    q_pe = torch.randn(total, nh, rope, generator=g).to(torch.bfloat16)
    ckv, k_pe = latent[:, :kvl], latent[:, kvl:]
    kv = (ckv @ kv_b.t()).view(total, nh, nope + vd)
    k_nope, v = kv.split([nope, vd], dim=-1)
    k = torch.cat([k_nope, k_pe[:, None, :].expand(total, nh, rope)], dim=-1).contiguous()
    q = torch.cat([q_nope, q_pe], dim=-1)
    backend = MlaDenseBackend({}, num_heads=nh, qk_nope=nope, qk_rope=rope, v_head_dim=vd,
                              kv_lora_rank=kvl, q_lora_rank=None, rms_eps=1e-6, softmax_scale=scale)
    ctx = _Ctx()
    ctx.cu_seqlens_q = list(np.cumsum(lens))
    out_nonabsorbed = backend._attn(0, q, k, v.contiguous(), ctx)

    # latent MQA attention at the real 512+64 width, decode rows, via the core
    g2 = torch.Generator().manual_seed(22)
    nh2, kvl2, rope2 = 16, 512, 64
    scale2 = 192 ** -0.5
    seqs = [130, 257]
    lat_tokens, q_lat, o_lat = [], [], []
    for kv_len in seqs:
        lt = torch.randn(kv_len, 1, kvl2 + rope2, generator=g2).to(torch.bfloat16)
        ql = torch.randn(1, nh2, kvl2 + rope2, generator=g2).to(torch.bfloat16)
        q_pad = torch.zeros(kv_len, nh2, kvl2 + rope2, dtype=torch.bfloat16)
        q_pad[-1:] = ql
        o = dense_causal_attention(q_pad, lt.expand(kv_len, nh2, kvl2 + rope2),
                                   lt.expand(kv_len, nh2, kvl2 + rope2), [kv_len], scale2)
        lat_tokens.append(lt)
        q_lat.append(ql)
        o_lat.append(o[-1:, :, :kvl2])
    return dict(nh=nh, nope=nope, rope=rope, vd=vd, kvl=kvl, scale=scale, kv_b=kv_b,
                w_uk=w_uk, w_uv=w_uv, latent=latent, q_nope=q_nope, q_pe=q_pe,
                cu=[int(c) for c in ctx.cu_seqlens_q], out_nonabsorbed=out_nonabsorbed,
                lat576=dict(seqs=seqs, scale=scale2, latent=lat_tokens, q=q_lat, o=o_lat))


def _install_vendor_norm_stub():
    """The reference's RMSNorm (auto_infer/layers/norm.py:5-9) is a call into the vendor module,
    which does not exist off the NPU.  The one function of it the MLA sub-block needs is stood
    in for here, by its documented arithmetic (normalise in fp32, round to the input type,
    scale by the weight); everything else in these fixtures is the reference's own code."""
    import types
    if "torch_npu" in sys.modules:
        return
    stub = types.ModuleType("torch_npu")

    def npu_rms_norm(x, weight, eps):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight, None

    stub.npu_rms_norm = npu_rms_norm
    sys.modules["torch_npu"] = stub


def mla_paged_cases():
    """Non-absorbed MLA at the real head widths (K 192 = 128 + 64, V 128): the reference's
    whole sub-block (``MlaDenseBackend.attention``: q-LoRA or plain q projection, kv_a, latent
    norm, kv_b, interleaved rotary embedding, per-head K / V, causal softmax, o_proj) on
    packed prefill sequences, the q / k / v it hands to its core, and decode / verify rows
    of the core obtained by zero-padding the query."""
    _install_vendor_norm_stub()
    out = {}
    for name, q_lora in (("plain_q", None), ("q_lora", 48)):
        g = torch.Generator().manual_seed(31 if q_lora is None else 32)
        nh, nope, rope, vd, kvl, hidden = 4, 128, 64, 128, 64, 96
        scale = (nope + rope) ** -0.5
        p = "model.layers.0.self_attn."

        def rnd(*shape, s=0.08):
            return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)

        w = {p + "kv_a_proj_with_mqa.weight": rnd(kvl + rope, hidden),
             p + "kv_a_layernorm.weight": (1 + 0.1 * torch.randn(kvl, generator=g)).to(torch.bfloat16),
             p + "kv_b_proj.weight": rnd(nh * (nope + vd), kvl, s=0.15),
             p + "o_proj.weight": rnd(hidden, nh * vd)}
        if q_lora is None:
            w[p + "q_proj.weight"] = rnd(nh * (nope + rope), hidden)
        else:
            w[p + "q_a_proj.weight"] = rnd(q_lora, hidden)
            w[p + "q_a_layernorm.weight"] = (1 + 0.1 * torch.randn(q_lora, generator=g)).to(torch.bfloat16)
            w[p + "q_b_proj.weight"] = rnd(nh * (nope + rope), q_lora, s=0.15)
        lens = [70, 9, 130]
        total = sum(lens)
        x = torch.randn(total, hidden, generator=g).to(torch.bfloat16)
        pos = torch.cat([torch.arange(n, dtype=torch.float32) for n in lens])
        inv = 1.0 / (10000.0 ** (torch.arange(0, rope, 2, dtype=torch.float32) / rope))
        ang = torch.cat([pos[:, None] * inv[None], pos[:, None] * inv[None]], dim=-1)
        cos = ang.cos()[:, None, :].to(torch.bfloat16)
        sin = ang.sin()[:, None, :].to(torch.bfloat16)
        backend = MlaDenseBackend(w, num_heads=nh, qk_nope=nope, qk_rope=rope, v_head_dim=vd,
                                  kv_lora_rank=kvl, q_lora_rank=q_lora, rms_eps=1e-6, softmax_scale=scale)
        seen = {}
        core = backend._attn

        def spy(layer_idx, q, k, v, ctx):
            seen["q"], seen["k"], seen["v"] = q.clone(), k.clone(), v.clone()
            seen["o"] = core(layer_idx, q, k, v, ctx)
            return seen["o"]

        backend._attn = spy
        ctx = _Ctx()
        ctx.cu_seqlens_q = [int(c) for c in np.cumsum(lens)]
        ctx.cos, ctx.sin = cos, sin
        block_out = backend.attention(0, x, ctx)
        out[name] = dict(nh=nh, nope=nope, rope=rope, vd=vd, kvl=kvl, hidden=hidden, q_lora=q_lora,
                         scale=scale, w=w, x=x, cos=cos, sin=sin, cu=ctx.cu_seqlens_q, lens=lens,
                         q=seen["q"], k=seen["k"], v=seen["v"], core_out=seen["o"], block_out=block_out)

    # decode (q_len 1) and verify (q_len 3) rows of the core over longer sequences
    g = torch.Generator().manual_seed(33)
    nh, scale = 4, 192 ** -0.5
    rows = []
    for q_len, kv_len in ((1, 200), (3, 131), (1, 64), (2, 65)):
        k = torch.randn(kv_len, nh, 192, generator=g).to(torch.bfloat16)
        v = torch.randn(kv_len, nh, 128, generator=g).to(torch.bfloat16)
        q = torch.randn(q_len, nh, 192, generator=g).to(torch.bfloat16)
        q_pad = torch.zeros(kv_len, nh, 192, dtype=torch.bfloat16)
        q_pad[kv_len - q_len:] = q
        o = dense_causal_attention(q_pad, k, v, [kv_len], scale)[kv_len - q_len:]
        rows.append(dict(q_len=q_len, kv_len=kv_len, q=q, k=k, v=v, o=o))
    out["decode_rows"] = dict(nh=nh, scale=scale, rows=rows)
    return out


def wrapper_case():
    """Whole GQA sub-block through the reference's DenseBackend.attention
    (packed projection, RoPE, core, o_proj) on one prefill sequence, bf16."""
    torch.manual_seed(3)
    t, hidden, n_q, n_kv, hd = 37, 64, 4, 2, 128
    p = "model.layers.0.self_attn."
    w = {
        p + "q_proj.weight": torch.randn(n_q * hd, hidden) * 0.2, p + "q_proj.bias": torch.randn(n_q * hd) * 0.1,
        p + "k_proj.weight": torch.randn(n_kv * hd, hidden) * 0.2, p + "k_proj.bias": torch.randn(n_kv * hd) * 0.1,
        p + "v_proj.weight": torch.randn(n_kv * hd, hidden) * 0.2, p + "v_proj.bias": torch.randn(n_kv * hd) * 0.1,
        p + "o_proj.weight": torch.randn(hidden, n_q * hd) * 0.1,
    }
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    pack_qwen2_projections(w, num_layers=1)
    x = torch.randn(t, hidden).to(torch.bfloat16)
    pos = torch.arange(t, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    ang = torch.cat([pos[:, None] * inv[None], pos[:, None] * inv[None]], dim=-1)
    cos = ang.cos()[:, None, :].to(torch.bfloat16)
    sin = ang.sin()[:, None, :].to(torch.bfloat16)
    ctx = _Ctx()
    ctx.cu_seqlens_q = [t]
    ctx.cos, ctx.sin = cos, sin
    backend = DenseBackend(n_q_heads=n_q, n_kv_heads=n_kv, head_dim=hd, scale=hd ** -0.5, w=w)
    out = backend.attention(0, x, ctx)
    return dict(t=t, hidden=hidden, n_q=n_q, n_kv=n_kv, hd=hd, w=w, x=x, cos=cos, sin=sin, out=out)


def _compact(obj):
    """Clone tensor views so a slice does not drag its whole storage into the file."""
    if isinstance(obj, torch.Tensor):
        return obj.detach().clone().contiguous()
    if isinstance(obj, dict):
        return {k: _compact(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_compact(v) for v in obj)
    return obj


def main():
    torch.set_num_threads(1)
    if "--mla-paged-only" in sys.argv:          # adds the newest file without touching the others
        torch.save(_compact(mla_paged_cases()), os.path.join(HERE, "reference_mla_paged.pt"))
        return
    small = dict(dense=dense_cases(), slots=slot_cases(), mla=mla_cases(), wrapper=wrapper_case())
    torch.save(_compact(small), os.path.join(HERE, "reference_small.pt"))
    torch.save(_compact(mla_paged_cases()), os.path.join(HERE, "reference_mla_paged.pt"))
    torch.save(_compact(dict(paged=paged_cases())), os.path.join(HERE, "reference_paged.pt"))
    for name in ("reference_small.pt", "reference_paged.pt"):
        print(name, os.path.getsize(os.path.join(HERE, name)) // 1024, "KiB")


if __name__ == "__main__":
    sys.exit(main())
