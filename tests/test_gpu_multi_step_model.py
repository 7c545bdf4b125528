"""A two-layer GQA model driven for a prefill step and a run of decode steps through
``B200GqaBackend.attention()`` with a growing paged cache, against a dense recompute of the
whole sequence on the CPU at every step - the shape of the reference's own parity gate
(tools/parity.py:46-68: paged engine vs eager recompute, argmax equality), in miniature and with
random weights.  What it adds to the single-step tests: the cache a step reads was written by
the kernels of earlier steps, through changing block tables and slot mappings."""
import pytest
import torch

from oracle import paged_attention_oracle as orc

pytestmark = pytest.mark.gpu

HIDDEN, N_Q, N_KV, HD, LAYERS, VOCAB, BS = 256, 4, 2, 128, 2, 97, 16


def _weights(g):
    def rnd(*shape, s):
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)
    w = {"embed": rnd(VOCAB, HIDDEN, s=1.0), "lm_head": rnd(VOCAB, HIDDEN, s=0.1)}
    for i in range(LAYERS):
        p = f"model.layers.{i}.self_attn."
        w[p + "qkv_proj.weight"] = rnd((N_Q + 2 * N_KV) * HD, HIDDEN, s=0.08)
        w[p + "qkv_proj.bias"] = rnd((N_Q + 2 * N_KV) * HD, s=0.05)
        w[p + "o_proj.weight"] = rnd(HIDDEN, N_Q * HD, s=0.05)
        w[p + "q_norm.weight"] = (torch.rand(HD, generator=g) + 0.5).to(torch.bfloat16)
        w[p + "k_norm.weight"] = (torch.rand(HD, generator=g) + 0.5).to(torch.bfloat16)
    return w


def _rope(positions):
    inv = 1.0 / (10000.0 ** (torch.arange(0, HD, 2, dtype=torch.float32) / HD))
    ang = torch.tensor(positions, dtype=torch.float32)[:, None] * inv[None]
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos()[:, None, :].to(torch.bfloat16), ang.sin()[:, None, :].to(torch.bfloat16)


def _dense_logits(w, tokens):
    """Eager recompute of one whole sequence (no cache): last-position logits."""
    t = len(tokens)
    x = w["embed"][torch.tensor(tokens)]
    cos, sin = _rope(list(range(t)))
    for i in range(LAYERS):
        cache = torch.zeros(2, (t + BS - 1) // BS, BS, N_KV, HD, dtype=torch.bfloat16)
        bt = torch.arange(cache.shape[1], dtype=torch.int32)[None]
        x = x + orc.gqa_attention_block(x, w, f"model.layers.{i}.", N_Q, N_KV, HD, HD ** -0.5, cos, sin, cache,
                                        list(range(t)), bt, [t], [t], rms_eps=1e-6)
    return (x[-1:].float() @ w["lm_head"].float().t())[0]


def test_prefill_then_decode_steps_follow_the_dense_recompute():
    from auto_infer_b200 import ops
    from auto_infer_b200.forward_context import ForwardContext
    from auto_infer_b200.gqa import B200GqaBackend
    g = torch.Generator().manual_seed(123)
    w = _weights(g)
    wd = {k: v.cuda() for k, v in w.items()}
    backend = B200GqaBackend(N_Q, N_KV, HD, HD ** -0.5, LAYERS, "cuda", torch.bfloat16, w=wd, rms_eps=1e-6)
    num_blocks = 24
    caches = backend.alloc_kv_caches(num_blocks, BS)
    free = torch.randperm(num_blocks, generator=g).tolist()
    # two requests with prompts of different lengths, decoded together
    seqs = [torch.randint(0, VOCAB, (n,), generator=g).tolist() for n in (21, 37)]
    blocks = [[], []]

    def ensure(b, length):
        while len(blocks[b]) * BS < length:
            blocks[b].append(free.pop())

    def forward(rows):
        """rows: per request the positions computed this step.  Returns last-row logits per request."""
        tok, pos, slots, cu, kv, acc = [], [], [], [], [], 0
        for b, positions in enumerate(rows):
            ensure(b, positions[-1] + 1)
            for p_ in positions:
                tok.append(seqs[b][p_])
                pos.append(p_)
                slots.append(blocks[b][p_ // BS] * BS + p_ % BS)
            acc += len(positions)
            cu.append(acc)
            kv.append(positions[-1] + 1)
        width = max(len(r) for r in blocks)
        bt = torch.zeros(len(rows), width, dtype=torch.int32)
        for b, r in enumerate(blocks):
            bt[b, :len(r)] = torch.tensor(r, dtype=torch.int32)
        cos, sin = _rope(pos)
        ctx = ForwardContext(None, None, torch.tensor(slots, dtype=torch.int32).cuda(), bt.cuda(), cu, kv, None,
                             backend, caches, False, cos=cos.cuda(), sin=sin.cuda())
        x = wd["embed"][torch.tensor(tok).cuda()]
        for i in range(LAYERS):
            x = x + backend.attention(i, x, ctx)
        last = torch.tensor([c - 1 for c in cu]).cuda()
        return (x[last].float() @ wd["lm_head"].float().t()).cpu()

    # prefill (wide-query kernel), then 12 decode steps (split-KV kernel, pooled refilled plan)
    logits = forward([list(range(len(s))) for s in seqs])
    for step in range(13):
        for b in range(2):
            want = _dense_logits(w, seqs[b])
            torch.testing.assert_close(logits[b], want, atol=6e-2, rtol=6e-2)
            # greedy continuation must agree wherever the dense top-2 margin is not a rounding matter
            top = torch.topk(want, 2).values
            if float(top[0] - top[1]) > 0.15:
                assert int(logits[b].argmax()) == int(want.argmax()), f"step {step}, request {b}"
            seqs[b].append(int(want.argmax()))
        if step < 12:
            logits = forward([[len(s) - 1] for s in seqs])
    assert ops.read_status("cuda") == 0
