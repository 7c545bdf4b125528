"""Graph mode on the GPU: ONE decode step is recorded into a CUDA graph and replayed for
other length sets without recapture, the way the reference's graph runners drive a gear
(auto_infer/worker/graph_decode_runner.py ``_capture`` / ``_prepare_graph``): static
per-gear buffers staged in place, padding rows on scratch blocks with kv_len 1
(auto_infer/worker/decode_input_stager.py:74-123), ``backend.update(ctx)`` with the step's
lengths, ``graph.replay()``.  Every replay must equal the oracle."""
from types import SimpleNamespace

import pytest
import torch

from oracle import paged_attention_oracle as orc
from tests.parity import assert_attention_close

pytestmark = pytest.mark.gpu

BS, GEAR, MAX_BLOCKS, NUM_BLOCKS, N_Q, N_KV, HD = 16, 4, 24, 64, 8, 2, 128
SCRATCH0 = NUM_BLOCKS                      # scratch blocks sit on top of the pool the engine hands out


def _stage(requests):
    """The reference stager's arithmetic for a decode gear: live rows first, then padding rows
    on their own scratch block.  requests: (position of the new token, block ids)."""
    slots, kv_lens = [], []
    bt = torch.zeros(GEAR, MAX_BLOCKS, dtype=torch.int32)
    for row, (pos, blocks) in enumerate(requests):
        slots.append(blocks[pos // BS] * BS + pos % BS)
        bt[row, :len(blocks)] = torch.tensor(blocks, dtype=torch.int32)
        kv_lens.append(pos + 1)
    for row in range(len(requests), GEAR):
        block = SCRATCH0 + row
        slots.append(block * BS)
        bt[row, 0] = block
        kv_lens.append(1)
    return torch.tensor(slots, dtype=torch.int32), bt, kv_lens


def test_one_captured_decode_step_replays_for_other_lengths():
    from auto_infer_b200 import ops, registry
    from auto_infer_b200.forward_context import ForwardContext
    from auto_infer_b200.gqa import B200GraphGqaBackend
    dev = torch.device("cuda")
    cfg = SimpleNamespace(head_dim=HD, num_layers=2, rms_eps=1e-6)
    model = SimpleNamespace(cfg=cfg, n_q_local=N_Q, n_kv_local=N_KV, w={}, layer_prefix=lambda i: f"model.layers.{i}.",
                            device=dev, dtype=torch.bfloat16, ATTENTION_FAMILY="gqa")
    backend, caches = registry.build_attention_backend(model, "graph", NUM_BLOCKS + GEAR, BS)
    assert isinstance(backend, B200GraphGqaBackend)
    g = torch.Generator().manual_seed(2024)
    for kc, vc in caches:                                   # a cache with history in every block
        kc.copy_(torch.randn(kc.shape, generator=g).to(torch.bfloat16))
        vc.copy_(torch.randn(vc.shape, generator=g).to(torch.bfloat16))

    # the gear's static buffers (what a captured graph is recorded against)
    q = torch.zeros(GEAR, N_Q, HD, dtype=torch.bfloat16, device=dev)
    k_new = torch.zeros(GEAR, N_KV, HD, dtype=torch.bfloat16, device=dev)
    v_new = torch.zeros(GEAR, N_KV, HD, dtype=torch.bfloat16, device=dev)
    slots = torch.zeros(GEAR, dtype=torch.int32, device=dev)
    block_table = torch.zeros(GEAR, MAX_BLOCKS, dtype=torch.int32, device=dev)
    cu_q = list(range(1, GEAR + 1))

    def ctx_for(kv_lens):
        return ForwardContext(None, None, slots, block_table, cu_q, kv_lens, None, backend, caches, True)

    def step(ctx):
        return [backend.paged_attention(layer, q, k_new, v_new, ctx) for layer in range(cfg.num_layers)]

    # capture on scratch rows only, as the reference does (kv_len 1 everywhere)
    s0, bt0, kv0 = _stage([])
    slots.copy_(s0)
    block_table.copy_(bt0)
    ctx = ctx_for(kv0)
    backend.capturing = False
    step(ctx)                                               # warm-up: plan buffers come to life here
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    backend.begin_capture()
    with torch.cuda.graph(graph):
        outs = step(ctx)
    backend.end_capture()
    gear_reg = backend.reg
    assert len(gear_reg) == cfg.num_layers and gear_reg[0].meta is gear_reg[1].meta

    perm = torch.randperm(NUM_BLOCKS, generator=g).tolist()
    length_sets = [
        [(5, perm[0:1]), (17, perm[1:3])],                                     # two live rows, two padding rows
        [(0, perm[3:4]), (300, perm[4:23]), (63, perm[23:27]), (16, perm[27:29])],   # full gear, long and short
        [(BS * MAX_BLOCKS - 1, perm[29:29 + MAX_BLOCKS])],                     # one row at the longest length
    ]
    for requests in length_sets:
        s_h, bt_h, kv_lens = _stage(requests)
        q_h = torch.randn(GEAR, N_Q, HD, generator=g).to(torch.bfloat16)
        k_h = torch.randn(GEAR, N_KV, HD, generator=g).to(torch.bfloat16)
        v_h = torch.randn(GEAR, N_KV, HD, generator=g).to(torch.bfloat16)
        for dst, src in ((q, q_h), (k_new, k_h), (v_new, v_h), (slots, s_h), (block_table, bt_h)):
            dst.copy_(src)
        # an eager step of another shape in between must not disturb the captured plan
        other = ForwardContext(None, None, slots[:1], block_table[:1], [1], [kv_lens[0]], None, backend, caches, True)
        ref_caches = [(kc.cpu().clone(), vc.cpu().clone()) for kc, vc in caches]
        backend.paged_attention(0, q[:1], k_new[:1], v_new[:1], other)
        backend.update_registrations(gear_reg, ctx_for(kv_lens))
        graph.replay()
        torch.cuda.synchronize()
        assert ops.read_status(dev) == 0
        live = len(requests)
        for layer in range(cfg.num_layers):
            kc, vc = ref_caches[layer]
            orc.write_kv(k_h, v_h, kc, vc, s_h.tolist())
            assert torch.equal(caches[layer][0].cpu(), kc) and torch.equal(caches[layer][1].cpu(), vc)
            ref, _ = orc.paged_attention(q_h, kc, vc, bt_h, cu_q, kv_lens, HD ** -0.5, return_lse=True)
            got = outs[layer].cpu()
            assert_attention_close(got[:live], ref[:live], what=f"layer {layer}, lengths {kv_lens}")
            assert torch.isfinite(got.float()).all()                          # padding rows: discarded, but sane
            assert_attention_close(got[live:], ref[live:], what="padding rows")


def test_one_captured_prefill_gear_replays_for_other_splits_of_its_tokens():
    """A prefill gear: a step of 48 query tokens recorded once (slot write, split-KV kernel for
    the narrow rows, wide-query kernel for the chunks) and replayed for other splits of the 48
    tokens into sequences - one chunk, two chunks over cached prefixes, decode rows beside a
    chunk, and a step without any wide row (the recorded wide-query launch then finds no item)."""
    from auto_infer_b200 import ops, registry
    from auto_infer_b200.forward_context import ForwardContext
    dev = torch.device("cuda")
    tokens, max_seqs = 48, 12
    cfg = SimpleNamespace(head_dim=HD, num_layers=1, rms_eps=1e-6)
    model = SimpleNamespace(cfg=cfg, n_q_local=N_Q, n_kv_local=N_KV, w={}, layer_prefix=lambda i: f"model.layers.{i}.",
                            device=dev, dtype=torch.bfloat16, ATTENTION_FAMILY="gqa")
    backend, caches = registry.build_attention_backend(model, "graph", NUM_BLOCKS, BS)
    assert backend.supports_prefill_graph
    g = torch.Generator().manual_seed(77)
    for kc, vc in caches:
        kc.copy_(torch.randn(kc.shape, generator=g).to(torch.bfloat16))
        vc.copy_(torch.randn(vc.shape, generator=g).to(torch.bfloat16))
    q = torch.zeros(tokens, N_Q, HD, dtype=torch.bfloat16, device=dev)
    k_new = torch.zeros(tokens, N_KV, HD, dtype=torch.bfloat16, device=dev)
    v_new = torch.zeros(tokens, N_KV, HD, dtype=torch.bfloat16, device=dev)
    slots = torch.zeros(tokens, dtype=torch.int32, device=dev)
    block_table = torch.zeros(max_seqs, MAX_BLOCKS, dtype=torch.int32, device=dev)
    perm = torch.randperm(NUM_BLOCKS, generator=g).tolist()

    def stage(seqs):
        """seqs: (q_len, kv_len) per sequence, kv_len including the q_len new tokens; the gear's
        unused sequence rows are left without query tokens."""
        assert sum(q_len for q_len, _ in seqs) == tokens
        bt = torch.zeros(max_seqs, MAX_BLOCKS, dtype=torch.int32)
        s_list, cu, kv, acc, cursor = [], [], [], 0, 0
        for b in range(max_seqs):
            q_len, kv_len = seqs[b] if b < len(seqs) else (0, 0)
            need = (kv_len + BS - 1) // BS
            row = perm[cursor:cursor + need]
            cursor += need
            bt[b, :need] = torch.tensor(row, dtype=torch.int32)
            for pos in range(kv_len - q_len, kv_len):
                s_list.append(row[pos // BS] * BS + pos % BS)
            acc += q_len
            cu.append(acc)
            kv.append(kv_len)
        return torch.tensor(s_list, dtype=torch.int32), bt, cu, kv

    def ctx_for(cu, kv):
        return ForwardContext(None, None, slots, block_table, cu, kv, None, backend, caches, False)

    s0, bt0, cu0, kv0 = stage([(48, 48)])                      # captured on one 48-token prompt
    slots.copy_(s0)
    block_table.copy_(bt0)
    ctx = ctx_for(cu0, kv0)
    backend.paged_attention(0, q, k_new, v_new, ctx)           # warm-up
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    backend.begin_capture()
    with torch.cuda.graph(graph):
        out = backend.paged_attention(0, q, k_new, v_new, ctx)
    backend.end_capture()
    gear_reg = backend.reg
    assert gear_reg[0].meta.prefill is not None and gear_reg[0].meta.prefill.replayable

    splits = [
        [(48, 48)],                                            # as captured
        [(30, 130), (18, 18)],                                 # two chunks, one over a cached prefix
        [(1, 90), (1, 17), (2, 40), (44, 44 + 64)],            # decode rows and a verify pair beside a chunk
        [(8, 40)] * 6,                                         # six short chunks
        [(4, 20), (4, 36), (4, 52), (4, 68), (4, 84), (28, 28)],
        [(4, 20 + 8 * i) for i in range(12)],                  # narrow rows only: the wide-query launch finds no item
    ]
    for seqs in splits:
        s_h, bt_h, cu, kv = stage(seqs)
        q_h = torch.randn(tokens, N_Q, HD, generator=g).to(torch.bfloat16)
        k_h = torch.randn(tokens, N_KV, HD, generator=g).to(torch.bfloat16)
        v_h = torch.randn(tokens, N_KV, HD, generator=g).to(torch.bfloat16)
        for dst, src in ((q, q_h), (k_new, k_h), (v_new, v_h), (slots, s_h), (block_table, bt_h)):
            dst.copy_(src)
        kc, vc = caches[0][0].cpu().clone(), caches[0][1].cpu().clone()
        backend.update_registrations(gear_reg, ctx_for(cu, kv))
        graph.replay()
        torch.cuda.synchronize()
        assert ops.read_status(dev) == 0
        orc.write_kv(k_h, v_h, kc, vc, s_h.tolist())
        assert torch.equal(caches[0][0].cpu(), kc) and torch.equal(caches[0][1].cpu(), vc)
        ref = orc.paged_attention(q_h, kc, vc, bt_h, cu, kv, HD ** -0.5)
        assert_attention_close(out.cpu(), ref, what=f"split {seqs}")
    assert gear_reg[0].meta.prefill.info.num_items == 0       # the last split had no wide row


def test_capture_without_a_warm_up_step_is_refused():
    from auto_infer_b200.forward_context import ForwardContext
    from auto_infer_b200.gqa import B200GraphGqaBackend
    dev = torch.device("cuda")
    backend = B200GraphGqaBackend(N_Q, N_KV, HD, HD ** -0.5, 1, dev, torch.bfloat16)
    caches = backend.alloc_kv_caches(8, BS)
    q = torch.zeros(1, N_Q, HD, dtype=torch.bfloat16, device=dev)
    ctx = ForwardContext(None, None, torch.zeros(1, dtype=torch.int32, device=dev),
                         torch.zeros(1, 4, dtype=torch.int32, device=dev), [1], [1], None, backend, caches, True)
    backend.begin_capture()
    with pytest.raises(RuntimeError, match="one eager step with the same context first"):
        backend._attn(0, q, None, None, ctx)
    backend.end_capture()


def test_mla_decode_gear_replays_for_other_lengths():
    """The absorbed-MLA family in mode "graph": latent write + latent attention of a decode
    gear recorded once, replayed after ``update_registrations`` for other length sets
    (sequences cut over several CTAs included), every replay against the oracle."""
    from auto_infer_b200 import ops, registry
    from auto_infer_b200.forward_context import ForwardContext
    from auto_infer_b200.mla import B200GraphMlaBackend
    dev = torch.device("cuda")
    heads, bs, gear, max_blocks, pool = 16, 16, 4, 80, 200
    cfg = SimpleNamespace(num_heads=heads, qk_nope=128, qk_rope=64, v_head_dim=128, kv_lora_rank=512,
                          q_lora_rank=None, rms_eps=1e-6, num_layers=2)
    model = SimpleNamespace(cfg=cfg, w={}, layer_prefix=lambda i: f"model.layers.{i}.", device=dev,
                            dtype=torch.bfloat16, _softmax_scale=192 ** -0.5, _mla_absorb=False,
                            ATTENTION_FAMILY="mla")
    backend, caches = registry.build_attention_backend(model, "graph", pool + gear, bs)
    assert isinstance(backend, B200GraphMlaBackend) and not backend.supports_prefill_graph
    g = torch.Generator().manual_seed(77)
    for latent, _ in caches:
        latent.copy_(torch.randn(latent.shape, generator=g).to(torch.bfloat16))

    q = torch.zeros(gear, heads, 576, dtype=torch.bfloat16, device=dev)
    k_new = torch.zeros(gear, 1, 576, dtype=torch.bfloat16, device=dev)
    slots = torch.zeros(gear, dtype=torch.int32, device=dev)
    block_table = torch.zeros(gear, max_blocks, dtype=torch.int32, device=dev)
    cu_q = list(range(1, gear + 1))

    def stage(requests):
        s, kv = [], []
        bt = torch.zeros(gear, max_blocks, dtype=torch.int32)
        for row, (pos, blocks) in enumerate(requests):
            s.append(blocks[pos // bs] * bs + pos % bs)
            bt[row, :len(blocks)] = torch.tensor(blocks, dtype=torch.int32)
            kv.append(pos + 1)
        for row in range(len(requests), gear):                 # padding rows on scratch blocks
            s.append((pool + row) * bs)
            bt[row, 0] = pool + row
            kv.append(1)
        return torch.tensor(s, dtype=torch.int32), bt, kv

    def ctx_for(kv_lens):
        return ForwardContext(None, None, slots, block_table, cu_q, kv_lens, None, backend, caches, True)

    def step(ctx):
        return [backend.latent_attention(layer, q, k_new, ctx) for layer in range(cfg.num_layers)]

    s0, bt0, kv0 = stage([])
    slots.copy_(s0)
    block_table.copy_(bt0)
    ctx = ctx_for(kv0)
    with pytest.raises(RuntimeError):                           # no warm-up step yet
        backend.begin_capture()
        try:
            step(ctx_for(kv0))
        finally:
            backend.end_capture()
    step(ctx)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    backend.begin_capture()
    with torch.cuda.graph(graph):
        outs = step(ctx)
    backend.end_capture()
    gear_reg = backend.reg
    assert len(gear_reg) == cfg.num_layers and gear_reg[0].plan is gear_reg[1].plan

    perm = torch.randperm(pool, generator=g).tolist()
    length_sets = [
        [(5, perm[0:1]), (40, perm[1:4])],
        [(0, perm[4:5]), (1200, perm[5:81]), (63, perm[81:85]), (16, perm[85:87])],
        [(bs * max_blocks - 1, perm[87:87 + max_blocks])],
    ]
    for requests in length_sets:
        s_h, bt_h, kv_lens = stage(requests)
        q_h = torch.randn(gear, heads, 576, generator=g).to(torch.bfloat16)
        k_h = torch.randn(gear, 1, 576, generator=g).to(torch.bfloat16)
        for dst, src in ((q, q_h), (k_new, k_h), (slots, s_h), (block_table, bt_h)):
            dst.copy_(src)
        ref_caches = [latent.cpu().clone() for latent, _ in caches]
        # an eager step of another batch size in between must not disturb the captured plan
        other = ForwardContext(None, None, slots[:1], block_table[:1], [1], [kv_lens[0]], None, backend, caches, True)
        backend._latent_attn(0, q[:1], other)
        backend.update_registrations(gear_reg, ctx_for(kv_lens))
        graph.replay()
        torch.cuda.synchronize()
        assert ops.read_status(dev) == 0
        live = len(requests)
        for layer in range(cfg.num_layers):
            lat = ref_caches[layer]
            orc.write_kv(k_h, None, lat, None, s_h.tolist())
            assert torch.equal(caches[layer][0].cpu(), lat)
            ref, _ = orc.paged_attention(q_h, lat, lat, bt_h, cu_q, kv_lens, 192 ** -0.5, return_lse=True)
            assert_attention_close(outs[layer].cpu()[:live], ref[:live, :, :512], what=f"layer {layer}")
    with pytest.raises(ValueError):                             # a wider query block needs an eager step
        backend.update_registrations(gear_reg, ForwardContext(None, None, slots, block_table, [2, 3, 4, 5],
                                                              [9, 9, 9, 9], None, backend, caches, False))
