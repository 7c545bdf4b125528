"""Host logic of the context-parallel path on CPU: page sharding, local causal
bases, and the one all-gather among real gloo ranks (world size 2).  The CUDA
kernels are not involved: each rank's partial comes from the oracle and the
merged answer must equal the unsplit oracle."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from auto_infer_b200 import context_parallel as cp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_lengths_cover_every_key_once():
    kv = [1, 127, 128, 129, 1000, 131072]
    cu = [1, 2, 4, 5, 6, 7]
    for size in (1, 2, 3, 8):
        total = [0] * len(kv)
        for r in range(size):
            local, off, base = cp.shard_lengths(kv, cu, 128, r, size)
            prev = 0
            for b in range(len(kv)):
                q_len = cu[b] - prev
                prev = cu[b]
                assert 0 <= local[b] <= kv[b] and off[b] + local[b] <= kv[b]
                assert base[b] == kv[b] - q_len - off[b]
                assert off[b] % 128 == 0 or local[b] == 0
                total[b] += local[b]
        assert total == kv


def test_shard_block_table_is_a_contiguous_page_run():
    bt = torch.arange(1, 25, dtype=torch.int32).view(2, 12)
    kv = [12 * 128, 5 * 128 + 3]
    parts = [cp.shard_block_table(bt, kv, 128, r, 4) for r in range(4)]
    assert torch.equal(torch.cat([p[0, :3] for p in parts]), bt[0])
    assert parts[0][1, :2].tolist() == bt[1, :2].tolist()
    assert parts[2][1, :2].tolist() == bt[1, 4:6].tolist()
    assert parts[3][1].abs().sum() == 0          # nothing left for the last rank


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    from oracle import paged_attention_oracle as orc
    from auto_infer_b200 import synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        # MTP-verify shaped rows so the mask crosses rank boundaries
        b = synth.build_gqa_batch("cp", [(2, 300), (1, 129), (2, 2), (1, 700)], 8, 2, 128, 80, 31,
                                  block_size=16)
        local, off, base = cp.shard_lengths(b.seqlens_kv, b.cu_seqlens_q, 16, rank, world)
        ranges = [(o, o + l) for o, l in zip(off, local)]
        o, lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table,
                                     b.cu_seqlens_q, b.seqlens_kv, b.scale, return_lse=True,
                                     kv_ranges=ranges)
        buf = cp.PartialBuffer(b.num_tokens, b.n_q, b.head_dim, "cpu")
        buf.clear()
        buf.o.copy_(o.float())
        buf.lse.copy_(lse)
        gathered = cp.all_gather_partials(buf.flat)
        assert gathered.shape == (world, buf.flat.numel())
        o_parts, lse_parts = cp.split_gathered(gathered, buf.rows, buf.head_dim)
        merged, _ = orc.lse_combine(o_parts, lse_parts)
        full = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table,
                                   b.cu_seqlens_q, b.seqlens_kv, b.scale)
        torch.testing.assert_close(merged.view_as(full).float(), full.float(), atol=2e-2, rtol=2e-2)
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_gloo_ranks_gather_and_merge():
    port = 29500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
        assert dict(ret) == {0: "ok", 1: "ok"}
