"""Context-parallel decode on GPUs.  On one GPU the R ranks are emulated one after
the other (each with its own local block table and causal base) and their packed
[o | lse] records merged by the CUDA merge kernel; with two or more GPUs the
real NCCL path runs as child processes (NVLS off, plain all-gather)."""
import os
import sys

import pytest
import torch

from oracle import paged_attention_oracle as orc
from tests.parity import assert_attention_close

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("ranks", [2, 3, 8])
def test_emulated_ranks_merge_to_the_unsplit_answer(ranks):
    from auto_infer_b200 import context_parallel as cp, ops, synth
    # MTP-verify rows (q_len 2) make the mask depend on global positions; the short
    # sequence leaves trailing ranks without keys
    b = synth.build_gqa_batch("cp", [(2, 1500), (1, 129), (2, 4096), (1, 2)], 32, 8, 128, 64, 17)
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                                       b.seqlens_kv, b.scale, return_lse=True)
    d = b.to("cuda")
    rows = b.num_tokens * b.n_q
    gathered = torch.empty(ranks, rows * (b.head_dim + 1), dtype=torch.float32, device="cuda")
    for r in range(ranks):
        local_kv, off, base = cp.shard_lengths(b.seqlens_kv, b.cu_seqlens_q, 128, r, ranks)
        local_bt = cp.shard_block_table(d.block_table, b.seqlens_kv, 128, r, ranks)
        plan = ops.DecodePlan(b.cu_seqlens_q, local_kv, b.n_q, b.n_kv, "cuda", causal_base=base)
        buf = cp.PartialBuffer(b.num_tokens, b.n_q, b.head_dim, "cuda")
        buf.flat.fill_(float("nan"))       # rows a rank has no keys for are written too (zeros, lse -inf)
        ops.paged_decode_gqa(d.q, d.kv_cache[0], d.kv_cache[1], local_bt, plan, b.scale,
                             out=buf.o, lse_out=buf.lse)
        gathered[r].copy_(buf.flat)
    o_parts, lse_parts = cp.split_gathered(gathered, rows, b.head_dim)
    lse = torch.empty(rows, dtype=torch.float32, device="cuda")
    out = ops.lse_combine(o_parts, lse_parts, lse_out=lse)
    assert_attention_close(out.view_as(ref).cpu(), ref, lse.view_as(ref_lse).cpu(), ref_lse,
                           f"{ranks} emulated ranks")
    assert ops.read_status("cuda") == 0


@pytest.mark.parametrize("ranks", [2, 4])
def test_emulated_ranks_with_prefill_chunks(ranks):
    """Context-parallel chunked prefill: every rank runs the wide-query kernel over its own
    slice of the keys (a chunk of 150 tokens over a 300-token prefix, a whole 200-token prompt,
    beside a decode row) and the partials merge to the unsplit answer - where the reference's
    context-parallel prefill gathers all K and V on every rank (auto_infer/models/qwen2.py:181-226).
    Rows that see none of a rank's keys come out as an empty part."""
    from auto_infer_b200 import context_parallel as cp, ops, synth
    b = synth.build_gqa_batch("cp_prefill", [(150, 450), (1, 700), (200, 200)], 16, 4, 128, 24, 19)
    ref, ref_lse = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                                       b.seqlens_kv, b.scale, return_lse=True)
    d = b.to("cuda")
    rows = b.num_tokens * b.n_q
    gathered = torch.empty(ranks, rows * (b.head_dim + 1), dtype=torch.float32, device="cuda")
    for r in range(ranks):
        local_bt = cp.shard_block_table(d.block_table, b.seqlens_kv, 128, r, ranks)
        step = cp.ContextParallelDecode(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, b.head_dim, 128, "cuda",
                                        cp_rank=r, cp_size=ranks)
        assert step.meta.prefill is not None
        step.partial.flat.fill_(float("nan"))
        step._local(d.q, d.kv_cache[0], d.kv_cache[1], local_bt, b.scale, step.partial.o, step.partial.lse)
        gathered[r].copy_(step.partial.flat)
    assert torch.isfinite(gathered[:, : rows * b.head_dim]).all()
    o_parts, lse_parts = cp.split_gathered(gathered, rows, b.head_dim)
    lse = torch.empty(rows, dtype=torch.float32, device="cuda")
    out = ops.lse_combine(o_parts, lse_parts, lse_out=lse)
    assert_attention_close(out.view_as(ref).cpu(), ref, lse.view_as(ref_lse).cpu(), ref_lse,
                           f"{ranks} emulated ranks, prefill chunks")
    assert ops.read_status("cuda") == 0


def test_exchange_wait_for_an_absent_peer_runs_out_and_the_next_step_works():
    """The fused exchange waits for its peers with a limit.  Two 'ranks' share this GPU, each
    with its own receive buffer and step counter, and run one after the other, so the first
    caller of a step never finds its peer's flag: its wait runs out (20 ms here), it reports
    B200_STATUS_WAIT_TIMEOUT and leaves `out` alone, and the context stays usable.  The rank
    that calls second finds both records and merges them."""
    from auto_infer_b200 import _lib, ops
    lib = _lib.load()
    rows, dim, world = 40, 128, 2
    g = torch.Generator().manual_seed(5)
    nfloats = lib.b200_cp_exchange_buffer_bytes(world, rows, dim) // 4
    bufs = [torch.zeros(nfloats, dtype=torch.float32, device="cuda") for _ in range(world)]
    ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda")
    states = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(world)]
    limit_ns = 20_000_000

    def record(step, rank):
        o = torch.randn(rows, dim, generator=g)
        lse = torch.randn(rows, generator=g) * 3
        return torch.cat([o.reshape(-1), lse]).cuda(), o, lse

    def call(rank, rec, out):
        return ops.cp_exchange_combine(rec, ptrs.data_ptr(), states[rank], rank, world, rows, dim, out,
                                       wait_limit_ns=limit_ns)

    ops.read_status("cuda")
    for step in range(2):                      # both receive slots
        recs = [record(step, r) for r in range(world)]
        want, _ = orc.lse_combine(torch.stack([recs[0][1], recs[1][1]]), torch.stack([recs[0][2], recs[1][2]]),
                                  out_dtype=torch.float32)
        first, second = (0, 1) if step == 0 else (1, 0)
        out_first = torch.full((rows, dim), 7.0, dtype=torch.float32, device="cuda")
        call(first, recs[first][0], out_first)
        torch.cuda.synchronize()
        assert ops.read_status("cuda") == _lib.STATUS_WAIT_TIMEOUT
        assert torch.equal(out_first, torch.full_like(out_first, 7.0))        # nothing merged, nothing written
        out_second = torch.zeros(rows, dim, dtype=torch.float32, device="cuda")
        call(second, recs[second][0], out_second)
        torch.cuda.synchronize()
        assert ops.read_status("cuda") == 0
        # the partial rows cross the link as bf16 (their log-sum-exp as fp32)
        torch.testing.assert_close(out_second.cpu(), want, atol=2e-2, rtol=2e-2)
    assert [int(s[0]) for s in states] == [2, 2]                              # both ranks are at step 2


def _nccl_worker(rank, world, port, ret, use_p2p=False):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from auto_infer_b200 import context_parallel as cp, synth
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        b = synth.build_gqa_batch("cp", [(1, 3000), (2, 700), (1, 130), (70, 400)], 16, 8, 128, 40, 23)
        d = b.to(f"cuda:{rank}")
        local_bt = cp.shard_block_table(d.block_table, b.seqlens_kv, 128, rank, world)
        exchange = cp.PeerExchange(b.num_tokens * b.n_q, b.head_dim, f"cuda:{rank}") if use_p2p else None
        step = cp.ContextParallelDecode(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, b.head_dim, 128,
                                        f"cuda:{rank}", cp_rank=rank, cp_size=world, exchange=exchange)
        ref = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q,
                                  b.seqlens_kv, b.scale)
        # the ranks reach this point at different times (the oracle above runs on the host):
        # line them up before the first exchange, whose wait for the peers is bounded
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(3):            # several steps: the step counter and both slots are exercised
            out = step.attend(d.q, d.kv_cache[0], d.kv_cache[1], local_bt, b.scale)
            assert_attention_close(out.cpu(), ref, what=f"rank {rank} of {world}")
        from auto_infer_b200 import ops
        assert ops.read_status(f"cuda:{rank}") == 0
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gpu_nccl_all_gather_and_merge():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 29600 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_nccl_worker, args=(2, port, ret), nprocs=2, join=True)
        assert dict(ret) == {0: "ok", 1: "ok"}


@pytest.mark.timeout(300)
def test_two_gpu_fused_peer_exchange_and_merge():
    """Same answer through the fused peer-to-peer exchange + merge kernel."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 29700 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_nccl_worker, args=(2, port, ret, True), nprocs=2, join=True)
        assert dict(ret) == {0: "ok", 1: "ok"}
