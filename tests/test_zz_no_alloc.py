"""The allocation-free decode entry point against the regular one.

``b200_paged_decode_gqa_static`` is for hosts that cannot allocate device memory
while a step runs (an engine whose KV pool already owns all free HBM; a decode
loop that cannot absorb the synchronisation an allocation causes).  It keeps the
split-KV partial records in a fixed array inside the library, so its results
must equal those of ``b200_paged_decode_gqa`` with a caller workspace — also on
a second call, when the array still holds the first call's records.

This file sorts last on purpose: a run that stops at the first failure has then
already been through every other test."""
import ctypes

import pytest
import torch

from oracle import paged_attention_oracle as orc
from tests.parity import assert_attention_close

pytestmark = pytest.mark.gpu


def _call_static(lib, b, plan, out, lse=None):
    from auto_infer_b200 import ops
    k_cache, v_cache = b.kv_cache[0], b.kv_cache[1]
    return lib.b200_paged_decode_gqa_static(
        b.q.data_ptr(), b.q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
        k_cache.shape[0], k_cache.shape[1], b.block_table.data_ptr(), b.block_table.stride(0),
        plan.dev.data_ptr(), ctypes.byref(plan.info), b.n_q, b.n_kv, b.head_dim, float(b.scale),
        out.data_ptr(), 1 if out.dtype == torch.float32 else 0,
        lse.data_ptr() if lse is not None else None,
        ops.status_word("cuda").data_ptr(), torch.cuda.current_stream().cuda_stream)


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    from auto_infer_b200 import _lib, ops, synth
    lib = _lib.load()
    # two different batches, so the second call meets stale records of another shape
    batches = [
        synth.build_gqa_batch("noalloc_a", [(1, 3000), (2, 777), (1, 64), (1, 5000)], 32, 8, 128, 80, 41),
        synth.build_gqa_batch("noalloc_b", [(2, 1500), (1, 129)], 16, 8, 128, 16, 42),
    ]
    for cpu_batch in batches:
        b = cpu_batch.to("cuda")
        plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, "cuda")
        assert 0 < plan.info.num_partials <= 1024
        want_lse = torch.empty(b.num_tokens, b.n_q, dtype=torch.float32, device="cuda")
        want = ops.paged_decode_gqa(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, plan, b.scale,
                                    lse_out=want_lse)
        got = torch.full_like(want, float("nan"))
        got_lse = torch.empty_like(want_lse)
        if cpu_batch is batches[0]:
            # the documented start-up call: the first call on a device looks the array's address up
            assert _call_static(lib, b, plan, got, got_lse) == 0, lib.b200_last_error()
            got.fill_(float("nan"))
        torch.cuda.synchronize()
        # the call must not allocate or free device memory: neither through torch's
        # allocator nor behind its back (free memory as the driver reports it)
        torch_bytes = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
        free_before, _ = torch.cuda.mem_get_info()
        rc = _call_static(lib, b, plan, got, got_lse)
        assert rc == 0, lib.b200_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == torch_bytes
        # same kernels, same plan, same fixed merge order: equal bit for bit
        assert torch.equal(got, want)
        assert torch.equal(got_lse, want_lse)
        ref, ref_lse = orc.paged_attention(cpu_batch.q, cpu_batch.kv_cache[0], cpu_batch.kv_cache[1],
                                           cpu_batch.block_table, cpu_batch.cu_seqlens_q,
                                           cpu_batch.seqlens_kv, cpu_batch.scale, return_lse=True)
        assert_attention_close(got.cpu(), ref, got_lse.cpu(), ref_lse, cpu_batch.name)
        assert ops.read_status("cuda") == 0


def test_static_scratch_entry_refuses_oversized_plans():
    from auto_infer_b200 import _lib, ops, synth
    lib = _lib.load()
    b = synth.build_gqa_batch("noalloc_big", [(1, 65536)] * 2, 16, 8, 128, 1024, 43, device="cuda")
    plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, "cuda", num_ctas=3000)
    assert plan.info.num_partials > 1024
    out = torch.zeros(b.q.shape, dtype=torch.bfloat16, device="cuda")
    rc = _call_static(lib, b, plan, out)
    assert rc == -5
    assert b"1024" in lib.b200_last_error()
    torch.cuda.synchronize()
    assert out.abs().sum() == 0            # nothing was launched
