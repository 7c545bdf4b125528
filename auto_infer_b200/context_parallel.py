"""Context-parallel decode over the ``cp`` axis of the mesh.

Each rank holds a contiguous run of every sequence's KV pages (auto-infer's CP
convention is contiguous chunks per rank, auto_infer/models/qwen2.py:189-190)
in its own local pool with its own local block table.  A step is: local split-KV
attention producing an fp32 partial (o, lse) per query row, ONE all-gather of
the packed [o | lse] record per rank, then the log-sum-exp merge kernel on local
memory.  The reference's only CP code gathers K and V per layer instead
(qwen2.py:211-212: two collectives moving O(context) bytes); here the exchange
is T*Hq*(D+1) floats per rank whatever the context length."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import ops
from .metadata import StepMetadata


def pages_per_rank(kv_len: int, block_size: int, cp_size: int) -> int:
    """Pages each rank owns of a sequence of kv_len tokens (the last rank may
    own fewer, trailing ranks none)."""
    pages = (kv_len + block_size - 1) // block_size
    return (pages + cp_size - 1) // cp_size


def shard_lengths(seqlens_kv: Sequence[int], cu_seqlens_q: Sequence[int], block_size: int,
                  cp_rank: int, cp_size: int) -> Tuple[List[int], List[int], List[int]]:
    """Per sequence: (local kv length, global position of local key 0, causal
    base in local coordinates).  Key j (local) of sequence b is visible to its
    query row i iff j <= causal_base[b] + i, i.e. the bottom-right causal mask
    evaluated at global positions."""
    local, offsets, bases = [], [], []
    prev = 0
    for kv_len, end in zip(seqlens_kv, cu_seqlens_q):
        q_len = end - prev
        prev = end
        span = pages_per_rank(kv_len, block_size, cp_size) * block_size
        lo = min(cp_rank * span, kv_len)
        hi = min(lo + span, kv_len)
        local.append(hi - lo)
        offsets.append(lo)
        bases.append(kv_len - q_len - lo)
    return local, offsets, bases


def shard_block_table(block_table: torch.Tensor, seqlens_kv: Sequence[int], block_size: int,
                      cp_rank: int, cp_size: int) -> torch.Tensor:
    """Columns of a global logical block table that rank cp_rank owns, left
    aligned and zero padded (used when one host deals pages to all ranks)."""
    rows = []
    for b, kv_len in enumerate(seqlens_kv):
        ppr = pages_per_rank(kv_len, block_size, cp_size)
        pages = (kv_len + block_size - 1) // block_size
        lo = min(cp_rank * ppr, pages)
        hi = min(lo + ppr, pages)
        rows.append(block_table[b, lo:hi])
    width = max((r.numel() for r in rows), default=1)
    out = torch.zeros(len(rows), max(width, 1), dtype=block_table.dtype, device=block_table.device)
    for b, r in enumerate(rows):
        out[b, :r.numel()] = r
    return out


class PartialBuffer:
    """One rank's packed partial result: T*Hq*D floats of o followed by T*Hq
    floats of lse, so the exchange is a single collective."""

    def __init__(self, num_tokens: int, num_q_heads: int, head_dim: int, device):
        self.rows = num_tokens * num_q_heads
        self.head_dim = head_dim
        self.flat = torch.empty(self.rows * (head_dim + 1), dtype=torch.float32, device=device)
        self.o = self.flat[: self.rows * head_dim].view(num_tokens, num_q_heads, head_dim)
        self.lse = self.flat[self.rows * head_dim:].view(num_tokens, num_q_heads)

    def clear(self) -> None:
        """Every row reads as an empty part (the decode plan writes every row of its
        sequences itself, also those a rank has no keys for; this is for buffers filled
        by hand)."""
        self.o.zero_()
        self.lse.fill_(float("-inf"))


def all_gather_partials(flat: torch.Tensor, group=None) -> torch.Tensor:
    """(world, len(flat)) tensor holding every rank's packed record; one
    ``all_gather_into_tensor`` (NCCL over NVLink on GPUs, gloo in CPU tests)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return flat.unsqueeze(0)
    out = torch.empty(world, flat.numel(), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(out.view(-1), flat, group=group)
    return out


def split_gathered(gathered: torch.Tensor, rows: int, head_dim: int):
    """Views (R, rows, D) and (R, rows) into the gathered records."""
    o = gathered[:, : rows * head_dim].unflatten(1, (rows, head_dim))
    lse = gathered[:, rows * head_dim:]
    return o, lse


class PeerExchange:
    """Symmetric receive buffers for the fused exchange + merge kernel: one buffer
    per rank, mapped into every peer of the group (torch symmetric memory does
    the handle exchange), plus this rank's step counter.  Collective: all ranks
    of the group construct it together."""

    def __init__(self, rows: int, head_dim: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.rows, self.head_dim = rows, head_dim
        nbytes = _lib.load().b200_cp_exchange_buffer_bytes(self.world, rows, head_dim)
        self.buffer = symm_mem.empty(nbytes // 4, dtype=torch.float32, device=device)
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        self.buffer.zero_()
        self.state = torch.zeros(4, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)          # every flag word is zero before anyone pushes
        self.recv_ptrs_dev = int(self.handle.buffer_ptrs_dev)


class ContextParallelDecode:
    """Holds the plan and buffers of one CP rank and runs layer-steps.  Buffers and
    the plan's device address are fixed for the object's life: ``replan()`` refills
    them for the next step's lengths, so a step costs host planning and one small
    copy, and a CUDA graph recorded by ``capture()`` stays valid."""

    def __init__(self, cu_seqlens_q: Sequence[int], seqlens_kv_global: Sequence[int],
                 num_q_heads: int, num_kv_heads: int, head_dim: int, block_size: int, device,
                 group=None, cp_rank: Optional[int] = None, cp_size: Optional[int] = None,
                 exchange: Optional["PeerExchange"] = None, capacity_seqs: Optional[int] = None):
        self.group = group
        self.exchange = exchange          # None: NCCL all-gather + merge kernel
        if cp_size is None:
            cp_size = dist.get_world_size(group) if dist.is_initialized() else 1
        if cp_rank is None:
            cp_rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.cp_rank, self.cp_size = cp_rank, cp_size
        self.block_size = block_size
        self.local_kv, self.offsets, self.bases = shard_lengths(
            seqlens_kv_global, cu_seqlens_q, block_size, cp_rank, cp_size)
        self.meta = StepMetadata(cu_seqlens_q, self.local_kv, num_q_heads, num_kv_heads, head_dim,
                                 device, causal_base=self.bases,
                                 capacity_seqs=capacity_seqs or len(cu_seqlens_q))
        self.num_tokens = self.meta.num_tokens
        self.partial = PartialBuffer(self.num_tokens, num_q_heads, head_dim, device)
        self.out = torch.empty(self.num_tokens, num_q_heads, head_dim, dtype=torch.bfloat16,
                               device=device)

    def replan(self, cu_seqlens_q: Sequence[int], seqlens_kv_global: Sequence[int]) -> None:
        """Lengths of the next step (same number of query tokens): the local plan is
        refilled in place."""
        if (cu_seqlens_q[-1] if len(cu_seqlens_q) else 0) != self.num_tokens:
            raise ValueError("replan() keeps the step's token count; build a new object for another shape")
        self.local_kv, self.offsets, self.bases = shard_lengths(
            seqlens_kv_global, cu_seqlens_q, self.block_size, self.cp_rank, self.cp_size)
        self.meta.rebuild(cu_seqlens_q, self.local_kv, causal_base=self.bases)

    def capture(self, q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                local_block_table: torch.Tensor, scale: float, before=None):
        """Record one layer-step (optional ``before`` callable, e.g. the slot write,
        then local attention, all-gather and merge) into a CUDA graph over the
        given fixed-address tensors and return it; ``graph.replay()`` then runs
        the step without per-kernel host launches.  The step runs eagerly a few
        times first so that every lazy initialisation (kernel attributes, tensor
        maps, NCCL channels) happens outside the capture.  All ranks of the group
        must call this together."""
        def step():
            if before is not None:
                before()
            return self.attend(q, key_cache, value_cache, local_block_table, scale)

        side = torch.cuda.Stream(device=q.device)
        side.wait_stream(torch.cuda.current_stream(q.device))
        with torch.cuda.stream(side):
            for _ in range(3):
                step()
        torch.cuda.current_stream(q.device).wait_stream(side)
        torch.cuda.synchronize(q.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
        torch.cuda.synchronize(q.device)
        return graph

    def _local(self, q, key_cache, value_cache, local_block_table, scale, out, lse_out=None):
        """This rank's attention over its own pages: decode-shaped rows through the split-KV
        kernel, wide query blocks (prefill chunks) through the tensor-core kernel.  Both take
        the causal base in local coordinates and write zeros / lse = -inf for rows that see
        none of this rank's keys, so every row of ``out`` is written."""
        if self.meta.decode.info.num_items or self.meta.decode.replayable:
            ops.paged_decode_gqa(q, key_cache, value_cache, local_block_table, self.meta.decode, scale,
                                 out=out, lse_out=lse_out)
        if self.meta.prefill is not None:
            ops.paged_prefill_gqa(q, key_cache, value_cache, local_block_table, self.meta.prefill, scale,
                                  out=out, lse_out=lse_out)

    def attend(self, q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
               local_block_table: torch.Tensor, scale: float) -> torch.Tensor:
        """One layer-step: local attention -> exchange -> merge.  Returns the bf16
        (T, Hq, D) output, identical on every rank.  Handles decode rows, multi-token
        verify rows and prefill chunks alike: where the reference's context-parallel
        prefill all-gathers K and V per layer (auto_infer/models/qwen2.py:181-226), the
        ranks here exchange T*Hq*(D+1) floats whatever the context length."""
        if self.cp_size == 1:
            self._local(q, key_cache, value_cache, local_block_table, scale, self.out)
            return self.out
        self._local(q, key_cache, value_cache, local_block_table, scale, self.partial.o, self.partial.lse)
        if self.exchange is not None:
            # one kernel: peer-to-peer push of [o | lse], flag wait, merge
            ops.cp_exchange_combine(self.partial.flat, self.exchange.recv_ptrs_dev, self.exchange.state,
                                    self.cp_rank, self.cp_size, self.partial.rows, self.partial.head_dim,
                                    self.out.view(self.partial.rows, -1))
            return self.out
        gathered = all_gather_partials(self.partial.flat, self.group)
        o_parts, lse_parts = split_gathered(gathered, self.partial.rows, self.partial.head_dim)
        ops.lse_combine(o_parts, lse_parts, out=self.out.view(self.partial.rows, -1))
        return self.out
