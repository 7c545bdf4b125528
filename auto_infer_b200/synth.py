"""Seeded synthetic workloads with the shapes of the five benchmark
configurations (Qwen3-0.6B decode, Qwen3-8B mixed prefill+decode, DeepSeek-style
absorbed-MLA decode, MiMo MTP verify, Qwen2.5-72B 128K context-parallel decode).
They stand in for serving traffic: lengths are drawn uniformly from the stated
ranges, block tables are a seeded permutation of the physical pool dealt out
consecutively, Q/K/V and the cache contents are N(0, 1).

Shared by the tests, the smoke entry point and the benchmark so that the CUDA
path and the CPU checker always see the same bytes."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

BLOCK_SIZE = 128
SEED_BASE = 20260


@dataclass
class PagedBatch:
    """One step's attention inputs in the reference's ForwardContext layout
    (auto_infer/forward_context.py:9-23): packed TND queries, the step's new
    K/V rows, flat slots, zero-padded block table, cumulative query lengths and
    per-sequence kv lengths that include the step's own tokens."""
    name: str
    n_q: int
    n_kv: int
    head_dim: int
    block_size: int
    scale: float
    q: torch.Tensor                      # (T, Hq, D)
    k_new: torch.Tensor                  # (T, Hkv, D)
    v_new: Optional[torch.Tensor]        # (T, Hkv, Dv) or None (latent cache)
    kv_cache: torch.Tensor               # (2, P, bs, Hkv, D)  or (P, bs, 1, 576) for the latent
    block_table: torch.Tensor            # (B, max_blocks) int32
    slot_mapping: torch.Tensor           # (T,) int32
    cu_seqlens_q: List[int]
    seqlens_kv: List[int]
    extra: dict = field(default_factory=dict)

    @property
    def num_tokens(self) -> int:
        return self.cu_seqlens_q[-1] if self.cu_seqlens_q else 0

    def to(self, device) -> "PagedBatch":
        def mv(x):
            return x.to(device) if isinstance(x, torch.Tensor) else x
        return PagedBatch(self.name, self.n_q, self.n_kv, self.head_dim, self.block_size, self.scale,
                          mv(self.q), mv(self.k_new), mv(self.v_new), mv(self.kv_cache),
                          mv(self.block_table), mv(self.slot_mapping), list(self.cu_seqlens_q),
                          list(self.seqlens_kv), {k: mv(v) for k, v in self.extra.items()})

    def kv_bytes(self) -> int:
        """Algorithmic KV bytes one attention pass reads (each cached row once)."""
        if self.kv_cache.dim() == 5:
            per_token = 2 * self.n_kv * self.head_dim * self.kv_cache.element_size()
        else:
            per_token = self.kv_cache.shape[-1] * self.kv_cache.element_size()
        return sum(self.seqlens_kv) * per_token


def _randn(shape, gen, device, dtype=torch.bfloat16):
    """N(0,1) drawn in fp32 then cast, on CPU; drawn directly in the target
    dtype when generating on the GPU (large caches)."""
    if torch.device(device).type == "cpu":
        return torch.randn(shape, generator=gen, dtype=torch.float32).to(dtype)
    return torch.randn(shape, generator=gen, dtype=dtype, device=device)


def deal_block_tables(seqs: Sequence[Tuple[int, int]], block_size: int, pool_blocks: int,
                      gen: torch.Generator, shared_prefix_tokens: Optional[Sequence[int]] = None):
    """Deal a seeded permutation of the pool to the sequences in order.  With
    ``shared_prefix_tokens[b] = p`` the first p/block_size blocks of sequence b
    alias those of the first sequence that declared a prefix at least as long
    (prefix-cache sharing: auto_infer/engine/kv_cache_manager.py:86-111)."""
    perm = torch.randperm(pool_blocks, generator=gen).tolist()
    cursor = 0
    rows = []
    donor: List[int] = []                  # longest shared document so far
    for b, (_, kv_len) in enumerate(seqs):
        need = (kv_len + block_size - 1) // block_size
        row: List[int] = []
        if shared_prefix_tokens is not None and shared_prefix_tokens[b] > 0:
            n_shared = shared_prefix_tokens[b] // block_size
            while len(donor) < n_shared:
                donor.append(perm[cursor])
                cursor += 1
            row.extend(donor[:n_shared])
        while len(row) < need:
            row.append(perm[cursor])
            cursor += 1
        if cursor > pool_blocks:
            raise ValueError("physical pool too small for the requested sequences")
        rows.append(row)
    max_blocks = max((len(r) for r in rows), default=1)
    table = torch.zeros(len(rows), max(max_blocks, 1), dtype=torch.int32)
    for b, row in enumerate(rows):
        table[b, :len(row)] = torch.tensor(row, dtype=torch.int32)
    return table, rows


def build_gqa_batch(name: str, seqs: Sequence[Tuple[int, int]], n_q: int, n_kv: int, head_dim: int,
                    pool_blocks: int, seed: int, device="cpu", block_size: int = BLOCK_SIZE,
                    shared_prefix_tokens: Optional[Sequence[int]] = None) -> PagedBatch:
    """seqs: (q_len, kv_len) per sequence, kv_len including the q_len new tokens."""
    cpu_gen = torch.Generator().manual_seed(seed)
    table, rows = deal_block_tables(seqs, block_size, pool_blocks, cpu_gen, shared_prefix_tokens)
    dev = torch.device(device)
    gen = cpu_gen if dev.type == "cpu" else torch.Generator(device=dev).manual_seed(seed)
    total_q = sum(q for q, _ in seqs)
    q = _randn((total_q, n_q, head_dim), gen, dev)
    k_new = _randn((total_q, n_kv, head_dim), gen, dev)
    v_new = _randn((total_q, n_kv, head_dim), gen, dev)
    kv_cache = _randn((2, pool_blocks, block_size, n_kv, head_dim), gen, dev)
    slots, cu, kv_lens, acc = [], [], [], 0
    for (q_len, kv_len), row in zip(seqs, rows):
        for pos in range(kv_len - q_len, kv_len):
            slots.append(row[pos // block_size] * block_size + pos % block_size)
        acc += q_len
        cu.append(acc)
        kv_lens.append(kv_len)
    return PagedBatch(name, n_q, n_kv, head_dim, block_size, head_dim ** -0.5, q, k_new, v_new,
                      kv_cache, table.to(dev), torch.tensor(slots, dtype=torch.int32, device=dev),
                      cu, kv_lens)


def build_mla_batch(name: str, seqs: Sequence[Tuple[int, int]], num_heads: int, pool_blocks: int,
                    seed: int, device="cpu", block_size: int = BLOCK_SIZE, kv_lora_rank: int = 512,
                    qk_rope: int = 64, qk_nope: int = 128, v_head_dim: int = 128) -> PagedBatch:
    """Absorbed-MLA decode inputs: latent cache (P, bs, 1, kvl+rope) stored
    once, q_nope / q_pe per head, absorbed weights W_UK / W_UV ~ N(0, 0.02)."""
    cpu_gen = torch.Generator().manual_seed(seed)
    table, rows = deal_block_tables(seqs, block_size, pool_blocks, cpu_gen)
    dev = torch.device(device)
    gen = cpu_gen if dev.type == "cpu" else torch.Generator(device=dev).manual_seed(seed)
    total_q = sum(q for q, _ in seqs)
    width = kv_lora_rank + qk_rope
    q_nope = _randn((total_q, num_heads, qk_nope), gen, dev)
    q_pe = _randn((total_q, num_heads, qk_rope), gen, dev)
    w_uk = (_randn((num_heads, qk_nope, kv_lora_rank), gen, dev, torch.float32) * 0.02).to(torch.bfloat16)
    w_uv = (_randn((num_heads, v_head_dim, kv_lora_rank), gen, dev, torch.float32) * 0.02).to(torch.bfloat16)
    latent_new = _randn((total_q, 1, width), gen, dev)
    cache = _randn((pool_blocks, block_size, 1, width), gen, dev)
    slots, cu, kv_lens, acc = [], [], [], 0
    for (q_len, kv_len), row in zip(seqs, rows):
        for pos in range(kv_len - q_len, kv_len):
            slots.append(row[pos // block_size] * block_size + pos % block_size)
        acc += q_len
        cu.append(acc)
        kv_lens.append(kv_len)
    q_latent = torch.cat([torch.einsum("tnp,npl->tnl", q_nope, w_uk), q_pe], dim=-1).contiguous()
    return PagedBatch(name, num_heads, 1, width, block_size, (qk_nope + qk_rope) ** -0.5, q_latent,
                      latent_new, None, cache, table.to(dev),
                      torch.tensor(slots, dtype=torch.int32, device=dev), cu, kv_lens,
                      extra=dict(q_nope=q_nope, q_pe=q_pe, w_uk=w_uk, w_uv=w_uv,
                                 kv_lora_rank=kv_lora_rank))


def _uniform_lengths(gen, n, lo, hi):
    return torch.randint(lo, hi + 1, (n,), generator=gen).tolist()


# --------------------------------------------------------------------------- #
# the five configurations
# --------------------------------------------------------------------------- #
def config1(device="cpu") -> PagedBatch:
    """Qwen3-0.6B-shaped decode: 16 q / 8 kv heads, batch 16, context U[512, 2048]."""
    g = torch.Generator().manual_seed(SEED_BASE + 1)
    ctx = _uniform_lengths(g, 16, 512, 2048)
    return build_gqa_batch("c1_qwen3_0.6b_decode", [(1, c) for c in ctx], 16, 8, 128, 512,
                           SEED_BASE + 1, device)


def config2(device="cpu") -> PagedBatch:
    """Qwen3-8B-shaped mixed batch in scheduler order: 60 decode rows
    (context U[256, 8192]) then four 512-token prefill chunks over prefixes of
    0 / 1024 / 2048 / 4096 tokens; the three non-empty prefixes are nested
    prefixes of one document and share physical blocks."""
    g = torch.Generator().manual_seed(SEED_BASE + 2)
    ctx = _uniform_lengths(g, 60, 256, 8192)
    prefixes = [0, 1024, 2048, 4096]
    seqs = [(1, c) for c in ctx] + [(512, p + 512) for p in prefixes]
    shared = [0] * 60 + prefixes
    return build_gqa_batch("c2_qwen3_8b_mixed", seqs, 32, 8, 128, 4096, SEED_BASE + 2, device,
                           shared_prefix_tokens=shared)


def config3(batch: int = 64, device="cpu") -> PagedBatch:
    """DeepSeek-V3/Moonlight-shaped absorbed-MLA decode: 16 heads, 512+64 latent."""
    g = torch.Generator().manual_seed(SEED_BASE + 3)
    ctx = _uniform_lengths(g, batch, 1024, 8192)
    return build_mla_batch(f"c3_mla_decode_b{batch}", [(1, c) for c in ctx], 16, 4096,
                           SEED_BASE + 3, device)


def config4(device="cpu") -> PagedBatch:
    """MiMo-7B-shaped MTP verify: 32 q / 8 kv heads, batch 16, 2 query rows per request."""
    g = torch.Generator().manual_seed(SEED_BASE + 4)
    ctx = _uniform_lengths(g, 16, 512, 4096)
    return build_gqa_batch("c4_mimo_mtp_verify", [(2, c) for c in ctx], 32, 8, 128, 1024,
                           SEED_BASE + 4, device)


def config5(device="cpu", cp_rank: int = 0, cp_size: int = 1, context: int = 131072,
            batch: int = 8) -> PagedBatch:
    """Qwen2.5-72B-shaped long-context decode: 64 q / 8 kv heads, batch 8, one
    query token over ``context`` cached tokens.  With cp_size > 1 the batch is
    rank ``cp_rank``'s contiguous slice of every sequence's pages in a local pool
    of 1/cp_size the blocks; queries are identical on all ranks (same seed)."""
    assert context % (BLOCK_SIZE * cp_size) == 0
    local_ctx = context // cp_size
    blocks_per_seq = local_ctx // BLOCK_SIZE
    pool = batch * blocks_per_seq
    seed = SEED_BASE + 5
    batch_obj = build_gqa_batch(f"c5_qwen2.5_72b_cp{cp_size}_rank{cp_rank}", [(1, local_ctx)] * batch,
                                64, 8, 128, pool, seed * 1000 + cp_rank, device)
    # identical queries on every rank
    qg = torch.Generator().manual_seed(seed)
    batch_obj.q = torch.randn((batch, 64, 128), generator=qg, dtype=torch.float32).to(torch.bfloat16).to(device)
    batch_obj.extra["global_context"] = context
    batch_obj.extra["kv_offset"] = cp_rank * local_ctx
    return batch_obj


CONFIGS = {"c1": config1, "c2": config2, "c3": config3, "c4": config4, "c5": config5}
