"""Test helper: lay packed per-sequence K / V rows out in a paged cache with shuffled pages."""
import torch


def page_out(k_rows, v_rows, lens, block_size, seed, spare_blocks=3, fill=0.0):
    """k_rows (sum(lens), H, Dk), v_rows (sum(lens), H, Dv) -> (k_cache, v_cache, block_table,
    slots) with every sequence's pages dealt from a shuffled pool.  ``fill`` is what unwritten
    slots hold."""
    g = torch.Generator().manual_seed(seed)
    h, dk = k_rows.shape[1], k_rows.shape[2]
    dv = v_rows.shape[2]
    need = [(n + block_size - 1) // block_size for n in lens]
    pool = sum(need) + spare_blocks
    order = torch.randperm(pool, generator=g).tolist()
    k_cache = torch.full((pool, block_size, h, dk), fill, dtype=k_rows.dtype)
    v_cache = torch.full((pool, block_size, h, dv), fill, dtype=v_rows.dtype)
    table = torch.zeros(len(lens), max(need), dtype=torch.int32)
    slots, start, nxt = [], 0, 0
    for b, n in enumerate(lens):
        pages = order[nxt:nxt + need[b]]
        nxt += need[b]
        table[b, :need[b]] = torch.tensor(pages, dtype=torch.int32)
        for pos in range(n):
            slots.append(pages[pos // block_size] * block_size + pos % block_size)
        start += n
    idx = torch.tensor(slots, dtype=torch.long)
    k_cache.view(-1, h, dk)[idx] = k_rows
    v_cache.view(-1, h, dv)[idx] = v_rows
    return k_cache, v_cache, table, slots
