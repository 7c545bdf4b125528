"""Slot arithmetic of the paged cache (auto_infer/engine/token_layout.py:1-4)."""


def slot_mapping(block_table, positions, block_size):
    """slot = block_table[pos // bs] * bs + pos % bs, for scalars or arrays."""
    return block_table[positions // block_size] * block_size + positions % block_size
