"""Per-step contract handed to every backend; field for field the dataclass of
auto_infer/forward_context.py:9-23, so a context built by the reference's
runners can be passed in unchanged."""
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class ForwardContext:
    token_ids: torch.Tensor
    positions: torch.Tensor
    slot_mapping: torch.Tensor
    block_table: torch.Tensor
    cu_seqlens_q: list          # cumulative query lengths (host list)
    seqlens_kv: list            # per-sequence kv lengths incl. this step's tokens (host list)
    attn_mask: Optional[torch.Tensor]
    attn_backend: object
    kv_caches: list
    is_decode: bool
    cos: Optional[torch.Tensor] = None
    sin: Optional[torch.Tensor] = None
    active_token_mask: Optional[torch.Tensor] = None
