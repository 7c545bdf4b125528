"""Backend seam shared by the attention families: the two-method
``AttentionBackend`` interface of auto-infer
(auto_infer/layers/attention/base.py:21-38) and the plain linear helper
(base.py:9-18, bf16 path only: the W8A8 tuple form is outside this package)."""
from abc import ABC, abstractmethod

import torch


def _lin(x: torch.Tensor, weight, bias=None) -> torch.Tensor:
    if isinstance(weight, tuple):
        raise NotImplementedError("W8A8 weights are not handled by the B200 attention backend")
    out = x @ weight.t()
    return out + bias if bias is not None else out


class AttentionBackend(ABC):
    """The backend owns the whole attention sub-block of one layer and returns a
    tensor ready to be added to the residual."""

    @abstractmethod
    def alloc_kv_caches(self, num_blocks: int, block_size: int) -> list:
        raise NotImplementedError

    @abstractmethod
    def attention(self, layer_idx: int, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError
