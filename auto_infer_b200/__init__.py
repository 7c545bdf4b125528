"""B200 (sm_100a) paged-attention backend for the auto-infer runtime.

The package holds the host side of one hot path only: the attention-backend
plug-in (registry, GQA and MLA backends, per-step metadata, context-parallel
merge) over a C-ABI CUDA library built from ``csrc/``.  Importing the package
does not need a GPU; calling an operator without the built library or without a
CUDA device raises."""

__all__ = ["ops", "registry", "build"]
__version__ = "0.1"
