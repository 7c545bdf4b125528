"""ctypes binding of the C-ABI library ``libb200attn.so`` (declared in
``include/b200_attention.h``).  There is no fallback: if the library has not
been built, loading raises and every operator of this package is unusable."""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200attn.so")

B200_OK = 0
STATUS_BAD_SLOT = 1
STATUS_BAD_BLOCK = 2
STATUS_WAIT_TIMEOUT = 4
STATUS_BAD_LAUNCH = 8


class DecodePlanInfo(ctypes.Structure):
    """Mirror of ``b200_decode_plan_info``."""
    _fields_ = [(name, c_int32) for name in (
        "num_ctas", "num_items", "num_partials", "num_multi",
        "total_tiles", "skipped_seqs", "plan_ints", "mode")]


class PrefillPlanInfo(ctypes.Structure):
    """Mirror of ``b200_prefill_plan_info``."""
    _fields_ = [(name, c_int32) for name in ("num_items", "total_tiles", "plan_ints", "num_tokens")]


class MhaPlanInfo(ctypes.Structure):
    """Mirror of ``b200_mha_plan_info``."""
    _fields_ = [("num_items", c_int32), ("num_splits", c_int32), ("num_tokens", c_int32),
                ("plan_ints", c_int32), ("narrow", c_int32), ("reserved", c_int32), ("total_tiles", c_int64)]


# name -> (restype, argtypes); one entry per function the header declares
SIGNATURES = {
    "b200_version": (c_char_p, []),
    "b200_last_error": (c_char_p, []),
    "b200_sm_count": (c_int, []),
    "b200_reshape_and_cache": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "b200_decode_plan_bytes": (c_size_t, [c_int, c_int, c_int]),
    "b200_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "b200_decode_plan": (c_int, [
        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
        c_void_p, c_size_t, POINTER(DecodePlanInfo)]),
    "b200_paged_decode_gqa": (c_int, [
        c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64,
        c_void_p, POINTER(DecodePlanInfo), c_int, c_int, c_int, c_float,
        c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_paged_decode_gqa_replayable": (c_int, [
        c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64,
        c_void_p, c_int, c_int, c_int, c_int, c_float,
        c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_paged_decode_gqa_write": (c_int, [
        c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_void_p, c_int64, c_void_p, POINTER(DecodePlanInfo), c_int,
        c_int, c_int, c_int, c_float,
        c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_paged_decode_gqa_static": (c_int, [
        c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64,
        c_void_p, POINTER(DecodePlanInfo), c_int, c_int, c_int, c_float,
        c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_prefill_plan_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "b200_prefill_plan": (c_int, [
        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
        c_void_p, c_size_t, POINTER(PrefillPlanInfo)]),
    "b200_paged_prefill_gqa": (c_int, [
        c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64,
        c_void_p, POINTER(PrefillPlanInfo), c_int, c_int, c_int, c_float,
        c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_paged_prefill_gqa_on": (c_int, [
        c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64,
        c_void_p, POINTER(PrefillPlanInfo), c_int, c_int, c_int, c_int, c_float,
        c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_paged_prefill_gqa_replayable": (c_int, [
        c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64,
        c_void_p, c_int, c_int, c_int, c_int, c_float,
        c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_mha_plan_bytes": (c_size_t, [c_int, c_int, c_int]),
    "b200_mha_workspace_bytes": (c_size_t, [c_int, c_int]),
    "b200_mha_plan": (c_int, [
        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
        c_void_p, c_size_t, POINTER(MhaPlanInfo)]),
    "b200_paged_mha": (c_int, [
        c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64,
        c_void_p, POINTER(MhaPlanInfo), c_int, c_int, c_int, c_float,
        c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_mla_decode_plan": (c_int, [
        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
        c_void_p, c_size_t, POINTER(DecodePlanInfo)]),
    "b200_mla_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "b200_mla_decode_absorbed": (c_int, [
        c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p, c_int64,
        c_void_p, POINTER(DecodePlanInfo), c_int, c_int, c_int, c_float,
        c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_cp_exchange_buffer_bytes": (c_size_t, [c_int, c_int64, c_int]),
    "b200_cp_exchange_combine": (c_int, [
        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int64,
        c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_gqa_rope_cache": (c_int, [
        c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64,
        c_void_p, c_void_p, c_float, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200_mla_rope_norm_cache": (c_int, [
        c_void_p, c_int64, c_void_p, c_float, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64,
        c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200_copy_blocks": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "b200_mla_decode_absorbed_replayable": (c_int, [
        c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p, c_int64,
        c_void_p, c_int, c_int, c_int, c_int, c_float,
        c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_lse_combine": (c_int, [
        c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64, c_int,
        c_void_p, c_int, c_void_p, c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library once and attach the signatures.  Raises RuntimeError
    with build instructions when the shared object is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m auto_infer_b200.build` "
            "(needs nvcc); this package has no CPU or eager fallback")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


class B200Error(RuntimeError):
    """A C-ABI call rejected its arguments or a CUDA call failed."""


def check(code: int, what: str) -> None:
    if code != B200_OK:
        msg = load().b200_last_error().decode("utf-8", "replace")
        raise B200Error(f"{what} failed with code {code}: {msg}")
