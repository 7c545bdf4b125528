"""Tensor-level wrappers over the C ABI.  Each function takes CUDA tensors,
passes raw pointers and the current stream to the library and returns torch
tensors.  CPU tensors are rejected: there is no host implementation."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import DecodePlanInfo, PrefillPlanInfo


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_ptr(device) -> int:
    """Raw cudaStream_t of torch's current stream on ``device``."""
    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def _on_device(device):
    """Device guard for a C call; free when ``device`` is already current (the calls
    of a step all are, and the guard object costs more than the call's own checks)."""
    if device.index is None or torch.cuda.current_device() == device.index:
        return _NO_GUARD
    return torch.cuda.device(device)


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "auto_infer_b200 operators run on CUDA tensors only (no CPU fallback); "
                f"got a tensor on {t.device}")


_status_words: dict = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 word the kernels OR fault bits into."""
    key = torch.device(device).index or 0
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _status_words[key]


def read_status(device, clear: bool = True) -> int:
    """Synchronising read of the device status word (0 = no fault seen)."""
    word = status_word(device)
    value = int(word.item())
    if clear and value:
        word.zero_()
    return value


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """SMs of ``device`` (the current one by default); asked once per device."""
    key = torch.device(device).index if device is not None else None
    if key is None:
        key = torch.cuda.current_device()
    if key not in _sm_counts:
        with torch.cuda.device(key):
            _sm_counts[key] = _lib.load().b200_sm_count()
    return _sm_counts[key]


# --------------------------------------------------------------------------- #
def reshape_and_cache(key: torch.Tensor, value: Optional[torch.Tensor],
                      key_cache: torch.Tensor, value_cache: Optional[torch.Tensor],
                      slot_mapping: torch.Tensor) -> None:
    """cache[slot // bs, slot % bs] = x[t]; replaces ``write_kv``
    (auto_infer/layers/attention/base.py:41-45).  key (T, Hkv, Dk) may be a
    strided view as long as each token row is contiguous."""
    _need_cuda(key, value, key_cache, value_cache, slot_mapping)
    lib = _lib.load()
    t, n_kv, k_dim = key.shape
    if t == 0:
        return
    if key.stride(2) != 1 or key.stride(1) != k_dim:
        key = key.contiguous()
    if not key_cache.is_contiguous():
        raise ValueError("key_cache must be contiguous")
    num_blocks, block_size = key_cache.shape[0], key_cache.shape[1]
    v_ptr = vc_ptr = None
    v_dim = 0
    v_stride = 0
    if value is not None:
        v_dim = value.shape[2]
        if value.stride(2) != 1 or value.stride(1) != v_dim:
            value = value.contiguous()
        if value_cache is None or not value_cache.is_contiguous():
            raise ValueError("value_cache must be a contiguous tensor when value is given")
        v_ptr, vc_ptr, v_stride = value.data_ptr(), value_cache.data_ptr(), value.stride(0)
    if slot_mapping.dtype != torch.int32:
        slot_mapping = slot_mapping.to(torch.int32)
    slot_mapping = slot_mapping.contiguous()
    with _on_device(key.device):
        rc = lib.b200_reshape_and_cache(
            key.data_ptr(), v_ptr, key_cache.data_ptr(), vc_ptr, slot_mapping.data_ptr(),
            t, n_kv, k_dim, v_dim, key.stride(0), v_stride, block_size, num_blocks,
            status_word(key.device).data_ptr(), _stream_ptr(key.device))
    _lib.check(rc, "b200_reshape_and_cache")


# --------------------------------------------------------------------------- #
class DecodePlan:
    """Host plan + device copy + workspace for one step of split-KV decode.
    Built once per step from the two host length lists and shared by all layers
    (the reference hands the same lists to its vendor op per layer,
    auto_infer/layers/attention/gqa.py:91-92).

    With ``capacity_seqs`` the plan is *replayable*: its device buffer and workspace
    are sized for any step of at most that many sequences and keep their
    addresses, ``refill()`` overwrites the plan in place, and the attention launch
    depends on ``num_ctas`` only, so a CUDA graph that recorded it serves later
    steps (what the reference's per-layer task update does on the host,
    auto_infer/layers/attention/graph_fia.py:70-104)."""

    def __init__(self, cu_seqlens_q: Sequence[int], seqlens_kv: Sequence[int], num_q_heads: int,
                 num_kv_heads: int, device, head_dim: int = 128, num_ctas: Optional[int] = None,
                 causal_base: Optional[Sequence[int]] = None, capacity_seqs: Optional[int] = None):
        lib = _lib.load()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("DecodePlan needs a CUDA device (no CPU fallback)")
        self.num_q_heads, self.num_kv_heads, self.head_dim = num_q_heads, num_kv_heads, head_dim
        self.num_ctas = int(num_ctas) if num_ctas else sm_count(self.device)
        self.replayable = capacity_seqs is not None
        self.capacity_seqs = max(int(capacity_seqs), len(cu_seqlens_q)) if self.replayable else len(cu_seqlens_q)
        self._nbytes = lib.b200_decode_plan_bytes(self.capacity_seqs, num_kv_heads, self.num_ctas)
        # two pinned staging buffers: a refill writes the one whose last copy has long left
        self._hosts = [torch.empty(self._nbytes // 4, dtype=torch.int32, pin_memory=True)
                       for _ in range(2 if self.replayable else 1)]
        self._copied = [None] * len(self._hosts)
        self._flip = 0
        self.host = self._hosts[0]
        self.info = DecodePlanInfo()
        self._build(cu_seqlens_q, seqlens_kv, causal_base)
        used = max(int(self.info.plan_ints), 16)
        if self.replayable:
            self.dev = torch.zeros(self._nbytes // 4, dtype=torch.int32, device=self.device)
            ws = self._capacity_workspace_bytes()
        else:
            self.dev = torch.empty(used, dtype=torch.int32, device=self.device)
            ws = (self.info.num_partials * (16 * head_dim + 16)) * 4 + 256
        self._upload(used)
        self.workspace = torch.empty(ws, dtype=torch.uint8, device=self.device)

    def _capacity_workspace_bytes(self) -> int:
        return _lib.load().b200_decode_workspace_bytes(self.capacity_seqs, self.num_kv_heads, self.num_ctas,
                                                       self.head_dim)

    def _call_planner(self, cu, kv, base) -> None:
        rc = _lib.load().b200_decode_plan(cu, kv, base, self.num_seqs,
                                          self.num_q_heads, self.num_kv_heads, self.num_ctas,
                                          self.host.data_ptr(), self._nbytes, ctypes.byref(self.info))
        _lib.check(rc, "b200_decode_plan")

    def _build(self, cu_seqlens_q, seqlens_kv, causal_base) -> None:
        self.num_seqs = len(cu_seqlens_q)
        if self.num_seqs > self.capacity_seqs:
            raise ValueError(f"{self.num_seqs} sequences exceed the plan's capacity of {self.capacity_seqs}")
        # plain C arrays: cheaper than tensors for a few dozen integers on the per-step path
        int_array = ctypes.c_int32 * self.num_seqs
        cu = int_array(*cu_seqlens_q)
        kv = int_array(*seqlens_kv)
        base = int_array(*causal_base) if causal_base is not None else None
        self._call_planner(cu, kv, base)

    def _upload(self, used: int) -> None:
        self.dev[:used].copy_(self.host[:used], non_blocking=True)
        if self.replayable:
            done = self._copied[self._flip]
            if done is None:                         # one event per staging buffer, recorded again each time
                done = self._copied[self._flip] = torch.cuda.Event()
            if self.device.index is None or torch.cuda.current_device() == self.device.index:
                done.record()                        # the current stream, where the copy was issued
            else:
                done.record(torch.cuda.current_stream(self.device))

    def refill(self, cu_seqlens_q: Sequence[int], seqlens_kv: Sequence[int],
               causal_base: Optional[Sequence[int]] = None) -> None:
        """Plan another step into the same device buffer: host planning into the idle
        staging buffer, then one pinned -> device copy on the current stream (ahead of
        the launches or the graph replay that read it).  The kernels of the previous
        step must be on the same stream (or finished): the copy overwrites their plan."""
        if not self.replayable:
            raise RuntimeError("refill() needs a plan built with capacity_seqs")
        self._flip ^= 1
        self.host = self._hosts[self._flip]
        if self._copied[self._flip] is not None:
            self._copied[self._flip].synchronize()      # its copy of two steps ago; normally long done
        self._build(cu_seqlens_q, seqlens_kv, causal_base)
        self._upload(max(int(self.info.plan_ints), 16))

    @property
    def skipped_seqs(self) -> int:
        return int(self.info.skipped_seqs)


def paged_decode_gqa(q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                     block_table: torch.Tensor, plan: DecodePlan, scale: float,
                     out: Optional[torch.Tensor] = None, out_f32: bool = False,
                     lse_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Paged GQA attention for decode-shaped rows (q_len * group <= 16).
    Replaces ``paged_fia`` (auto_infer/layers/attention/base.py:48-61).  Rows of
    sequences the plan skipped are left untouched in ``out``."""
    _need_cuda(q, key_cache, value_cache, block_table)
    lib = _lib.load()
    t, n_q, d = q.shape
    if q.stride(2) != 1 or q.stride(1) != d:
        q = q.contiguous()
    if not (key_cache.is_contiguous() and value_cache.is_contiguous()):
        raise ValueError("KV caches must be contiguous (num_blocks, block_size, Hkv, D)")
    num_blocks, block_size, n_kv, _ = key_cache.shape
    if block_table.dtype != torch.int32:
        block_table = block_table.to(torch.int32)
    if block_table.stride(1) != 1:
        block_table = block_table.contiguous()
    if out is None:
        out = torch.empty(t, n_q, d, dtype=torch.float32 if out_f32 else q.dtype, device=q.device)
    elif not out.is_contiguous():
        raise ValueError("out must be contiguous")
    with _on_device(q.device):
        if plan.replayable:
            rc = lib.b200_paged_decode_gqa_replayable(
                q.data_ptr(), q.stride(0), key_cache.data_ptr(), value_cache.data_ptr(),
                num_blocks, block_size, block_table.data_ptr(), block_table.stride(0),
                plan.dev.data_ptr(), plan.num_ctas, n_q, n_kv, d, float(scale),
                plan.workspace.data_ptr(), plan.workspace.numel(), out.data_ptr(),
                1 if out.dtype == torch.float32 else 0,
                lse_out.data_ptr() if lse_out is not None else None,
                status_word(q.device).data_ptr(), _stream_ptr(q.device))
        else:
            rc = lib.b200_paged_decode_gqa(
                q.data_ptr(), q.stride(0), key_cache.data_ptr(), value_cache.data_ptr(),
                num_blocks, block_size, block_table.data_ptr(), block_table.stride(0),
                plan.dev.data_ptr(), ctypes.byref(plan.info), n_q, n_kv, d, float(scale),
                plan.workspace.data_ptr(), plan.workspace.numel(), out.data_ptr(),
                1 if out.dtype == torch.float32 else 0,
                lse_out.data_ptr() if lse_out is not None else None,
                status_word(q.device).data_ptr(), _stream_ptr(q.device))
    _lib.check(rc, "b200_paged_decode_gqa")
    return out


def paged_decode_gqa_write(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                           slot_mapping: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                           block_table: torch.Tensor, plan: DecodePlan, scale: float,
                           out: Optional[torch.Tensor] = None, out_f32: bool = False,
                           lse_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``write_kv`` + ``paged_fia`` of a decode-shaped step in one launch
    (auto_infer/layers/attention/base.py:41-61): the CTA that streams the KV tile a new row
    falls in takes the row from ``k_new`` / ``v_new`` and stores it to its slot itself.  Same
    bits as ``reshape_and_cache`` followed by ``paged_decode_gqa``.  The plan must cover every
    sequence of the step (no rows left to the wide-query kernel)."""
    _need_cuda(q, k_new, v_new, slot_mapping, key_cache, value_cache, block_table)
    lib = _lib.load()
    t, n_q, d = q.shape
    if plan.info.skipped_seqs:
        raise ValueError("the plan leaves sequences to the wide-query kernel: write their rows with "
                         "reshape_and_cache and attend with paged_decode_gqa / paged_prefill_gqa")
    if q.stride(2) != 1 or q.stride(1) != d:
        q = q.contiguous()
    for name, x in (("k_new", k_new), ("v_new", v_new)):
        if x.shape[0] != t or x.stride(2) != 1 or x.stride(1) != d:
            raise ValueError(f"{name}: (T, Hkv, D) with each token's heads contiguous")
    if not (key_cache.is_contiguous() and value_cache.is_contiguous()):
        raise ValueError("KV caches must be contiguous (num_blocks, block_size, Hkv, D)")
    num_blocks, block_size, n_kv, _ = key_cache.shape
    if block_table.dtype != torch.int32:
        block_table = block_table.to(torch.int32)
    if block_table.stride(1) != 1:
        block_table = block_table.contiguous()
    if slot_mapping.dtype != torch.int32 or not slot_mapping.is_contiguous():
        slot_mapping = slot_mapping.to(torch.int32).contiguous()
    if out is None:
        out = torch.empty(t, n_q, d, dtype=torch.float32 if out_f32 else q.dtype, device=q.device)
    elif not out.is_contiguous():
        raise ValueError("out must be contiguous")
    with _on_device(q.device):
        rc = lib.b200_paged_decode_gqa_write(
            q.data_ptr(), q.stride(0), k_new.data_ptr(), k_new.stride(0), v_new.data_ptr(), v_new.stride(0),
            slot_mapping.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
            num_blocks, block_size, block_table.data_ptr(), block_table.stride(0),
            plan.dev.data_ptr(), None if plan.replayable else ctypes.byref(plan.info), plan.num_ctas,
            n_q, n_kv, d, float(scale), plan.workspace.data_ptr(), plan.workspace.numel(), out.data_ptr(),
            1 if out.dtype == torch.float32 else 0,
            lse_out.data_ptr() if lse_out is not None else None,
            status_word(q.device).data_ptr(), _stream_ptr(q.device))
    _lib.check(rc, "b200_paged_decode_gqa_write")
    return out


class MlaDecodePlan(DecodePlan):
    """Host plan + device copy + workspace of the absorbed-MLA decode kernel (32-token latent
    tiles, one shared latent head).  ``capacity_seqs`` makes it replayable like ``DecodePlan``:
    fixed addresses, ``refill()`` in place, a launch that depends on ``num_ctas`` only."""

    def __init__(self, cu_seqlens_q: Sequence[int], seqlens_kv: Sequence[int], num_heads: int,
                 device, kv_lora_rank: int = 512, num_ctas: Optional[int] = None,
                 causal_base: Optional[Sequence[int]] = None, capacity_seqs: Optional[int] = None):
        self.num_heads = num_heads
        super().__init__(cu_seqlens_q, seqlens_kv, num_heads, 1, device, head_dim=kv_lora_rank,
                         num_ctas=num_ctas, causal_base=causal_base, capacity_seqs=capacity_seqs)

    def _capacity_workspace_bytes(self) -> int:
        return _lib.load().b200_mla_decode_workspace_bytes(self.capacity_seqs, self.num_ctas, self.head_dim)

    def _call_planner(self, cu, kv, base) -> None:
        rc = _lib.load().b200_mla_decode_plan(cu, kv, base, self.num_seqs, self.num_heads, self.num_ctas,
                                              self.host.data_ptr(), self._nbytes, ctypes.byref(self.info))
        _lib.check(rc, "b200_mla_decode_plan")


def mla_decode_absorbed(q_latent: torch.Tensor, latent_cache: torch.Tensor,
                        block_table: torch.Tensor, plan: MlaDecodePlan, scale: float,
                        kv_lora_rank: int = 512, out: Optional[torch.Tensor] = None,
                        out_f32: bool = False, lse_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Latent MQA attention of the absorbed MLA path
    (auto_infer/layers/attention/mla.py:115-120): q_latent (T, H, kvl+rope) over
    latent_cache (num_blocks, block_size, 1, kvl+rope) -> (T, H, kvl)."""
    _need_cuda(q_latent, latent_cache, block_table)
    lib = _lib.load()
    t, h, width = q_latent.shape
    if q_latent.stride(2) != 1 or q_latent.stride(1) != width:
        q_latent = q_latent.contiguous()
    if not latent_cache.is_contiguous():
        raise ValueError("latent cache must be contiguous (num_blocks, block_size, 1, kvl+rope)")
    num_blocks, block_size = latent_cache.shape[0], latent_cache.shape[1]
    if block_table.dtype != torch.int32:
        block_table = block_table.to(torch.int32)
    if block_table.stride(1) != 1:
        block_table = block_table.contiguous()
    if out is None:
        out = torch.empty(t, h, kv_lora_rank, dtype=torch.float32 if out_f32 else q_latent.dtype,
                          device=q_latent.device)
    tail = (h, kv_lora_rank, width - kv_lora_rank, float(scale),
            plan.workspace.data_ptr(), plan.workspace.numel(), out.data_ptr(),
            1 if out.dtype == torch.float32 else 0,
            lse_out.data_ptr() if lse_out is not None else None,
            status_word(q_latent.device).data_ptr(), _stream_ptr(q_latent.device))
    with _on_device(q_latent.device):
        if plan.replayable:
            rc = lib.b200_mla_decode_absorbed_replayable(
                q_latent.data_ptr(), q_latent.stride(0), latent_cache.data_ptr(), num_blocks, block_size,
                block_table.data_ptr(), block_table.stride(0), plan.dev.data_ptr(), plan.num_ctas, *tail)
        else:
            rc = lib.b200_mla_decode_absorbed(
                q_latent.data_ptr(), q_latent.stride(0), latent_cache.data_ptr(), num_blocks, block_size,
                block_table.data_ptr(), block_table.stride(0), plan.dev.data_ptr(), ctypes.byref(plan.info),
                *tail)
    _lib.check(rc, "b200_mla_decode_absorbed")
    return out


class PrefillPlan:
    """Host plan + device copy for the wide-query attention kernel: 128-row work
    items of every (sequence, kv head) pair whose q_len * group exceeds
    ``min_rows``, longest first.

    With ``capacity_tokens`` (and ``capacity_seqs``) the plan is *replayable*: its device
    buffer is sized for any step of at most that many query tokens and sequences and keeps
    its address, ``refill()`` overwrites it in place and the attention launch does not depend
    on the step, so a CUDA graph that recorded it serves later steps."""

    def __init__(self, cu_seqlens_q: Sequence[int], seqlens_kv: Sequence[int], num_q_heads: int,
                 num_kv_heads: int, device, min_rows: int = 16,
                 causal_base: Optional[Sequence[int]] = None, capacity_tokens: Optional[int] = None,
                 capacity_seqs: Optional[int] = None):
        lib = _lib.load()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("PrefillPlan needs a CUDA device (no CPU fallback)")
        self.num_q_heads, self.num_kv_heads, self.min_rows = num_q_heads, num_kv_heads, int(min_rows)
        num_seqs = len(cu_seqlens_q)
        num_tokens = int(cu_seqlens_q[-1]) if num_seqs else 0
        self.replayable = capacity_tokens is not None
        self.capacity_tokens = max(int(capacity_tokens), num_tokens) if self.replayable else num_tokens
        self.capacity_seqs = max(int(capacity_seqs or 0), num_seqs) if self.replayable else num_seqs
        self._nbytes = max(lib.b200_prefill_plan_bytes(self.capacity_seqs, self.capacity_tokens, num_q_heads,
                                                       num_kv_heads), 64)
        self._hosts = [torch.empty(self._nbytes // 4, dtype=torch.int32, pin_memory=True)
                       for _ in range(2 if self.replayable else 1)]
        self._copied = [None] * len(self._hosts)
        self._flip = 0
        self.host = self._hosts[0]
        self.info = PrefillPlanInfo()
        self._build(cu_seqlens_q, seqlens_kv, causal_base)
        used = max(int(self.info.plan_ints), 16)
        self.dev = torch.zeros(self._nbytes // 4 if self.replayable else used, dtype=torch.int32,
                               device=self.device)
        self._upload(used)

    def _build(self, cu_seqlens_q, seqlens_kv, causal_base) -> None:
        lib = _lib.load()
        num_seqs = len(cu_seqlens_q)
        num_tokens = int(cu_seqlens_q[-1]) if num_seqs else 0
        if num_seqs > self.capacity_seqs or num_tokens > self.capacity_tokens:
            raise ValueError(f"step of {num_seqs} sequences / {num_tokens} tokens exceeds the plan's capacity "
                             f"({self.capacity_seqs} / {self.capacity_tokens})")
        int_array = ctypes.c_int32 * max(num_seqs, 1)
        cu = int_array(*cu_seqlens_q)
        kv = int_array(*seqlens_kv)
        base = int_array(*causal_base) if causal_base is not None else None
        rc = lib.b200_prefill_plan(cu, kv, base, num_seqs, self.num_q_heads, self.num_kv_heads, self.min_rows,
                                   self.host.data_ptr(), self.host.numel() * 4, ctypes.byref(self.info))
        _lib.check(rc, "b200_prefill_plan")

    def _upload(self, used: int) -> None:
        self.dev[:used].copy_(self.host[:used], non_blocking=True)
        if self.replayable:
            done = torch.cuda.Event()
            done.record(torch.cuda.current_stream(self.device))
            self._copied[self._flip] = done

    def refill(self, cu_seqlens_q: Sequence[int], seqlens_kv: Sequence[int],
               causal_base: Optional[Sequence[int]] = None) -> None:
        """Plan another step into the same device buffer (see ``DecodePlan.refill``)."""
        if not self.replayable:
            raise RuntimeError("refill() needs a plan built with capacity_tokens")
        self._flip ^= 1
        self.host = self._hosts[self._flip]
        if self._copied[self._flip] is not None:
            self._copied[self._flip].synchronize()
        self._build(cu_seqlens_q, seqlens_kv, causal_base)
        self._upload(max(int(self.info.plan_ints), 16))


def paged_prefill_gqa(q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                      block_table: torch.Tensor, plan: PrefillPlan, scale: float,
                      out: Optional[torch.Tensor] = None, out_f32: bool = False,
                      lse_out: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
    """Paged GQA attention for wide query blocks (chunked prefill, multi-token
    verify); replaces ``paged_fia`` (auto_infer/layers/attention/base.py:48-61)
    for the sequences in ``plan``.  Other rows of ``out`` are left untouched.
    ``max_ctas`` > 0 keeps the launch to that many SMs (a mixed step runs the decode
    kernel on the others at the same time)."""
    _need_cuda(q, key_cache, value_cache, block_table)
    lib = _lib.load()
    t, n_q, d = q.shape
    if q.stride(2) != 1 or q.stride(1) != d:
        q = q.contiguous()
    if not (key_cache.is_contiguous() and value_cache.is_contiguous()):
        raise ValueError("KV caches must be contiguous (num_blocks, block_size, Hkv, D)")
    num_blocks, block_size, n_kv, _ = key_cache.shape
    if block_table.dtype != torch.int32:
        block_table = block_table.to(torch.int32)
    if block_table.stride(1) != 1:
        block_table = block_table.contiguous()
    if out is None:
        out = torch.empty(t, n_q, d, dtype=torch.float32 if out_f32 else q.dtype, device=q.device)
    elif not out.is_contiguous():
        raise ValueError("out must be contiguous")
    with _on_device(q.device):
        if plan.replayable:
            if t > plan.capacity_tokens:
                raise ValueError("q holds more rows than the plan was sized for")
            rc = lib.b200_paged_prefill_gqa_replayable(
                q.data_ptr(), q.stride(0), key_cache.data_ptr(), value_cache.data_ptr(),
                num_blocks, block_size, block_table.data_ptr(), block_table.stride(0),
                plan.dev.data_ptr(), t, n_q, n_kv, d, float(scale),
                out.data_ptr(), 1 if out.dtype == torch.float32 else 0,
                lse_out.data_ptr() if lse_out is not None else None,
                status_word(q.device).data_ptr(), _stream_ptr(q.device))
        elif max_ctas > 0:
            rc = lib.b200_paged_prefill_gqa_on(
                q.data_ptr(), q.stride(0), key_cache.data_ptr(), value_cache.data_ptr(),
                num_blocks, block_size, block_table.data_ptr(), block_table.stride(0),
                plan.dev.data_ptr(), ctypes.byref(plan.info), int(max_ctas), n_q, n_kv, d, float(scale),
                out.data_ptr(), 1 if out.dtype == torch.float32 else 0,
                lse_out.data_ptr() if lse_out is not None else None,
                status_word(q.device).data_ptr(), _stream_ptr(q.device))
        else:
            rc = lib.b200_paged_prefill_gqa(
                q.data_ptr(), q.stride(0), key_cache.data_ptr(), value_cache.data_ptr(),
                num_blocks, block_size, block_table.data_ptr(), block_table.stride(0),
                plan.dev.data_ptr(), ctypes.byref(plan.info), n_q, n_kv, d, float(scale),
                out.data_ptr(), 1 if out.dtype == torch.float32 else 0,
                lse_out.data_ptr() if lse_out is not None else None,
                status_word(q.device).data_ptr(), _stream_ptr(q.device))
    _lib.check(rc, "b200_paged_prefill_gqa")
    return out


class MhaPlan:
    """Host plan + device copy + workspace of the K-192 / V-128 multi-head kernel (non-absorbed
    MLA): blocks of 64 query positions per head, keys cut into equal splits when the step has
    too few blocks for the SMs."""

    def __init__(self, cu_seqlens_q: Sequence[int], seqlens_kv: Sequence[int], num_heads: int, device,
                 num_ctas: Optional[int] = None, causal_base: Optional[Sequence[int]] = None):
        lib = _lib.load()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("MhaPlan needs a CUDA device (no CPU fallback)")
        num_seqs = len(cu_seqlens_q)
        num_tokens = int(cu_seqlens_q[-1]) if num_seqs else 0
        self.num_heads = num_heads
        self.num_ctas = int(num_ctas) if num_ctas else sm_count(self.device)
        nbytes = lib.b200_mha_plan_bytes(num_seqs, num_tokens, num_heads)
        self.host = torch.empty(max(nbytes // 4, 16), dtype=torch.int32, pin_memory=True)
        cu = torch.tensor(list(cu_seqlens_q), dtype=torch.int32)
        kv = torch.tensor(list(seqlens_kv), dtype=torch.int32)
        base_ptr = None
        if causal_base is not None:
            base = torch.tensor(list(causal_base), dtype=torch.int32)
            base_ptr = base.data_ptr()
        self.info = _lib.MhaPlanInfo()
        rc = lib.b200_mha_plan(cu.data_ptr(), kv.data_ptr(), base_ptr, num_seqs, num_heads, self.num_ctas,
                               self.host.data_ptr(), self.host.numel() * 4, ctypes.byref(self.info))
        _lib.check(rc, "b200_mha_plan")
        used = max(int(self.info.plan_ints), 16)
        self.dev = torch.empty(used, dtype=torch.int32, device=self.device)
        self.dev.copy_(self.host[:used], non_blocking=True)
        self.workspace = None
        if self.info.num_splits > 1:
            ws = int(self.info.num_splits) * num_tokens * num_heads * (128 + 1) * 4 + 16
            self.workspace = torch.empty(ws, dtype=torch.uint8, device=self.device)


def paged_mha(q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, block_table: torch.Tensor,
              plan: MhaPlan, scale: float, out: Optional[torch.Tensor] = None, out_f32: bool = False,
              lse_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Paged attention of the non-absorbed MLA form (auto_infer/layers/attention/mla.py:56-63,
    243-254): q (T, H, 192) over key_cache (num_blocks, block_size, H, 192) and value_cache
    (num_blocks, block_size, H, 128) -> (T, H, 128); decode rows and prefill chunks alike."""
    _need_cuda(q, key_cache, value_cache, block_table)
    lib = _lib.load()
    t, h, dk = q.shape
    if q.stride(2) != 1 or q.stride(1) != dk:
        q = q.contiguous()
    if not (key_cache.is_contiguous() and value_cache.is_contiguous()):
        raise ValueError("KV caches must be contiguous (num_blocks, block_size, H, D)")
    num_blocks, block_size, n_kv, _ = key_cache.shape
    dv = value_cache.shape[3]
    if n_kv != h or value_cache.shape[:3] != key_cache.shape[:3]:
        raise ValueError("one K and one V row per query head: caches (num_blocks, block_size, H, 192 / 128)")
    if t != plan.info.num_tokens:
        raise ValueError(f"the plan covers {plan.info.num_tokens} tokens, q has {t}")
    if block_table.dtype != torch.int32:
        block_table = block_table.to(torch.int32)
    if block_table.stride(1) != 1:
        block_table = block_table.contiguous()
    if out is None:
        out = torch.empty(t, h, dv, dtype=torch.float32 if out_f32 else q.dtype, device=q.device)
    elif not out.is_contiguous():
        raise ValueError("out must be contiguous")
    ws = plan.workspace
    with _on_device(q.device):
        rc = lib.b200_paged_mha(
            q.data_ptr(), q.stride(0), key_cache.data_ptr(), value_cache.data_ptr(), num_blocks, block_size,
            block_table.data_ptr(), block_table.stride(0), plan.dev.data_ptr(), ctypes.byref(plan.info),
            h, dk, dv, float(scale), ws.data_ptr() if ws is not None else None,
            ws.numel() if ws is not None else 0, out.data_ptr(), 1 if out.dtype == torch.float32 else 0,
            lse_out.data_ptr() if lse_out is not None else None,
            status_word(q.device).data_ptr(), _stream_ptr(q.device))
    _lib.check(rc, "b200_paged_mha")
    return out


def lse_combine(o_parts: torch.Tensor, lse_parts: torch.Tensor,
                out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None,
                lse_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Merge (R, rows, D) fp32 partial outputs with their (R, rows) fp32 lse.
    Parts may be strided along dim 0 (e.g. views into an all-gather buffer)."""
    _need_cuda(o_parts, lse_parts)
    lib = _lib.load()
    r, rows, d = o_parts.shape
    if o_parts.stride(2) != 1 or o_parts.stride(1) != d or lse_parts.stride(1) != 1:
        raise ValueError("each part must be contiguous (rows, D) / (rows,)")
    if out is None:
        out = torch.empty(rows, d, dtype=out_dtype, device=o_parts.device)
    with _on_device(o_parts.device):
        rc = lib.b200_lse_combine(
            o_parts.data_ptr(), lse_parts.data_ptr(), o_parts.stride(0), lse_parts.stride(0),
            r, rows, d, out.data_ptr(), 1 if out.dtype == torch.float32 else 0,
            lse_out.data_ptr() if lse_out is not None else None, _stream_ptr(o_parts.device))
    _lib.check(rc, "b200_lse_combine")
    return out


def cp_exchange_combine(local_record: torch.Tensor, recv_ptrs_dev: int, state: torch.Tensor, rank: int,
                        world: int, rows: int, head_dim: int, out: torch.Tensor,
                        lse_out: Optional[torch.Tensor] = None, wait_limit_ns: int = 0) -> torch.Tensor:
    """Fused context-parallel exchange + merge: push this rank's packed fp32
    record [o | lse] to every rank's receive buffer over NVLink, wait for all
    ranks' records and merge them into ``out`` (rows, head_dim).  ``recv_ptrs_dev``
    is the device address of the array of receive-buffer pointers;
    ``wait_limit_ns`` bounds the wait for a peer (0 = one second)."""
    _need_cuda(local_record, state, out)
    lib = _lib.load()
    with _on_device(out.device):
        rc = lib.b200_cp_exchange_combine(
            local_record.data_ptr(), recv_ptrs_dev, state.data_ptr(), rank, world, rows, head_dim,
            int(wait_limit_ns), out.data_ptr(), 1 if out.dtype == torch.float32 else 0,
            lse_out.data_ptr() if lse_out is not None else None,
            status_word(out.device).data_ptr(), _stream_ptr(out.device))
    _lib.check(rc, "b200_cp_exchange_combine")
    return out


def _cache_tensors(layer):
    return layer if isinstance(layer, tuple) else (layer,)


def copy_blocks(source_caches, target_caches, block_ids, target_block_ids=None) -> None:
    """Copy selected physical blocks between caches with identical layouts; same contract as
    ``copy_blocks`` of auto_infer/pd/connector.py:30-51 (a tensor cache is the dense
    ``(2, blocks, ...)`` layout, a tuple holds separate key / value tensors whose leading
    axis is the block axis), one kernel launch per cache tensor instead of one copy per
    block.  ``target_block_ids`` (optional, beyond the reference) lands the pages on other
    block ids of the target pool."""
    if len(source_caches) != len(target_caches):
        raise ValueError("source and target cache layer counts must match")
    lib = _lib.load()
    ids = torch.as_tensor(block_ids, dtype=torch.int32)
    if ids.numel() == 0:
        return
    dst_ids = None
    if target_block_ids is not None:
        dst_ids = torch.as_tensor(target_block_ids, dtype=torch.int32)
        if dst_ids.numel() != ids.numel():
            raise ValueError("block_ids and target_block_ids must have the same length")
    ids_dev = {}
    for source_layer, target_layer in zip(source_caches, target_caches):
        source_tensors = _cache_tensors(source_layer)
        target_tensors = _cache_tensors(target_layer)
        if len(source_tensors) != len(target_tensors):
            raise ValueError("source and target cache layouts must match")
        separate_kv = isinstance(source_layer, tuple)
        for source, target in zip(source_tensors, target_tensors):
            block_axis = 0 if separate_kv else 1
            same = (source.shape == target.shape) if dst_ids is None else (
                source.shape[:block_axis] + source.shape[block_axis + 1:] ==
                target.shape[:block_axis] + target.shape[block_axis + 1:])
            if not same:
                raise ValueError("source and target cache shapes must match")
            _need_cuda(source, target)
            if not (source.is_contiguous() and target.is_contiguous()):
                raise ValueError("caches must be contiguous")
            # the dense layout is two stacked pools: K pages, then V pages
            halves = [(source, target)] if separate_kv else [(source[0], target[0]), (source[1], target[1])]
            dev = source.device
            if dev not in ids_dev:
                ids_dev[dev] = (ids.to(dev), dst_ids.to(dev) if dst_ids is not None else None)
            src_ids, tgt_ids = ids_dev[dev]
            for src, dst in halves:
                page_bytes = src[0].numel() * src.element_size()
                with _on_device(dev):
                    rc = lib.b200_copy_blocks(
                        src.data_ptr(), dst.data_ptr(), src_ids.data_ptr(),
                        tgt_ids.data_ptr() if tgt_ids is not None else None, ids.numel(), page_bytes,
                        src.shape[0], dst.shape[0], status_word(dev).data_ptr(), _stream_ptr(dev))
                _lib.check(rc, "b200_copy_blocks")


def gqa_rope_cache(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                   key_cache: torch.Tensor, value_cache: torch.Tensor, slot_mapping: torch.Tensor,
                   q_norm_weight: Optional[torch.Tensor] = None, k_norm_weight: Optional[torch.Tensor] = None,
                   eps: float = 1e-6, want_k: bool = False):
    """Fused prologue of the GQA sub-block (auto_infer/layers/attention/gqa.py:40-47): optional
    per-head RMSNorm of q / k, NeoX rotary embedding of q / k, slot write of k and v.
    q / k / v are (T, H*, 128) views (of the packed projection, typically); returns the rotated
    q (T, Hq, 128) and, with ``want_k``, the rotated k."""
    _need_cuda(q, k, v, cos, sin, key_cache, value_cache, slot_mapping)
    lib = _lib.load()
    t, n_q, d = q.shape
    n_kv = k.shape[1]
    for name, x in (("q", q), ("k", k), ("v", v)):
        if x.stride(2) != 1 or x.stride(1) != d:
            raise ValueError(f"{name}: each token's heads must be contiguous")
    if cos.stride(-1) != 1 or sin.stride(-1) != 1 or cos.stride(0) != sin.stride(0):
        raise ValueError("cos / sin must be (T, 1, D) with contiguous rows and equal token strides")
    if not (key_cache.is_contiguous() and value_cache.is_contiguous()):
        raise ValueError("KV caches must be contiguous (num_blocks, block_size, Hkv, D)")
    if slot_mapping.dtype != torch.int32:
        slot_mapping = slot_mapping.to(torch.int32)
    q_out = torch.empty(t, n_q, d, dtype=q.dtype, device=q.device)
    k_out = torch.empty(t, n_kv, d, dtype=k.dtype, device=k.device) if want_k else None
    num_blocks, block_size = key_cache.shape[0], key_cache.shape[1]
    with _on_device(q.device):
        rc = lib.b200_gqa_rope_cache(
            q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
            cos.data_ptr(), sin.data_ptr(), cos.stride(0),
            q_norm_weight.data_ptr() if q_norm_weight is not None else None,
            k_norm_weight.data_ptr() if k_norm_weight is not None else None, float(eps),
            q_out.data_ptr(), q_out.stride(0), k_out.data_ptr() if k_out is not None else None,
            key_cache.data_ptr(), value_cache.data_ptr(), slot_mapping.contiguous().data_ptr(),
            t, n_q, n_kv, d, block_size, num_blocks, status_word(q.device).data_ptr(), _stream_ptr(q.device))
    _lib.check(rc, "b200_gqa_rope_cache")
    return (q_out, k_out) if want_k else q_out


def mla_rope_norm_cache(ckv_full: torch.Tensor, norm_weight: torch.Tensor, eps: float, q_pe: torch.Tensor,
                        q_pe_out: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                        latent_cache: torch.Tensor, slot_mapping: torch.Tensor, kv_lora_rank: int = 512,
                        want_k_latent: bool = False) -> Optional[torch.Tensor]:
    """Fused prologue of the absorbed-MLA sub-block (auto_infer/layers/attention/mla.py:96-113):
    latent RMSNorm, interleaved rotary embedding of the decoupled key and of every head's q_pe
    (written to ``q_pe_out``, any (T, H, 64) view), slot write of the latent row."""
    _need_cuda(ckv_full, norm_weight, q_pe, q_pe_out, cos, sin, latent_cache, slot_mapping)
    lib = _lib.load()
    t, width = ckv_full.shape
    rope = width - kv_lora_rank
    h = q_pe.shape[1]
    if ckv_full.stride(1) != 1 or q_pe.stride(2) != 1 or q_pe_out.stride(2) != 1:
        raise ValueError("rows must be contiguous along their last axis")
    if not latent_cache.is_contiguous():
        raise ValueError("latent cache must be contiguous (num_blocks, block_size, 1, kvl+rope)")
    if slot_mapping.dtype != torch.int32:
        slot_mapping = slot_mapping.to(torch.int32)
    k_latent = torch.empty(t, 1, width, dtype=ckv_full.dtype, device=ckv_full.device) if want_k_latent else None
    num_blocks, block_size = latent_cache.shape[0], latent_cache.shape[1]
    with _on_device(ckv_full.device):
        rc = lib.b200_mla_rope_norm_cache(
            ckv_full.data_ptr(), ckv_full.stride(0), norm_weight.data_ptr(), float(eps),
            q_pe.data_ptr(), q_pe.stride(0), q_pe.stride(1), q_pe_out.data_ptr(), q_pe_out.stride(0),
            q_pe_out.stride(1), cos.data_ptr(), sin.data_ptr(), cos.stride(0), latent_cache.data_ptr(),
            k_latent.data_ptr() if k_latent is not None else None, slot_mapping.contiguous().data_ptr(),
            t, h, kv_lora_rank, rope, block_size, num_blocks, status_word(ckv_full.device).data_ptr(),
            _stream_ptr(ckv_full.device))
    _lib.check(rc, "b200_mla_rope_norm_cache")
    return k_latent
