"""The C-ABI shared library loads without a GPU and exports every function the
public header declares; argument validation runs on the host."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from auto_infer_b200 import _lib, build
    build.build()
    return _lib.load()


def _declared():
    text = open(os.path.join(ROOT, "include", "b200_attention.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from auto_infer_b200 import _lib
    names = _declared()
    assert len(names) >= 9
    for name in names:
        assert hasattr(lib, name), name
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names
    assert b"sm_100a" in lib.b200_version()


def test_plan_is_pure_host_code(lib):
    import torch
    from auto_infer_b200._lib import DecodePlanInfo
    cu = torch.tensor([1, 2, 4], dtype=torch.int32)
    kv = torch.tensor([100, 65, 130], dtype=torch.int32)
    nbytes = lib.b200_decode_plan_bytes(3, 2, 4)
    buf = torch.zeros(nbytes // 4, dtype=torch.int32)
    info = DecodePlanInfo()
    rc = lib.b200_decode_plan(cu.data_ptr(), kv.data_ptr(), None, 3, 8, 2, 4, buf.data_ptr(), nbytes,
                              ctypes.byref(info))
    assert rc == 0
    tiles = (2 + 2 + 3) * 2
    assert info.total_tiles == tiles and info.num_ctas == 4
    hdr = buf[:16].tolist()
    cta_off = buf[hdr[5]:hdr[5] + 5].tolist()
    items = buf[hdr[6]:hdr[6] + 12 * info.num_items].view(-1, 12).tolist()
    per_cta = [sum(it[3] - it[2] for it in items[cta_off[c]:cta_off[c + 1]]) for c in range(4)]
    assert sum(per_cta) == tiles and max(per_cta) - min(per_cta) <= 1
    # every (seq, head) pair is covered exactly once, in order
    cover = {}
    for it in items:
        cover.setdefault((it[0], it[1]), []).append((it[2], it[3]))
    for (seq, _), runs in cover.items():
        assert runs[0][0] == 0 and all(a[1] == b[0] for a, b in zip(runs, runs[1:]))
        assert runs[-1][1] == (kv[seq].item() + 63) // 64
    # partial records are numbered consecutively per pair and listed for the merge
    multi = buf[hdr[7]:hdr[7] + 8 * info.num_multi].view(-1, 8).tolist()
    assert sum(m[4] - m[3] for m in multi) == info.num_partials
    assert all((it[9] == 1) == (it[8] == -1) for it in items)


def test_plan_rejects_bad_arguments(lib):
    import torch
    from auto_infer_b200._lib import DecodePlanInfo
    info = DecodePlanInfo()
    buf = torch.zeros(1024, dtype=torch.int32)
    cu = torch.tensor([1], dtype=torch.int32)
    kv = torch.tensor([5], dtype=torch.int32)
    assert lib.b200_decode_plan(cu.data_ptr(), kv.data_ptr(), None, 1, 7, 2, 4, buf.data_ptr(), 4096,
                                ctypes.byref(info)) == -1          # heads not divisible
    assert lib.b200_decode_plan(cu.data_ptr(), kv.data_ptr(), None, 1, 8, 2, 4, buf.data_ptr(), 16,
                                ctypes.byref(info)) == -6          # buffer too small
    assert b"plan buffer" in lib.b200_last_error()
    # too many query rows for the decode kernel: left to the prefill kernel
    cu2 = torch.tensor([9], dtype=torch.int32)
    kv2 = torch.tensor([9], dtype=torch.int32)
    assert lib.b200_decode_plan(cu2.data_ptr(), kv2.data_ptr(), None, 1, 8, 2, 4, buf.data_ptr(), 4096,
                                ctypes.byref(info)) == 0
    assert info.skipped_seqs == 1 and info.num_items == 0


def test_operators_refuse_cpu_tensors():
    import torch
    from auto_infer_b200 import ops
    x = torch.zeros(1, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.lse_combine(torch.zeros(1, 1, 4), torch.zeros(1, 1))
    with pytest.raises(RuntimeError):
        ops.DecodePlan([1], [5], 2, 2, "cpu")
