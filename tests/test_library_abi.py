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


def _plan(lib, cu, kv, n_q, n_kv, num_ctas, mla=False):
    """(info, header, per-CTA item lists, items, multi groups) of a host-built plan."""
    import torch
    from auto_infer_b200._lib import DecodePlanInfo
    cu_t = torch.tensor(cu, dtype=torch.int32)
    kv_t = torch.tensor(kv, dtype=torch.int32)
    heads = 1 if mla else n_kv
    nbytes = lib.b200_decode_plan_bytes(len(cu), heads, num_ctas)
    buf = torch.zeros(nbytes // 4, dtype=torch.int32)
    info = DecodePlanInfo()
    if mla:
        rc = lib.b200_mla_decode_plan(cu_t.data_ptr(), kv_t.data_ptr(), None, len(cu), n_q, num_ctas,
                                      buf.data_ptr(), nbytes, ctypes.byref(info))
    else:
        rc = lib.b200_decode_plan(cu_t.data_ptr(), kv_t.data_ptr(), None, len(cu), n_q, n_kv, num_ctas,
                                  buf.data_ptr(), nbytes, ctypes.byref(info))
    assert rc == 0, lib.b200_last_error()
    hdr = buf[:16].tolist()
    assert hdr[1] == num_ctas and hdr[2] == info.num_items and hdr[10] == info.mode
    assert info.plan_ints == hdr[6] + 12 * info.num_items and info.plan_ints * 4 <= nbytes
    recs = buf[hdr[5]:hdr[5] + 16 * num_ctas].view(-1, 16).tolist()
    items = buf[hdr[6]:hdr[6] + 12 * info.num_items].view(-1, 12).tolist()
    multi = buf[hdr[7]:hdr[7] + 8 * info.num_multi].view(-1, 8).tolist()
    assert hdr[7] + 8 * info.num_multi <= hdr[6]             # the groups end before the items start
    per_cta = []
    for rec in recs:
        mine = items[rec[0]:rec[1]]
        if mine:
            assert rec[4:16] == mine[0]                      # the record carries a copy of the first item
        per_cta.append(mine)
    return info, hdr, per_cta, items, multi


def _check_cover(items, multi, kv, n_kv, tile, info):
    """Every (seq, head) pair is covered exactly once; the records of a cut pair are numbered
    consecutively in tile order and listed in its group."""
    cover = {}
    for it in items:
        cover.setdefault((it[0], it[1]), []).append((it[2], it[3], it[8], it[9], it[10]))
    assert len(cover) == sum(1 for k in kv if k > 0) * n_kv
    parts = 0
    for (seq, _), runs in cover.items():
        runs.sort()
        assert runs[0][0] == 0 and all(a[1] == b[0] for a, b in zip(runs, runs[1:]))
        assert runs[-1][1] == (kv[seq] + tile - 1) // tile
        if len(runs) == 1:
            assert runs[0][2] == -1 and runs[0][3] == 1
        else:
            group = multi[runs[0][4]]
            assert [r[2] for r in runs] == list(range(group[3], group[4]))
            assert all(r[3] == 0 and r[4] == runs[0][4] for r in runs)
            parts += len(runs)
    assert parts == info.num_partials == sum(m[4] - m[3] for m in multi)


def test_plan_is_pure_host_code(lib):
    cu, kv = [1, 2, 4], [100, 65, 130]
    info, hdr, per_cta, items, multi = _plan(lib, cu, kv, 8, 2, 4)
    tiles = (2 + 2 + 3) * 2
    assert info.total_tiles == tiles and info.num_ctas == 4
    assert sum(it[3] - it[2] for it in items) == tiles
    _check_cover(items, multi, kv, 2, 64, info)


def test_plan_modes_on_the_benchmark_shapes(lib):
    """Small steps and many-pair steps keep pairs whole (no partial records at all where the
    pairs fit); the 128K-context step is cut into equal streams."""
    from auto_infer_b200 import synth
    import torch
    g = torch.Generator().manual_seed(synth.SEED_BASE + 1)
    c1 = synth._uniform_lengths(g, 16, 512, 2048)
    info, _, per_cta, items, multi = _plan(lib, list(range(1, 17)), c1, 16, 8, 148)
    assert info.mode == 1 and info.num_partials == 0 and info.num_items == 128
    _check_cover(items, multi, c1, 8, 64, info)
    assert max(len(m) for m in per_cta) <= 3

    g = torch.Generator().manual_seed(synth.SEED_BASE + 2)
    c2 = synth._uniform_lengths(g, 60, 256, 8192)
    info, _, per_cta, items, multi = _plan(lib, list(range(1, 61)), c2, 32, 8, 148)
    assert info.mode == 1 and info.num_partials == 0 and info.num_items == 480
    loads = [sum(it[3] - it[2] for it in mine) for mine in per_cta]
    assert max(loads) <= 1.10 * sum(loads) / 148
    _check_cover(items, multi, c2, 8, 64, info)

    # config 5 on one GPU: long streams, cut to equal cost
    kv = [131072] * 8
    info, _, per_cta, items, multi = _plan(lib, list(range(1, 9)), kv, 64, 8, 148)
    assert info.mode == 0
    loads = [sum(it[3] - it[2] for it in mine) for mine in per_cta]
    assert max(loads) - min(loads) <= 20 and max(len(m) for m in per_cta) <= 3
    assert sum(1 for mine in per_cta for it in mine if it[9] == 0) == info.num_partials
    assert max(sum(1 for it in mine if it[9] == 0) for mine in per_cta) <= 2
    _check_cover(items, multi, kv, 8, 64, info)
    # one of eight context-parallel ranks: every pair in two halves, one piece per CTA
    kv = [131072 // 8] * 8
    info, _, per_cta, items, multi = _plan(lib, list(range(1, 9)), kv, 64, 8, 148)
    assert info.mode == 1 and info.num_items == 128 and info.num_multi == 64
    assert max(len(m) for m in per_cta) == 1
    _check_cover(items, multi, kv, 8, 64, info)

    # the latent kernel is not bandwidth-shared: uneven packing is never taken for it
    g = torch.Generator().manual_seed(synth.SEED_BASE + 3)
    c3 = synth._uniform_lengths(g, 64, 1024, 8192)
    info, _, per_cta, items, multi = _plan(lib, list(range(1, 65)), c3, 16, 1, 148, mla=True)
    loads = [sum(it[3] - it[2] for it in mine) for mine in per_cta]
    assert max(loads) <= 1.12 * sum(loads) / 148 + 8
    _check_cover(items, multi, c3, 1, 32, info)


def _mha_plan(lib, cu, kv, heads, num_ctas, base=None):
    from auto_infer_b200._lib import MhaPlanInfo
    n = len(cu)
    tokens = cu[-1] if cu else 0
    nbytes = lib.b200_mha_plan_bytes(n, tokens, heads)
    host = (ctypes.c_int32 * max(nbytes // 4, 16))()
    cu_a, kv_a = (ctypes.c_int32 * max(n, 1))(*cu), (ctypes.c_int32 * max(n, 1))(*kv)
    base_a = (ctypes.c_int32 * n)(*base) if base is not None else None
    info = MhaPlanInfo()
    rc = lib.b200_mha_plan(cu_a, kv_a, base_a, n, heads, num_ctas, host, nbytes, ctypes.byref(info))
    assert rc == 0, lib.b200_last_error()
    items = [tuple(host[16 + 12 * i + k] for k in range(9)) for i in range(info.num_items)]
    return info, list(host[:16]), items


def test_mha_plan_covers_every_row_and_key_once(lib):
    """Blocks of 64 query positions per head; the tiles a block can see are dealt to the
    splits without gap or overlap; long items come first."""
    cu, kv, heads = [1, 131, 136, 136], [5000, 1000, 5, 77], 4
    for num_ctas in (1, 148, 4000):
        info, hdr, items = _mha_plan(lib, cu, kv, heads, num_ctas)
        assert hdr[1] == info.num_items == len(items) and hdr[2] == info.num_splits and hdr[3] == 136
        assert 1 <= info.num_splits <= 8
        lengths = [it[5] - it[4] for it in items]
        assert lengths == sorted(lengths, reverse=True)
        seen = {}
        for seq, head, tok0, n_rows, t0, t1, kv_len, limit0, split in items:
            assert 0 < n_rows <= 64 and kv_len == kv[seq] and 0 <= t0 <= t1
            seen.setdefault((tok0, head), []).append((split, t0, t1, seq, n_rows, limit0))
        prev, blocks = 0, []
        for b, end in enumerate(cu):
            for r in range(0, end - prev, 64):
                blocks.append((prev + r, b, min(64, end - prev - r), kv[b] - (end - prev) + r))
            prev = end
        assert len(seen) == len(blocks) * heads
        for tok0, b, n_rows, limit0 in blocks:
            for h in range(heads):
                parts = sorted(seen[(tok0, h)])
                assert [p[0] for p in parts] == list(range(info.num_splits))
                assert all(p[3:] == (b, n_rows, limit0) for p in parts)
                n_tiles = min(limit0 + n_rows - 1, kv[b] - 1) // 64 + 1
                at = 0
                for _, t0, t1, *_ in parts:
                    assert t0 == min(at, n_tiles) and t1 >= t0
                    at = t1
                assert at == n_tiles
        assert info.total_tiles == sum(lengths)
    # a step with a block of more than 16 rows is not "narrow"; decode / verify steps are
    assert _mha_plan(lib, cu, kv, heads, 148)[0].narrow == 0
    assert _mha_plan(lib, [1, 3, 19], [500, 70, 9000], heads, 148)[0].narrow == 1
    assert _mha_plan(lib, [1, 18], [500, 70], heads, 148)[0].narrow == 0
    # one CTA wanted: no splits; many: the longest block is cut
    assert _mha_plan(lib, cu, kv, heads, 1)[0].num_splits == 1
    assert _mha_plan(lib, cu, kv, heads, 4000)[0].num_splits == 8
    # an empty step is an empty plan
    info, _, items = _mha_plan(lib, [], [], heads, 148)
    assert info.num_items == 0 and not items


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
