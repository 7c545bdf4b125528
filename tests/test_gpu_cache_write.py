"""Bit-exact parity of the CUDA KV-cache slot write with the oracle scatter,
called through the C ABI."""
import pytest
import torch

from oracle import paged_attention_oracle as orc

pytestmark = pytest.mark.gpu


def _run(num_blocks, bs, n_kv, kd, vd, slots, seed, strided=False):
    from auto_infer_b200 import ops
    g = torch.Generator().manual_seed(seed)
    t = len(slots)
    if strided:   # K and V as column slices of a packed projection, like qkv.split() gives
        packed = torch.randn(t, n_kv * (kd + vd) + 64, generator=g).to(torch.bfloat16)
        k = packed[:, 64:64 + n_kv * kd].view(t, n_kv, kd)
        v = packed[:, 64 + n_kv * kd:].view(t, n_kv, vd)
    else:
        k = torch.randn(t, n_kv, kd, generator=g).to(torch.bfloat16)
        v = torch.randn(t, n_kv, vd, generator=g).to(torch.bfloat16)
    kc = torch.randn(num_blocks, bs, n_kv, kd, generator=g).to(torch.bfloat16)
    vc = torch.randn(num_blocks, bs, n_kv, vd, generator=g).to(torch.bfloat16)
    kc_d, vc_d = kc.cuda(), vc.cuda()
    k_d, v_d = k.cuda(), v.cuda()
    if strided:
        packed_d = packed.cuda()
        k_d = packed_d[:, 64:64 + n_kv * kd].view(t, n_kv, kd)
        v_d = packed_d[:, 64 + n_kv * kd:].view(t, n_kv, vd)
    ops.reshape_and_cache(k_d, v_d, kc_d, vc_d, torch.tensor(slots, dtype=torch.int32).cuda())
    keep = [i for i, s in enumerate(slots) if s >= 0]
    orc.write_kv(k[keep], v[keep], kc, vc, [slots[i] for i in keep])
    assert torch.equal(kc_d.cpu(), kc) and torch.equal(vc_d.cpu(), vc)
    assert ops.read_status("cuda") == 0


def test_known_answer_slots_block_size_4():
    # slots of the reference's stager tests: decode [33, 13], MTP verify [33, 34, 13, 14],
    # mixed prefill [20..23, 29, 30]
    _run(12, 4, 2, 8, 8, [33, 13], 1)
    _run(12, 4, 2, 8, 8, [33, 34, 13, 14], 2)
    _run(12, 4, 1, 16, 16, [20, 21, 22, 23, 29, 30], 3)


def test_page_128_qwen_shapes_and_strided_rows():
    _run(16, 128, 8, 128, 128, [0, 127, 128, 129, 2047, 1000], 4)
    _run(16, 128, 8, 128, 128, list(range(300, 300 + 77)), 5, strided=True)


def test_unequal_k_v_width_and_padding_rows():
    # non-absorbed MLA: K 192 wide, V 128 wide; negative slots are padding rows
    _run(8, 16, 4, 192, 128, [5, -1, 100, 17, -1], 6)
    # odd width: falls to the 2-byte path
    _run(8, 16, 3, 7, 5, [1, 2, 127], 7)


def test_latent_cache_single_copy():
    from auto_infer_b200 import ops
    g = torch.Generator().manual_seed(8)
    lat = torch.randn(9, 1, 576, generator=g).to(torch.bfloat16)
    cache = torch.zeros(4, 128, 1, 576, dtype=torch.bfloat16)
    slots = [0, 1, 2, 130, 131, 300, 301, 302, 511]
    cache_d = cache.cuda()
    ops.reshape_and_cache(lat.cuda(), None, cache_d, None, torch.tensor(slots, dtype=torch.int32).cuda())
    orc.write_kv(lat, None, cache, None, slots)
    assert torch.equal(cache_d.cpu(), cache)


def test_out_of_pool_slot_is_skipped_and_flagged():
    from auto_infer_b200 import ops
    cache = torch.zeros(2, 4, 1, 8, dtype=torch.bfloat16).cuda()
    guard = cache.clone()
    k = torch.ones(2, 1, 8, dtype=torch.bfloat16).cuda()
    ops.reshape_and_cache(k, k, cache, cache.clone(), torch.tensor([8, 3], dtype=torch.int32).cuda())
    assert ops.read_status("cuda") & 1
    guard.view(-1, 1, 8)[3] = 1
    assert torch.equal(cache, guard)


def test_cpu_tensor_is_rejected():
    from auto_infer_b200 import ops
    k = torch.zeros(1, 1, 8, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        ops.reshape_and_cache(k, k, k.view(1, 1, 1, 8), k.view(1, 1, 1, 8), torch.zeros(1, dtype=torch.int32))
