"""The CUDA stand-in for the vendor module (``auto_infer_b200/vendor_shim.py``): the functions
auto-infer imports from ``torch_npu``, with the call shapes of its own call sites
(auto_infer/layers/attention/base.py:41-61, layers/norm.py:5-17, layers/mlp.py:16-20)."""
import sys

import pytest
import torch

from oracle import paged_attention_oracle as orc


def test_elementwise_stand_ins_match_their_definitions():
    from auto_infer_b200 import vendor_shim as shim
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, 64, generator=g).to(torch.bfloat16)
    r = torch.randn(5, 64, generator=g).to(torch.bfloat16)
    w = (torch.rand(64, generator=g) + 0.5).to(torch.bfloat16)
    out, _ = shim.npu_rms_norm(x, w, 1e-6)
    assert torch.equal(out, orc.rms_norm(x, w, 1e-6))
    normed, _, new_res = shim.npu_add_rms_norm(x, r, w, 1e-6)
    assert torch.equal(new_res, r + x) and torch.equal(normed, orc.rms_norm(r + x, w, 1e-6))
    gate_up = torch.randn(5, 32, generator=g).to(torch.bfloat16)
    assert torch.equal(shim.npu_swiglu(gate_up), torch.nn.functional.silu(gate_up[:, :16]) * gate_up[:, 16:])


def test_install_serves_the_reference_layers():
    """With the shim installed the reference's own norm / MLP layers run (here on CPU tensors)
    and its device helper is redirected.  Skipped where auto-infer is not importable."""
    from auto_infer_b200 import vendor_shim as shim
    from tests.test_registry_and_backends_host import _reference_registry
    _reference_registry()                                    # puts the reference on sys.path or skips
    had = sys.modules.get("torch_npu")
    done = shim.install()
    try:
        import torch_npu
        if had is None:
            assert torch_npu is shim and "torch_npu" in done
        from auto_infer import platform as ref_platform
        from auto_infer.layers.mlp import swiglu_mlp
        from auto_infer.layers.norm import add_rms_norm, rms_norm
        assert ref_platform.npu_device is shim.cuda_device
        g = torch.Generator().manual_seed(2)
        x = torch.randn(3, 32, generator=g).to(torch.bfloat16)
        w = (torch.rand(32, generator=g) + 0.5).to(torch.bfloat16)
        assert torch.equal(rms_norm(x, w, 1e-6), orc.rms_norm(x, w, 1e-6))
        normed, res = add_rms_norm(x, x, w, 1e-6)
        assert torch.equal(res, x + x)
        weights = {"mlp.gate_proj.weight": torch.randn(48, 32, generator=g).to(torch.bfloat16),
                   "mlp.up_proj.weight": torch.randn(48, 32, generator=g).to(torch.bfloat16),
                   "mlp.down_proj.weight": torch.randn(32, 48, generator=g).to(torch.bfloat16)}
        assert swiglu_mlp(x, weights, "mlp.").shape == (3, 32)
        if not torch.cuda.is_available():
            with pytest.raises(RuntimeError, match="no CPU fallback"):
                ref_platform.npu_device(0)
    finally:
        if had is None:
            sys.modules.pop("torch_npu", None)


@pytest.mark.gpu
def test_paged_operators_with_the_reference_call_shapes():
    """What GqaFIABackend._write_kv / ._attn do (auto_infer/layers/attention/gqa.py:76-94):
    the slot write, then the attention op on 3-D cache views with the two host lists, for a
    mixed step (decode row, verify pair, prefill chunk)."""
    from auto_infer_b200 import ops, synth
    from auto_infer_b200 import vendor_shim as torch_npu
    from tests.parity import assert_attention_close
    b = synth.build_gqa_batch("shim", [(1, 500), (2, 131), (80, 80 + 256)], 16, 4, 128, 24, 77)
    d = b.to("cuda")
    key_cache, value_cache = d.kv_cache[0], d.kv_cache[1]
    torch_npu._npu_reshape_and_cache(key=d.k_new, value=d.v_new, key_cache=key_cache, value_cache=value_cache,
                                     slot_indices=d.slot_mapping)
    orc.write_kv(b.k_new, b.v_new, b.kv_cache[0], b.kv_cache[1], b.slot_mapping.tolist())
    assert torch.equal(d.kv_cache.cpu(), b.kv_cache)
    num_blocks, block_size = key_cache.shape[0], key_cache.shape[1]
    k_fia = key_cache.view(num_blocks, block_size, b.n_kv * b.head_dim)
    v_fia = value_cache.view(num_blocks, block_size, b.n_kv * b.head_dim)
    mask = ~torch.tril(torch.ones((2048, 2048), dtype=torch.bool, device="cuda"))
    for _ in range(2):                                        # the second layer's call reuses the step's plan
        out, _ = torch_npu.npu_fused_infer_attention_score(
            query=d.q, key=k_fia, value=v_fia, block_table=d.block_table, input_layout="TND",
            block_size=block_size, actual_seq_lengths=b.cu_seqlens_q, actual_seq_lengths_kv=b.seqlens_kv,
            num_key_value_heads=b.n_kv, num_heads=b.n_q, scale=b.scale, atten_mask=mask, sparse_mode=3)
    ref = orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, b.cu_seqlens_q, b.seqlens_kv,
                              b.scale)
    assert_attention_close(out.cpu(), ref, what="vendor-op call shape")
    assert len(torch_npu._plan_cache) >= 1
    assert ops.read_status("cuda") == 0


@pytest.mark.gpu
def test_non_absorbed_mla_call_shape():
    """What MlaFIABackend._write_kv / ._attn do in the default, non-absorbed form
    (auto_infer/layers/attention/mla.py:243-255): K rows 192 wide, V rows 128 wide, one kv head
    per query head, a decode row and a prefill chunk in one step."""
    from auto_infer_b200 import ops
    from auto_infer_b200 import vendor_shim as torch_npu
    from tests.paging import page_out
    from tests.parity import assert_attention_close
    g = torch.Generator().manual_seed(8)
    nh, bs = 4, 16
    seqs = [(1, 300), (70, 70), (2, 65)]
    lens = [kv for _, kv in seqs]
    k = torch.randn(sum(lens), nh, 192, generator=g).to(torch.bfloat16)
    v = torch.randn(sum(lens), nh, 128, generator=g).to(torch.bfloat16)
    q = torch.randn(sum(ql for ql, _ in seqs), nh, 192, generator=g).to(torch.bfloat16)
    k_cache, v_cache, table, slots = page_out(k, v, lens, bs, 9)
    # the step's own rows arrive through the slot write, as in the reference
    new_rows, cu, at = [], [], 0
    for ql, kv in seqs:
        new_rows += list(range(at + kv - ql, at + kv))
        at += kv
        cu.append((cu[-1] if cu else 0) + ql)
    kc, vc = k_cache.clone(), v_cache.clone()
    new_slots = [slots[i] for i in new_rows]
    kc.view(-1, nh, 192)[new_slots] = 0
    vc.view(-1, nh, 128)[new_slots] = 0
    kc, vc = kc.cuda(), vc.cuda()
    torch_npu._npu_reshape_and_cache(key=k[new_rows].cuda(), value=v[new_rows].cuda(), key_cache=kc, value_cache=vc,
                                     slot_indices=torch.tensor(new_slots, dtype=torch.int32, device="cuda"))
    assert torch.equal(kc.cpu(), k_cache) and torch.equal(vc.cpu(), v_cache)
    nb = kc.shape[0]
    out, _ = torch_npu.npu_fused_infer_attention_score(
        query=q.cuda(), key=kc.view(nb, bs, nh * 192), value=vc.view(nb, bs, nh * 128), block_table=table.cuda(),
        input_layout="TND", block_size=bs, actual_seq_lengths=cu, actual_seq_lengths_kv=lens,
        num_key_value_heads=nh, num_heads=nh, scale=192 ** -0.5, atten_mask=None, sparse_mode=3)
    ref = orc.paged_attention(q, k_cache, v_cache, table, cu, lens, 192 ** -0.5)
    assert_attention_close(out.cpu(), ref, what="non-absorbed MLA call shape")
    with pytest.raises(NotImplementedError):                  # any other unequal widths
        torch_npu.npu_fused_infer_attention_score(
            query=q.cuda(), key=kc.view(nb, bs, nh * 192), value=vc.view(nb, bs, nh * 128)[..., :nh * 64].contiguous(),
            block_table=table.cuda(), input_layout="TND", block_size=bs, actual_seq_lengths=cu,
            actual_seq_lengths_kv=lens, num_key_value_heads=nh, num_heads=nh, scale=1.0)
    assert ops.read_status("cuda") == 0
