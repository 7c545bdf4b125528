"""Runs the kernels of one workload a few times on a bounded case, for profilers.

    python -m auto_infer_b200.profile_case --case decode --batch 1 --context 131072 --iters 3

Cases: ``decode`` (config-5-shaped split-KV GQA decode; 512 MiB of KV per
sequence at the default context, larger than L2), ``c1`` / ``c4`` (small decode
configurations), ``c2`` (mixed prefill + decode), ``c3`` (absorbed-MLA decode,
``--batch`` 4 / 16 / 64).  Inputs are generated on the device; a 256 MiB fill
flushes L2 before every iteration."""
from __future__ import annotations

import argparse

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="decode", choices=["decode", "c1", "c2", "c3", "c4"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=131072)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    from . import ops, synth
    from .metadata import StepMetadata
    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    if args.case == "c3":
        b = synth.config3(args.batch, dev)
        plan = ops.MlaDecodePlan(b.cu_seqlens_q, b.seqlens_kv, 16, dev)
        out = torch.empty(b.num_tokens, 16, 512, dtype=torch.bfloat16, device=dev)

        def step():
            ops.reshape_and_cache(b.k_new, None, b.kv_cache, None, b.slot_mapping)
            ops.mla_decode_absorbed(b.q, b.kv_cache, b.block_table, plan, b.scale, out=out)
    else:
        if args.case == "decode":
            b = synth.config5(dev, context=args.context, batch=args.batch)
        elif args.case == "c2":
            b = synth.config2(dev)
        else:
            b = synth.CONFIGS[args.case]().to(dev)
        meta = StepMetadata(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, b.head_dim, dev)
        out = torch.empty(b.q.shape, dtype=torch.bfloat16, device=dev)

        def step():
            ops.reshape_and_cache(b.k_new, b.v_new, b.kv_cache[0], b.kv_cache[1], b.slot_mapping)
            ops.paged_decode_gqa(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, meta.decode,
                                 b.scale, out=out)
            if meta.prefill is not None:
                ops.paged_prefill_gqa(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, meta.prefill,
                                      b.scale, out=out)
    for _ in range(args.iters):
        flush.zero_()
        step()
    torch.cuda.synchronize()
    status = ops.read_status(dev)
    print(f"{b.name}: {args.iters} iterations, kv bytes per step {b.kv_bytes()}, status {status}")
    if status:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
