"""Runs one kernel of the path a few times on a bounded case, for profilers.

    python -m auto_infer_b200.profile_case --case decode --batch 1 --context 131072 --iters 3

Cases: ``decode`` (config-5-shaped split-KV GQA decode), ``c1`` / ``c4`` (the
small decode configurations).  Inputs are generated on the device and are larger
than L2 for ``decode`` at the default size (512 MiB of KV per sequence)."""
from __future__ import annotations

import argparse

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="decode", choices=["decode", "c1", "c4"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=131072)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    from . import ops, synth
    dev = torch.device("cuda", 0)
    if args.case == "decode":
        b = synth.config5(dev, context=args.context, batch=args.batch)
    else:
        b = synth.CONFIGS[args.case]().to(dev)
    plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, dev)
    out = torch.empty(b.q.shape, dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(args.iters):
        flush.zero_()
        ops.reshape_and_cache(b.k_new, b.v_new, b.kv_cache[0], b.kv_cache[1], b.slot_mapping)
        ops.paged_decode_gqa(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, plan, b.scale, out=out)
    torch.cuda.synchronize()
    status = ops.read_status(dev)
    print(f"{b.name}: {args.iters} iterations, kv bytes per launch {b.kv_bytes()}, status {status}")
    if status:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
