#!/usr/bin/env python
"""Benchmark of the paged-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One "step" is one layer-step of the path on the Qwen2.5-72B-shaped long-context
decode workload (64 q / 8 kv heads, head_dim 128, bf16, 128-token pages, batch
8, 131072 cached tokens per sequence): KV slot write of the step's token,
split-KV paged attention and, on N > 1 GPUs (context parallel: every rank holds
a contiguous 1/N of each sequence's pages), the exchange of the per-rank
(o, lse) partials fused with the log-sum-exp merge.  Total work is fixed as N
grows (strong scaling).  The metric is achieved HBM throughput over the
algorithmic KV bytes of the step, whole job; microseconds per layer-step are
reported beside it.  Rank 0 prints one JSON line.

``--impl reference`` times the reference's eager torch attention arithmetic
(restated for paged KV in oracle/) on the host cores, one sequence of the batch
per step.

``--case c1|c2|c3|c4|decode|mha --iters N`` runs the kernels of one workload N times
on a bounded case and exits (what the profiler commands under profiles/ run).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "paged_attn_decode_achieved_hbm"
UNIT = "TB/s"
CONTEXT = 131072
BATCH = 8
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--no-side-configs", action="store_true",
                    help="skip the kernel-only timings of the smaller configurations")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="auto", choices=["auto", "p2p", "nccl"],
                    help="context-parallel exchange: fused peer-to-peer kernel or NCCL all-gather")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the step's kernels one by one instead of replaying a CUDA graph")
    ap.add_argument("--case", default=None, choices=["decode", "c1", "c2", "c3", "c4", "merges", "mha"],
                    help="profiler mode: run one workload's kernels --iters times and exit")
    ap.add_argument("--iters", type=int, default=3)
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s: the burst figure (kernels here are timed alone)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["bf16_tflops"])
    except Exception:
        return 1590.0


def ncu_traffic(workload: str):
    """DRAM bytes per launch of the dominant kernel from the committed ncu
    summary (profiles/roofline_traffic.txt), or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "roofline_traffic.txt")) as fh:
            return json.load(fh).get(workload)
    except Exception:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed
    region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        load = [c for c, w in zip(sm, power) if w >= 0.5 * max(power)] if power else sm
        return {"sm_mhz": statistics.median(load) if load else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "samples_under_load": len(load),
                "power_w_max": max(power) if power else None, "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- #
def scale_free_ok(out: torch.Tensor, ref: torch.Tensor, atol_rms=2e-2, rtol=2.0 ** -7, rel_l2=1e-2):
    """The check the parity tests use for long contexts: error bounds relative to each
    reference row's own size (the rows are ~0.005 here, far below any absolute tolerance)."""
    o, r = out.float(), ref.float()
    rms = r.pow(2).mean(-1, keepdim=True).sqrt()
    err = (o - r).abs()
    elem_ok = bool((err <= atol_rms * rms + rtol * r.abs()).all())
    l2_ok = bool(((o - r).pow(2).sum(-1).sqrt() <= rel_l2 * r.pow(2).sum(-1).sqrt()).all())
    return elem_ok and l2_ok and bool(torch.isfinite(o).all()) and float(r.abs().max()) > 0


def unroll_for(steps: int) -> int:
    """Layer-steps recorded per CUDA graph (an engine replays all layers of a model from one
    graph, not one graph per layer): the largest divisor of ``steps`` up to 25, or all of them
    when ``steps`` is a prime of moderate size."""
    best = max(d for d in range(1, 26) if steps % d == 0)
    if best == 1 and 1 < steps <= 64:
        return steps
    return best


def capture_graph(fn, device, reps: int):
    """Record ``reps`` calls of ``fn`` into one CUDA graph (after eager warm-up calls, so that
    lazy initialisations happen outside the capture)."""
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()
    torch.cuda.current_stream(device).wait_stream(side)
    torch.cuda.synchronize(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for _ in range(reps):
            fn()
    torch.cuda.synchronize(device)
    return graph


def timed_batches(run_steps, steps, barrier, n_batches):
    """Device time (ms) of ``n_batches`` batches of exactly ``steps`` steps, each bracketed by
    a barrier and a synchronize on both sides."""
    out = []
    for _ in range(n_batches):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        run_steps(steps)
        e1.record()
        barrier()
        out.append(e0.elapsed_time(e1))
    return out


def max_over_ranks(value: float, device, world: int) -> float:
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def layer_rotation_time(make_step, layers, device, reps=12):
    """Per-layer-step device time (us) of a step replayed from ONE graph over ``layers``
    distinct caches (as the layers of a model are): graph-launch latency is paid once per
    model step, consecutive layers overlap their prologues, and every layer's reads come
    from HBM because the other layers' traffic (far more than L2 holds) passes in between."""
    steps = [make_step(i) for i in range(layers)]

    def all_layers():
        for s in steps:
            s()

    graph = capture_graph(all_layers, device, 1)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize(device)
    ts = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize(device)
        ts.append(e0.elapsed_time(e1) * 1e3 / layers)
    ts.sort()
    return statistics.median(ts), ts[0]


def side_config(name, device):
    """Layer-step time of one of the other configurations (slot write + attention) with its
    roofline fractions against the measured peaks."""
    from auto_infer_b200 import ops, synth
    hbm_peak, _ = measured_peak()
    tensor_peak = measured_tensor_peak()
    how = "one graph over {} layer caches (reuse distance > L2), time / layers"
    if name.startswith("c3"):
        batch = int(name.split("_b")[1])
        b = synth.config3(batch, device)
        plan = ops.MlaDecodePlan(b.cu_seqlens_q, b.seqlens_kv, 16, device)
        out = torch.empty(b.num_tokens, 16, 512, dtype=torch.bfloat16, device=device)
        layers = 8
        caches = [b.kv_cache] + [b.kv_cache.clone() for _ in range(layers - 1)]

        def make(i):
            def step():
                ops.reshape_and_cache(b.k_new, None, caches[i], None, b.slot_mapping)
                ops.mla_decode_absorbed(b.q, caches[i], b.block_table, plan, b.scale, out=out)
            return step

        us, best = layer_rotation_time(make, layers, device)
        bytes_ = sum(b.seqlens_kv) * 1152 + b.num_tokens * 16 * (576 + 512) * 2
        flops = sum(b.seqlens_kv) * 34816
        return {"us_per_layer_step": round(us, 2), "best_us": round(best, 2),
                "algorithmic_mb": round(bytes_ / 1e6, 2), "achieved_gbs": round(bytes_ / us / 1e3, 1),
                "hbm_frac": round(bytes_ / us / 1e3 / hbm_peak, 3), "bound": "hbm",
                "tflops": round(flops / us / 1e6, 1),
                "tensor_frac": round(flops / us / 1e6 / tensor_peak, 4), "batch": batch,
                "timing": how.format(layers)}
    if name == "c2":
        b = synth.config2(device)
        from auto_infer_b200.metadata import StepMetadata
        meta = StepMetadata(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, b.head_dim, device)
        out = torch.empty(b.q.shape, dtype=torch.bfloat16, device=device)
        layers = 4
        caches = [b.kv_cache] + [b.kv_cache.clone() for _ in range(layers - 1)]

        def make_full(i):
            def step():
                ops.reshape_and_cache(b.k_new, b.v_new, caches[i][0], caches[i][1], b.slot_mapping)
                ops.paged_decode_gqa(b.q, caches[i][0], caches[i][1], b.block_table, meta.decode, b.scale, out=out)
                ops.paged_prefill_gqa(b.q, caches[i][0], caches[i][1], b.block_table, meta.prefill, b.scale, out=out)
            return step

        def make_dec(i):
            return lambda: ops.paged_decode_gqa(b.q, caches[i][0], caches[i][1], b.block_table, meta.decode,
                                                b.scale, out=out)

        def make_pre(i):
            return lambda: ops.paged_prefill_gqa(b.q, caches[i][0], caches[i][1], b.block_table, meta.prefill,
                                                 b.scale, out=out)

        us_seq, _ = layer_rotation_time(make_full, layers, device)
        us_dec, _ = layer_rotation_time(make_dec, layers, device)
        us_pre, _ = layer_rotation_time(make_pre, layers, device)
        # the step as the backend runs it: the two kernels side by side on disjoint SMs (the decode
        # plan built for its share), when the cost model expects a gain
        from auto_infer_b200.metadata import mixed_split, scan_step
        _, dec_b, pre_t, pre_items, pre_longest = scan_step(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, b.head_dim)
        n_pre = mixed_split(dec_b, pre_t, ops.sm_count(device), pre_items, pre_longest)
        us, best = us_seq, us_seq
        if n_pre:
            split = StepMetadata(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, b.head_dim, device,
                                 prefill_ctas=n_pre)
            side = torch.cuda.Stream(device)

            def make_side_by_side(i):
                def step():
                    ops.reshape_and_cache(b.k_new, b.v_new, caches[i][0], caches[i][1], b.slot_mapping)
                    cur = torch.cuda.current_stream(device)
                    fork, join = torch.cuda.Event(), torch.cuda.Event()
                    fork.record(cur)
                    side.wait_event(fork)
                    with torch.cuda.stream(side):
                        ops.paged_prefill_gqa(b.q, caches[i][0], caches[i][1], b.block_table, split.prefill,
                                              b.scale, out=out, max_ctas=n_pre)
                        join.record(side)
                    ops.paged_decode_gqa(b.q, caches[i][0], caches[i][1], b.block_table, split.decode, b.scale,
                                         out=out)
                    cur.wait_event(join)
                return step

            us, best = layer_rotation_time(make_side_by_side, layers, device)
        # causal-aware flops of the four 512-token chunks over prefixes 0/1024/2048/4096
        flops = sum(4 * 32 * 128 * (512 * p + 131328) for p in (0, 1024, 2048, 4096))
        dec_bytes = sum(b.seqlens_kv[:60]) * 4096 + 2 * 60 * 32 * 128 * 2
        return {"us_per_layer_step": round(us, 2), "best_us": round(best, 2),
                "one_after_the_other_us": round(us_seq, 2), "prefill_sms_side_by_side": n_pre,
                "decode_rows_us": round(us_dec, 2), "decode_rows_gbs": round(dec_bytes / us_dec / 1e3, 1),
                "decode_rows_hbm_frac": round(dec_bytes / us_dec / 1e3 / hbm_peak, 3),
                "prefill_chunks_us": round(us_pre, 2), "prefill_gflop": round(flops / 1e9, 2),
                "prefill_tflops": round(flops / us_pre / 1e6, 1),
                "prefill_tensor_frac": round(flops / us_pre / 1e6 / tensor_peak, 4),
                "bound": "tensor (chunks) + hbm (decode rows)", "tokens": b.num_tokens,
                "timing": how.format(layers)}
    b = synth.CONFIGS[name]().to(device)
    plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, device)
    out = torch.empty(b.q.shape, dtype=torch.bfloat16, device=device)
    layers = 8
    caches = [b.kv_cache] + [b.kv_cache.clone() for _ in range(layers - 1)]

    def make(i):
        return lambda: ops.paged_decode_gqa_write(b.q, b.k_new, b.v_new, b.slot_mapping, caches[i][0],
                                                  caches[i][1], b.block_table, plan, b.scale, out=out)

    us, best = layer_rotation_time(make, layers, device)
    bytes_ = b.kv_bytes() + 2 * b.q.numel() * 2
    return {"us_per_layer_step": round(us, 2), "best_us": round(best, 2),
            "algorithmic_mb": round(bytes_ / 1e6, 2), "achieved_gbs": round(bytes_ / us / 1e3, 1),
            "hbm_frac": round(bytes_ / us / 1e3 / hbm_peak, 3), "bound": "hbm",
            "batch": len(b.seqlens_kv), "tokens": b.num_tokens, "timing": how.format(layers)}


def cpu_baseline_sample(args, threads):
    """The oracle (reference eager arithmetic) on one sequence of the workload."""
    from oracle import paged_attention_oracle as orc
    from auto_infer_b200 import synth
    torch.set_num_threads(threads)
    b = synth.config5("cpu", context=args.context, batch=1)
    warm = synth.config5("cpu", context=4096, batch=1)
    orc.paged_attention(warm.q, warm.kv_cache[0], warm.kv_cache[1], warm.block_table,
                        warm.cu_seqlens_q, warm.seqlens_kv, warm.scale, literal_max_kv=0)
    return b, orc


def run_reference(args, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    b, orc = cpu_baseline_sample(args, threads)
    bytes_step = b.kv_bytes()

    def step():
        orc.write_kv(b.k_new, b.v_new, b.kv_cache[0], b.kv_cache[1], b.slot_mapping.tolist())
        return orc.paged_attention(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table,
                                   b.cu_seqlens_q, b.seqlens_kv, b.scale, literal_max_kv=0)

    # each step is a bounded sample (one sequence, ~0.2-1 s of host work): the stated warm-up
    # and step counts are run as given
    warmup = max(args.warmup, 1)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = bytes_step / dt / 1e12
    sample = f"1 of {args.batch} sequences per step ({args.context} tokens, all 64 heads)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": warmup, "ms_per_step": dt * 1e3,
        "us_per_layer_step_full_batch": dt * 1e6 * args.batch,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(args, max(args.gpus, 1)),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, n):
    return {"workload": "c5: Qwen2.5-72B-shaped context-parallel long-context decode",
            "q_heads": 64, "kv_heads": 8, "head_dim": 128, "block_size": 128,
            "batch": args.batch, "context": args.context, "q_len": 1,
            "parallelism": f"cp{n}", "l2": "inputs larger than L2 (KV read per rank per step "
            f"{args.batch * args.context * 4096 // n // 2**20} MiB, never re-read)"}


# --------------------------------------------------------------------------- #
def profile_case(args):
    """Bounded runs for profilers: the kernels of one workload ``--iters`` times, a 256 MiB
    fill between iterations so that every iteration reads from HBM."""
    from auto_infer_b200 import ops, synth
    from auto_infer_b200.metadata import StepMetadata
    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    batch = args.batch or 1
    if args.case == "merges":
        # the small stand-alone kernels on config-5-sized operands: merge of 8 ranks' records
        # (512 rows x 128), the fused exchange with one rank (push to and merge from this GPU's own
        # buffer), the prologue kernels, the page copy
        from auto_infer_b200 import _lib
        g = torch.Generator(device=dev).manual_seed(1)
        o = torch.randn(8, 512, 128, generator=g, device=dev)
        lse = torch.randn(8, 512, generator=g, device=dev)
        rec = torch.cat([o[0].reshape(-1), lse[0]]).contiguous()
        nfloats = _lib.load().b200_cp_exchange_buffer_bytes(1, 512, 128) // 4
        xbuf = torch.zeros(nfloats, dtype=torch.float32, device=dev)
        xptr = torch.tensor([xbuf.data_ptr()], dtype=torch.int64, device=dev)
        xstate = torch.zeros(4, dtype=torch.int32, device=dev)
        xout = torch.empty(512, 128, dtype=torch.bfloat16, device=dev)
        t, n_q, n_kv = 2048, 32, 8
        qkv = torch.randn(t, (n_q + 2 * n_kv) * 128, generator=g, device=dev).to(torch.bfloat16)
        q, k, v = qkv.split((n_q * 128, n_kv * 128, n_kv * 128), dim=-1)
        cos = torch.randn(t, 1, 128, generator=g, device=dev).to(torch.bfloat16)
        sin = torch.randn(t, 1, 128, generator=g, device=dev).to(torch.bfloat16)
        nw = torch.ones(128, dtype=torch.bfloat16, device=dev)
        cache = torch.zeros(2, 512, 128, n_kv, 128, dtype=torch.bfloat16, device=dev)
        cache2 = torch.zeros_like(cache)
        slots = torch.randperm(512 * 128, generator=g, device=dev)[:t].to(torch.int32)
        ckv = torch.randn(t, 576, generator=g, device=dev).to(torch.bfloat16)
        qm = torch.randn(t, 16, 192, generator=g, device=dev).to(torch.bfloat16)
        ql = torch.empty(t, 16, 576, dtype=torch.bfloat16, device=dev)
        lat = torch.zeros(512, 128, 1, 576, dtype=torch.bfloat16, device=dev)
        cs64 = cos[..., :64].contiguous()
        sn64 = sin[..., :64].contiguous()
        ids = torch.randperm(512, generator=g, device=dev)[:256].tolist()
        name = "lse_combine, cp_exchange (1 rank), rope/cache prologues, copy_blocks"

        def step():
            ops.lse_combine(o, lse)
            ops.cp_exchange_combine(rec, xptr.data_ptr(), xstate, 0, 1, 512, 128, xout)
            ops.gqa_rope_cache(q.view(t, n_q, 128), k.view(t, n_kv, 128), v.view(t, n_kv, 128), cos, sin,
                               cache[0], cache[1], slots, q_norm_weight=nw, k_norm_weight=nw)
            ops.mla_rope_norm_cache(ckv, torch.ones(512, dtype=torch.bfloat16, device=dev), 1e-6, qm[..., 128:],
                                    ql[..., 512:], cs64, sn64, lat, slots)
            ops.copy_blocks([cache], [cache2], ids)
    elif args.case == "mha":
        # config 3's sequences (16 heads, contexts 1 024-8 192) in the reference's default,
        # non-absorbed cache layout: per head K 192 / V 128
        b3 = synth.config3(batch if args.batch else 16)
        name = "non-absorbed MLA decode, K 192 / V 128 per head, lengths of " + b3.name
        lens, bs = b3.seqlens_kv, b3.block_size
        del b3
        pages = [(n + bs - 1) // bs for n in lens]
        pool = sum(pages)
        g = torch.Generator(device=dev).manual_seed(5)
        order = torch.randperm(pool, generator=torch.Generator().manual_seed(5)).to(torch.int32)
        table = torch.zeros(len(lens), max(pages), dtype=torch.int32)
        at = 0
        for i, n in enumerate(pages):
            table[i, :n] = order[at:at + n]
            at += n
        table = table.to(dev)
        kc = torch.randn(pool, bs, 16, 192, generator=g, device=dev).to(torch.bfloat16)
        vc = torch.randn(pool, bs, 16, 128, generator=g, device=dev).to(torch.bfloat16)
        qh = torch.randn(len(lens), 16, 192, generator=g, device=dev).to(torch.bfloat16)
        plan = ops.MhaPlan(list(range(1, len(lens) + 1)), lens, 16, dev)
        out = torch.empty(len(lens), 16, 128, dtype=torch.bfloat16, device=dev)

        def step():
            ops.paged_mha(qh, kc, vc, table, plan, 192 ** -0.5, out=out)
    elif args.case == "c3":
        b = synth.config3(batch if args.batch else 64, dev)
        name = b.name
        plan = ops.MlaDecodePlan(b.cu_seqlens_q, b.seqlens_kv, 16, dev)
        out = torch.empty(b.num_tokens, 16, 512, dtype=torch.bfloat16, device=dev)

        def step():
            ops.reshape_and_cache(b.k_new, None, b.kv_cache, None, b.slot_mapping)
            ops.mla_decode_absorbed(b.q, b.kv_cache, b.block_table, plan, b.scale, out=out)
    else:
        if args.case == "decode":
            b = synth.config5(dev, context=args.context, batch=batch)
        elif args.case == "c2":
            b = synth.config2(dev)
        else:
            b = synth.CONFIGS[args.case]().to(dev)
        name = b.name
        meta = StepMetadata(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, b.head_dim, dev)
        out = torch.empty(b.q.shape, dtype=torch.bfloat16, device=dev)

        def step():
            if meta.prefill is None:
                ops.paged_decode_gqa_write(b.q, b.k_new, b.v_new, b.slot_mapping, b.kv_cache[0], b.kv_cache[1],
                                           b.block_table, meta.decode, b.scale, out=out)
                return
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
    print(f"{name}: {args.iters} iterations, status {status}")
    if status:
        raise SystemExit(1)


# --------------------------------------------------------------------------- #
def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.case:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py --case needs a CUDA device")
        profile_case(args)
        return
    if args.batch is None:
        args.batch = BATCH
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 path has no CPU fallback")

    import torch.distributed as dist
    from auto_infer_b200 import ops, synth
    from auto_infer_b200.context_parallel import ContextParallelDecode
    from auto_infer_b200.forward_context import ForwardContext
    from auto_infer_b200.gqa import B200GqaBackend

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL's own log (NCCL_DEBUG as the caller set it) goes to stderr, so that rank 0's
        # stdout carries the JSON line only
        if os.environ.get("NCCL_DEBUG") and not os.environ.get("NCCL_DEBUG_FILE"):
            os.environ["NCCL_DEBUG_FILE"] = "/dev/stderr"
        dist.init_process_group("nccl", device_id=device)

    # ---- workload: this rank's slice of every sequence's pages -------------
    b = synth.config5(device, cp_rank=rank, cp_size=world, context=args.context, batch=args.batch)
    k_cache, v_cache = b.kv_cache[0], b.kv_cache[1]
    global_kv = [args.context] * args.batch
    exchange, exchange_kind = None, "none"
    if world > 1:
        exchange_kind = "nccl all-gather + merge kernel"
        if args.exchange != "nccl":
            try:
                from auto_infer_b200.context_parallel import PeerExchange
                exchange = PeerExchange(args.batch * b.n_q, b.head_dim, device)
                exchange_kind = "fused peer-to-peer push + merge kernel"
            except Exception as exc:          # no symmetric memory on this box: keep the NCCL exchange
                if args.exchange == "p2p":
                    raise
                print(f"peer exchange unavailable ({exc!r}); using NCCL", file=sys.stderr)
    cpd = ContextParallelDecode(b.cu_seqlens_q, global_kv, b.n_q, b.n_kv, b.head_dim, b.block_size,
                                device, cp_rank=rank, cp_size=world, exchange=exchange)
    assert cpd.local_kv == b.seqlens_kv
    owner_of_new_token = (rank == world - 1)        # the rank holding position context-1

    def write_new_token():
        if owner_of_new_token:
            ops.reshape_and_cache(b.k_new, b.v_new, k_cache, v_cache, b.slot_mapping)

    def one_launch_step():
        # one GPU: slot write and attention are one launch (the CTA that streams the tile the
        # new row falls in stores it); this is also the dominant kernel the roofline is about
        return ops.paged_decode_gqa_write(b.q, b.k_new, b.v_new, b.slot_mapping, k_cache, v_cache,
                                          b.block_table, cpd.meta.decode, b.scale, out=cpd.out)

    def layer_step():
        if world == 1:
            return one_launch_step()
        write_new_token()
        return cpd.attend(b.q, k_cache, v_cache, b.block_table, b.scale)

    def decode_only():
        if world > 1:
            ops.paged_decode_gqa(b.q, k_cache, v_cache, b.block_table, cpd.meta.decode, b.scale,
                                 out=cpd.partial.o, lse_out=cpd.partial.lse)
        else:
            one_launch_step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Layer-steps are recorded into CUDA graphs of `unroll` steps each and replayed: the
    # engine's graph mode replays all layers of a model from one graph the same way.
    unroll = 1 if args.no_graph else unroll_for(args.steps)
    barrier()                                       # ranks lined up before the first exchange
    graph = None if args.no_graph else capture_graph(layer_step, device, unroll)
    kgraph = None if args.no_graph else capture_graph(decode_only, device, unroll)

    def run_steps(n):
        if graph is None:
            for _ in range(n):
                layer_step()
        else:
            for _ in range(n // unroll):
                graph.replay()

    def run_kernel(n):
        if kgraph is None:
            for _ in range(n):
                decode_only()
        else:
            for _ in range(n // unroll):
                kgraph.replay()

    total_kv_bytes = args.batch * args.context * 2 * b.n_kv * b.head_dim * 2
    local_kv_bytes = b.kv_bytes()

    # ---- timed region: batches of exactly K steps, device events, max over ranks --------
    warm = max(args.warmup, 3)
    barrier()
    run_steps(unroll * math.ceil(warm / unroll))
    barrier()
    probe = timed_batches(run_steps, args.steps, barrier, 1)[0]
    # enough batches for half a second of timed work (clock samples come every 20 ms)
    n_batches = int(min(200, max(10, math.ceil(500.0 / max(probe, 1e-3)))))
    if world > 1:
        nb = torch.tensor([n_batches], device=device)
        dist.all_reduce(nb, op=dist.ReduceOp.MAX)
        n_batches = int(nb.item())
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)                      # let the sampler come up before the timed region
    batches = timed_batches(run_steps, args.steps, barrier, n_batches)
    ms_per_step = max_over_ranks(statistics.median(batches), device, world) / args.steps
    value = total_kv_bytes / (ms_per_step * 1e-3) / 1e12
    launches_per_step = 1 if world == 1 else (1 if owner_of_new_token else 0) + 2

    # ---- the dominant kernel alone, replayed the same way, for the roofline -------------
    run_kernel(unroll * 2)
    kbatches = timed_batches(run_kernel, args.steps, barrier, max(5, n_batches // 4))
    my_kernel_ms = statistics.median(kbatches) / args.steps
    kernel_ms = max_over_ranks(my_kernel_ms, device, world)
    clocks = sampler.stop() if rank == 0 else None
    peak, peak_kind = measured_peak()
    algorithmic = local_kv_bytes + 2 * b.q.numel() * 2
    achieved = algorithmic / (kernel_ms * 1e-3) / 1e9
    traffic = ncu_traffic("c5") if world == 1 else None

    # ---- where a context-parallel step's time goes (per rank) ---------------------------
    breakdown = None
    if world > 1:
        def exchange_only():
            if exchange is not None:
                ops.cp_exchange_combine(cpd.partial.flat, exchange.recv_ptrs_dev, exchange.state, rank, world,
                                        cpd.partial.rows, cpd.partial.head_dim, cpd.out.view(cpd.partial.rows, -1))
            else:
                from auto_infer_b200.context_parallel import all_gather_partials, split_gathered
                gathered = all_gather_partials(cpd.partial.flat, None)
                o_parts, lse_parts = split_gathered(gathered, cpd.partial.rows, cpd.partial.head_dim)
                ops.lse_combine(o_parts, lse_parts, out=cpd.out.view(cpd.partial.rows, -1))

        barrier()
        xgraph = exchange_only if args.no_graph else capture_graph(exchange_only, device, unroll)

        def run_exchange(n):
            if args.no_graph:
                for _ in range(n):
                    exchange_only()
            else:
                for _ in range(n // unroll):
                    xgraph.replay()

        run_exchange(unroll * 2)
        xb = timed_batches(run_exchange, args.steps, barrier, 5)
        my_exchange_us = statistics.median(xb) / args.steps * 1e3
        write_us = 0.0
        if owner_of_new_token:
            wgraph = capture_graph(write_new_token, device, unroll)
            torch.cuda.synchronize()
            wt = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.steps // unroll):
                    wgraph.replay()
                e1.record()
                torch.cuda.synchronize()
                wt.append(e0.elapsed_time(e1) / args.steps * 1e3)
            write_us = statistics.median(wt)
        mine = torch.tensor([my_kernel_ms * 1e3, my_exchange_us, write_us], device=device, dtype=torch.float64)
        allr = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        dec = [round(float(t[0]), 2) for t in allr]
        breakdown = {"decode_us_per_rank": dec,
                     "decode_us_spread": round(max(dec) - min(dec), 2),
                     "exchange_us_per_rank": [round(float(t[1]), 2) for t in allr],
                     "write_us_owner_rank": round(float(allr[-1][2]), 2),
                     "step_us": round(ms_per_step * 1e3, 2),
                     "note": "each leg replayed alone from its own graph; the exchange leg contains "
                             "the wait for the slowest peer of that leg"}

    # ---- does the timed computation give the right rows?  (untimed) ---------------------
    verified, verify_how = None, None
    try:
        if world == 1:
            from oracle import paged_attention_oracle as orc
            run_steps(unroll)
            torch.cuda.synchronize()
            seq = 0
            ids = b.block_table[seq].long()
            bt = torch.arange(ids.numel(), dtype=torch.int32)[None]
            torch.set_num_threads(os.cpu_count() or 1)
            ref = orc.paged_attention(b.q[seq:seq + 1].cpu(), k_cache[ids].cpu(), v_cache[ids].cpu(), bt, [1],
                                      [b.seqlens_kv[seq]], b.scale, literal_max_kv=0)
            verified = scale_free_ok(cpd.out[seq:seq + 1].cpu(), ref)
            verify_how = "sequence 0 of the timed step against the CPU oracle, row-relative tolerance"
        else:
            # sequence 0's pages of every rank are gathered on rank 0, which runs the
            # single-GPU kernel over the whole sequence and compares the rows
            run_steps(unroll)
            torch.cuda.synchronize()
            ids = b.block_table[0].long()
            mine_k, mine_v = k_cache[ids].contiguous(), v_cache[ids].contiguous()
            ks = [torch.empty_like(mine_k) for _ in range(world)] if rank == 0 else None
            vs = [torch.empty_like(mine_v) for _ in range(world)] if rank == 0 else None
            dist.gather(mine_k, ks, dst=0)
            dist.gather(mine_v, vs, dst=0)
            if rank == 0:
                full_k, full_v = torch.cat(ks), torch.cat(vs)
                bt = torch.arange(full_k.shape[0], dtype=torch.int32, device=device)[None]
                plan1 = ops.DecodePlan([1], [args.context], b.n_q, b.n_kv, device)
                one = ops.paged_decode_gqa(b.q[0:1], full_k, full_v, bt, plan1, b.scale, out_f32=True)
                torch.cuda.synchronize()
                verified = scale_free_ok(cpd.out[0:1], one)
                verify_how = (f"sequence 0: the {world}-rank result against the single-GPU kernel run on "
                              "rank 0 over the gathered pages, row-relative tolerance")
                del full_k, full_v, ks, vs
    except Exception as exc:                  # verification must never take the measurement down
        verify_how = f"verification did not run: {exc!r}"

    # ---- end to end through the backend call with host buffers -------------
    # one backend object per staging set: each keeps its own refillable plan, so the plan of
    # step k + 1 can travel while the kernels of step k still read theirs
    from auto_infer_b200.metadata import step_metadata
    # (context parallel: two attention objects over the one peer exchange, for the same reason)
    cpds = [cpd]
    if world > 1:
        cpds.append(ContextParallelDecode(b.cu_seqlens_q, global_kv, b.n_q, b.n_kv, b.head_dim, b.block_size,
                                          device, cp_rank=rank, cp_size=world, exchange=exchange))
    backends = [B200GqaBackend(b.n_q, b.n_kv, b.head_dim, b.scale, 1, device, torch.bfloat16) for _ in range(2)]
    # The step's inputs live in one pinned staging arena on the host (as an engine's input
    # stager keeps them) and travel in one copy; the tensors below are views into it.
    srcs = {k: getattr(b, k).cpu().contiguous() for k in ("q", "k_new", "v_new", "slot_mapping", "block_table")}
    offs, total = {}, 0
    for k, v in srcs.items():
        offs[k] = total
        total += (v.numel() * v.element_size() + 255) // 256 * 256
    host_arena = torch.empty(total, dtype=torch.uint8).pin_memory()
    depth = 2
    dev_arenas = [torch.empty(total, dtype=torch.uint8, device=device) for _ in range(depth)]

    def _view(arena, k):
        v = srcs[k]
        n = v.numel() * v.element_size()
        return arena[offs[k]:offs[k] + n].view(v.dtype).view(v.shape)

    host = {k: _view(host_arena, k) for k in srcs}
    for k in srcs:
        host[k].copy_(srcs[k])
    devs = [{k: _view(arena, k) for k in srcs} for arena in dev_arenas]
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    # Two staging sets (device input arena, pinned result buffer) and two copy streams, as an
    # engine's input stager and output thread work: step k + 1's inputs travel while step k's
    # kernels run, step k's result travels while step k + 1's kernels run, and a set is reused
    # when its result has reached the host (step k + 2).  Every step still copies its inputs in
    # and its result out inside the timed region, and the region ends with all results on the
    # host.
    out_hosts = [torch.empty(b.q.shape, dtype=torch.bfloat16).pin_memory() for _ in range(depth)]
    out_done = [None] * depth
    d2h = out_hosts[0].numel() * out_hosts[0].element_size()
    e2e_count = [0]
    # Copy streams pay when the device step is long against the host's own work per step; a
    # step of ~100 us (eight ranks) is bound by the host, where two more stream switches per
    # step cost more than the copies they hide: there everything stays on one stream.
    overlap_copies = ms_per_step > 0.15               # the same on all ranks (max over ranks)
    main_stream = torch.cuda.current_stream(device)
    copy_in = torch.cuda.Stream(device) if overlap_copies else main_stream
    copy_out = torch.cuda.Stream(device) if overlap_copies else main_stream

    def e2e_compute(i, dev, ctx):
        if world == 1:
            if ctx is None:
                ctx = ForwardContext(None, None, dev["slot_mapping"], dev["block_table"],
                                     b.cu_seqlens_q, b.seqlens_kv, None, backends[i], [b.kv_cache], True)
            return backends[i].paged_attention(0, dev["q"], dev["k_new"], dev["v_new"], ctx)
        if owner_of_new_token:
            ops.reshape_and_cache(dev["k_new"], dev["v_new"], k_cache, v_cache, dev["slot_mapping"])
        return cpds[i].attend(dev["q"], k_cache, v_cache, dev["block_table"], b.scale)

    def e2e_step():
        # a step as the engine drives it: inputs from the host, this step's lengths planned on
        # the host (into buffers the backend keeps), kernels, result back to the host
        i = e2e_count[0] % depth
        e2e_count[0] += 1
        if out_done[i] is not None:
            out_done[i].synchronize()                # set i is free: its result is on the host
        dev = devs[i]
        done = torch.cuda.Event()
        if not overlap_copies:                       # everything in order on the compute stream
            dev_arenas[i].copy_(host_arena, non_blocking=True)
            if world > 1:
                cpds[i].replan(b.cu_seqlens_q, global_kv)
            out_hosts[i].copy_(e2e_compute(i, dev, None), non_blocking=True)
            done.record()
            out_done[i] = done
            return
        arrived, computed = torch.cuda.Event(), torch.cuda.Event()
        ctx = None
        with torch.cuda.stream(copy_in):             # the step's plan is built and uploaded beside its inputs
            dev_arenas[i].copy_(host_arena, non_blocking=True)
            if world == 1:
                ctx = ForwardContext(None, None, dev["slot_mapping"], dev["block_table"],
                                     b.cu_seqlens_q, b.seqlens_kv, None, backends[i], [b.kv_cache], True)
                step_metadata(ctx, b.n_q, b.n_kv, b.head_dim, device, pool=backends[i]._meta_pool,
                              split_mixed=backends[i]._overlap_mixed)
            else:
                cpds[i].replan(b.cu_seqlens_q, global_kv)
            arrived.record(copy_in)
        main_stream.wait_event(arrived)
        o = e2e_compute(i, dev, ctx)
        computed.record(main_stream)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(computed)
            out_hosts[i].copy_(o, non_blocking=True)
            o.record_stream(copy_out)
            done.record(copy_out)
        out_done[i] = done

    def e2e_drain():
        for ev in out_done:
            if ev is not None:
                ev.synchronize()

    for _ in range(3):
        e2e_step()
    e2e_drain()
    e2e_runs = []
    for _ in range(5):
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        e2e_drain()
        barrier()
        e2e_runs.append((time.perf_counter() - t0) * 1e3 / args.steps)
    e2e_ms = max_over_ranks(statistics.median(e2e_runs), device, world)
    e2e_value = total_kv_bytes / (e2e_ms * 1e-3) / 1e12
    status = ops.read_status(device)

    # ---- smaller configurations and the CPU baseline (rank 0, N = 1) --------
    side, cpu = {}, None
    if rank == 0 and world == 1:
        if not args.no_side_configs:
            for name in ("c1", "c2", "c3_b4", "c3_b16", "c3_b64", "c4"):
                side[name] = side_config(name, device)
                torch.cuda.empty_cache()
        if not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            cb, orc = cpu_baseline_sample(args, threads)
            t0 = time.perf_counter()
            reps = 0
            while reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 50):
                orc.write_kv(cb.k_new, cb.v_new, cb.kv_cache[0], cb.kv_cache[1], cb.slot_mapping.tolist())
                orc.paged_attention(cb.q, cb.kv_cache[0], cb.kv_cache[1], cb.block_table,
                                    cb.cu_seqlens_q, cb.seqlens_kv, cb.scale, literal_max_kv=0)
                reps += 1
            dt = (time.perf_counter() - t0) / reps
            cpu = {"value": cb.kv_bytes() / dt / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"1 of {args.batch} sequences ({args.context} tokens, all heads), "
                             f"{reps} repetitions, {dt * 1e3:.0f} ms each"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_per_step,
            "us_per_layer_step": ms_per_step * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": dict(workload_config(args, world), exchange=exchange_kind),
            "timing": {"batches": n_batches, "steps_per_batch": args.steps, "reported": "median batch",
                       "layer_steps_per_graph": unroll if not args.no_graph else 0,
                       "batch_ms_min": min(batches), "batch_ms_max": max(batches)},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_kind": peak_kind,
                         "kernel": "paged_decode_gqa_kernel (cut pairs merged in-kernel)",
                         "kernel_us": kernel_ms * 1e3, "algorithmic_bytes": algorithmic,
                         "frac_of_nominal_8tbs": achieved / 8000.0,
                         "timed": "same graph replay as the step, the attention kernel alone"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "copies": ("on two copy streams, overlapped with the neighbouring steps' kernels" if overlap_copies
                               else "on the compute stream (host-bound step)"),
                    "results_in_flight": depth},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks, "device_status": status,
            "verified": verified, "verified_how": verify_how,
        }
        if breakdown is not None:
            line["cp_breakdown"] = breakdown
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if side:
            line["other_configs"] = side
        print(json.dumps(line), flush=True)
    if world > 1:
        # graphs first (they hold the kernels' arguments), then the communicator
        graph = kgraph = None
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
