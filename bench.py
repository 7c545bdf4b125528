#!/usr/bin/env python
"""Benchmark of the paged-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One "step" is one layer-step of the path on the Qwen2.5-72B-shaped long-context
decode workload (64 q / 8 kv heads, head_dim 128, bf16, 128-token pages, batch
8, 131072 cached tokens per sequence): KV slot write of the step's token,
split-KV paged attention and, on N > 1 GPUs (context parallel: every rank holds
a contiguous 1/N of each sequence's pages), one all-gather of the per-rank
(o, lse) partials plus the log-sum-exp merge.  Total work is fixed as N grows
(strong scaling).  The metric is achieved HBM throughput over the algorithmic KV
bytes of the step, whole job; microseconds per layer-step are reported beside
it.  Rank 0 prints one JSON line.

``--impl reference`` times the reference's eager torch attention arithmetic
(restated for paged KV in oracle/) on the host cores, one sequence of the batch
per step.
"""
from __future__ import annotations

import argparse
import json
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
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--no-side-configs", action="store_true",
                    help="skip the kernel-only timings of the smaller configurations")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="auto", choices=["auto", "p2p", "nccl"],
                    help="context-parallel exchange: fused peer-to-peer kernel or NCCL all-gather")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the step's kernels one by one instead of replaying a CUDA graph")
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
def time_events(fn, steps, warmup, pre=None):
    """Per-iteration device times (ms) with CUDA events on the current stream."""
    for _ in range(warmup):
        if pre:
            pre()
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(steps):
        if pre:
            pre()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
    return out


def _graph_time(step, flush, iters=40):
    """Trimmed-mean / best device time (us) of ``step`` replayed from a CUDA graph, L2
    flushed before every replay (host launch overhead excluded)."""
    step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        step()
        with torch.cuda.graph(graph, stream=side):
            step()
    torch.cuda.synchronize()
    times = sorted(time_events(graph.replay, iters, 5, pre=flush.zero_))
    # CUDA event stamps tick every ~2 us on this part: the mean of the middle 60 % resolves
    # finer than the median of equally quantised samples
    core = times[len(times) // 5: len(times) - len(times) // 5]
    return statistics.fmean(core) * 1e3, times[0] * 1e3


def side_config(name, device, flush):
    """Kernel-only time of one of the other configurations (slot write +
    attention), with its roofline fractions against the measured peaks."""
    from auto_infer_b200 import ops, synth
    hbm_peak, _ = measured_peak()
    tensor_peak = measured_tensor_peak()
    if name.startswith("c3"):
        batch = int(name.split("_b")[1])
        b = synth.config3(batch, device)
        plan = ops.MlaDecodePlan(b.cu_seqlens_q, b.seqlens_kv, 16, device)
        out = torch.empty(b.num_tokens, 16, 512, dtype=torch.bfloat16, device=device)

        def step():
            ops.reshape_and_cache(b.k_new, None, b.kv_cache, None, b.slot_mapping)
            ops.mla_decode_absorbed(b.q, b.kv_cache, b.block_table, plan, b.scale, out=out)

        us, best = _graph_time(step, flush)
        bytes_ = sum(b.seqlens_kv) * 1152 + b.num_tokens * 16 * (576 + 512) * 2
        flops = sum(b.seqlens_kv) * 34816
        return {"us_per_layer_step": round(us, 2), "best_us": round(best, 2),
                "algorithmic_mb": round(bytes_ / 1e6, 2), "achieved_gbs": round(bytes_ / us / 1e3, 1),
                "hbm_frac": round(bytes_ / us / 1e3 / hbm_peak, 3), "bound": "hbm",
                "tflops": round(flops / us / 1e6, 1),
                "tensor_frac": round(flops / us / 1e6 / tensor_peak, 4), "batch": batch}
    if name == "c2":
        b = synth.config2(device)
        from auto_infer_b200.metadata import StepMetadata
        meta = StepMetadata(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, b.head_dim, device)
        out = torch.empty(b.q.shape, dtype=torch.bfloat16, device=device)
        k_cache, v_cache = b.kv_cache[0], b.kv_cache[1]

        def write():
            ops.reshape_and_cache(b.k_new, b.v_new, k_cache, v_cache, b.slot_mapping)

        def decode():
            ops.paged_decode_gqa(b.q, k_cache, v_cache, b.block_table, meta.decode, b.scale, out=out)

        def prefill():
            ops.paged_prefill_gqa(b.q, k_cache, v_cache, b.block_table, meta.prefill, b.scale, out=out)

        def step():
            write()
            decode()
            prefill()

        us, best = _graph_time(step, flush)
        us_dec, _ = _graph_time(decode, flush)
        us_pre, _ = _graph_time(prefill, flush)
        # causal-aware flops of the four 512-token chunks over prefixes 0/1024/2048/4096
        flops = sum(4 * 32 * 128 * (512 * p + 131328) for p in (0, 1024, 2048, 4096))
        dec_bytes = sum(b.seqlens_kv[:60]) * 4096 + 2 * 60 * 32 * 128 * 2
        return {"us_per_layer_step": round(us, 2), "best_us": round(best, 2),
                "decode_rows_us": round(us_dec, 2), "decode_rows_gbs": round(dec_bytes / us_dec / 1e3, 1),
                "decode_rows_hbm_frac": round(dec_bytes / us_dec / 1e3 / hbm_peak, 3),
                "prefill_chunks_us": round(us_pre, 2), "prefill_gflop": round(flops / 1e9, 2),
                "prefill_tflops": round(flops / us_pre / 1e6, 1),
                "prefill_tensor_frac": round(flops / us_pre / 1e6 / tensor_peak, 4),
                "bound": "tensor (chunks) + hbm (decode rows)", "tokens": b.num_tokens}
    b = synth.CONFIGS[name]().to(device)
    plan = ops.DecodePlan(b.cu_seqlens_q, b.seqlens_kv, b.n_q, b.n_kv, device)
    out = torch.empty(b.q.shape, dtype=torch.bfloat16, device=device)

    def step():
        ops.reshape_and_cache(b.k_new, b.v_new, b.kv_cache[0], b.kv_cache[1], b.slot_mapping)
        ops.paged_decode_gqa(b.q, b.kv_cache[0], b.kv_cache[1], b.block_table, plan, b.scale, out=out)

    us, best = _graph_time(step, flush)
    bytes_ = b.kv_bytes() + 2 * b.q.numel() * 2
    return {"us_per_layer_step": round(us, 2), "best_us": round(best, 2),
            "algorithmic_mb": round(bytes_ / 1e6, 2), "achieved_gbs": round(bytes_ / us / 1e3, 1),
            "hbm_frac": round(bytes_ / us / 1e3 / hbm_peak, 3), "bound": "hbm",
            "batch": len(b.seqlens_kv), "tokens": b.num_tokens}


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

    for _ in range(min(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = bytes_step / dt / 1e12
    sample = f"1 of {args.batch} sequences per step ({args.context} tokens, all 64 heads)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3,
        "us_per_layer_step_full_batch": dt * 1e6 * args.batch,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(args, 1),
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
def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
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
        # NCCL prints its version banner to stdout at VERSION/INFO level; rank 0's stdout must
        # carry the JSON line only
        if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "INFO", "TRACE") and \
                not os.environ.get("B200_BENCH_KEEP_NCCL_DEBUG"):
            os.environ["NCCL_DEBUG"] = "WARN"
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

    # the layer-step (slot write, attention, all-gather, merge) is recorded once into a
    # CUDA graph and replayed: the engine's graph mode does the same for whole decode steps
    graph = None
    if not args.no_graph:
        graph = cpd.capture(b.q, k_cache, v_cache, b.block_table, b.scale, before=write_new_token)

    def step():
        if graph is not None:
            graph.replay()
            return cpd.out
        write_new_token()
        return cpd.attend(b.q, k_cache, v_cache, b.block_table, b.scale)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    total_kv_bytes = args.batch * args.context * 2 * b.n_kv * b.head_dim * 2
    local_kv_bytes = b.kv_bytes()

    # ---- timed region: K steps, device events, max over ranks --------------
    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)                      # let the sampler come up before the timed region
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = total_kv_bytes / (ms_per_step * 1e-3) / 1e12
    launches_per_step = (1 if owner_of_new_token else 0) + 1 + \
        (1 if cpd.meta.decode.info.num_multi else 0) + (1 if world > 1 else 0)

    # ---- dominant kernel alone (decode + its merge), for the roofline -------
    if world > 1:
        out32 = cpd.partial
        kern = lambda: ops.paged_decode_gqa(b.q, k_cache, v_cache, b.block_table, cpd.meta.decode,
                                            b.scale, out=out32.o, lse_out=out32.lse)
    else:
        kern = lambda: ops.paged_decode_gqa(b.q, k_cache, v_cache, b.block_table, cpd.meta.decode,
                                            b.scale, out=cpd.out)
    ktimes = time_events(kern, args.steps, 3)
    kernel_ms = sum(ktimes) / len(ktimes)
    if world > 1:
        t = torch.tensor([kernel_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        kernel_ms = float(t.item())
    peak, peak_kind = measured_peak()
    algorithmic = local_kv_bytes + 2 * b.q.numel() * 2
    achieved = algorithmic / (kernel_ms * 1e-3) / 1e9
    traffic = ncu_traffic("c5") if world == 1 else None

    # ---- end to end through the backend call with host buffers -------------
    backend = B200GqaBackend(b.n_q, b.n_kv, b.head_dim, b.scale, 1, device, torch.bfloat16)
    # The step's inputs live in one pinned staging arena on the host (as an engine's input
    # stager keeps them) and travel in one copy; the tensors below are views into it.
    srcs = {k: getattr(b, k).cpu().contiguous() for k in ("q", "k_new", "v_new", "slot_mapping", "block_table")}
    offs, total = {}, 0
    for k, v in srcs.items():
        offs[k] = total
        total += (v.numel() * v.element_size() + 255) // 256 * 256
    host_arena = torch.empty(total, dtype=torch.uint8).pin_memory()
    dev_arena = torch.empty(total, dtype=torch.uint8, device=device)

    def _view(arena, k):
        v = srcs[k]
        n = v.numel() * v.element_size()
        return arena[offs[k]:offs[k] + n].view(v.dtype).view(v.shape)

    host = {k: _view(host_arena, k) for k in srcs}
    for k in srcs:
        host[k].copy_(srcs[k])
    dev = {k: _view(dev_arena, k) for k in srcs}
    out_host = torch.empty(b.q.shape, dtype=torch.bfloat16).pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step():
        dev_arena.copy_(host_arena, non_blocking=True)
        if world == 1:
            ctx = ForwardContext(None, None, dev["slot_mapping"], dev["block_table"],
                                 b.cu_seqlens_q, b.seqlens_kv, None, backend, [b.kv_cache], True)
            o = backend.paged_attention(0, dev["q"], dev["k_new"], dev["v_new"], ctx)
        else:
            plan = ContextParallelDecode(b.cu_seqlens_q, global_kv, b.n_q, b.n_kv, b.head_dim,
                                         b.block_size, device, cp_rank=rank, cp_size=world,
                                         exchange=exchange)
            if owner_of_new_token:
                ops.reshape_and_cache(dev["k_new"], dev["v_new"], k_cache, v_cache, dev["slot_mapping"])
            o = plan.attend(dev["q"], k_cache, v_cache, dev["block_table"], b.scale)
        out_host.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = total_kv_bytes / (e2e_ms * 1e-3) / 1e12
    status = ops.read_status(device)
    # the sampler ran from before the timed region to the end of the end-to-end loop
    clocks = sampler.stop() if rank == 0 else None

    # ---- smaller configurations and the CPU baseline (rank 0, N = 1) --------
    side, cpu = {}, None
    if rank == 0 and world == 1:
        if not args.no_side_configs:
            flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
            for name in ("c1", "c2", "c3_b4", "c3_b16", "c3_b64", "c4"):
                side[name] = side_config(name, device, flush)
                torch.cuda.empty_cache()
            del flush
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
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "us_per_layer_step": ms_per_step * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": dict(workload_config(args, world), exchange=exchange_kind),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_kind": peak_kind,
                         "kernel": "paged_decode_gqa_kernel (+ decode_merge_kernel, one C call)",
                         "kernel_us": kernel_ms * 1e3, "algorithmic_bytes": algorithmic,
                         "frac_of_nominal_8tbs": achieved / 8000.0},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks, "device_status": status,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if side:
            line["other_configs"] = side
        print(json.dumps(line), flush=True)
    if world > 1:
        # Tear down in dependency order: a CUDA graph that recorded NCCL kernels has to go
        # before its communicator, and the exit must not wait on peers that already left.
        graph = None
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
