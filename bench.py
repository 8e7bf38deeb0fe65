"""Benchmark of the attention / gated-delta hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--extras 0|1]

Headline metric: split-k GQA decode attention HBM GB/s (16 query / 4 KV heads, head_dim 256, BF16 head-major KV
cache, batch 1, context 32768, split 256).  A step is one decode call (partition + combine kernels) through the
C ABI; `value` counts the algorithmic bytes of the step (4096 * context + 24576: the live K and V rows once,
plus q, gate and the output) per second, inputs resident in HBM.  With N > 1 ranks every rank decodes its own
sequence with no collective (weak scaling) and `value` is the sum over ranks divided by the slowest rank's time.

`e2e` is the same step driven from host buffers: the new token's q, k, v, gate are copied from pinned host memory,
the call is made, and the output is read back, every step (the KV cache is device-resident state by the
reference's design, cpp/execution/qwen35_executor.cu:2027-2055).

`--impl reference` times the CPU path of the same workload on the host cores: the oracle's restatement of
cpp/reference/qwen35.cpp:316-370 (the reference's fused layer has no decode entry, so it cannot run this
workload).  This is the only leg that executes the oracle; the product path never does.

Synthetic operands: N(0,1) rounded to BF16, seeded; there is no dataset behind this path.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HQ, HKV, D = 16, 4, 256
CONTEXT = 32768
ROTATION = 4  # distinct KV caches visited round-robin: 4 x 134 MB > the 126 MB L2


def algorithmic_bytes(context: int) -> int:
    return 2 * HKV * context * D * 2 + 3 * HQ * D * 2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        peaks = json.load(open(path))
        return float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            if len(row) < 6:
                continue
            try:
                clocks.append(float(row[0]))
                maxima.append(float(row[1]))
            except ValueError:
                continue
            for name, cell in zip(names, row[2:6]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": sorted(reasons), "samples": len(clocks)}


def workload_config(context: int, cache_bytes: int):
    """The `config` object of the JSON line: the same for the GPU arm and for the CPU reference arm."""
    return {"workload": f"split-k decode attention, batch 1 per GPU, context {context}, 16q/4kv heads, head_dim 256, "
                        "BF16 head-major KV, partition 256",
            "l2": f"{ROTATION} KV caches of {cache_bytes / 1e6:.0f} MB visited round-robin (working set > L2)",
            "sharding": "one sequence per GPU, no collective"}


def profiled_traffic(context: int):
    """DRAM bytes (read + written) of one decode launch at `context`, from the ncu capture recorded beside its
    summary; None when no capture of that context is on record."""
    path = os.path.join(ROOT, "profiles", f"decode_partition_ctx{context}.json")
    try:
        record = json.load(open(path))
        return float(record["dram_bytes_read"]) + float(record["dram_bytes_write"])
    except (OSError, KeyError, ValueError):
        return None


def cpu_decode_baseline(context: int, repeats: int, threads: int):
    """Times the oracle's attention core (decode row over a BF16 head-major cache) on the host cores."""
    import numpy as np

    from oracle import bindings as ob
    from raftinfer_b200 import synth

    seed = 0xB2000020
    q = synth.round_bf16(synth.normal(seed, 0, (1, HQ, D)))
    gate = synth.round_bf16(synth.normal(seed, 1, (1, HQ, D)))
    rng = np.random.default_rng(seed)
    cache = synth.bf16_bits(rng.standard_normal((2, HKV, context, D), dtype=np.float32))
    ob.attention_core_cache(q, gate, cache, context, context - 1, threads=threads)  # warm
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        ob.attention_core_cache(q, gate, cache, context, context - 1, threads=threads)
        times.append(time.perf_counter() - t0)
    seconds = statistics.median(times)
    return algorithmic_bytes(context) / seconds / 1e9, seconds


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = max(1, len(os.sched_getaffinity(0)))
    steps = max(1, args.steps)
    for _ in range(max(0, args.warmup)):
        cpu_decode_baseline(CONTEXT, 1, threads)
    t0 = time.perf_counter()
    gbs, _ = cpu_decode_baseline(CONTEXT, steps, threads)
    total = time.perf_counter() - t0
    sample = f"{steps} full decode rows at context {CONTEXT} (16 q heads), oracle attention core, {threads} threads"
    line = {
        "impl": "reference", "metric": "split-k decode attention HBM GB/s", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": algorithmic_bytes(CONTEXT) / gbs / 1e6, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64 dot / f32 accumulate (CPU)", "data": "synthetic",
        "config": workload_config(CONTEXT, 2 * HKV * CONTEXT * D * 2),
        "arithmetic": "CPU reference arithmetic (one pass over the context, no split) on the host cores; the cache "
                      "rotation and the sharding named in config describe the GPU arm's run of the same workload",
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_seconds": total,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--extras", type=int, default=1, help="also time the other kernels of the path (rank 0, N=1)")
    ap.add_argument("--context", type=int, default=CONTEXT)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import numpy as np
    import torch

    from raftinfer_b200 import kernels as K

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    ctx = args.context
    torch.cuda.set_stream(torch.cuda.Stream(device=dev))  # the library rejects the NULL stream
    stream = torch.cuda.current_stream()

    gen = torch.Generator(device=dev)
    gen.manual_seed(0xB2000000 + rank)

    def randn_bf16(*shape):
        return torch.randn(*shape, device=dev, generator=gen, dtype=torch.float32).to(torch.bfloat16)

    shape = K.Qwen35AttentionShape(1, HQ, HKV, D, ctx, ctx - 1)
    plan = K.qwen35_online_decode_plan(shape, K.SPLIT_K_256, ctx)
    layout = K.qwen35_online_decode_workspace_layout(shape, plan.resolved_mode)
    caches = [randn_bf16(2, HKV, ctx, D) for _ in range(ROTATION)]
    cache_bytes = caches[0].numel() * 2
    q, gate = randn_bf16(HQ, D), randn_bf16(HQ, D)
    k_new, v_new = randn_bf16(HKV, D), randn_bf16(HKV, D)
    out = torch.zeros(HQ, D, device=dev, dtype=torch.bfloat16)
    ws = torch.zeros(layout.bytes // 4, device=dev)

    def step(i, q_=q, k_=k_new, v_=v_new, g_=gate):
        K.qwen35_online_attention_decode(q_, k_, v_, g_, out, caches[i % ROTATION], cache_bytes, ws, layout.bytes,
                                         shape, K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, plan, None, stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing ---------------------------------------------------------------
    # The clock sampler (an nvidia-smi process polling every 100 ms) is started before the warm-up and is already
    # delivering samples when the timed region begins: its start-up would otherwise fall into the region, which at
    # 20 steps lasts less than a millisecond.
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for i in range(warmup):
        step(i)
    barrier()
    if rank == 0:
        deadline = time.time() + 3.0
        i = 0
        while not sampler.rows and time.time() < deadline:  # keep the GPU busy until the first sample is in
            step(i)
            i += 1
            if i % 64 == 0:
                torch.cuda.synchronize()
    # The K steps are captured once in a CUDA graph and replayed, which is how the reference's executor runs its decode
    # steps (one captured graph per context bucket, cpp/execution/qwen35_executor.cu:2191-2225): the host then enqueues
    # one graph, not 2 K kernels.  If capture is refused the steps are launched one by one and the line says so.
    def run_block():
        for i in range(steps):
            step(i)

    launch_mode = "direct launches"
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run_block()
        graph.replay()  # first replay uploads the graph
        torch.cuda.synchronize()
        run_block = graph.replay
        launch_mode = f"{steps} steps captured in one CUDA graph and replayed"
    except Exception:  # capture refused (by torch, the driver or the library): fall back to launching every step
        torch.cuda.synchronize()

        def run_block():
            for i in range(steps):
                step(i)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record(stream)
    run_block()
    stop.record(stream)
    barrier()
    device_ms = max_over_ranks(start.elapsed_time(stop))
    # the same K steps five more times: the spread of the figure from block to block
    block_ms = []
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        run_block()
        b.record(stream)
        torch.cuda.synchronize()
        block_ms.append(a.elapsed_time(b) / steps)
    block_cv = statistics.pstdev(block_ms) / statistics.mean(block_ms)
    # keep the GPU under the same load a little longer so the clock sampler sees it
    t_end = time.time() + 0.6
    i = 0
    while time.time() < t_end:
        step(i)
        i += 1
        if i % 64 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    assert K.device_status(stream) == 0

    # ---- host-buffer timing (end to end) --------------------------------------------------------
    # the token's q | k | v | gate rows sit back to back in one pinned buffer: one copy brings them over
    rows = (HQ, HKV, HKV, HQ)
    host_packed = torch.randn(sum(rows), D, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).pin_memory()
    dev_packed = torch.empty_like(host_packed, device=dev)
    offsets = [sum(rows[:i]) for i in range(len(rows) + 1)]
    dev_in = [dev_packed[offsets[i]:offsets[i + 1]] for i in range(len(rows))]
    host_in = [host_packed]
    host_out = torch.empty(HQ, D, dtype=torch.bfloat16).pin_memory()
    e2e_steps = min(steps, 200)

    def e2e_step(i):
        # the library's host-buffer entry point: copy in, the decode step, copy out, synchronise
        K.online_attention_decode_from_host(host_packed, host_out, dev_packed, out, caches[i % ROTATION], cache_bytes,
                                            ws, layout.bytes, shape, K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, plan, None,
                                            stream)

    for i in range(3):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)
    barrier()

    step_bytes = algorithmic_bytes(ctx)
    value = world * step_bytes * steps / (device_ms * 1e-3) / 1e9
    e2e_value = world * step_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e9
    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    per_gpu_gbs = value / world

    line = {
        "metric": "split-k decode attention HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": device_ms / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 operands, f32 softmax/accumulate", "data": "synthetic",
        "config": workload_config(ctx, cache_bytes),
        "cv": block_cv, "block_ms_per_step": [round(ms, 6) for ms in block_ms],
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": sum(t.numel() * 2 for t in host_in),
                "d2h_bytes_per_step": host_out.numel() * 2, "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": 2 * steps,
        "launch": launch_mode,
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": hbm_peak, "unit": "GB/s",
                     "frac": per_gpu_gbs / hbm_peak, "traffic": None, "peak_kind": f"of {peak_kind}",
                     "frac_of_nominal_8000": per_gpu_gbs / 8000.0,
                     "note": "duration is the whole decode step (partition + combine kernels, overlapped by "
                             "programmatic dependent launch); the partition kernel moves all the algorithmic bytes"},
        "clocks": clocks,
    }
    line["roofline"]["traffic"] = profiled_traffic(ctx)

    if rank == 0 and world == 1:
        threads = max(1, len(os.sched_getaffinity(0)))
        gbs, seconds = cpu_decode_baseline(ctx, 3, threads)
        gbs1, seconds1 = cpu_decode_baseline(ctx, 3, 1)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": f"3 full decode rows at context {ctx} (median {seconds * 1e3:.0f} ms each), "
                                          "oracle restatement of cpp/reference/qwen35.cpp:316-370 over the BF16 cache; "
                                          "the threads are this harness's loop over query heads, the reference's "
                                          "own code is single-threaded",
                                "single_thread": {"value": gbs1, "unit": "GB/s", "cores": 1,
                                                  "sample": f"the same 3 rows on one thread (median "
                                                            f"{seconds1 * 1e3:.0f} ms each)"}}
        if args.extras:
            from raftinfer_b200 import benchmarks

            line["extra"] = benchmarks.run(dev, stream, hbm_peak, tensor_peak)
    if world > 1 and args.extras:
        from raftinfer_b200 import benchmarks

        extra = benchmarks.run_distributed(dev, stream, hbm_peak, tensor_peak, rank, world, dist)
        line["extra"] = extra
    if "extra" in line:
        # last in the line, so that a reader of its tail finds every kernel's figure: name -> [ms, fraction of the
        # measured roofline (HBM copy bandwidth or BF16 tensor peak, whichever bounds that kernel)]
        from raftinfer_b200 import benchmarks

        line["summary"] = benchmarks.summarize(line["extra"])
        line["summary"]["decode_ctx%d" % ctx] = [round(device_ms / steps, 5), round(per_gpu_gbs / hbm_peak, 4)]
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
