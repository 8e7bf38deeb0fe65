"""Timings of the other kernels of the path, reported next to the headline decode number (bench.py "extra").

Each entry is the median of `reps` CUDA-event timings after warm-up, inputs resident in HBM, with the
algorithmic bytes or flops the figure is computed from.  Buffers are rotated or larger than L2 where the
working set would otherwise be served from L2.
"""
from __future__ import annotations

import statistics

import torch

from . import kernels as K
from .sharding import assign_sequences

HQ, HKV, D = 16, 4, 256
HK, HV, DK = 16, 32, 128


def _median_ms(fn, stream, warmup=5, reps=20, calls=1):
    """Median over `reps` of the CUDA-event time of `calls` consecutive fn() calls, per call.  calls > 1 keeps the
    stream fed, so that a kernel of a few microseconds is not measured as the host's launch latency."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    times = []
    for i in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for c in range(calls):
            fn(i * calls + c)
        b.record(stream)
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) / calls)
    return statistics.median(times), (statistics.pstdev(times) / statistics.mean(times) if len(times) > 1 else 0.0)


def _graph_ms(fn, stream, calls, warmup=3, reps=10):
    """Per-call device time of `calls` consecutive fn() calls captured into one CUDA graph and replayed: for kernels
    of a few microseconds, whose launch from Python costs more host time than they run."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for i in range(calls):
            fn(i)
    ms, cv = _median_ms(lambda i: graph.replay(), stream, warmup=2, reps=reps)
    return ms / calls, cv


def _bf16(gen, dev, *shape):
    return torch.randn(*shape, device=dev, generator=gen, dtype=torch.float32).to(torch.bfloat16)


def decode_contexts(dev, stream, hbm_peak, contexts=(4096, 131072), early_kv_fetch_contexts=(32768,)):
    """Single-sequence decode steps on caches visited round-robin.  For `early_kv_fetch_contexts` the same loop is
    also timed through rib200_online_attention_decode_early_kv_fetch: no step of the loop writes a cache row another
    one reads, which is what that entry point asks of the caller."""
    out = {}
    contexts = tuple(contexts) + tuple(c for c in early_kv_fetch_contexts if c not in contexts)
    gen = torch.Generator(device=dev).manual_seed(11)
    for ctx in contexts:
        rotation = max(2, min(16, -(-600_000_000 // (4096 * ctx))))
        shape = K.Qwen35AttentionShape(1, HQ, HKV, D, ctx, ctx - 1)
        plan = K.qwen35_online_decode_plan(shape, K.SPLIT_K_256, ctx)
        layout = K.qwen35_online_decode_workspace_layout(shape, plan.resolved_mode)
        caches = [_bf16(gen, dev, 2, HKV, ctx, D) for _ in range(rotation)]
        q, gate, k, v = _bf16(gen, dev, HQ, D), _bf16(gen, dev, HQ, D), _bf16(gen, dev, HKV, D), _bf16(gen, dev, HKV, D)
        o = torch.zeros(HQ, D, device=dev, dtype=torch.bfloat16)
        ws = torch.zeros(layout.bytes // 4, device=dev)

        def fn(i):
            K.qwen35_online_attention_decode(q, k, v, gate, o, caches[i % rotation], caches[0].numel() * 2, ws,
                                             layout.bytes, shape, K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, plan, None,
                                             stream)

        # steps replayed from one CUDA graph (how the reference's executor runs decode steps); for the long contexts
        # also launched one by one from the host, eight between two events
        ms, cv = _graph_ms(fn, stream, max(8, rotation))
        nbytes = 4096 * ctx + 24576
        out[f"decode_ctx{ctx}"] = {"ms": ms, "cv": cv, "bytes": nbytes, "GB/s": nbytes / ms / 1e6,
                                   "frac_of_measured_hbm": nbytes / ms / 1e6 / hbm_peak, "caches_rotated": rotation,
                                   "launch": "cuda graph replay"}
        if ctx > 8192:
            out[f"decode_ctx{ctx}"]["ms_direct_launches"] = _median_ms(fn, stream, warmup=5, reps=10, calls=8)[0]
        if ctx in early_kv_fetch_contexts:
            def fn_early(i):
                K.online_attention_decode_early_kv_fetch(q, k, v, gate, o, caches[i % rotation], caches[0].numel() * 2,
                                                         ws, layout.bytes, shape, K.DTYPE_BF16, K.KV_BF16,
                                                         K.HEAD_MAJOR, plan, stream)

            ms, cv = _graph_ms(fn_early, stream, max(8, rotation))
            out[f"decode_ctx{ctx}_early_kv_fetch"] = {
                "ms": ms, "cv": cv, "bytes": nbytes, "GB/s": nbytes / ms / 1e6,
                "frac_of_measured_hbm": nbytes / ms / 1e6 / hbm_peak, "launch": "cuda graph replay",
                "ms_direct_launches": _median_ms(fn_early, stream, warmup=5, reps=10, calls=8)[0]}
        del caches
    return out


def batched_serving_decode(dev, stream, hbm_peak, batch=64, lo=1024, hi=32768, seed=0xB2000004):
    """64 ragged sequences: one attention decode step + one gated-delta decode step per sequence."""
    gen = torch.Generator(device=dev).manual_seed(seed)
    cpu_gen = torch.Generator().manual_seed(seed)
    lengths = torch.randint(lo, hi + 1, (batch,), generator=cpu_gen).tolist()
    caps = [-(-n // 256) * 256 for n in lengths]
    largest = max(caps)
    caches = [_bf16(gen, dev, 2, HKV, c, D) for c in caps]
    ptrs = torch.tensor([c.data_ptr() for c in caches], device=dev, dtype=torch.int64)
    dcaps = torch.tensor(caps, device=dev, dtype=torch.int32)
    dpos = torch.tensor([n - 1 for n in lengths], device=dev, dtype=torch.int32)
    q, gate = _bf16(gen, dev, batch, HQ, D), _bf16(gen, dev, batch, HQ, D)
    k, v = _bf16(gen, dev, batch, HKV, D), _bf16(gen, dev, batch, HKV, D)
    o = torch.zeros(batch, HQ, D, device=dev, dtype=torch.bfloat16)
    ws_bytes = K.batched_decode_workspace_bytes(batch, largest)
    ws = torch.zeros(ws_bytes // 4, device=dev)
    states = [torch.zeros(HV, DK, DK, device=dev) for _ in range(batch)]
    sptrs = torch.tensor([s.data_ptr() for s in states], device=dev, dtype=torch.int64)
    gq = torch.nn.functional.normalize(torch.randn(batch, HK, DK, device=dev, generator=gen), dim=-1)
    gk = torch.nn.functional.normalize(torch.randn(batch, HK, DK, device=dev, generator=gen), dim=-1)
    gq, gk = (gq / DK ** 0.5).to(torch.bfloat16), gk.to(torch.bfloat16)
    gv = _bf16(gen, dev, batch, HV, DK)
    beta = torch.sigmoid(torch.randn(batch, HV, device=dev, generator=gen))
    logd = -torch.nn.functional.softplus(torch.randn(batch, HV, device=dev, generator=gen))
    go = torch.zeros(batch, HV, DK, device=dev)

    def attn(i):
        K.batched_decode_attention(q, k, v, gate, o, ptrs, dcaps, dpos, batch, largest, ws, ws_bytes, stream)

    def gdn(i):
        K.batched_gdn_decode(gq, gk, gv, beta, logd, sptrs, go, batch, HK, HV, stream)

    def both(i):
        attn(i)
        gdn(i)

    # the same contexts served from a pool of 256-token pages handed out in shuffled order
    blocks = [c // K.PAGE_TOKENS for c in caps]
    pool_pages = sum(blocks)
    pool = _bf16(gen, dev, pool_pages, 2, HKV, K.PAGE_TOKENS, D)
    order = torch.randperm(pool_pages, generator=cpu_gen).tolist()
    table_rows, handed = [], 0
    for n in blocks:
        table_rows.append(order[handed:handed + n] + [0] * (max(blocks) - n))
        handed += n
    tables = torch.tensor(table_rows, device=dev, dtype=torch.int32)

    def paged(i):
        K.paged_decode_attention(q, k, v, gate, o, pool, pool_pages, tables, max(blocks), dpos, batch, ws, ws_bytes,
                                 stream)

    attn_bytes = sum(4096 * n + 24576 for n in lengths)
    gdn_bytes = batch * 2 * HV * DK * DK * 4
    res = {"sequences": batch, "total_context_tokens": sum(lengths)}
    for name, fn, nbytes in (("attention", attn, attn_bytes), ("attention_paged", paged, attn_bytes),
                             ("gdn_decode", gdn, gdn_bytes), ("attention+gdn_decode", both, attn_bytes + gdn_bytes)):
        ms, cv = _median_ms(fn, stream, warmup=3, reps=10, calls=4)
        res[name] = {"ms": ms, "cv": cv, "bytes": nbytes, "GB/s": nbytes / ms / 1e6,
                     "frac_of_measured_hbm": nbytes / ms / 1e6 / hbm_peak}
    return res


def batched_gdn_decode_only(dev, stream, hbm_peak, batch=64):
    """The gated-delta half of the serving step alone (64 sequences' FP32 states, 134 MB read and written): small
    enough to profile."""
    gen = torch.Generator(device=dev).manual_seed(0xB2000005)
    states = [0.05 * torch.randn(HV, DK, DK, device=dev, generator=gen) for _ in range(batch)]
    sptrs = torch.tensor([s.data_ptr() for s in states], device=dev, dtype=torch.int64)
    gq, gk = _bf16(gen, dev, batch, HK, DK), _bf16(gen, dev, batch, HK, DK)
    gv = _bf16(gen, dev, batch, HV, DK)
    beta = torch.rand(batch, HV, device=dev, generator=gen)
    logd = -torch.rand(batch, HV, device=dev, generator=gen)
    go = torch.zeros(batch, HV, DK, device=dev)

    def gdn(i):
        K.batched_gdn_decode(gq, gk, gv, beta, logd, sptrs, go, batch, HK, HV, stream)

    ms, cv = _median_ms(gdn, stream, warmup=3, reps=10, calls=4)
    nbytes = batch * 2 * HV * DK * DK * 4
    return {"sequences": batch, "ms": ms, "cv": cv, "bytes": nbytes, "GB/s": nbytes / ms / 1e6,
            "frac_of_measured_hbm": nbytes / ms / 1e6 / hbm_peak}


def gdn_layer(dev, stream, hbm_peak, tensor_peak, tokens=4096, decode_steps=128):
    """configs[3]: chunked prefill over `tokens`, then `decode_steps` recurrent steps on the same state."""
    gen = torch.Generator(device=dev).manual_seed(13)
    total = tokens + decode_steps
    q = torch.nn.functional.normalize(torch.randn(total, HK, DK, device=dev, generator=gen), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(total, HK, DK, device=dev, generator=gen), dim=-1)
    q, k = (q / DK ** 0.5).to(torch.bfloat16), k.to(torch.bfloat16)
    v = _bf16(gen, dev, total, HV, DK)
    beta = torch.sigmoid(torch.randn(total, HV, device=dev, generator=gen))
    logd = -torch.nn.functional.softplus(torch.randn(total, HV, device=dev, generator=gen))
    state = torch.zeros(HV, DK, DK, device=dev)
    out = torch.zeros(total, HV, DK, device=dev)
    ws_bytes = K.gdn_core_workspace_bytes(tokens, HK, HV, DK, DK)
    ws = torch.zeros(max(ws_bytes // 4, 4), device=dev)

    def prefill(i):
        state.zero_()
        K.gdn_core(q, k, v, beta, logd, state, out, ws, ws_bytes, tokens, HK, HV, DK, DK, K.DTYPE_BF16, stream)

    def decode(i):
        t = tokens + (i % decode_steps)
        K.gdn_core(q[t], k[t], v[t], beta[t], logd[t], state, out[t], None, 0, 1, HK, HV, DK, DK, K.DTYPE_BF16, stream)

    chunk = 64
    flops = (tokens // chunk) * HV * (2 * chunk * chunk * (3 * DK + 2 * DK) + 6 * chunk * DK * DK)
    ms, cv = _median_ms(prefill, stream, warmup=3, reps=10)
    res = {"prefill": {"tokens": tokens, "ms": ms, "cv": cv, "flops": flops, "TFLOP/s": flops / ms / 1e9,
                       "frac_of_measured_bf16_peak": flops / ms / 1e9 / tensor_peak,
                       "note": "time includes a 2 MiB state memset"}}
    # a step is a few microseconds of device time, less than one launch from Python costs on the host
    ms, cv = _graph_ms(decode, stream, decode_steps, warmup=3, reps=8)
    nbytes = 2 * HV * DK * DK * 4
    res["decode_step"] = {"ms": ms, "cv": cv, "bytes": nbytes, "effective GB/s": nbytes / ms / 1e6,
                          "steps_per_graph": decode_steps,
                          "note": "single sequence: the 2 MiB state is L2-resident, this is latency not HBM bandwidth"}
    return res


def gdn_packed_layer(dev, stream, hbm_peak, tensor_peak, tokens=4096, decode_steps=128, width=4):
    """The reference's own entry point, qwen35_gated_delta: packed input [q | k | v | b | a | z] per token in BF16,
    FP32 weights, causal conv of `width` + SiLU, L2 norm, gates, the recurrence, RMSNorm * SiLU(z).  Prefill over
    `tokens` (states reset in front of every call), then single-token calls replayed from a graph."""
    gen = torch.Generator(device=dev).manual_seed(31)
    hidden = HV * DK
    conv_dim = 2 * HK * DK + hidden
    stride = conv_dim + 2 * HV + hidden
    packed = _bf16(gen, dev, tokens + decode_steps, stride)
    conv_w = 0.3 * torch.randn(conv_dim, width, device=dev, generator=gen)
    rec_a = -torch.exp(0.3 * torch.randn(HV, device=dev, generator=gen))
    dt_bias = 0.5 * torch.randn(HV, device=dev, generator=gen)
    norm_w = 1.0 + 0.1 * torch.randn(DK, device=dev, generator=gen)
    conv_state = torch.zeros(conv_dim, width - 1, device=dev)
    rec_state = torch.zeros(HV, DK, DK, device=dev)
    out = torch.zeros(tokens + decode_steps, hidden, device=dev, dtype=torch.bfloat16)
    shape = K.GatedDeltaShape(tokens, hidden, HK, HV, DK, DK, width, 1.0e-6)
    one = K.GatedDeltaShape(1, hidden, HK, HV, DK, DK, width, 1.0e-6)
    ws_bytes = K.qwen35_gated_delta_workspace_bytes(shape)
    ws = torch.zeros(ws_bytes // 4, device=dev)
    policy, policy_one = K.qwen35_gated_delta_select_policy(shape, tokens), K.qwen35_gated_delta_select_policy(one, 1)

    def prefill(i):
        rec_state.zero_()
        conv_state.zero_()
        K.qwen35_gated_delta(packed, conv_w, rec_a, dt_bias, norm_w, out, conv_state, rec_state, ws, ws_bytes, shape,
                             K.DTYPE_BF16, K.DTYPE_F32, stream, policy)

    def decode(i):
        t = tokens + (i % decode_steps)
        K.qwen35_gated_delta(packed[t], conv_w, rec_a, dt_bias, norm_w, out[t], conv_state, rec_state, ws, ws_bytes,
                             one, K.DTYPE_BF16, K.DTYPE_F32, stream, policy_one)

    chunk = 64
    flops = (tokens // chunk) * HV * (2 * chunk * chunk * (3 * DK + 2 * DK) + 6 * chunk * DK * DK)
    io_bytes = tokens * stride * 2 + tokens * hidden * 2  # the packed input read once, the output written once
    ms, cv = _median_ms(prefill, stream, warmup=3, reps=10)
    res = {"prefill": {"tokens": tokens, "ms": ms, "cv": cv, "flops": flops, "TFLOP/s": flops / ms / 1e9,
                       "frac_of_measured_bf16_peak": flops / ms / 1e9 / tensor_peak, "io_bytes": io_bytes,
                       "io_GB/s": io_bytes / ms / 1e6,
                       "note": "whole layer call: prologue (conv, SiLU, norms, gates), chunked recurrence, epilogue; "
                               "time includes two state memsets"}}
    ms, cv = _graph_ms(decode, stream, decode_steps, warmup=3, reps=8)
    nbytes = 2 * HV * DK * DK * 4
    res["decode_step"] = {"ms": ms, "cv": cv, "bytes": nbytes, "effective GB/s": nbytes / ms / 1e6,
                          "steps_per_graph": decode_steps,
                          "note": "single sequence, state L2-resident: latency of the three launches of a layer step"}
    return res


def prefill_attention(dev, stream, tensor_peak, token_counts=(128, 512, 4096)):
    gen = torch.Generator(device=dev).manual_seed(17)
    res = {}
    cases = [(t, 0) for t in token_counts] + [(512, 3584)]
    for tokens, past in cases:
        max_ctx = past + tokens
        shape = K.Qwen35AttentionShape(tokens, HQ, HKV, D, max_ctx, past)
        q, gate = _bf16(gen, dev, tokens, HQ, D), _bf16(gen, dev, tokens, HQ, D)
        k, v = _bf16(gen, dev, tokens, HKV, D), _bf16(gen, dev, tokens, HKV, D)
        o = torch.zeros(tokens, HQ, D, device=dev, dtype=torch.bfloat16)
        cache = _bf16(gen, dev, 2, HKV, max_ctx, D)

        def fn(i):
            K.qwen35_online_attention_prefill(q, k, v, gate, o, cache, cache.numel() * 2, shape, K.DTYPE_BF16, K.KV_BF16,
                                              K.HEAD_MAJOR, stream)

        ms, cv = _graph_ms(fn, stream, 8) if tokens <= 512 else _median_ms(fn, stream, warmup=3, reps=10, calls=4)
        flops = 4 * HQ * D * (tokens * past + tokens * (tokens + 1) // 2)
        res[f"T{tokens}_past{past}"] = {"ms": ms, "cv": cv, "flops": flops, "TFLOP/s": flops / ms / 1e9,
                                        "frac_of_measured_bf16_peak": flops / ms / 1e9 / tensor_peak}
        if tokens == max(token_counts) and past == 0:
            # the same call on FP32 activations (what the reference's executor passes): Q is rounded to BF16 inside
            # the kernel, K and V by the append kernel in front of it
            q32, g32, k32, v32 = q.float(), gate.float(), k.float(), v.float()
            o32 = torch.zeros(tokens, HQ, D, device=dev)

            def fn32(i):
                K.qwen35_online_attention_prefill(q32, k32, v32, g32, o32, cache, cache.numel() * 2, shape, K.DTYPE_F32,
                                                  K.KV_BF16, K.HEAD_MAJOR, stream)

            ms, cv = _median_ms(fn32, stream, warmup=3, reps=10, calls=4)
            res[f"T{tokens}_past{past}_f32_activations"] = {
                "ms": ms, "cv": cv, "flops": flops, "TFLOP/s": flops / ms / 1e9,
                "frac_of_measured_bf16_peak": flops / ms / 1e9 / tensor_peak}
    return res


def attention_prologue(dev, stream, hbm_peak, tokens=4096, rotary=64):
    """The step in front of attention on FP32 projections (what the executor's full layers produce): query/gate
    split, RMSNorm with weight and partial RoPE on q and k, casts of gate and v to BF16 - as one launch, and as the
    reference's sequence of three calls (split, qk_norm_rope on q, qk_norm_rope on k) in FP32."""
    gen = torch.Generator(device=dev).manual_seed(29)
    packed = torch.randn(tokens, HQ, 2 * D, device=dev, generator=gen)
    k = torch.randn(tokens, HKV, D, device=dev, generator=gen)
    v = torch.randn(tokens, HKV, D, device=dev, generator=gen)
    qw = 1.0 + 0.1 * torch.randn(D, device=dev, generator=gen)
    kw = 1.0 + 0.1 * torch.randn(D, device=dev, generator=gen)
    bf = lambda *shape: torch.zeros(*shape, device=dev, dtype=torch.bfloat16)
    fq, fg, fk, fv = bf(tokens, HQ, D), bf(tokens, HQ, D), bf(tokens, HKV, D), bf(tokens, HKV, D)
    shape = K.Qwen35AttentionShape(tokens, HQ, HKV, D, tokens, 0)

    def fused(i):
        K.attention_prologue(packed, k, v, qw, kw, fq, fg, fk, fv, shape, rotary, 1.0e7, 1.0e-6, K.DTYPE_F32,
                             K.DTYPE_F32, K.DTYPE_BF16, stream)

    q0, g0 = torch.zeros(tokens, HQ, D, device=dev), torch.zeros(tokens, HQ, D, device=dev)
    qn, kn = torch.zeros_like(q0), torch.zeros_like(k)

    def three_calls(i):
        K.qwen35_split_full_query_gate(packed, q0, g0, tokens, HQ, D, K.DTYPE_F32, stream)
        K.qwen35_qk_norm_rope(q0, qw, qn, K.QkNormRopeShape(tokens, HQ, D, rotary, 0, 1.0e7), 1.0e-6, K.DTYPE_F32,
                              K.DTYPE_F32, stream)
        K.qwen35_qk_norm_rope(k, kw, kn, K.QkNormRopeShape(tokens, HKV, D, rotary, 0, 1.0e7), 1.0e-6, K.DTYPE_F32,
                              K.DTYPE_F32, stream)

    elements = tokens * (2 * HQ + 2 * HKV) * D
    fused_bytes = elements * 4 + elements * 2          # every projection element read once, written once as BF16
    three_bytes = tokens * HQ * D * 4 * (2 + 2 + 2) + tokens * HKV * D * 4 * 2  # split r+w, q r+w, k r+w
    ms, cv = _median_ms(fused, stream, warmup=3, reps=10, calls=4)
    ms3, cv3 = _median_ms(three_calls, stream, warmup=3, reps=10, calls=4)
    return {"tokens": tokens,
            "fused": {"ms": ms, "cv": cv, "bytes": fused_bytes, "GB/s": fused_bytes / ms / 1e6,
                      "frac_of_measured_hbm": fused_bytes / ms / 1e6 / hbm_peak},
            "three_calls_f32": {"ms": ms3, "cv": cv3, "bytes": three_bytes, "GB/s": three_bytes / ms3 / 1e6,
                                "frac_of_measured_hbm": three_bytes / ms3 / 1e6 / hbm_peak}}


def summarize(extra):
    """{name: [ms, fraction of the measured roofline]} for every timed entry of an `extra` object, flat and short."""
    flat = {}

    def walk(prefix, node):
        if not isinstance(node, dict):
            return
        ms = node.get("ms", node.get("ms_fused_peer_stores"))
        if isinstance(ms, float):
            frac = None
            for key, value in node.items():
                if key.startswith("frac_of_") and isinstance(value, float):
                    frac = value
                    break
            flat[prefix] = [round(ms, 5), None if frac is None else round(frac, 4)]
        for key, value in node.items():
            walk(f"{prefix}.{key}" if prefix else key, value)

    for section, node in extra.items():
        short = {"decode_attention": "dec", "batched_serving_decode": "serve", "gated_delta": "gdn", "gated_delta_layer": "gdn_layer",
                 "prefill_attention": "pre", "attention_prologue": "prol", "sharded_serving_decode": "serve_sharded",
                 "head_split_prefill": "head_split"}.get(section, section)
        walk(short, node)
    return flat


def run(dev, stream, hbm_peak, tensor_peak):
    extra = {}
    for name, fn in (("decode_attention", lambda: decode_contexts(dev, stream, hbm_peak)),
                     ("batched_serving_decode", lambda: batched_serving_decode(dev, stream, hbm_peak)),
                     ("gated_delta", lambda: gdn_layer(dev, stream, hbm_peak, tensor_peak)),
                     ("gated_delta_layer", lambda: gdn_packed_layer(dev, stream, hbm_peak, tensor_peak)),
                     ("prefill_attention", lambda: prefill_attention(dev, stream, tensor_peak)),
                     ("attention_prologue", lambda: attention_prologue(dev, stream, hbm_peak))):
        try:
            extra[name] = fn()
        except (K.Qwen35PrimitiveError, K.Qwen35DeltaError) as err:
            extra[name] = {"unavailable": str(err)}
        torch.cuda.empty_cache()
    return extra


def _timed_max_over_ranks(fn, stream, dist, dev, warmup=3, reps=10, calls=1):
    """Median over `reps` of the slowest rank's CUDA-event time per fn(i) call; a barrier precedes every repetition.
    calls > 1 puts that many consecutive calls between the two events, so that a step of tens of microseconds is not
    measured as the host's launch latency (only for steps that need no rank to wait for another)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    times = []
    for i in range(reps):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for c in range(calls):
            fn(i * calls + c)
        b.record(stream)
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / calls], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t.item()))
    return statistics.median(times)


def sharded_serving_decode(dev, stream, hbm_peak, rank, world, dist, batch=64, lo=1024, hi=32768, seed=0xB2000004):
    """The 64-sequence ragged decode step with the sequences sharded over the ranks: no collective on the data
    path, each rank steps its own sequences (attention + gated-delta decode)."""
    cpu_gen = torch.Generator().manual_seed(seed)
    lengths = torch.randint(lo, hi + 1, (batch,), generator=cpu_gen).tolist()
    owner, load = assign_sequences(lengths, world)
    mine = [n for n, r in zip(lengths, owner) if r == rank]
    gen = torch.Generator(device=dev).manual_seed(seed + rank)
    b = len(mine)
    caps = [-(-n // 256) * 256 for n in mine]
    largest = max(caps)
    caches = [_bf16(gen, dev, 2, HKV, c, D) for c in caps]
    ptrs = torch.tensor([c.data_ptr() for c in caches], device=dev, dtype=torch.int64)
    dcaps = torch.tensor(caps, device=dev, dtype=torch.int32)
    dpos = torch.tensor([n - 1 for n in mine], device=dev, dtype=torch.int32)
    q, gate = _bf16(gen, dev, b, HQ, D), _bf16(gen, dev, b, HQ, D)
    k, v = _bf16(gen, dev, b, HKV, D), _bf16(gen, dev, b, HKV, D)
    o = torch.zeros(b, HQ, D, device=dev, dtype=torch.bfloat16)
    ws_bytes = K.batched_decode_workspace_bytes(b, largest)
    ws = torch.zeros(ws_bytes // 4, device=dev)
    states = [torch.zeros(HV, DK, DK, device=dev) for _ in range(b)]
    sptrs = torch.tensor([s.data_ptr() for s in states], device=dev, dtype=torch.int64)
    gq = (torch.nn.functional.normalize(torch.randn(b, HK, DK, device=dev, generator=gen), dim=-1) / DK ** 0.5)
    gk = torch.nn.functional.normalize(torch.randn(b, HK, DK, device=dev, generator=gen), dim=-1)
    gq, gk, gv = gq.to(torch.bfloat16), gk.to(torch.bfloat16), _bf16(gen, dev, b, HV, DK)
    beta = torch.sigmoid(torch.randn(b, HV, device=dev, generator=gen))
    logd = -torch.nn.functional.softplus(torch.randn(b, HV, device=dev, generator=gen))
    go = torch.zeros(b, HV, DK, device=dev)

    def step(i):
        K.batched_decode_attention(q, k, v, gate, o, ptrs, dcaps, dpos, b, largest, ws, ws_bytes, stream)
        K.batched_gdn_decode(gq, gk, gv, beta, logd, sptrs, go, b, HK, HV, stream)

    ms = _timed_max_over_ranks(step, stream, dist, dev, calls=4)
    nbytes = sum(4096 * n + 24576 for n in lengths) + batch * 2 * HV * DK * DK * 4
    return {"sequences": batch, "ranks": world, "context_tokens_per_rank": load, "ms": ms, "bytes": nbytes,
            "GB/s": nbytes / ms / 1e6, "frac_of_measured_hbm_all_ranks": nbytes / ms / 1e6 / (hbm_peak * world),
            "collective": "none"}


def head_split_prefill(dev, stream, tensor_peak, rank, world, dist, tokens=4096):
    """Prefill split by KV-head group: a rank computes 16/world query heads (with 8 ranks two ranks share a KV
    head, each holding a copy).  Two ways to assemble [tokens][16][256] on every rank: one NCCL all-gather plus a
    layout permute (the baseline), and the fused form, whose epilogue stores every tile into all ranks' buffers
    over NVLink, followed by a device-side rendezvous."""
    from .peer import SharedBuffer

    hq = HQ // world
    hkv = max(1, HKV // world)
    gen = torch.Generator(device=dev).manual_seed(23 + rank)
    q, gate = _bf16(gen, dev, tokens, hq, D), _bf16(gen, dev, tokens, hq, D)
    k, v = _bf16(gen, dev, tokens, hkv, D), _bf16(gen, dev, tokens, hkv, D)
    cache = _bf16(gen, dev, 2, hkv, tokens, D)
    local = torch.zeros(tokens, hq, D, device=dev, dtype=torch.bfloat16)
    gathered = torch.zeros(world, tokens, hq, D, device=dev, dtype=torch.bfloat16)
    full = torch.zeros(tokens, HQ, D, device=dev, dtype=torch.bfloat16)
    shape = K.Qwen35AttentionShape(tokens, hq, hkv, D, tokens, 0)

    def kernel_only(i):
        K.qwen35_online_attention_prefill(q, k, v, gate, local, cache, cache.numel() * 2, shape, K.DTYPE_BF16, K.KV_BF16,
                                          K.HEAD_MAJOR, stream)

    def with_gather(i):
        kernel_only(i)
        dist.all_gather_into_tensor(gathered, local)
        full.view(tokens, world, hq, D).copy_(gathered.permute(1, 0, 2, 3))

    shared_out = SharedBuffer((tokens, HQ, D), torch.bfloat16, rank, world, dist, dev)
    shared_flags = SharedBuffer((world,), torch.int32, rank, world, dist, dev)
    epoch = [0]

    def fused(i):
        epoch[0] += 1
        K.online_attention_prefill_scatter(q, k, v, gate, shared_out.pointers, rank, HQ, rank * hq, cache,
                                           cache.numel() * 2, shape, K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, stream)
        K.peer_rendezvous(shared_flags.pointers, rank, epoch[0], stream)

    flops = 4 * HQ * D * (tokens * (tokens + 1) // 2)
    ms_kernel = _timed_max_over_ranks(kernel_only, stream, dist, dev)
    ms_total = _timed_max_over_ranks(with_gather, stream, dist, dev)
    ms_fused = _timed_max_over_ranks(fused, stream, dist, dev)
    torch.cuda.synchronize()
    same = bool(torch.equal(shared_out.local, full))
    status = K.device_status(stream)
    shared_flags.close()
    shared_out.close()
    if not same or status != 0:
        raise K.Qwen35PrimitiveError(f"fused head-split prefill differs from the all-gather form (status {status})")
    return {"tokens": tokens, "ranks": world, "query_heads_per_rank": hq, "kv_heads_per_rank": hkv,
            "ms_kernel": ms_kernel, "ms_with_all_gather": ms_total, "ms_fused_peer_stores": ms_fused, "flops": flops,
            "TFLOP/s": flops / ms_fused / 1e9, "TFLOP/s_with_all_gather": flops / ms_total / 1e9,
            "TFLOP/s_kernel_only": flops / ms_kernel / 1e9,
            "frac_of_measured_bf16_peak_all_ranks": flops / ms_fused / 1e9 / (tensor_peak * world),
            "fused_matches_all_gather": same,
            "collective": "fused: tile stores into every rank's buffer + device-side rendezvous; "
                          "baseline: ncclAllGather of outputs + layout permute",
            "peer_store_bytes_per_rank": (world - 1) * tokens * hq * D * 2}


def run_distributed(dev, stream, hbm_peak, tensor_peak, rank, world, dist):
    """Sections that need every rank (called by bench.py under torchrun)."""
    extra = {}
    for name, fn in (("sharded_serving_decode", lambda: sharded_serving_decode(dev, stream, hbm_peak, rank, world, dist)),
                     ("head_split_prefill", lambda: head_split_prefill(dev, stream, tensor_peak, rank, world, dist))):
        try:
            extra[name] = fn()
        except (K.Qwen35PrimitiveError, K.Qwen35DeltaError) as err:
            extra[name] = {"unavailable": str(err)}
        torch.cuda.empty_cache()
    return extra


def main(argv=None):
    """python -m raftinfer_b200.benchmarks [decode] [serving] [gdn] [gdnlayer] [gdndecode] [prefill] [prologue] [--tokens N]

    Prints one JSON object with the requested sections (all when none is named)."""
    import argparse
    import json
    import os

    ap = argparse.ArgumentParser()
    ap.add_argument("sections", nargs="*", default=[])
    ap.add_argument("--tokens", type=int, nargs="*", default=None, help="prefill token counts")
    ap.add_argument("--contexts", type=int, nargs="*", default=None, help="decode contexts")
    ap.add_argument("--gdn-tokens", type=int, default=4096, help="gated-delta prefill length")
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.cuda.set_stream(torch.cuda.Stream(device=dev))
    stream = torch.cuda.current_stream()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    peaks_path = os.path.join(root, "MEASURED_PEAKS.json")
    hbm, tensor = 6650.0, 1590.0
    if os.path.exists(peaks_path):
        peaks = json.load(open(peaks_path))
        hbm, tensor = float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"])
    want = set(args.sections) or {"decode", "serving", "gdn", "gdnlayer", "prefill", "prologue"}
    out = {}
    if "decode" in want:
        out["decode_attention"] = decode_contexts(dev, stream, hbm, tuple(args.contexts or (4096, 32768, 131072)))
    if "serving" in want:
        out["batched_serving_decode"] = batched_serving_decode(dev, stream, hbm)
    if "gdndecode" in want:
        out["batched_gdn_decode"] = batched_gdn_decode_only(dev, stream, hbm)
    if "gdn" in want:
        out["gated_delta"] = gdn_layer(dev, stream, hbm, tensor, tokens=args.gdn_tokens)
    if "gdnlayer" in want:
        out["gated_delta_layer"] = gdn_packed_layer(dev, stream, hbm, tensor, tokens=args.gdn_tokens)
    if "prefill" in want:
        out["prefill_attention"] = prefill_attention(dev, stream, tensor, tuple(args.tokens or (128, 512, 4096)))
    if "prologue" in want:
        out["attention_prologue"] = attention_prologue(dev, stream, hbm)
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
