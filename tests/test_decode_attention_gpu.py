"""Split-k / single-block GQA decode attention on the GPU against the CPU oracle, through the C ABI.

Cases follow the reference's decode tests (cpp/tests/qwen35_cuda_attention_test.cu:768-1101: boundary contexts,
two consecutive steps through a device-side position, appended cache rows, split-k partials, untouched workspace
below the threshold) and extend them to N(0,1) operands and to the 4K / 32K / 128K contexts.  Tolerance for BF16
outputs against the fp32-accumulated oracle: max abs <= 3e-2 and relative L2 <= 1e-2; FP32 outputs are held to
1e-3 / 1e-4, which the two-term BF16 operand split is expected to meet."""
import numpy as np
import pytest
import torch

from oracle import bindings as ob
from raftinfer_b200 import kernels as K
from raftinfer_b200 import synth

from gpu_util import (D, HKV, HQ, NAN_BITS, act_tensor, bf16_tensor, cache_bits_of, cache_to_device, compare,
                      decode_operands, dev, gate_bf16_outputs, make_cache, to_numpy_f32)

pytestmark = pytest.mark.gpu
SENTINEL = -12345.0


def run_decode(ctx, max_ctx, mode, dtype, seed, device_position=False, q_scale=1.0, check_partials=True):
    pos = ctx - 1
    q, gate, k, v = decode_operands(seed, ctx, q_scale)
    shape = K.Qwen35AttentionShape(1, HQ, HKV, D, max_ctx, 0 if device_position else pos)
    plan = K.qwen35_online_decode_plan(shape, mode, ctx)
    layout = K.qwen35_online_decode_workspace_layout(shape, plan.resolved_mode)
    cache = cache_to_device(make_cache(k, v, max_ctx, pos))
    dq, dg = act_tensor(q, dtype), act_tensor(gate, dtype)
    dk, dv = act_tensor(k[pos], dtype), act_tensor(v[pos], dtype)
    out = torch.full((HQ, D), 7.0, device=dev(), dtype=torch.float32 if dtype == K.DTYPE_F32 else torch.bfloat16)
    ws = torch.full((max(layout.bytes // 4, 1),), SENTINEL, device=dev(), dtype=torch.float32)
    dpos = torch.tensor([pos], device=dev(), dtype=torch.int32) if device_position else None
    stream = torch.cuda.current_stream()
    K.qwen35_online_attention_decode(dq, dk, dv, dg, out, cache, cache.numel() * 2, ws if layout.bytes else None,
                                     layout.bytes, shape, dtype, K.KV_BF16, K.HEAD_MAJOR, plan, dpos, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0

    full = make_cache(k, v, max_ctx, ctx)
    got_cache = cache_bits_of(cache).reshape(full.shape)
    assert np.array_equal(got_cache, full), "cache rows: appended row must be the rounded input, others untouched"
    want = ob.attention_core_cache(q[None], gate[None], full, max_ctx, pos)[0]
    metrics = compare(to_numpy_f32(out), want)
    if dtype == K.DTYPE_F32:
        assert metrics["nonfinite"] == 0 and metrics["max_abs"] <= 1.0e-3 and metrics["rel_l2"] <= 1.0e-4, metrics
    else:
        gate_bf16_outputs(metrics)
        assert metrics["rel_l2"] <= 4.0e-3, metrics

    host_ws = ws.cpu().numpy()
    split = plan.partition_tokens != 0 and ctx >= plan.split_k_threshold_tokens
    if layout.bytes and not split:
        assert (host_ws == SENTINEL).all(), "workspace must stay untouched below the split-k threshold"
    if split and check_partials:
        pc = layout.partial_count
        max_parts = pc // HQ
        parts = -(-ctx // plan.partition_tokens)
        pmax = host_ws[:pc].reshape(HQ, max_parts)
        psum = host_ws[pc:2 * pc].reshape(HQ, max_parts)
        pval = host_ws[2 * pc:2 * pc + pc * D].reshape(HQ, max_parts, D)
        wmax, wsum, wval = ob.decode_partials(q, full, max_ctx, ctx, plan.partition_tokens)
        assert np.abs(pmax[:, :parts] - wmax[:, :parts]).max() <= 1.0e-4
        assert np.abs(psum[:, :parts] / wsum[:, :parts] - 1.0).max() <= 1.0e-4
        assert np.abs(pval[:, :parts] - wval[:, :parts]).max() <= 2.0e-3 * max(1.0, np.abs(wval[:, :parts]).max())
        assert (pmax[:, parts:] == SENTINEL).all() and (pval[:, parts:] == SENTINEL).all()
    return metrics


@pytest.mark.parametrize("ctx", [1, 2, 15, 16, 17, 255, 256, 257, 511, 512, 513, 777, 1024])
@pytest.mark.parametrize("dtype", [K.DTYPE_BF16, K.DTYPE_F32])
def test_split_k_256_boundary_contexts(ctx, dtype):
    run_decode(ctx, 1024, K.SPLIT_K_256, dtype, seed=0xB2000100 + ctx)


@pytest.mark.parametrize("ctx", [1, 511, 512, 513, 777, 1024])
def test_split_k_512(ctx):
    run_decode(ctx, 1024, K.SPLIT_K_512, K.DTYPE_BF16, seed=0xB2000200 + ctx)


@pytest.mark.parametrize("ctx", [1, 32, 128, 129, 300, 1000])
@pytest.mark.parametrize("dtype", [K.DTYPE_BF16, K.DTYPE_F32])
def test_single_block(ctx, dtype):
    run_decode(ctx, 1024, K.SINGLE_BLOCK, dtype, seed=0xB2000300 + ctx)


def test_cache_capacity_not_a_partition_multiple():
    run_decode(700, 777, K.SPLIT_K_256, K.DTYPE_BF16, seed=0xB2000310)
    run_decode(777, 777, K.SPLIT_K_256, K.DTYPE_F32, seed=0xB2000311)


@pytest.mark.parametrize("ctx", [4096, 32768, 131072])
def test_long_contexts(ctx):
    metrics = run_decode(ctx, ctx, K.SPLIT_K_256, K.DTYPE_BF16, seed=0xB2000400 + ctx, device_position=True,
                         check_partials=ctx <= 32768)
    assert metrics["rel_l2"] <= 4.0e-3


def test_large_logits_stay_finite():
    # scores of order +-80: the running-max rescale must neither overflow nor lose the dominant key
    run_decode(600, 1024, K.SPLIT_K_256, K.DTYPE_F32, seed=0xB2000500, q_scale=80.0)
    run_decode(200, 1024, K.SINGLE_BLOCK, K.DTYPE_BF16, seed=0xB2000501, q_scale=80.0)


def test_two_steps_through_a_device_position_and_plan_less_overload():
    max_ctx, ctx0 = 1024, 300
    q, gate, k, v = decode_operands(0xB2000600, ctx0 + 2)
    shape = K.Qwen35AttentionShape(1, HQ, HKV, D, max_ctx, 0)
    plan = K.qwen35_online_decode_plan(shape, K.SPLIT_K_256, ctx0 + 2)
    layout = K.qwen35_online_decode_workspace_layout(shape, plan.resolved_mode)
    cache = cache_to_device(make_cache(k, v, max_ctx, ctx0))
    ws = torch.zeros(layout.bytes // 4, device=dev())
    dpos = torch.tensor([ctx0], device=dev(), dtype=torch.int32)
    stream = torch.cuda.current_stream()
    outs = []
    for step in range(2):
        pos = ctx0 + step
        out = torch.zeros(HQ, D, device=dev(), dtype=torch.bfloat16)
        K.qwen35_online_attention_decode(act_tensor(q, K.DTYPE_BF16), act_tensor(k[pos], K.DTYPE_BF16),
                                         act_tensor(v[pos], K.DTYPE_BF16), act_tensor(gate, K.DTYPE_BF16), out, cache,
                                         cache.numel() * 2, ws, layout.bytes, shape, K.DTYPE_BF16, K.KV_BF16,
                                         K.HEAD_MAJOR, plan, dpos, stream)
        dpos += 1
        outs.append(out)
    torch.cuda.synchronize()
    full = make_cache(k, v, max_ctx, ctx0 + 2)
    assert np.array_equal(cache_bits_of(cache).reshape(full.shape), full)
    for step, out in enumerate(outs):
        want = ob.attention_core_cache(q[None], gate[None], full, max_ctx, ctx0 + step)[0]
        gate_bf16_outputs(compare(to_numpy_f32(out), want))
    # the plan-less overload (cpp/kernels/qwen35_online_attention.cuh:65-68) and the dispatcher with tokens == 1
    shape3 = K.Qwen35AttentionShape(1, HQ, HKV, D, max_ctx, ctx0 + 1)
    for call in ("decode", "dispatch"):
        out = torch.zeros(HQ, D, device=dev(), dtype=torch.bfloat16)
        args = (act_tensor(q, K.DTYPE_BF16), act_tensor(k[ctx0 + 1], K.DTYPE_BF16),
                act_tensor(v[ctx0 + 1], K.DTYPE_BF16), act_tensor(gate, K.DTYPE_BF16), out, cache, cache.numel() * 2)
        if call == "decode":
            K.qwen35_online_attention_decode(*args, None, 0, shape3, K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, None, None,
                                             stream)
        else:
            K.qwen35_causal_attention(*args, None, 0, shape3, K.DTYPE_BF16,
                                      K.Qwen35AttentionLaunchPolicy(K.ONLINE_TILED, K.KV_BF16, K.HEAD_MAJOR), stream)
        torch.cuda.synchronize()
        want = ob.attention_core_cache(q[None], gate[None], full, max_ctx, ctx0 + 1)[0]
        gate_bf16_outputs(compare(to_numpy_f32(out), want))


def test_capacity_guard_sets_a_status_bit_instead_of_trapping():
    """The reference traps when a replayed position needs more partitions than the captured plan holds
    (cpp/kernels/qwen35_online_attention.cu:714-717).  Here the combine kernel records the condition in the
    device status word, leaves the output alone, and the context stays usable."""
    max_ctx = 2048
    q, gate, k, v = decode_operands(0xB2000700, 601)
    shape = K.Qwen35AttentionShape(1, HQ, HKV, D, max_ctx, 0)
    plan = K.qwen35_online_decode_plan(shape, K.SPLIT_K_256, 400)  # bucket 512 -> capacity 2
    assert plan.active_partition_capacity == 2
    layout = K.qwen35_online_decode_workspace_layout(shape, plan.resolved_mode)
    cache = cache_to_device(make_cache(k, v, max_ctx, 600))
    ws = torch.zeros(layout.bytes // 4, device=dev())
    out = torch.full((HQ, D), 3.0, device=dev(), dtype=torch.bfloat16)
    stream = torch.cuda.current_stream()
    dpos = torch.tensor([600], device=dev(), dtype=torch.int32)  # context 601 needs 3 partitions
    K.qwen35_online_attention_decode(act_tensor(q, K.DTYPE_BF16), act_tensor(k[600], K.DTYPE_BF16),
                                     act_tensor(v[600], K.DTYPE_BF16), act_tensor(gate, K.DTYPE_BF16), out, cache,
                                     cache.numel() * 2, ws, layout.bytes, shape, K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR,
                                     plan, dpos, stream)
    assert K.device_status(stream) == K.DEVICE_DECODE_CAPACITY_EXCEEDED
    assert (out.float() == 3.0).all()
    assert K.device_status(stream) == 0  # reading clears it
    dpos.fill_(max_ctx)  # a position outside the cache
    K.qwen35_online_attention_decode(act_tensor(q, K.DTYPE_BF16), act_tensor(k[600], K.DTYPE_BF16),
                                     act_tensor(v[600], K.DTYPE_BF16), act_tensor(gate, K.DTYPE_BF16), out, cache,
                                     cache.numel() * 2, ws, layout.bytes, shape, K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR,
                                     plan, dpos, stream)
    assert K.device_status(stream) == K.DEVICE_POSITION_OUT_OF_RANGE
    assert (out.float() == 3.0).all()


def test_decode_replays_inside_a_cuda_graph():
    """One captured graph serves every position of its context bucket (the reference's decode-graph contract,
    cpp/execution/qwen35_executor.cu:2191-2225): position, query and the new K/V row live in device buffers."""
    max_ctx, ctx0, steps = 1024, 520, 3
    q, gate, k, v = decode_operands(0xB2000800, ctx0 + steps)
    shape = K.Qwen35AttentionShape(1, HQ, HKV, D, max_ctx, 0)
    plan = K.qwen35_online_decode_plan(shape, K.SPLIT_K_256, ctx0 + steps)
    layout = K.qwen35_online_decode_workspace_layout(shape, plan.resolved_mode)
    cache = cache_to_device(make_cache(k, v, max_ctx, ctx0))
    ws = torch.zeros(layout.bytes // 4, device=dev())
    dq, dg = act_tensor(q, K.DTYPE_BF16), act_tensor(gate, K.DTYPE_BF16)
    dk = torch.zeros(HKV, D, device=dev(), dtype=torch.bfloat16)
    dv = torch.zeros(HKV, D, device=dev(), dtype=torch.bfloat16)
    out = torch.zeros(HQ, D, device=dev(), dtype=torch.bfloat16)
    dpos = torch.tensor([ctx0], device=dev(), dtype=torch.int32)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())

    def call(stream):
        K.qwen35_online_attention_decode(dq, dk, dv, dg, out, cache, cache.numel() * 2, ws, layout.bytes, shape,
                                         K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, plan, dpos, stream)

    with torch.cuda.stream(side):
        dk.copy_(act_tensor(k[ctx0], K.DTYPE_BF16))
        dv.copy_(act_tensor(v[ctx0], K.DTYPE_BF16))
        call(side)  # warm-up outside capture (first call sets the shared-memory attribute)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            call(side)
    full = make_cache(k, v, max_ctx, ctx0 + steps)
    for step in range(steps):
        pos = ctx0 + step
        dk.copy_(act_tensor(k[pos], K.DTYPE_BF16))
        dv.copy_(act_tensor(v[pos], K.DTYPE_BF16))
        dpos.fill_(pos)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        want = ob.attention_core_cache(q[None], gate[None], full, max_ctx, pos)[0]
        gate_bf16_outputs(compare(to_numpy_f32(out), want))
    assert np.array_equal(cache_bits_of(cache).reshape(full.shape), full)


def test_back_to_back_steps_keep_stream_order():
    """Both kernels of a step are launched with programmatic stream serialisation and wait for their predecessor on
    the device.  A chain in which every step's query is made, by a kernel on the same stream and with no host
    synchronisation, from the previous step's output must give what the same chain gives with a synchronisation
    after every operation."""
    max_ctx, ctx0, steps = 4096, 3000, 6
    q, gate, k, v = decode_operands(0xB2000900, ctx0 + steps)
    shape_of = lambda pos: K.Qwen35AttentionShape(1, HQ, HKV, D, max_ctx, pos)
    plan = K.qwen35_online_decode_plan(shape_of(ctx0), K.SPLIT_K_256, ctx0 + steps)
    layout = K.qwen35_online_decode_workspace_layout(shape_of(ctx0), plan.resolved_mode)
    dg = act_tensor(gate, K.DTYPE_BF16)
    rows_k = [act_tensor(k[ctx0 + i], K.DTYPE_BF16) for i in range(steps)]
    rows_v = [act_tensor(v[ctx0 + i], K.DTYPE_BF16) for i in range(steps)]
    stream = torch.cuda.current_stream()

    def chain(synchronise):
        cache = cache_to_device(make_cache(k, v, max_ctx, ctx0))
        ws = torch.zeros(layout.bytes // 4, device=dev())
        dq = act_tensor(q, K.DTYPE_BF16).clone()
        outs = []
        for i in range(steps):
            out = torch.zeros(HQ, D, device=dev(), dtype=torch.bfloat16)
            K.qwen35_online_attention_decode(dq, rows_k[i], rows_v[i], dg, out, cache, cache.numel() * 2, ws,
                                             layout.bytes, shape_of(ctx0 + i), K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR,
                                             plan, None, stream)
            if synchronise:
                torch.cuda.synchronize()
            dq = (dq.float() * 0.5 + out.float() * 4.0).to(torch.bfloat16)  # the next query depends on this output
            if synchronise:
                torch.cuda.synchronize()
            outs.append(out)
        torch.cuda.synchronize()
        return torch.stack(outs), cache

    loose, loose_cache = chain(False)
    strict, strict_cache = chain(True)
    assert K.device_status(stream) == 0
    assert torch.equal(loose, strict)
    assert torch.equal(loose_cache, strict_cache)


def test_early_kv_fetch_gives_the_same_bits():
    """Through the early-cache-fetch entry point the partition kernel reads cache rows before the kernels in front of
    it have finished.  Under the conditions that entry point asks for, the results are those of the default ordering:
    (a) steps enqueued back to back on different caches, none of which writes a row another one reads; (b) a chain on
    one cache with advancing positions in which ordinary kernels sit between the steps: they rewrite the query AND the
    gate directly in front of each step, so a step that read either of them too early would show."""
    max_ctx, ctx0, steps = 8192, 6000, 8
    q, gate, k, v = decode_operands(0xB2000B00, ctx0 + steps)
    shape_of = lambda pos: K.Qwen35AttentionShape(1, HQ, HKV, D, max_ctx, pos)
    plan = K.qwen35_online_decode_plan(shape_of(ctx0), K.SPLIT_K_256, ctx0 + steps)
    layout = K.qwen35_online_decode_workspace_layout(shape_of(ctx0), plan.resolved_mode)
    dg = act_tensor(gate, K.DTYPE_BF16)
    rows_k = [act_tensor(k[ctx0 + i], K.DTYPE_BF16) for i in range(steps)]
    rows_v = [act_tensor(v[ctx0 + i], K.DTYPE_BF16) for i in range(steps)]
    queries = [act_tensor(q * (1.0 + 0.1 * i), K.DTYPE_BF16) for i in range(steps)]
    stream = torch.cuda.current_stream()

    def call(early, *args):
        if early:
            K.online_attention_decode_early_kv_fetch(*args, stream)
        else:
            K.qwen35_online_attention_decode(*args, None, stream)

    def independent(early):
        caches = [cache_to_device(make_cache(k, v, max_ctx, ctx0)) for _ in range(steps)]
        ws = torch.zeros(layout.bytes // 4, device=dev())
        outs = [torch.zeros(HQ, D, device=dev(), dtype=torch.bfloat16) for _ in range(steps)]
        torch.cuda.synchronize()
        for i in range(steps):
            call(early, queries[i], rows_k[0], rows_v[0], dg, outs[i], caches[i], caches[i].numel() * 2, ws,
                 layout.bytes, shape_of(ctx0), K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, plan)
        torch.cuda.synchronize()
        return torch.stack(outs), torch.stack(caches)

    def chain(early, moving_gate=True):
        cache = cache_to_device(make_cache(k, v, max_ctx, ctx0))
        ws = torch.zeros(layout.bytes // 4, device=dev())
        dq = queries[0].clone()
        step_gate = dg.clone()
        outs = []
        for i in range(steps):
            out = torch.zeros(HQ, D, device=dev(), dtype=torch.bfloat16)
            call(early, dq, rows_k[i], rows_v[i], step_gate, out, cache, cache.numel() * 2, ws, layout.bytes,
                 shape_of(ctx0 + i), K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, plan)
            dq = (dq.float() * 0.5 + out.float() * 4.0).to(torch.bfloat16)
            if moving_gate:  # rewritten in place, at the same address, by an ordinary kernel
                step_gate.copy_((step_gate.float() * 0.75 - out.float() * 3.0).to(torch.bfloat16))
            outs.append(out)
        torch.cuda.synchronize()
        return torch.stack(outs), cache

    plain = independent(False), chain(False)
    early = independent(True), chain(True)
    assert K.device_status(stream) == 0
    for (want_out, want_cache), (got_out, got_cache) in zip(plain, early):
        assert torch.equal(got_out, want_out)
        assert torch.equal(got_cache, want_cache)
    # the chain's gates really moved: its outputs differ from those of a chain whose gate is held constant
    assert not torch.equal(plain[1][0], chain(False, moving_gate=False)[0])


def test_decode_from_host_buffers():
    """The host-buffer entry point (copy in, step, copy out, synchronise) gives what the device-buffer call gives."""
    ctx, max_ctx = 1500, 2048
    pos = ctx - 1
    q, gate, k, v = decode_operands(0xB2000A00, ctx)
    shape = K.Qwen35AttentionShape(1, HQ, HKV, D, max_ctx, pos)
    plan = K.qwen35_online_decode_plan(shape, K.SPLIT_K_256, ctx)
    layout = K.qwen35_online_decode_workspace_layout(shape, plan.resolved_mode)
    stream = torch.cuda.current_stream()
    token = np.concatenate([q, k[pos], v[pos], gate], axis=0)  # rows q | k | v | gate
    host_token = bf16_tensor(token).cpu().pin_memory()
    host_out = torch.zeros(HQ, D, dtype=torch.bfloat16).pin_memory()
    dev_token = torch.zeros(2 * HQ + 2 * HKV, D, device=dev(), dtype=torch.bfloat16)
    dev_out = torch.zeros(HQ, D, device=dev(), dtype=torch.bfloat16)
    ws = torch.zeros(layout.bytes // 4, device=dev())
    cache = cache_to_device(make_cache(k, v, max_ctx, pos))
    K.online_attention_decode_from_host(host_token, host_out, dev_token, dev_out, cache, cache.numel() * 2, ws,
                                        layout.bytes, shape, K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, plan, None, stream)
    # no synchronisation here: the call has returned, so the host buffer holds the result
    got = host_out.clone()
    ref_out = torch.zeros(HQ, D, device=dev(), dtype=torch.bfloat16)
    cache2 = cache_to_device(make_cache(k, v, max_ctx, pos))
    K.qwen35_online_attention_decode(bf16_tensor(q), bf16_tensor(k[pos]), bf16_tensor(v[pos]), bf16_tensor(gate),
                                     ref_out, cache2, cache2.numel() * 2, ws, layout.bytes, shape, K.DTYPE_BF16,
                                     K.KV_BF16, K.HEAD_MAJOR, plan, None, stream)
    torch.cuda.synchronize()
    assert torch.equal(got, ref_out.cpu()) and torch.equal(cache, cache2)
    # pageable host buffers: the result comes back through device_output and a copy
    cache3 = cache_to_device(make_cache(k, v, max_ctx, pos))
    pageable_out = torch.zeros(HQ, D, dtype=torch.bfloat16)
    K.online_attention_decode_from_host(bf16_tensor(token).cpu(), pageable_out, dev_token, dev_out, cache3,
                                        cache3.numel() * 2, ws, layout.bytes, shape, K.DTYPE_BF16, K.KV_BF16,
                                        K.HEAD_MAJOR, plan, None, stream)
    assert torch.equal(pageable_out, ref_out.cpu()) and torch.equal(dev_out, ref_out) and torch.equal(cache3, cache2)
    with pytest.raises(K.Qwen35PrimitiveError):
        K.online_attention_decode_from_host(None, host_out, dev_token, dev_out, cache, cache.numel() * 2, ws,
                                            layout.bytes, shape, K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, plan, None,
                                            stream)


def test_batched_ragged_decode():
    """Five independent sequences with ragged contexts in one launch pair (the batched serving entry point)."""
    contexts = [1, 200, 256, 1000, 2049]
    batch = len(contexts)
    rng_seed = 0xB2000900
    caps = [-(-c // 256) * 256 for c in contexts]
    largest = max(caps)
    qs, gs, ks, vs, caches, fulls = [], [], [], [], [], []
    for i, ctx in enumerate(contexts):
        q, gate, k, v = decode_operands(rng_seed + i, ctx)
        qs.append(q), gs.append(gate), ks.append(k[ctx - 1]), vs.append(v[ctx - 1])
        caches.append(cache_to_device(make_cache(k, v, caps[i], ctx - 1)))
        fulls.append(make_cache(k, v, caps[i], ctx))
    dq, dg = act_tensor(np.stack(qs), K.DTYPE_BF16), act_tensor(np.stack(gs), K.DTYPE_BF16)
    dk, dv = act_tensor(np.stack(ks), K.DTYPE_BF16), act_tensor(np.stack(vs), K.DTYPE_BF16)
    out = torch.zeros(batch, HQ, D, device=dev(), dtype=torch.bfloat16)
    ptrs = torch.tensor([c.data_ptr() for c in caches], device=dev(), dtype=torch.int64)
    dcaps = torch.tensor(caps, device=dev(), dtype=torch.int32)
    dpos = torch.tensor([c - 1 for c in contexts], device=dev(), dtype=torch.int32)
    ws_bytes = K.batched_decode_workspace_bytes(batch, largest)
    ws = torch.zeros(ws_bytes // 4, device=dev())
    stream = torch.cuda.current_stream()
    K.batched_decode_attention(dq, dk, dv, dg, out, ptrs, dcaps, dpos, batch, largest, ws, ws_bytes, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0
    got = to_numpy_f32(out)
    for i, ctx in enumerate(contexts):
        assert np.array_equal(cache_bits_of(caches[i]).reshape(fulls[i].shape), fulls[i])
        want = ob.attention_core_cache(qs[i][None], gs[i][None], fulls[i], caps[i], ctx - 1)[0]
        gate_bf16_outputs(compare(got[i], want))


def paged_setup(contexts, seed, spare_pages=3, shuffle_seed=5):
    """Contiguous per-sequence caches and the same rows scattered over a page pool in a shuffled page order."""
    batch = len(contexts)
    caps = [-(-c // K.PAGE_TOKENS) * K.PAGE_TOKENS for c in contexts]
    max_blocks = max(caps) // K.PAGE_TOKENS
    qs, gs, ks, vs, before, after = [], [], [], [], [], []
    for i, ctx in enumerate(contexts):
        q, gate, k, v = decode_operands(seed + i, ctx)
        qs.append(q), gs.append(gate), ks.append(k[ctx - 1]), vs.append(v[ctx - 1])
        before.append(make_cache(k, v, caps[i], ctx - 1))
        after.append(make_cache(k, v, caps[i], ctx))
    pool_pages = sum(c // K.PAGE_TOKENS for c in caps) + spare_pages
    order = np.random.default_rng(shuffle_seed).permutation(pool_pages)
    pool = np.full((pool_pages, 2, HKV, K.PAGE_TOKENS, D), NAN_BITS, dtype=np.uint16)
    want_pool = pool.copy()
    tables = np.full((batch, max_blocks), 0xFFFFFFFF, dtype=np.uint32)  # entries past the live context: never read
    nxt = 0
    for i, cap in enumerate(caps):
        for b in range(cap // K.PAGE_TOKENS):
            page = int(order[nxt])
            nxt += 1
            tables[i, b] = page
            rows = slice(b * K.PAGE_TOKENS, (b + 1) * K.PAGE_TOKENS)
            pool[page] = before[i][:, :, rows]
            want_pool[page] = after[i][:, :, rows]
    return dict(batch=batch, caps=caps, max_blocks=max_blocks, qs=qs, gs=gs, ks=ks, vs=vs, before=before, after=after,
                pool=pool, want_pool=want_pool, tables=tables, pool_pages=pool_pages)


def test_paged_decode_matches_the_contiguous_batched_step():
    """The paged form reads the same rows through a block table: outputs are bit-identical to the batched step over
    contiguous caches, the appended rows land in the right pages, and every other page byte is untouched (unused
    pages and table entries past the live context hold NaNs / an invalid page number)."""
    contexts = [1, 200, 256, 257, 1000, 2049, 4096]
    s = paged_setup(contexts, 0xB2000C00)
    batch, largest = s["batch"], max(s["caps"])
    dq, dg = act_tensor(np.stack(s["qs"]), K.DTYPE_BF16), act_tensor(np.stack(s["gs"]), K.DTYPE_BF16)
    dk, dv = act_tensor(np.stack(s["ks"]), K.DTYPE_BF16), act_tensor(np.stack(s["vs"]), K.DTYPE_BF16)
    dpos = torch.tensor([c - 1 for c in contexts], device=dev(), dtype=torch.int32)
    ws_bytes = K.batched_decode_workspace_bytes(batch, largest)
    stream = torch.cuda.current_stream()

    caches = [cache_to_device(c) for c in s["before"]]
    ptrs = torch.tensor([c.data_ptr() for c in caches], device=dev(), dtype=torch.int64)
    dcaps = torch.tensor(s["caps"], device=dev(), dtype=torch.int32)
    out_flat = torch.zeros(batch, HQ, D, device=dev(), dtype=torch.bfloat16)
    ws = torch.zeros(ws_bytes // 4, device=dev())
    K.batched_decode_attention(dq, dk, dv, dg, out_flat, ptrs, dcaps, dpos, batch, largest, ws, ws_bytes, stream)

    pool = cache_to_device(s["pool"])
    tables = torch.from_numpy(s["tables"].view(np.int32)).to(dev())
    out_paged = torch.zeros(batch, HQ, D, device=dev(), dtype=torch.bfloat16)
    ws2 = torch.zeros(ws_bytes // 4, device=dev())
    K.paged_decode_attention(dq, dk, dv, dg, out_paged, pool, s["pool_pages"], tables, s["max_blocks"], dpos, batch,
                             ws2, ws_bytes, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0
    assert torch.equal(out_paged, out_flat)
    assert np.array_equal(cache_bits_of(pool).reshape(s["want_pool"].shape), s["want_pool"])
    got = to_numpy_f32(out_paged)
    for i, ctx in enumerate(contexts):
        want = ob.attention_core_cache(s["qs"][i][None], s["gs"][i][None], s["after"][i], s["caps"][i], ctx - 1)[0]
        gate_bf16_outputs(compare(got[i], want))


def test_paged_decode_flags_a_page_outside_the_pool():
    """A live table entry that names a page the pool does not hold is reported through the status word; the kernel
    does not touch memory for it, and the other sequences of the batch are served as usual."""
    contexts = [300, 700]
    s = paged_setup(contexts, 0xB2000D00)
    s["tables"][0, 1] = s["pool_pages"] + 7
    batch, largest = s["batch"], max(s["caps"])
    dq, dg = act_tensor(np.stack(s["qs"]), K.DTYPE_BF16), act_tensor(np.stack(s["gs"]), K.DTYPE_BF16)
    dk, dv = act_tensor(np.stack(s["ks"]), K.DTYPE_BF16), act_tensor(np.stack(s["vs"]), K.DTYPE_BF16)
    dpos = torch.tensor([c - 1 for c in contexts], device=dev(), dtype=torch.int32)
    ws_bytes = K.batched_decode_workspace_bytes(batch, largest)
    ws = torch.zeros(ws_bytes // 4, device=dev())
    pool = cache_to_device(s["pool"])
    tables = torch.from_numpy(s["tables"].view(np.int32)).to(dev())
    out = torch.zeros(batch, HQ, D, device=dev(), dtype=torch.bfloat16)
    stream = torch.cuda.current_stream()
    K.paged_decode_attention(dq, dk, dv, dg, out, pool, s["pool_pages"], tables, s["max_blocks"], dpos, batch, ws,
                             ws_bytes, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == K.DEVICE_PAGE_OUT_OF_RANGE
    want = ob.attention_core_cache(s["qs"][1][None], s["gs"][1][None], s["after"][1], s["caps"][1], contexts[1] - 1)[0]
    gate_bf16_outputs(compare(to_numpy_f32(out)[1], want))
    with pytest.raises(K.Qwen35PrimitiveError):
        K.paged_decode_attention(dq, dk, dv, dg, out, pool, s["pool_pages"], tables, s["max_blocks"], dpos, batch, ws,
                                 ws_bytes // 2, stream)


def test_serving_decode_64_ragged_sequences_at_full_size():
    """The batched serving configuration at its full size: 64 sequences, contexts uniform in [1024, 32768] from a
    seed (about 1.1 M tokens, 4.7 GB of caches), one launch pair.  The caches are drawn on the device; the oracle runs
    on the shortest, the longest and four more sequences, whose caches are copied back, and every sequence's appended
    row and output are checked for the properties that need no oracle: the row equals the new token's K and V bit for
    bit, nothing else in the cache moved (a checksum of the other rows), the output is finite."""
    batch, lo, hi, seed = 64, 1024, 32768, 0xB2000004
    cpu_gen = torch.Generator().manual_seed(seed)
    lengths = torch.randint(lo, hi + 1, (batch,), generator=cpu_gen).tolist()
    caps = [-(-n // 256) * 256 for n in lengths]
    largest = max(caps)
    gen = torch.Generator(device=dev()).manual_seed(seed)
    rand = lambda *shape: torch.randn(*shape, device=dev(), generator=gen, dtype=torch.float32).to(torch.bfloat16)
    caches = [rand(2, HKV, c, D) for c in caps]
    q, gate = rand(batch, HQ, D), rand(batch, HQ, D)
    k, v = rand(batch, HKV, D), rand(batch, HKV, D)
    out = torch.zeros(batch, HQ, D, device=dev(), dtype=torch.bfloat16)
    ptrs = torch.tensor([c.data_ptr() for c in caches], device=dev(), dtype=torch.int64)
    dcaps = torch.tensor(caps, device=dev(), dtype=torch.int32)
    dpos = torch.tensor([n - 1 for n in lengths], device=dev(), dtype=torch.int32)
    ws_bytes = K.batched_decode_workspace_bytes(batch, largest)
    ws = torch.zeros(ws_bytes // 4, device=dev())
    # checksums of everything but the row that is appended (as 16-bit integers, wrapping 64-bit sums)
    def checksum(cache, row):
        bits = cache.view(torch.int16).to(torch.int64)
        return int(bits.sum().item()) - int(bits[:, :, row].sum().item())
    before = [checksum(c, n - 1) for c, n in zip(caches, lengths)]
    stream = torch.cuda.current_stream()
    K.batched_decode_attention(q, k, v, gate, out, ptrs, dcaps, dpos, batch, largest, ws, ws_bytes, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0
    assert torch.isfinite(out.float()).all()
    for i, n in enumerate(lengths):
        assert torch.equal(caches[i][0, :, n - 1], k[i]) and torch.equal(caches[i][1, :, n - 1], v[i])
        assert checksum(caches[i], n - 1) == before[i], f"sequence {i}: a row other than the appended one changed"
    order = sorted(range(batch), key=lambda i: lengths[i])
    sampled = {order[0], order[-1], order[batch // 2], 0, 17, 63}
    got = to_numpy_f32(out)
    for i in sampled:
        bits = cache_bits_of(caches[i])
        want = ob.attention_core_cache(to_numpy_f32(q[i])[None], to_numpy_f32(gate[i])[None], bits, caps[i],
                                       lengths[i] - 1)[0]
        gate_bf16_outputs(compare(got[i], want))
