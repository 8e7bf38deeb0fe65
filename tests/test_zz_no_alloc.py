"""The decode entry point that allocates nothing (rib200_online_attention_decode_static_scratch).

Some hosts cannot give the library a workspace or call cudaMalloc on the decode path: a runtime whose device
memory all went to a pool at start-up, a plugin that only sees the operator's own tensors, a serving thread that
cannot afford cudaMalloc's device-wide synchronisation.  For them the split-k partials live in an array inside the
library.  This file checks, through the C ABI, that the entry point gives the same output and the same appended
cache row as the workspace entry point on the same inputs, on two calls in a row that share the built-in array
(different positions, the second one shorter so stale partials of the first stay behind it), that both agree with the
CPU oracle, that the largest cache the array was built for (32768 rows, last partition) works, and that it refuses
caches beyond that size.  It is collected last on purpose.
"""
import numpy as np
import pytest
import torch

from oracle import bindings as ob
from raftinfer_b200 import kernels as K

from gpu_util import (D, HKV, HQ, act_tensor, cache_bits_of, cache_to_device, compare, decode_operands, dev,
                      gate_bf16_outputs, make_cache, to_numpy_f32)


def _both_entry_points(ctx, max_ctx, dtype, seed, device_position):
    pos = ctx - 1
    q, gate, k, v = decode_operands(seed, ctx)
    stream = torch.cuda.current_stream()
    dq, dg = act_tensor(q, dtype), act_tensor(gate, dtype)
    dk, dv = act_tensor(k[pos], dtype), act_tensor(v[pos], dtype)
    out_dtype = torch.float32 if dtype == K.DTYPE_F32 else torch.bfloat16
    dpos = torch.tensor([pos], device=dev(), dtype=torch.int32) if device_position else None
    shape = K.Qwen35AttentionShape(1, HQ, HKV, D, max_ctx, 0 if device_position else pos)

    cache_a = cache_to_device(make_cache(k, v, max_ctx, pos))
    plan = K.qwen35_online_decode_plan(shape, K.SPLIT_K_256, ctx)
    layout = K.qwen35_online_decode_workspace_layout(shape, plan.resolved_mode)
    ws = torch.zeros(layout.bytes // 4, device=dev())
    out_a = torch.zeros(HQ, D, device=dev(), dtype=out_dtype)
    K.qwen35_online_attention_decode(dq, dk, dv, dg, out_a, cache_a, cache_a.numel() * 2, ws, layout.bytes, shape,
                                     dtype, K.KV_BF16, K.HEAD_MAJOR, plan, dpos, stream)

    cache_b = cache_to_device(make_cache(k, v, max_ctx, pos))
    out_b = torch.full((HQ, D), 9.0, device=dev(), dtype=out_dtype)
    K.online_attention_decode_static_scratch(dq, dk, dv, dg, out_b, cache_b, cache_b.numel() * 2, shape, dtype, dpos,
                                             stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0
    metrics = compare(to_numpy_f32(out_b), to_numpy_f32(out_a))
    gate_bf16_outputs(metrics)  # max abs <= 3e-2, relative L2 <= 1e-2: the tolerance of the decode tests
    assert np.array_equal(cache_bits_of(cache_b), cache_bits_of(cache_a))
    # and against the CPU oracle on the cache as the step leaves it (the new row appended)
    full = make_cache(k, v, max_ctx, ctx)
    assert np.array_equal(cache_bits_of(cache_b).reshape(full.shape), full)
    want = ob.attention_core_cache(q[None], gate[None], full, max_ctx, pos)[0]
    gate_bf16_outputs(compare(to_numpy_f32(out_b), want))
    return metrics


@pytest.mark.gpu
def test_static_scratch_decode_matches_workspace_decode_on_two_calls_in_a_row():
    first = _both_entry_points(2049, 4096, K.DTYPE_BF16, 0xB2003000, device_position=True)
    second = _both_entry_points(777, 1024, K.DTYPE_F32, 0xB2003001, device_position=False)
    third = _both_entry_points(100, 1024, K.DTYPE_BF16, 0xB2003002, device_position=False)  # below the threshold
    for metrics in (first, second, third):
        assert metrics["max_abs"] <= 3.0e-2 and metrics["rel_l2"] <= 1.0e-2


@pytest.mark.gpu
@pytest.mark.parametrize("ctx,max_ctx", [(32768, 32768), (32700, 32700), (32513, 32768)])
def test_static_scratch_decode_at_the_size_limit_of_its_array(ctx, max_ctx):
    """The built-in array holds 16 heads x 128 partitions: a 32768-row cache with the position in the last partition
    uses its last partial, and a capacity that is not a multiple of 256 rounds the partition count up to the same
    128.  An array one partial too small, or an offset computed from the wrong partition count, shows here."""
    _both_entry_points(ctx, max_ctx, K.DTYPE_BF16, 0xB2003010 + ctx, device_position=False)
    # a short call straight afterwards, in the other activation type, finds the long call's partials still in the array
    _both_entry_points(300, 512, K.DTYPE_F32, 0xB2003020, device_position=True)


def test_static_scratch_decode_refuses_caches_beyond_its_array():
    fake = 0x1000
    too_large = K.Qwen35AttentionShape(1, HQ, HKV, D, 32769, 0)
    with pytest.raises(K.Qwen35PrimitiveError) as err:
        K.online_attention_decode_static_scratch(fake, fake, fake, fake, fake, fake, 1 << 40, too_large, K.DTYPE_BF16,
                                                 None, fake)
    assert err.value.code == K.INVALID_ARGUMENT and "32768" in str(err.value)
    with pytest.raises(K.Qwen35PrimitiveError):
        K.online_attention_decode_static_scratch(fake, fake, fake, fake, fake, fake, 1 << 40,
                                                 K.Qwen35AttentionShape(1, HQ, HKV, D, 1024, 0), K.DTYPE_BF16, None,
                                                 None)
