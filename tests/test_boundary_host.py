"""Host-side contract of the C ABI, runnable without a GPU: exported symbols, size/plan arithmetic and the
refusals that happen before any CUDA call.  Expected values follow the reference's contract tests
(cpp/tests/qwen35_cuda_attention_test.cu:205-440,1466-1516; cpp/tests/qwen35_cuda_delta_test.cu:785-908)."""
import ctypes
import os
import re

import pytest

from raftinfer_b200 import _lib
from raftinfer_b200 import kernels as K

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MODEL = K.Qwen35AttentionShape(1, 16, 4, 256, 4096, 0)
BF16_HEAD = K.Qwen35AttentionLaunchPolicy(K.ONLINE_TILED, K.KV_BF16, K.HEAD_MAJOR)
FAKE = 0x1000  # non-null, 16-byte aligned address that is never dereferenced on the host


def test_every_declared_symbol_is_exported():
    header = open(os.path.join(ROOT, "include", "rib200.h")).read()
    declared = set(re.findall(r"\b(rib200_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 20
    for name in sorted(declared):
        assert hasattr(_lib.lib, name), name
    assert set(_lib.PROTOTYPES) | {"rib200_version"} == declared
    assert K.version().startswith("rib200")


def test_cache_and_workspace_sizes():
    shape = K.Qwen35AttentionShape(1, 2, 1, 7, 4, 0)
    ref_policy = K.Qwen35AttentionLaunchPolicy(K.MATERIALIZED_REFERENCE, K.KV_F32, K.TOKEN_MAJOR)
    bf16_online = K.Qwen35AttentionLaunchPolicy(K.ONLINE_TILED, K.KV_BF16, K.TOKEN_MAJOR)
    assert K.qwen35_attention_cache_bytes(shape, ref_policy) == 2 * 4 * 1 * 7 * 4
    assert K.qwen35_attention_workspace_bytes(shape, ref_policy) == 1 * 2 * 1 * 4
    assert K.qwen35_attention_workspace_floats(shape) == 2
    assert K.qwen35_attention_cache_bytes(shape, bf16_online) == 2 * 4 * 1 * 7 * 2
    assert K.qwen35_attention_workspace_bytes(shape, bf16_online) == 0
    assert K.qwen35_online_attention_workspace_bytes(shape) == 0
    assert K.qwen35_attention_cache_bytes(K.Qwen35AttentionShape(1, 16, 4, 256, 32768, 0), BF16_HEAD) == 4096 * 32768


def test_decode_plans_and_layout():
    single = K.qwen35_online_decode_plan(MODEL, K.SINGLE_BLOCK, 128)
    assert (single.resolved_mode, single.context_bucket_tokens, single.active_partition_capacity) == (K.SINGLE_BLOCK, 512, 1)
    assert K.qwen35_online_decode_workspace_layout(MODEL, single.resolved_mode).bytes == 0
    for mode in (K.AUTO_SELECT, K.SPLIT_K_256):
        plan = K.qwen35_online_decode_plan(MODEL, mode, 513)
        assert plan == K.Qwen35OnlineDecodePlan(K.SPLIT_K_256, 256, 256, 1024, 4)
    plan512 = K.qwen35_online_decode_plan(MODEL, K.SPLIT_K_512, 513)
    assert plan512 == K.Qwen35OnlineDecodePlan(K.SPLIT_K_512, 512, 512, 1024, 2)
    layout = K.qwen35_online_decode_workspace_layout(MODEL, K.SPLIT_K_256)
    assert layout.partial_count == 16 * 16
    assert (layout.max_offset_bytes, layout.sum_offset_bytes, layout.value_offset_bytes) == (0, 1024, 2048)
    assert layout.bytes == (2 * 256 + 256 * 256) * 4 == 264192
    # bucket: smallest power of two >= context starting at 512, capped by the cache capacity
    big = K.Qwen35AttentionShape(1, 16, 4, 256, 131072, 0)
    for ctx, bucket in ((1, 512), (512, 512), (513, 1024), (4096, 4096), (32768, 32768), (100000, 131072)):
        assert K.qwen35_online_decode_plan(big, K.SPLIT_K_256, ctx).context_bucket_tokens == bucket
    odd = K.Qwen35AttentionShape(1, 16, 4, 256, 777, 0)
    assert K.qwen35_online_decode_plan(odd, K.SPLIT_K_256, 600).context_bucket_tokens == 777
    assert K.qwen35_online_decode_plan(odd, K.SPLIT_K_256, 600).active_partition_capacity == 4


def test_decode_plan_refusals():
    with pytest.raises(K.Qwen35PrimitiveError):
        K.qwen35_online_decode_plan(MODEL, K.SINGLE_BLOCK, 0)
    with pytest.raises(K.Qwen35PrimitiveError):
        K.qwen35_online_decode_plan(MODEL, K.SINGLE_BLOCK, 4097)
    other = K.Qwen35AttentionShape(1, 16, 4, 255, 4096, 0)
    with pytest.raises(K.Qwen35PrimitiveError):
        K.qwen35_online_decode_plan(other, K.SPLIT_K_256, 513)
    with pytest.raises(K.Qwen35PrimitiveError):
        K.qwen35_online_decode_workspace_layout(other, K.SPLIT_K_256)
    with pytest.raises(K.Qwen35PrimitiveError):
        K.qwen35_online_decode_workspace_layout(MODEL, K.AUTO_SELECT)
    # a single-block plan is available for any shape
    assert K.qwen35_online_decode_plan(other, K.SINGLE_BLOCK, 5).partition_tokens == 0


def test_prefill_supported_matrix():
    shape = K.Qwen35AttentionShape(4, 16, 4, 256, 4, 0)
    assert K.qwen35_online_attention_prefill_supported(shape, K.DTYPE_F32, BF16_HEAD)
    assert K.qwen35_online_attention_prefill_supported(shape, K.DTYPE_BF16, BF16_HEAD)
    assert not K.qwen35_online_attention_prefill_supported(shape, K.DTYPE_F16, BF16_HEAD)
    assert not K.qwen35_online_attention_prefill_supported(
        shape, K.DTYPE_F32, K.Qwen35AttentionLaunchPolicy(K.MATERIALIZED_REFERENCE, K.KV_BF16, K.HEAD_MAJOR))
    assert not K.qwen35_online_attention_prefill_supported(
        shape, K.DTYPE_F32, K.Qwen35AttentionLaunchPolicy(K.ONLINE_TILED, K.KV_BF16, 99))
    assert not K.qwen35_online_attention_prefill_supported(K.Qwen35AttentionShape(1, 16, 4, 256, 4, 0), K.DTYPE_F32, BF16_HEAD)
    assert not K.qwen35_online_attention_prefill_supported(K.Qwen35AttentionShape(4, 16, 4, 257, 4, 0), K.DTYPE_F32, BF16_HEAD)
    assert not K.qwen35_online_attention_prefill_supported(K.Qwen35AttentionShape(4, 16, 4, 256, 6, 3), K.DTYPE_F32, BF16_HEAD)
    # the narrowing of this library: other caches are declined, not served by a second path
    assert not K.qwen35_online_attention_prefill_supported(
        shape, K.DTYPE_F32, K.Qwen35AttentionLaunchPolicy(K.ONLINE_TILED, K.KV_F32, K.TOKEN_MAJOR))


def _decode(shape=MODEL, plan=None, ws=FAKE, ws_bytes=None, stream=FAKE, q=FAKE, cache_bytes=None,
            cache_dtype=K.KV_BF16, layout=K.HEAD_MAJOR, dtype=K.DTYPE_BF16, cache=FAKE, device_position=None):
    plan = plan or K.qwen35_online_decode_plan(shape, K.SPLIT_K_256, shape.past_tokens + 1)
    if ws_bytes is None:
        ws_bytes = K.qwen35_online_decode_workspace_layout(shape, plan.resolved_mode).bytes
    if cache_bytes is None:
        cache_bytes = 2 * shape.max_context_tokens * 4 * 256 * 4
    K.qwen35_online_attention_decode(q, FAKE, FAKE, FAKE, FAKE, cache, cache_bytes, ws, ws_bytes, shape, dtype,
                                     cache_dtype, layout, plan, device_position, stream)


def test_decode_refusals_before_any_launch():
    good = K.qwen35_online_decode_plan(MODEL, K.SPLIT_K_256, 1)
    cases = [
        dict(q=None), dict(stream=None), dict(cache=None),
        dict(shape=K.Qwen35AttentionShape(1, 16, 4, 128, 4096, 0), plan=good),
        dict(shape=K.Qwen35AttentionShape(2, 16, 4, 256, 4096, 0), plan=good),
        dict(shape=K.Qwen35AttentionShape(1, 16, 4, 256, 4096, 4096), plan=good),
        dict(dtype=K.DTYPE_F16),
        dict(plan=K.Qwen35OnlineDecodePlan(K.AUTO_SELECT, 256, 256, 512, 2)),
        dict(plan=K.Qwen35OnlineDecodePlan(K.SPLIT_K_256, 512, 256, 512, 2)),
        dict(plan=K.Qwen35OnlineDecodePlan(K.SPLIT_K_256, 256, 128, 512, 2)),
        dict(plan=K.Qwen35OnlineDecodePlan(K.SPLIT_K_256, 256, 256, 0, 2)),
        dict(plan=K.Qwen35OnlineDecodePlan(K.SPLIT_K_256, 256, 256, 8192, 32)),
        dict(plan=K.Qwen35OnlineDecodePlan(K.SPLIT_K_256, 256, 256, 512, 3)),
        dict(plan=K.Qwen35OnlineDecodePlan(K.SINGLE_BLOCK, 0, 0, 512, 2), ws=None, ws_bytes=0),
        dict(plan=K.Qwen35OnlineDecodePlan(K.SINGLE_BLOCK, 0, 0, 512, 1), ws_bytes=16),
        dict(shape=K.Qwen35AttentionShape(1, 16, 4, 256, 4096, 600), plan=good),  # context beyond the bucket
        dict(ws=None), dict(ws_bytes=264191), dict(cache_bytes=2 * 4096 * 1024 * 2 - 1),
        dict(q=FAKE + 2),
    ]
    for kw in cases:
        with pytest.raises(K.Qwen35PrimitiveError) as err:
            _decode(**kw)
        assert err.value.code == K.INVALID_ARGUMENT, kw
    for kw in (dict(cache_dtype=K.KV_F32), dict(layout=K.TOKEN_MAJOR)):
        with pytest.raises(K.Qwen35PrimitiveError) as err:
            _decode(**kw)
        assert err.value.code == K.UNSUPPORTED, kw


def test_causal_attention_dispatch_refusals():
    shape = K.Qwen35AttentionShape(4, 16, 4, 256, 8, 0)
    args = dict(query=FAKE, key=FAKE, value=FAKE, gate=FAKE, output=FAKE, kv_cache=FAKE,
                kv_cache_bytes=2 * 8 * 1024 * 2, workspace=None, workspace_bytes=0, shape=shape,
                activation_dtype=K.DTYPE_BF16, policy=BF16_HEAD, stream=FAKE)
    for change, code in [
        (dict(workspace=FAKE, workspace_bytes=64), K.INVALID_ARGUMENT),  # online path forbids a workspace
        (dict(stream=None), K.INVALID_ARGUMENT),
        (dict(kv_cache_bytes=100), K.INVALID_ARGUMENT),
        (dict(shape=K.Qwen35AttentionShape(4, 16, 4, 256, 8, 5)), K.INVALID_ARGUMENT),  # context exceeds capacity
        (dict(shape=K.Qwen35AttentionShape(4, 16, 3, 256, 8, 0)), K.INVALID_ARGUMENT),
        (dict(activation_dtype=7), K.INVALID_ARGUMENT),
        (dict(policy=K.Qwen35AttentionLaunchPolicy(K.MATERIALIZED_REFERENCE, K.KV_F32, K.TOKEN_MAJOR),
              kv_cache_bytes=1 << 20, workspace=FAKE, workspace_bytes=1 << 20), K.UNSUPPORTED),
        (dict(activation_dtype=K.DTYPE_F16), K.INVALID_ARGUMENT),  # F16 is refused by the online prefill signature
    ]:
        with pytest.raises(K.Qwen35PrimitiveError) as err:
            K.qwen35_causal_attention(**{**args, **change})
        assert err.value.code == code, change


DELTA = K.GatedDeltaShape(3, 4096, 16, 32, 128, 128, 4, 1.0e-6)


def test_gated_delta_sizes_and_policy():
    conv_dim = 2 * 16 * 128 + 4096
    assert K.qwen35_gated_delta_workspace_bytes(DELTA) == 3 * (conv_dim + 4096 + 64) * 4
    policy = K.qwen35_gated_delta_select_policy(DELTA, 3)
    assert (policy.schedule, policy.warps_per_block, policy.transposed_boundary_state) == (0, 4, False)
    diag = K.qwen35_gated_delta_schedule_diagnostic(DELTA, 1)
    assert (diag.bucket_tokens, diag.key_dim, diag.value_dim) == (1, 128, 128)
    assert diag.candidate_schedule == 2 and diag.schedule == 0 and not diag.candidate_accepted
    assert diag.rejection_reason == b"not_tuned"
    assert K.qwen35_gated_delta_schedule_diagnostic(DELTA, 128).candidate_schedule == 1


def _delta(shape=DELTA, policy=None, dtype=K.DTYPE_BF16, wdtype=K.DTYPE_F32, ws_bytes=None, **ptrs):
    p = dict(input=FAKE, conv_weight=FAKE, recurrent_a=FAKE, dt_bias=FAKE, output_norm_weight=FAKE, output=FAKE,
             convolution_state=FAKE, recurrent_state=FAKE, workspace=FAKE, stream=FAKE)
    p.update(ptrs)
    if ws_bytes is None:
        ws_bytes = 1 << 30
    K.qwen35_gated_delta(p["input"], p["conv_weight"], p["recurrent_a"], p["dt_bias"], p["output_norm_weight"],
                         p["output"], p["convolution_state"], p["recurrent_state"], p["workspace"], ws_bytes, shape,
                         dtype, wdtype, p["stream"], policy=policy or K.GatedDeltaLaunchPolicy())


def test_gated_delta_refusals_before_any_launch():
    import dataclasses
    bad_shapes = [dict(tokens=0), dict(hidden_size=0), dict(key_heads=0), dict(value_heads=0), dict(key_dim=0),
                  dict(value_dim=0), dict(conv_width=0), dict(epsilon=-1.0), dict(epsilon=float("nan")),
                  dict(value_heads=33), dict(hidden_size=4095)]
    for change in bad_shapes:
        with pytest.raises(K.Qwen35DeltaError) as err:
            _delta(shape=dataclasses.replace(DELTA, **change))
        assert err.value.code == K.INVALID_ARGUMENT, change
        with pytest.raises(K.Qwen35DeltaError):
            K.qwen35_gated_delta_workspace_bytes(dataclasses.replace(DELTA, **change))
    for name in ("input", "conv_weight", "recurrent_a", "dt_bias", "output_norm_weight", "output",
                 "convolution_state", "recurrent_state", "workspace", "stream"):
        with pytest.raises(K.Qwen35DeltaError) as err:
            _delta(**{name: None})
        assert err.value.code == K.INVALID_ARGUMENT, name
    # misaligned pointers (cpp/tests/qwen35_cuda_delta_test.cu:850-908)
    for name in ("input", "output"):
        with pytest.raises(K.Qwen35DeltaError):
            _delta(**{name: FAKE + 1})
    for name in ("conv_weight", "recurrent_a", "dt_bias", "output_norm_weight", "convolution_state",
                 "recurrent_state", "workspace"):
        with pytest.raises(K.Qwen35DeltaError):
            _delta(**{name: FAKE + 2})
    with pytest.raises(K.Qwen35DeltaError):
        _delta(ws_bytes=K.qwen35_gated_delta_workspace_bytes(DELTA) - 1)
    for policy in (K.GatedDeltaLaunchPolicy(0, 8, False), K.GatedDeltaLaunchPolicy(0, 4, True),
                   K.GatedDeltaLaunchPolicy(9, 4, False), K.GatedDeltaLaunchPolicy(2, 4, False)):
        with pytest.raises(K.Qwen35DeltaError):
            _delta(policy=policy)
    with pytest.raises(K.Qwen35DeltaError):
        _delta(dtype=K.DTYPE_BF16, wdtype=K.DTYPE_F16)
    small = K.GatedDeltaShape(2, 28, 2, 4, 5, 7, 3, 1.0e-6)
    with pytest.raises(K.Qwen35DeltaError) as err:
        _delta(shape=small)
    assert err.value.code == K.UNSUPPORTED


def test_status_struct_matches_reference_layout():
    # RaftInferStatus is {enum code; const char* message} (cpp/include/raftinfer/status.h:17-20)
    assert ctypes.sizeof(_lib.Status) == 16 and _lib.Status.message.offset == 8
