"""Host-side mirror of RAFTInfer's kernel-launcher API (namespace raftinfer::kernels) over librib200.so.

Function names, argument order and refusal behaviour follow cpp/kernels/qwen35_attention.cuh:29-51,
cpp/kernels/qwen35_online_attention.cuh:33-68 and cpp/kernels/qwen35_delta.cuh:64-102; a non-OK status
from the C ABI is raised as Qwen35PrimitiveError / Qwen35DeltaError, the exception types the reference throws
(cpp/kernels/qwen35_primitives.cuh:15-19, cpp/kernels/qwen35_delta.cuh:14-18).  Pointer arguments accept a
torch tensor, an int address or None; `stream` accepts a torch.cuda.Stream or an int handle.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from . import _lib
from ._lib import lib

# RaftInferDataType, cpp/include/raftinfer/tensor.h:10-15
DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 1, 2, 3
# cpp/execution/qwen35_execution_policy.hpp:7-27
MATERIALIZED_REFERENCE, ONLINE_TILED = 0, 1
AUTO_SELECT, SINGLE_BLOCK, SPLIT_K_256, SPLIT_K_512 = 0, 1, 2, 3
KV_F32, KV_BF16 = 0, 1
TOKEN_MAJOR, HEAD_MAJOR = 0, 1
# status codes, cpp/include/raftinfer/status.h:7-20
OK, INVALID_ARGUMENT, UNAVAILABLE, CUDA_ERROR, INTERNAL, UNSUPPORTED, RESOURCE_EXHAUSTED = range(7)
# device status bits
DEVICE_DECODE_CAPACITY_EXCEEDED, DEVICE_POSITION_OUT_OF_RANGE, DEVICE_WAIT_TIMED_OUT = 1, 2, 4
DEVICE_PAGE_OUT_OF_RANGE = 8
DEVICE_POINTER_MISALIGNED = 16


class Qwen35PrimitiveError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(message)
        self.code = code


class Qwen35DeltaError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(message)
        self.code = code


def _check(status, exc=Qwen35PrimitiveError):
    if status.code != OK:
        raise exc(status.code, (status.message or b"").decode())


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()


def _stream(stream):
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


@dataclass(frozen=True)
class Qwen35AttentionShape:
    tokens: int
    query_heads: int
    kv_heads: int
    head_dim: int
    max_context_tokens: int
    past_tokens: int

    def c(self):
        return _lib.AttentionShape(self.tokens, self.query_heads, self.kv_heads, self.head_dim,
                                   self.max_context_tokens, self.past_tokens)


@dataclass(frozen=True)
class Qwen35AttentionLaunchPolicy:
    implementation: int = ONLINE_TILED
    kv_cache_dtype: int = KV_BF16
    kv_cache_layout: int = HEAD_MAJOR

    def c(self):
        return _lib.AttentionLaunchPolicy(self.implementation, self.kv_cache_dtype, self.kv_cache_layout)


@dataclass(frozen=True)
class Qwen35OnlineDecodePlan:
    resolved_mode: int = SINGLE_BLOCK
    partition_tokens: int = 0
    split_k_threshold_tokens: int = 0
    context_bucket_tokens: int = 0
    active_partition_capacity: int = 1

    def c(self):
        return _lib.OnlineDecodePlan(self.resolved_mode, self.partition_tokens, self.split_k_threshold_tokens,
                                     self.context_bucket_tokens, self.active_partition_capacity)


@dataclass(frozen=True)
class Qwen35OnlineDecodeWorkspaceLayout:
    partial_count: int = 0
    max_offset_bytes: int = 0
    sum_offset_bytes: int = 0
    value_offset_bytes: int = 0
    bytes: int = 0


@dataclass(frozen=True)
class GatedDeltaShape:
    tokens: int
    hidden_size: int
    key_heads: int
    value_heads: int
    key_dim: int
    value_dim: int
    conv_width: int
    epsilon: float

    def c(self):
        return _lib.GatedDeltaShape(self.tokens, self.hidden_size, self.key_heads, self.value_heads, self.key_dim,
                                    self.value_dim, self.conv_width, self.epsilon)


@dataclass(frozen=True)
class GatedDeltaLaunchPolicy:
    schedule: int = 0
    warps_per_block: int = 4
    transposed_boundary_state: bool = False

    def c(self):
        return _lib.GatedDeltaLaunchPolicy(self.schedule, self.warps_per_block,
                                           1 if self.transposed_boundary_state else 0)


# ---- attention: sizes and plans ----------------------------------------------------------------
def qwen35_attention_workspace_floats(shape):
    out = C.c_size_t()
    s = shape.c()
    _check(lib.rib200_attention_workspace_floats(C.byref(s), C.byref(out)))
    return out.value


def qwen35_attention_cache_bytes(shape, policy):
    out = C.c_size_t()
    s = shape.c()
    _check(lib.rib200_attention_cache_bytes(C.byref(s), policy.c(), C.byref(out)))
    return out.value


def qwen35_attention_workspace_bytes(shape, policy=None):
    out = C.c_size_t()
    s = shape.c()
    if policy is None:  # the reference's one-argument overload: the materialized logits buffer in bytes
        policy = Qwen35AttentionLaunchPolicy(MATERIALIZED_REFERENCE, KV_F32, TOKEN_MAJOR)
    _check(lib.rib200_attention_workspace_bytes(C.byref(s), policy.c(), C.byref(out)))
    return out.value


def qwen35_online_decode_plan(shape, requested, context_tokens):
    plan = _lib.OnlineDecodePlan()
    s = shape.c()
    _check(lib.rib200_online_decode_plan(C.byref(s), requested, context_tokens, C.byref(plan)))
    return Qwen35OnlineDecodePlan(*plan.as_tuple())


def qwen35_online_decode_workspace_layout(shape, resolved_mode):
    layout = _lib.OnlineDecodeWorkspaceLayout()
    s = shape.c()
    _check(lib.rib200_online_decode_workspace_layout(C.byref(s), resolved_mode, C.byref(layout)))
    return Qwen35OnlineDecodeWorkspaceLayout(layout.partial_count, layout.max_offset_bytes,
                                             layout.sum_offset_bytes, layout.value_offset_bytes, layout.bytes)


def qwen35_online_attention_prefill_supported(shape, activation_dtype, policy):
    out = C.c_int32()
    s = shape.c()
    _check(lib.rib200_online_attention_prefill_supported(C.byref(s), activation_dtype, policy.c(), C.byref(out)))
    return bool(out.value)


def qwen35_online_attention_workspace_bytes(shape):
    out = C.c_size_t()
    s = shape.c()
    _check(lib.rib200_online_attention_workspace_bytes(C.byref(s), C.byref(out)))
    return out.value


# ---- attention: launchers ----------------------------------------------------------------------
def qwen35_causal_attention(query, key, value, gate, output, kv_cache, kv_cache_bytes, workspace, workspace_bytes,
                            shape, activation_dtype, policy, stream):
    s = shape.c()
    _check(lib.rib200_causal_attention(_ptr(query), _ptr(key), _ptr(value), _ptr(gate), _ptr(output),
                                       _ptr(kv_cache), kv_cache_bytes, _ptr(workspace), workspace_bytes,
                                       C.byref(s), activation_dtype, policy.c(), _stream(stream)))


def qwen35_online_attention_prefill(query, key, value, gate, output, kv_cache, kv_cache_bytes, shape,
                                    activation_dtype, cache_dtype, cache_layout, stream):
    s = shape.c()
    _check(lib.rib200_online_attention_prefill(_ptr(query), _ptr(key), _ptr(value), _ptr(gate), _ptr(output),
                                               _ptr(kv_cache), kv_cache_bytes, C.byref(s), activation_dtype,
                                               cache_dtype, cache_layout, _stream(stream)))


@dataclass(frozen=True)
class QkNormRopeShape:
    """cpp/kernels/qwen35_primitives.cuh:32-39"""
    tokens: int
    heads: int
    head_dim: int
    rotary_dim: int
    position_offset: int
    rope_base: float

    def c(self):
        return _lib.QkNormRopeShape(self.tokens, self.heads, self.head_dim, self.rotary_dim, self.position_offset,
                                    self.rope_base)


def qwen35_qk_norm_rope(input, weight, output, shape, epsilon, dtype, weight_dtype, stream, device_position=None):
    """cpp/kernels/qwen35_primitives.cuh:61-66"""
    s = shape.c()
    _check(lib.rib200_qk_norm_rope(_ptr(input), _ptr(weight), _ptr(output), C.byref(s), epsilon, dtype, weight_dtype,
                                   _stream(stream), _ptr(device_position)))


def qwen35_split_full_query_gate(query_gate, query, gate, tokens, heads, head_dim, dtype, stream):
    """cpp/kernels/qwen35_primitives.cuh:90-93"""
    _check(lib.rib200_split_full_query_gate(_ptr(query_gate), _ptr(query), _ptr(gate), tokens, heads, head_dim, dtype,
                                            _stream(stream)))


def attention_prologue(query_gate, key, value, query_norm_weight, key_norm_weight, query, gate, key_out, value_out,
                       shape, rotary_dim, rope_base, epsilon, dtype, weight_dtype, output_dtype, stream,
                       device_position=None):
    """The executor's three pre-attention calls (cpp/execution/qwen35_executor.cu:1989-2015) as one launch."""
    s = shape.c()
    _check(lib.rib200_attention_prologue(_ptr(query_gate), _ptr(key), _ptr(value), _ptr(query_norm_weight),
                                         _ptr(key_norm_weight), _ptr(query), _ptr(gate), _ptr(key_out),
                                         _ptr(value_out), C.byref(s), rotary_dim, rope_base, epsilon, dtype,
                                         weight_dtype, output_dtype, _ptr(device_position), _stream(stream)))


def online_attention_decode_from_host(host_token, host_output, device_token, device_output, kv_cache, kv_cache_bytes,
                                      workspace, workspace_bytes, shape, activation_dtype, cache_dtype, cache_layout,
                                      plan, device_position, stream):
    """One decode step driven from (pinned) host memory: rows q | k | v | gate go up, the [16][256] output comes
    back, and the call returns when it is there.  No counterpart in the reference."""
    s = shape.c()
    p = plan.c()
    _check(lib.rib200_online_attention_decode_from_host(_ptr(host_token), _ptr(host_output), _ptr(device_token),
                                                        _ptr(device_output), _ptr(kv_cache), kv_cache_bytes,
                                                        _ptr(workspace), workspace_bytes, C.byref(s),
                                                        activation_dtype, cache_dtype, cache_layout, C.byref(p),
                                                        _ptr(device_position), _stream(stream)))


def online_attention_prefill_scatter(query, key, value, gate, outputs, rank, total_query_heads, head_offset, kv_cache,
                                     kv_cache_bytes, shape, activation_dtype, cache_dtype, cache_layout, stream):
    """Head-sharded prefill: `outputs` lists every rank's full-width output buffer (pointers or tensors valid on
    this device), outputs[rank] being this rank's own; this rank's heads land at `head_offset` in each of them.
    No counterpart in the reference."""
    s = shape.c()
    array = (C.c_void_p * len(outputs))(*[_ptr(o) for o in outputs])
    _check(lib.rib200_online_attention_prefill_scatter(_ptr(query), _ptr(key), _ptr(value), _ptr(gate), array,
                                                       len(outputs), rank, total_query_heads, head_offset,
                                                       _ptr(kv_cache),
                                                       kv_cache_bytes, C.byref(s), activation_dtype, cache_dtype,
                                                       cache_layout, _stream(stream)))


def peer_rendezvous(flag_arrays, rank, epoch, stream):
    """Device-side rendezvous of the ranks behind the work already queued on `stream`."""
    array = (C.c_void_p * len(flag_arrays))(*[_ptr(f) for f in flag_arrays])
    _check(lib.rib200_peer_rendezvous(array, len(flag_arrays), rank, epoch, _stream(stream)))


def peer_rendezvous_bounded(flag_arrays, rank, epoch, limit_cycles, stream):
    """The rendezvous with the caller's bound on the device-side wait, in SM clock cycles."""
    array = (C.c_void_p * len(flag_arrays))(*[_ptr(f) for f in flag_arrays])
    _check(lib.rib200_peer_rendezvous_bounded(array, len(flag_arrays), rank, epoch, limit_cycles, _stream(stream)))


def shared_alloc(nbytes):
    """Zero-filled device memory other processes can map: (pointer, 64-byte handle)."""
    ptr = C.c_void_p()
    handle = (C.c_uint8 * 64)()
    _check(lib.rib200_shared_alloc(nbytes, C.byref(ptr), handle))
    return ptr.value, bytes(handle)


def shared_open(handle):
    ptr = C.c_void_p()
    raw = (C.c_uint8 * 64)(*handle)
    _check(lib.rib200_shared_open(raw, C.byref(ptr)))
    return ptr.value


def shared_close(pointer):
    _check(lib.rib200_shared_close(pointer))


def shared_free(pointer):
    _check(lib.rib200_shared_free(pointer))


def qwen35_online_attention_decode(query, key, value, gate, output, kv_cache, kv_cache_bytes, workspace,
                                   workspace_bytes, shape, activation_dtype, cache_dtype, cache_layout, plan,
                                   device_position, stream):
    """Plan overload (cpp/kernels/qwen35_online_attention.cuh:55-63).  Pass plan=None for the reference's
    plan-less overload (:65-68), which resolves to single-block mode and takes no workspace."""
    s = shape.c()
    if plan is None:
        plan = qwen35_online_decode_plan(shape, SINGLE_BLOCK, shape.past_tokens + 1)
        workspace, workspace_bytes = None, 0
    p = plan.c()
    _check(lib.rib200_online_attention_decode(_ptr(query), _ptr(key), _ptr(value), _ptr(gate), _ptr(output),
                                              _ptr(kv_cache), kv_cache_bytes, _ptr(workspace), workspace_bytes,
                                              C.byref(s), activation_dtype, cache_dtype, cache_layout, C.byref(p),
                                              _ptr(device_position), _stream(stream)))


def online_attention_decode_static_scratch(query, key, value, gate, output, kv_cache, kv_cache_bytes, shape,
                                           activation_dtype, device_position, stream):
    """Split-k decode whose partials live in an array built into the library (no workspace argument, nothing
    allocated): for hosts that cannot allocate on the decode path.  Caches of at most 32768 tokens; calls that
    overlap on one GPU race on the shared array.  See include/rib200.h."""
    s = shape.c()
    _check(lib.rib200_online_attention_decode_static_scratch(_ptr(query), _ptr(key), _ptr(value), _ptr(gate),
                                                             _ptr(output), _ptr(kv_cache), kv_cache_bytes,
                                                             C.byref(s), activation_dtype, _ptr(device_position),
                                                             _stream(stream)))


def batched_decode_workspace_bytes(batch, max_context_tokens):
    out = C.c_size_t()
    _check(lib.rib200_batched_decode_workspace_bytes(batch, max_context_tokens, C.byref(out)))
    return out.value


def batched_decode_attention(query, key, value, gate, output, kv_caches, max_context_tokens, positions, batch,
                             largest_max_context_tokens, workspace, workspace_bytes, stream):
    _check(lib.rib200_batched_decode_attention(_ptr(query), _ptr(key), _ptr(value), _ptr(gate), _ptr(output),
                                               _ptr(kv_caches), _ptr(max_context_tokens), _ptr(positions), batch,
                                               largest_max_context_tokens, _ptr(workspace), workspace_bytes,
                                               _stream(stream)))


PAGE_TOKENS = 256


def paged_decode_attention(query, key, value, gate, output, page_pool, pool_pages, block_tables, max_blocks_per_sequence,
                           positions, batch, workspace, workspace_bytes, stream):
    """Batched decode step over a pool of 256-token pages ([2][4][256][256] BF16 each) named by per-sequence block
    tables (uint32, device memory)."""
    _check(lib.rib200_paged_decode_attention(_ptr(query), _ptr(key), _ptr(value), _ptr(gate), _ptr(output),
                                             _ptr(page_pool), pool_pages, _ptr(block_tables), max_blocks_per_sequence,
                                             _ptr(positions), batch, _ptr(workspace), workspace_bytes,
                                             _stream(stream)))


# ---- gated delta ---------------------------------------------------------------------------------
def qwen35_gated_delta_workspace_bytes(shape):
    out = C.c_size_t()
    s = shape.c()
    _check(lib.rib200_gated_delta_workspace_bytes(C.byref(s), C.byref(out)), Qwen35DeltaError)
    return out.value


def qwen35_gated_delta_select_policy(shape, bucket_tokens):
    pol = _lib.GatedDeltaLaunchPolicy()
    s = shape.c()
    _check(lib.rib200_gated_delta_select_policy(C.byref(s), bucket_tokens, C.byref(pol)), Qwen35DeltaError)
    return GatedDeltaLaunchPolicy(pol.schedule, pol.warps_per_block, bool(pol.transposed_boundary_state))


def qwen35_gated_delta_schedule_diagnostic(shape, bucket_tokens):
    diag = _lib.GatedDeltaScheduleDiagnostic()
    s = shape.c()
    _check(lib.rib200_gated_delta_schedule_diagnostic(C.byref(s), bucket_tokens, C.byref(diag)), Qwen35DeltaError)
    return diag


def qwen35_gated_delta(input, conv_weight, recurrent_a, dt_bias, output_norm_weight, output, convolution_state,
                       recurrent_state, workspace, workspace_bytes, shape, dtype, weight_dtype, stream,
                       policy=None):
    s = shape.c()
    if policy is None:
        policy = qwen35_gated_delta_select_policy(shape, shape.tokens)
    _check(lib.rib200_gated_delta(_ptr(input), _ptr(conv_weight), _ptr(recurrent_a), _ptr(dt_bias),
                                  _ptr(output_norm_weight), _ptr(output), _ptr(convolution_state),
                                  _ptr(recurrent_state), _ptr(workspace), workspace_bytes, C.byref(s), policy.c(),
                                  dtype, weight_dtype, _stream(stream)), Qwen35DeltaError)


def gdn_core_workspace_bytes(tokens, key_heads, value_heads, key_dim, value_dim):
    out = C.c_size_t()
    _check(lib.rib200_gdn_core_workspace_bytes(tokens, key_heads, value_heads, key_dim, value_dim, C.byref(out)),
           Qwen35DeltaError)
    return out.value


def gdn_core(q, k, v, beta, log_decay, state, out, workspace, workspace_bytes, tokens, key_heads, value_heads,
             key_dim, value_dim, qkv_dtype, stream):
    _check(lib.rib200_gdn_core(_ptr(q), _ptr(k), _ptr(v), _ptr(beta), _ptr(log_decay), _ptr(state), _ptr(out),
                               _ptr(workspace), workspace_bytes, tokens, key_heads, value_heads, key_dim,
                               value_dim, qkv_dtype, _stream(stream)), Qwen35DeltaError)


def batched_gdn_decode(q, k, v, beta, log_decay, states, out, batch, key_heads, value_heads, stream):
    _check(lib.rib200_batched_gdn_decode(_ptr(q), _ptr(k), _ptr(v), _ptr(beta), _ptr(log_decay), _ptr(states),
                                         _ptr(out), batch, key_heads, value_heads, _stream(stream)),
           Qwen35DeltaError)


def online_attention_decode_early_kv_fetch(query, key, value, gate, output, kv_cache, kv_cache_bytes, workspace,
                                           workspace_bytes, shape, activation_dtype, cache_dtype, cache_layout, plan,
                                           stream):
    """rib200_online_attention_decode_early_kv_fetch: the decode step with a host position whose partition kernel
    fetches cache rows before the kernel in front of it has finished.  The caller promises that no work in flight
    writes the cache rows the step reads (see include/rib200.h)."""
    s, p = shape.c(), plan.c()
    _check(lib.rib200_online_attention_decode_early_kv_fetch(_ptr(query), _ptr(key), _ptr(value), _ptr(gate),
                                                             _ptr(output), _ptr(kv_cache), kv_cache_bytes,
                                                             _ptr(workspace), workspace_bytes, C.byref(s),
                                                             activation_dtype, cache_dtype, cache_layout, C.byref(p),
                                                             _stream(stream)))


def device_status(stream):
    bits = C.c_uint32()
    _check(lib.rib200_device_status(_stream(stream), C.byref(bits)))
    return bits.value


def version():
    return lib.rib200_version().decode()
