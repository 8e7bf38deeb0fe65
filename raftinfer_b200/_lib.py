"""Loads librib200.so (the CUDA library built from raftinfer_b200/csrc) and declares its C ABI.

There is no fallback of any kind: if the library is missing the import of this module raises, and the
operators in `raftinfer_b200.kernels` cannot be used.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librib200.so")

sz = C.c_size_t
vp = C.c_void_p


class Status(C.Structure):
    _fields_ = [("code", C.c_int32), ("message", C.c_char_p)]


class AttentionShape(C.Structure):
    _fields_ = [("tokens", sz), ("query_heads", sz), ("kv_heads", sz), ("head_dim", sz),
                ("max_context_tokens", sz), ("past_tokens", sz)]


class QkNormRopeShape(C.Structure):
    _fields_ = [("tokens", sz), ("heads", sz), ("head_dim", sz), ("rotary_dim", sz), ("position_offset", sz),
                ("rope_base", C.c_float)]


class AttentionLaunchPolicy(C.Structure):
    _fields_ = [("implementation", C.c_uint8), ("kv_cache_dtype", C.c_uint8), ("kv_cache_layout", C.c_uint8)]


class OnlineDecodePlan(C.Structure):
    _fields_ = [("resolved_mode", C.c_uint8), ("partition_tokens", sz), ("split_k_threshold_tokens", sz),
                ("context_bucket_tokens", sz), ("active_partition_capacity", sz)]

    def as_tuple(self):
        return (self.resolved_mode, self.partition_tokens, self.split_k_threshold_tokens,
                self.context_bucket_tokens, self.active_partition_capacity)


class OnlineDecodeWorkspaceLayout(C.Structure):
    _fields_ = [("partial_count", sz), ("max_offset_bytes", sz), ("sum_offset_bytes", sz),
                ("value_offset_bytes", sz), ("bytes", sz)]


class GatedDeltaShape(C.Structure):
    _fields_ = [("tokens", sz), ("hidden_size", sz), ("key_heads", sz), ("value_heads", sz), ("key_dim", sz),
                ("value_dim", sz), ("conv_width", sz), ("epsilon", C.c_float)]


class GatedDeltaLaunchPolicy(C.Structure):
    _fields_ = [("schedule", C.c_uint8), ("warps_per_block", C.c_uint32), ("transposed_boundary_state", C.c_uint8)]


class GatedDeltaScheduleDiagnostic(C.Structure):
    _fields_ = [("bucket_tokens", sz), ("key_dim", sz), ("value_dim", sz), ("candidate_schedule", C.c_uint8),
                ("schedule", C.c_uint8), ("warps_per_block", C.c_uint32), ("transposed_boundary_state", C.c_uint8),
                ("candidate_accepted", C.c_uint8), ("correctness_passed", C.c_uint8),
                ("current_median_ms", C.c_float), ("candidate_median_ms", C.c_float),
                ("rejection_reason", C.c_char * 32)]


# name -> argument types (every function returns Status except rib200_version)
PROTOTYPES = {
    "rib200_attention_workspace_floats": [C.POINTER(AttentionShape), C.POINTER(sz)],
    "rib200_attention_cache_bytes": [C.POINTER(AttentionShape), AttentionLaunchPolicy, C.POINTER(sz)],
    "rib200_attention_workspace_bytes": [C.POINTER(AttentionShape), AttentionLaunchPolicy, C.POINTER(sz)],
    "rib200_online_decode_plan": [C.POINTER(AttentionShape), C.c_uint8, sz, C.POINTER(OnlineDecodePlan)],
    "rib200_online_decode_workspace_layout": [C.POINTER(AttentionShape), C.c_uint8,
                                              C.POINTER(OnlineDecodeWorkspaceLayout)],
    "rib200_online_attention_prefill_supported": [C.POINTER(AttentionShape), C.c_int32, AttentionLaunchPolicy,
                                                  C.POINTER(C.c_int32)],
    "rib200_online_attention_workspace_bytes": [C.POINTER(AttentionShape), C.POINTER(sz)],
    "rib200_gated_delta_workspace_bytes": [C.POINTER(GatedDeltaShape), C.POINTER(sz)],
    "rib200_gated_delta_select_policy": [C.POINTER(GatedDeltaShape), sz, C.POINTER(GatedDeltaLaunchPolicy)],
    "rib200_gated_delta_schedule_diagnostic": [C.POINTER(GatedDeltaShape), sz,
                                               C.POINTER(GatedDeltaScheduleDiagnostic)],
    "rib200_causal_attention": [vp, vp, vp, vp, vp, vp, sz, vp, sz, C.POINTER(AttentionShape), C.c_int32,
                                AttentionLaunchPolicy, vp],
    "rib200_online_attention_prefill": [vp, vp, vp, vp, vp, vp, sz, C.POINTER(AttentionShape), C.c_int32,
                                        C.c_uint8, C.c_uint8, vp],
    "rib200_online_attention_decode": [vp, vp, vp, vp, vp, vp, sz, vp, sz, C.POINTER(AttentionShape), C.c_int32,
                                       C.c_uint8, C.c_uint8, C.POINTER(OnlineDecodePlan), vp, vp],
    "rib200_online_attention_decode_from_host": [vp, vp, vp, vp, vp, sz, vp, sz, C.POINTER(AttentionShape), C.c_int32,
                                                 C.c_uint8, C.c_uint8, C.POINTER(OnlineDecodePlan), vp, vp],
    "rib200_online_attention_prefill_scatter": [vp, vp, vp, vp, C.POINTER(vp), sz, sz, sz, sz, vp, sz,
                                                C.POINTER(AttentionShape), C.c_int32, C.c_uint8, C.c_uint8, vp],
    "rib200_peer_rendezvous": [C.POINTER(vp), sz, sz, C.c_uint32, vp],
    "rib200_peer_rendezvous_bounded": [C.POINTER(vp), sz, sz, C.c_uint32, C.c_uint64, vp],
    "rib200_qk_norm_rope": [vp, vp, vp, C.POINTER(QkNormRopeShape), C.c_float, C.c_int32, C.c_int32, vp, vp],
    "rib200_split_full_query_gate": [vp, vp, vp, sz, sz, sz, C.c_int32, vp],
    "rib200_attention_prologue": [vp, vp, vp, vp, vp, vp, vp, vp, vp, C.POINTER(AttentionShape), sz, C.c_float,
                                  C.c_float, C.c_int32, C.c_int32, C.c_int32, vp, vp],
    "rib200_shared_alloc": [sz, C.POINTER(vp), C.POINTER(C.c_uint8)],
    "rib200_shared_open": [C.POINTER(C.c_uint8), C.POINTER(vp)],
    "rib200_shared_close": [vp],
    "rib200_shared_free": [vp],
    "rib200_gated_delta": [vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, C.POINTER(GatedDeltaShape),
                           GatedDeltaLaunchPolicy, C.c_int32, C.c_int32, vp],
    "rib200_gdn_core_workspace_bytes": [sz, sz, sz, sz, sz, C.POINTER(sz)],
    "rib200_gdn_core": [vp, vp, vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, sz, sz, C.c_int32, vp],
    "rib200_batched_decode_workspace_bytes": [sz, sz, C.POINTER(sz)],
    "rib200_batched_decode_attention": [vp, vp, vp, vp, vp, vp, vp, vp, sz, sz, vp, sz, vp],
    "rib200_batched_gdn_decode": [vp, vp, vp, vp, vp, vp, vp, sz, sz, sz, vp],
    "rib200_online_attention_decode_static_scratch": [vp, vp, vp, vp, vp, vp, sz, C.POINTER(AttentionShape), C.c_int32,
                                                      vp, vp],
    "rib200_online_attention_decode_early_kv_fetch": [vp, vp, vp, vp, vp, vp, sz, vp, sz, C.POINTER(AttentionShape),
                                                      C.c_int32, C.c_uint8, C.c_uint8,
                                                      C.POINTER(OnlineDecodePlan), vp],
    "rib200_paged_decode_attention": [vp, vp, vp, vp, vp, vp, sz, vp, sz, vp, sz, vp, sz, vp],
    "rib200_device_status": [vp, C.POINTER(C.c_uint32)],
}

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
        "(or `make -C raftinfer_b200/csrc`). raftinfer_b200 has no CPU or PyTorch fallback.")

lib = C.CDLL(LIB_PATH)
for _name, _args in PROTOTYPES.items():
    _fn = getattr(lib, _name)  # AttributeError here means the library is stale: rebuild it
    _fn.argtypes = _args
    _fn.restype = Status
lib.rib200_version.argtypes = []
lib.rib200_version.restype = C.c_char_p
