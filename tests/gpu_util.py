"""Helpers shared by the GPU parity tests: seeded operands, device buffers, oracle calls, tolerance gates."""
import numpy as np
import torch

from oracle import bindings as ob
from raftinfer_b200 import kernels as K
from raftinfer_b200 import synth

HQ, HKV, D = 16, 4, 256
NAN_BITS = 0x7FC1  # BF16 NaN pattern for cache rows that must never be read


def dev():
    return torch.device("cuda:0")


def bf16_tensor(values_f32):
    """float32 numpy (already BF16-representable or not) -> torch.bfloat16 on the device, nearest even."""
    bits = synth.bf16_bits(np.ascontiguousarray(values_f32, dtype=np.float32))
    return torch.from_numpy(bits.view(np.int16)).to(dev()).view(torch.bfloat16)


def act_tensor(values_f32, dtype):
    if dtype == K.DTYPE_F32:
        return torch.from_numpy(np.ascontiguousarray(values_f32, dtype=np.float32)).to(dev())
    if dtype == K.DTYPE_F16:
        return torch.from_numpy(np.ascontiguousarray(values_f32, dtype=np.float32).astype(np.float16)).to(dev())
    return bf16_tensor(values_f32)


def to_numpy_f32(t):
    return t.detach().float().cpu().numpy()


def cache_bits_of(t):
    return t.detach().cpu().view(torch.int16).numpy().view(np.uint16)


def make_cache(k, v, max_ctx, rows):
    """Head-major BF16 cache [2][HKV][max_ctx][D] as uint16 bits holding rows [0, rows) of k, v
    ([ctx][HKV][D] float, BF16-representable); everything else is the NaN pattern."""
    cache = np.full((2, HKV, max_ctx, D), NAN_BITS, dtype=np.uint16)
    if rows:
        cache[0, :, :rows] = synth.bf16_bits(k[:rows]).transpose(1, 0, 2)
        cache[1, :, :rows] = synth.bf16_bits(v[:rows]).transpose(1, 0, 2)
    return cache


def cache_to_device(cache_bits):
    return torch.from_numpy(cache_bits.view(np.int16)).to(dev())


def decode_operands(seed, ctx, q_scale=1.0):
    """q, gate [HQ][D]; k, v [ctx][HKV][D]; all BF16-representable float32."""
    q = synth.round_bf16(synth.normal(seed, 0, (HQ, D)) * q_scale)
    gate = synth.round_bf16(synth.normal(seed, 1, (HQ, D)))
    k = synth.round_bf16(synth.normal(seed, 2, (ctx, HKV, D)))
    v = synth.round_bf16(synth.normal(seed, 3, (ctx, HKV, D)))
    return q, gate, k, v


def gate_bf16_outputs(metrics):
    """BF16 outputs against the fp32-accumulated oracle: max abs <= 3e-2 and relative L2 <= 1e-2."""
    assert metrics["nonfinite"] == 0, metrics
    assert metrics["max_abs"] <= 3.0e-2, metrics
    assert metrics["rel_l2"] <= 1.0e-2, metrics


def compare(candidate, reference):
    return ob.compare(np.asarray(candidate, dtype=np.float32), np.asarray(reference, dtype=np.float32))
