"""The step in front of the attention kernels - query/gate split, per-head RMSNorm with weight, partial RoPE -
against the CPU oracle (oracle.qk_norm_rope restates cpp/reference/qwen35.cpp:125-186,298-313 and is pinned
through the reference's fused layer), through the C ABI.

Cases follow the reference's tests of the two primitives (cpp/tests/qwen35_cuda_primitives_test.cu:318-341 and
:465-471 values against a CPU restatement with a position offset, :393-410 the split, :608-665 the throwing
argument checks) at the shapes this library serves (head_dim 256 and 128; the model's rotary 64, base 1e7), plus
BF16 tensors and weights, a device-side position and positions far into a long context.  FP32 results must agree with the
oracle to 2e-6 of the value range; BF16 results to one rounding."""
import numpy as np
import pytest
import torch

from oracle import bindings as ob
from raftinfer_b200 import kernels as K
from raftinfer_b200 import synth

from gpu_util import act_tensor, cache_to_device, compare, dev, gate_bf16_outputs, to_numpy_f32

pytestmark = pytest.mark.gpu
BASE, EPS = 1.0e7, 1.0e-6


def vectors(seed, tokens, heads, head_dim, bf16):
    x = synth.normal(seed, 0, (tokens, heads, head_dim)).astype(np.float32) * 1.7
    w = (1.0 + 0.1 * synth.normal(seed, 1, (head_dim,))).astype(np.float32)
    if bf16:
        x = synth.round_bf16(x)
    return x, w


@pytest.mark.parametrize("dtype", [K.DTYPE_F32, K.DTYPE_BF16])
@pytest.mark.parametrize("weight_bf16", [False, True])
@pytest.mark.parametrize("tokens,heads,head_dim,rotary,position", [
    (1, 16, 256, 64, 0), (17, 16, 256, 64, 111), (33, 4, 256, 64, 4095), (5, 16, 256, 64, 250000),
    (9, 3, 128, 64, 7), (6, 2, 128, 128, 1000), (4, 2, 256, 256, 31)])
def test_qk_norm_rope_matches_the_oracle(tokens, heads, head_dim, rotary, position, dtype, weight_bf16):
    bf16 = dtype == K.DTYPE_BF16
    x, w = vectors(0xB2001000 + tokens, tokens, heads, head_dim, bf16)
    if weight_bf16:
        w = synth.round_bf16(w)
    want = ob.qk_norm_rope(x, w, rotary, position, BASE, EPS)
    out = torch.zeros(tokens, heads, head_dim, device=dev(), dtype=torch.bfloat16 if bf16 else torch.float32)
    shape = K.QkNormRopeShape(tokens, heads, head_dim, rotary, position, BASE)
    K.qwen35_qk_norm_rope(act_tensor(x, dtype), act_tensor(w, K.DTYPE_BF16 if weight_bf16 else K.DTYPE_F32), out,
                          shape, EPS, dtype, K.DTYPE_BF16 if weight_bf16 else K.DTYPE_F32, torch.cuda.current_stream())
    torch.cuda.synchronize()
    got = to_numpy_f32(out)
    if bf16:
        # one BF16 rounding of the oracle's value, with room for a last-place difference before the rounding
        assert np.all(np.abs(got - want) <= np.abs(want) * 2.0 ** -8 + 1.0e-6)
    else:
        assert np.abs(got - want).max() <= 2.0e-6 * max(1.0, np.abs(want).max())


def test_qk_norm_rope_device_position():
    tokens, heads, head_dim, rotary, position = 1, 16, 256, 64, 777
    x, w = vectors(0xB2001100, tokens, heads, head_dim, False)
    want = ob.qk_norm_rope(x, w, rotary, position, BASE, EPS)
    out = torch.zeros(tokens, heads, head_dim, device=dev())
    dpos = torch.tensor([position], device=dev(), dtype=torch.int32)
    shape = K.QkNormRopeShape(tokens, heads, head_dim, rotary, 5, BASE)  # the host offset is ignored
    K.qwen35_qk_norm_rope(act_tensor(x, K.DTYPE_F32), act_tensor(w, K.DTYPE_F32), out, shape, EPS, K.DTYPE_F32,
                          K.DTYPE_F32, torch.cuda.current_stream(), dpos)
    torch.cuda.synchronize()
    assert np.abs(to_numpy_f32(out) - want).max() <= 2.0e-6 * np.abs(want).max()


@pytest.mark.parametrize("dtype,torch_dtype", [(K.DTYPE_F32, torch.float32), (K.DTYPE_BF16, torch.bfloat16)])
def test_split_full_query_gate_is_exact(dtype, torch_dtype):
    tokens, heads, head_dim = 19, 16, 256
    packed = synth.round_bf16(synth.normal(0xB2001200, 0, (tokens, heads, 2, head_dim)))
    src = act_tensor(packed, dtype)
    q = torch.zeros(tokens, heads, head_dim, device=dev(), dtype=torch_dtype)
    g = torch.zeros_like(q)
    K.qwen35_split_full_query_gate(src, q, g, tokens, heads, head_dim, dtype, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert torch.equal(q, src[:, :, 0]) and torch.equal(g, src[:, :, 1])


@pytest.mark.parametrize("dtype,out_dtype", [(K.DTYPE_F32, K.DTYPE_F32), (K.DTYPE_F32, K.DTYPE_BF16),
                                             (K.DTYPE_BF16, K.DTYPE_BF16)])
def test_fused_prologue_equals_the_three_calls(dtype, out_dtype):
    tokens, hq, hkv, d, rotary, past = 37, 16, 4, 256, 64, 300
    stream = torch.cuda.current_stream()
    bf16_in = dtype == K.DTYPE_BF16
    packed = synth.normal(0xB2001300, 0, (tokens, hq, 2, d)).astype(np.float32)
    k = synth.normal(0xB2001300, 1, (tokens, hkv, d)).astype(np.float32)
    v = synth.normal(0xB2001300, 2, (tokens, hkv, d)).astype(np.float32)
    if bf16_in:
        packed, k, v = synth.round_bf16(packed), synth.round_bf16(k), synth.round_bf16(v)
    qw = (1.0 + 0.1 * synth.normal(0xB2001300, 3, (d,))).astype(np.float32)
    kw = (1.0 + 0.1 * synth.normal(0xB2001300, 4, (d,))).astype(np.float32)
    t_in = torch.bfloat16 if bf16_in else torch.float32
    t_out = torch.bfloat16 if out_dtype == K.DTYPE_BF16 else torch.float32
    d_packed, d_k, d_v = act_tensor(packed, dtype), act_tensor(k, dtype), act_tensor(v, dtype)
    d_qw, d_kw = act_tensor(qw, K.DTYPE_F32), act_tensor(kw, K.DTYPE_F32)

    # the reference's sequence, in the input dtype
    q0 = torch.zeros(tokens, hq, d, device=dev(), dtype=t_in)
    g0 = torch.zeros_like(q0)
    K.qwen35_split_full_query_gate(d_packed, q0, g0, tokens, hq, d, dtype, stream)
    qn = torch.zeros_like(q0)
    kn = torch.zeros(tokens, hkv, d, device=dev(), dtype=t_in)
    K.qwen35_qk_norm_rope(q0, d_qw, qn, K.QkNormRopeShape(tokens, hq, d, rotary, past, BASE), EPS, dtype, K.DTYPE_F32,
                          stream)
    K.qwen35_qk_norm_rope(d_k, d_kw, kn, K.QkNormRopeShape(tokens, hkv, d, rotary, past, BASE), EPS, dtype,
                          K.DTYPE_F32, stream)

    fq = torch.zeros(tokens, hq, d, device=dev(), dtype=t_out)
    fg, fk, fv = torch.zeros_like(fq), torch.zeros(tokens, hkv, d, device=dev(), dtype=t_out), None
    fv = torch.zeros_like(fk)
    shape = K.Qwen35AttentionShape(tokens, hq, hkv, d, past + tokens, past)
    K.attention_prologue(d_packed, d_k, d_v, d_qw, d_kw, fq, fg, fk, fv, shape, rotary, BASE, EPS, dtype, K.DTYPE_F32,
                         out_dtype, stream)
    torch.cuda.synchronize()
    assert torch.equal(fq, qn.to(t_out)) and torch.equal(fk, kn.to(t_out))
    assert torch.equal(fg, g0.to(t_out)) and torch.equal(fv, d_v.to(t_out))


def test_prologue_then_prefill_matches_the_oracle_layer_core():
    """FP32 projections -> fused prologue (BF16 out) -> prefill attention, against qk_norm_rope + attention_core of
    the oracle (the composition that reproduces the reference's fused layer in tests/test_oracle_pins.py)."""
    tokens, hq, hkv, d, rotary = 200, 16, 4, 256, 64
    stream = torch.cuda.current_stream()
    packed = synth.normal(0xB2001400, 0, (tokens, hq, 2, d)).astype(np.float32)
    k = synth.normal(0xB2001400, 1, (tokens, hkv, d)).astype(np.float32)
    v = synth.normal(0xB2001400, 2, (tokens, hkv, d)).astype(np.float32)
    qw = (1.0 + 0.1 * synth.normal(0xB2001400, 3, (d,))).astype(np.float32)
    kw = (1.0 + 0.1 * synth.normal(0xB2001400, 4, (d,))).astype(np.float32)
    bf = lambda *s: torch.zeros(*s, device=dev(), dtype=torch.bfloat16)
    fq, fg, fk, fv = bf(tokens, hq, d), bf(tokens, hq, d), bf(tokens, hkv, d), bf(tokens, hkv, d)
    shape = K.Qwen35AttentionShape(tokens, hq, hkv, d, tokens, 0)
    K.attention_prologue(act_tensor(packed, K.DTYPE_F32), act_tensor(k, K.DTYPE_F32), act_tensor(v, K.DTYPE_F32),
                         act_tensor(qw, K.DTYPE_F32), act_tensor(kw, K.DTYPE_F32), fq, fg, fk, fv, shape, rotary,
                         BASE, EPS, K.DTYPE_F32, K.DTYPE_F32, K.DTYPE_BF16, stream)
    out = bf(tokens, hq, d)
    cache = bf(2, hkv, tokens, d)
    K.qwen35_online_attention_prefill(fq, fk, fv, fg, out, cache, cache.numel() * 2, shape, K.DTYPE_BF16, K.KV_BF16,
                                      K.HEAD_MAJOR, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0
    qn = ob.qk_norm_rope(packed[:, :, 0], qw, rotary, 0, BASE, EPS)
    kn = ob.qk_norm_rope(k, kw, rotary, 0, BASE, EPS)
    want = ob.attention_core(qn, kn, v, packed[:, :, 1])
    gate_bf16_outputs(compare(to_numpy_f32(out), want))


def test_argument_checks_follow_the_reference():
    stream = torch.cuda.current_stream()
    x = torch.zeros(2, 4, 256, device=dev())
    w = torch.zeros(256, device=dev())
    ok = K.QkNormRopeShape(2, 4, 256, 64, 0, BASE)
    bad_shapes = [K.QkNormRopeShape(0, 4, 256, 64, 0, BASE), K.QkNormRopeShape(2, 0, 256, 64, 0, BASE),
                  K.QkNormRopeShape(2, 4, 256, 0, 0, BASE), K.QkNormRopeShape(2, 4, 256, 258, 0, BASE),
                  K.QkNormRopeShape(2, 4, 256, 63, 0, BASE), K.QkNormRopeShape(2, 4, 256, 64, 0, -1.0),
                  K.QkNormRopeShape(2, 4, 256, 64, 0, float("inf"))]
    for shape in bad_shapes:
        with pytest.raises(K.Qwen35PrimitiveError):
            K.qwen35_qk_norm_rope(x, w, x, shape, EPS, K.DTYPE_F32, K.DTYPE_F32, stream)
    with pytest.raises(K.Qwen35PrimitiveError):
        K.qwen35_qk_norm_rope(None, w, x, ok, EPS, K.DTYPE_F32, K.DTYPE_F32, stream)
    with pytest.raises(K.Qwen35PrimitiveError):
        K.qwen35_qk_norm_rope(x, w, x, ok, -1.0, K.DTYPE_F32, K.DTYPE_F32, stream)
    with pytest.raises(K.Qwen35PrimitiveError):
        K.qwen35_qk_norm_rope(x, w, x, ok, EPS, K.DTYPE_F32, K.DTYPE_F32, None)
    with pytest.raises(K.Qwen35PrimitiveError):
        K.qwen35_qk_norm_rope(x, w, x, ok, EPS, 9, K.DTYPE_F32, stream)
    with pytest.raises(K.Qwen35PrimitiveError):
        K.qwen35_split_full_query_gate(x, x, None, 2, 4, 128, K.DTYPE_F32, stream)
    with pytest.raises(K.Qwen35PrimitiveError):
        K.qwen35_split_full_query_gate(x, x, x, 0, 4, 128, K.DTYPE_F32, stream)
