"""Pins the CPU oracle (oracle/oracle.cpp) before anything is checked against it.

Three anchors: the reference's literal known answers (cpp/tests/qwen35_reference_test.cpp:59-156), the
Hugging Face golden layer fixture the reference ships (cpp/tests/qwen35_fixture_test.cpp:234-295, 1e-5 abs-or-rel),
and outputs of the reference's own CPU library at model shape (committed in ref_model_shape.npz, and re-derived
live from oracle/_ref when that library is present).
"""
import json
import os

import numpy as np
import pytest

from oracle import bindings as ob
from raftinfer_b200 import synth


def near(actual, expected, tol=1.0e-5):
    actual = np.asarray(actual, dtype=np.float64).reshape(-1)
    expected = np.asarray(expected, dtype=np.float64).reshape(-1)
    assert actual.shape == expected.shape
    err = np.abs(actual - expected)
    scale = np.maximum(np.abs(actual), np.abs(expected))
    bad = (err > tol) & (err > tol * scale)
    assert not bad.any(), f"max err {err.max()}"


@pytest.fixture(scope="module")
def known(golden_dir):
    return json.load(open(os.path.join(golden_dir, "known_answers.json")))


@pytest.fixture(scope="module")
def hf(golden_dir):
    return json.load(open(os.path.join(golden_dir, "hf_tiny_layer.json")))


def test_known_answer_full_attention(known):
    case = known["attention"]
    a = case["args"]
    out = ob.full_attention_layer(case["input"], case["query_norm_weight"], case["key_norm_weight"],
                                  case["output_weight"], tokens=a["tokens"], hidden=a["hidden_size"],
                                  q_heads=a["query_heads"], kv_heads=a["kv_heads"], head_dim=a["head_dim"],
                                  rotary=a["rotary_dim"], pos_offset=a["position_offset"],
                                  rope_base=a["rope_base"], eps=a["epsilon"])
    assert np.abs(out.reshape(-1) - np.array(case["expected"])).max() <= 1.0e-5


def test_known_answer_gated_delta(known):
    case = known["gated_delta"]
    a = case["args"]
    shape = (a["tokens"], a["hidden_size"], a["key_heads"], a["value_heads"], a["key_dim"], a["value_dim"],
             a["conv_width"], a["epsilon"])
    conv_dim = 2 * a["key_heads"] * a["key_dim"] + a["value_heads"] * a["value_dim"]
    cs = np.zeros((conv_dim, a["conv_width"] - 1), dtype=np.float32)
    rs = np.zeros((a["value_heads"], a["key_dim"], a["value_dim"]), dtype=np.float32)
    out, cs1, rs1 = ob.gated_delta_layer(case["input"], case["conv_weight"], case["recurrent_a"], case["dt_bias"],
                                         case["output_norm_weight"], cs, rs, shape)
    assert np.abs(out.reshape(-1) - np.array(case["expected"])).max() <= 1.0e-5
    # step == prefill (reference test :137-155): feed one token at a time, carrying both states.
    stride = conv_dim + 2 * a["value_heads"] + a["hidden_size"]
    inp = np.array(case["input"], dtype=np.float32).reshape(a["tokens"], stride)
    cs2, rs2, rows = cs.reshape(-1), rs.reshape(-1), []
    for t in range(a["tokens"]):
        o, cs2, rs2 = ob.gated_delta_layer(inp[t], case["conv_weight"], case["recurrent_a"], case["dt_bias"],
                                           case["output_norm_weight"], cs2, rs2, (1,) + shape[1:])
        rows.append(o)
    near(np.concatenate(rows), out)
    near(cs2, cs1)
    near(rs2, rs1)


def test_hf_fixture_full_attention(hf):
    a, v = hf["full"], hf["vectors"]
    out = ob.full_attention_layer(v["full_input"], v["full_query_norm_weight"], v["full_key_norm_weight"],
                                  v["full_output_weight"], tokens=a["tokens"], hidden=a["hidden_size"],
                                  q_heads=a["query_heads"], kv_heads=a["kv_heads"], head_dim=a["head_dim"],
                                  rotary=a["rotary_dim"], pos_offset=a["position_offset"],
                                  rope_base=a["rope_base"], eps=a["epsilon"])
    near(out, v["full_expected_output"])


def test_hf_fixture_gated_delta(hf):
    a, v = hf["delta"], hf["vectors"]
    shape = (a["tokens"], a["hidden_size"], a["key_heads"], a["value_heads"], a["key_dim"], a["value_dim"],
             a["conv_width"], a["epsilon"])
    out, cs, rs = ob.gated_delta_layer(v["delta_input"], v["delta_conv_weight"], v["delta_recurrent_a"],
                                       v["delta_dt_bias"], v["delta_output_norm_weight"],
                                       v["delta_initial_convolution"], v["delta_initial_recurrent"], shape)
    near(out, v["delta_expected_output"])
    near(cs, v["delta_expected_convolution"])
    near(rs, v["delta_expected_recurrent"])


def _attn_model_inputs(meta):
    T, Hq, Hkv, D, rotary, pos, seed = [int(x) for x in meta]
    hidden = Hq * D
    q = synth.round_bf16(synth.normal(seed, 0, (T, Hq * D)))
    k = synth.round_bf16(synth.normal(seed, 1, (T, Hkv * D)))
    v = synth.round_bf16(synth.normal(seed, 2, (T, Hkv * D)))
    g = synth.round_bf16(synth.normal(seed, 3, (T, hidden)))
    qw = 1.0 + 0.1 * synth.normal(seed, 4, (D,))
    kw = 1.0 + 0.1 * synth.normal(seed, 5, (D,))
    return T, Hq, Hkv, D, rotary, pos, q, k, v, g, qw, kw


def test_model_shape_attention_core_matches_reference_library(golden_dir):
    """The core extraction (pre-normalised operands, no projection) against the reference's fused layer with an
    identity projection: the extraction must agree to rounding (1e-6)."""
    z = np.load(os.path.join(golden_dir, "ref_model_shape.npz"))
    T, Hq, Hkv, D, rotary, pos, q, k, v, g, qw, kw = _attn_model_inputs(z["attn_meta"])
    qn = ob.qk_norm_rope(q.reshape(T, Hq, D), qw, rotary, pos, 1.0e7, 1.0e-6)
    kn = ob.qk_norm_rope(k.reshape(T, Hkv, D), kw, rotary, pos, 1.0e7, 1.0e-6)
    out = ob.attention_core(qn, kn, v.reshape(T, Hkv, D), g.reshape(T, Hq, D))
    assert np.abs(out.reshape(T, -1) - z["attn_out"]).max() <= 1.0e-6
    if ob.ref() is not None:
        live = ob.ref_full_attention_layer(np.concatenate([q, k, v, g], axis=1), qw, kw,
                                           np.eye(Hq * D, dtype=np.float32), tokens=T, hidden=Hq * D, q_heads=Hq,
                                           kv_heads=Hkv, head_dim=D, rotary=rotary, pos_offset=pos, rope_base=1.0e7,
                                           eps=1.0e-6)
        assert np.array_equal(live, z["attn_out"])


def test_model_shape_cache_accessor_equals_dense(golden_dir):
    """Reading K/V through the BF16 head-major cache gives bit-identical results to dense float K/V."""
    T, Hq, Hkv, D, past, max_ctx = 3, 16, 4, 256, 37, 64
    seed = 0xB2000012
    q = synth.round_bf16(synth.normal(seed, 0, (T, Hq, D)))
    g = synth.round_bf16(synth.normal(seed, 1, (T, Hq, D)))
    k = synth.round_bf16(synth.normal(seed, 2, (past + T, Hkv, D)))
    v = synth.round_bf16(synth.normal(seed, 3, (past + T, Hkv, D)))
    cache = np.full((2, Hkv, max_ctx, D), 0x7FC1, dtype=np.uint16)  # NaN where never written
    cache[0, :, : past + T] = synth.bf16_bits(k).transpose(1, 0, 2)
    cache[1, :, : past + T] = synth.bf16_bits(v).transpose(1, 0, 2)
    dense = ob.attention_core(q, k, v, g, past=past)
    cached = ob.attention_core_cache(q, g, cache, max_ctx, past)
    assert np.array_equal(dense, cached)
    assert np.isfinite(cached).all()


def test_model_shape_gated_delta_matches_reference_library(golden_dir):
    z = np.load(os.path.join(golden_dir, "ref_model_shape.npz"))
    T, Hk, Hv, dk, dv, W, seed = [int(x) for x in z["delta_meta"]]
    hidden = Hv * dv
    conv_dim = 2 * Hk * dk + hidden
    stride = conv_dim + 2 * Hv + hidden
    inp = synth.round_bf16(synth.normal(seed, 0, (T, stride)))
    conv_w = (0.3 * synth.normal(seed, 1, (conv_dim, W))).astype(np.float32)
    rec_a = (-np.exp(0.3 * synth.normal(seed, 2, (Hv,)))).astype(np.float32)
    dt_bias = (0.5 * synth.normal(seed, 3, (Hv,))).astype(np.float32)
    norm_w = (1.0 + 0.1 * synth.normal(seed, 4, (dv,))).astype(np.float32)
    cs = (0.5 * synth.normal(seed, 5, (conv_dim, W - 1))).astype(np.float32)
    rs = (0.1 * synth.normal(seed, 6, (Hv, dk, dv))).astype(np.float32)
    out, cs1, rs1 = ob.gated_delta_layer(inp, conv_w, rec_a, dt_bias, norm_w, cs, rs,
                                         (T, hidden, Hk, Hv, dk, dv, W, 1.0e-6))
    assert np.abs(out - z["delta_out"]).max() <= 1.0e-6
    assert np.abs(cs1.reshape(conv_dim, W - 1) - z["delta_conv_state"].reshape(conv_dim, W - 1)).max() == 0.0
    assert np.abs(rs1[::61] - z["delta_state_sample"]).max() <= 1.0e-6
    assert abs(rs1.astype(np.float64).sum() - z["delta_state_sum"][0]) <= 1.0e-3


def test_partials_recombine_to_core():
    """Split-k partials (max, sum, acc) merged with the rescale rule reproduce the un-split attention row."""
    Hq, Hkv, D, max_ctx, ctx, part = 16, 4, 256, 1024, 777, 256
    seed = 0xB2000013
    q = synth.round_bf16(synth.normal(seed, 0, (1, Hq, D)))
    k = synth.round_bf16(synth.normal(seed, 1, (ctx, Hkv, D)))
    v = synth.round_bf16(synth.normal(seed, 2, (ctx, Hkv, D)))
    cache = np.full((2, Hkv, max_ctx, D), 0x7FC1, dtype=np.uint16)
    cache[0, :, :ctx] = synth.bf16_bits(k).transpose(1, 0, 2)
    cache[1, :, :ctx] = synth.bf16_bits(v).transpose(1, 0, 2)
    pmax, psum, pval = ob.decode_partials(q[0], cache, max_ctx, ctx, part)
    parts = -(-ctx // part)
    m = pmax[:, :parts].max(axis=1, keepdims=True)
    w = np.exp(pmax[:, :parts] - m)
    merged = (w[:, :, None] * pval[:, :parts]).sum(axis=1) / (w * psum[:, :parts]).sum(axis=1, keepdims=True)
    zero_gate = np.full((1, Hq, D), 50.0, dtype=np.float32)  # sigmoid(50) == 1 in float
    want = ob.attention_core_cache(q, zero_gate, cache, max_ctx, ctx - 1)[0]
    assert np.abs(merged - want).max() <= 2.0e-6
    assert np.isnan(pmax[:, parts:]).all()


def test_compare_matches_reference_metrics():
    rng = np.random.default_rng(5)
    a = rng.standard_normal(1000).astype(np.float32)
    b = (a + 1e-3 * rng.standard_normal(1000)).astype(np.float32)
    b[7] = np.inf
    a[7] = np.inf
    b[9] = np.nan
    m = ob.compare(b, a)
    assert m["nonfinite"] == 1
    if ob.ref() is not None:
        out = np.zeros(4)
        assert ob.ref().ref_compare(b, a, a.size, 1e-12, out) == 0
        assert np.allclose(out, [m["max_abs"], m["max_rel"], m["cosine"], m["nonfinite"]], rtol=0, atol=0)
