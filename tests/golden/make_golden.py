"""Regenerates the golden fixtures under tests/golden/ from the RAFTInfer reference checkout.

Run where the reference checkout exists (its location is the REF environment variable) after `make -C oracle`:

    python tests/golden/make_golden.py

It writes
  * hf_tiny_layer.json      - the reference's Hugging Face golden layer fixture
                              (tests/fixtures/qwen35/tiny-layer-v1.bin, decoded per
                              cpp/tests/qwen35_fixture_test.cpp:105-161) as JSON;
  * known_answers.json      - the literal known-answer inputs/outputs of
                              cpp/tests/qwen35_reference_test.cpp:59-156, lifted from that file's text;
  * ref_model_shape.npz     - outputs of the reference's own CPU library (oracle/_ref) at the model
                              shapes on seeded operands (raftinfer_b200.synth), so that machines without
                              the reference checkout can still pin the oracle at D=256 / dk=dv=128.
The GPU box never runs this script; it reads the committed files.
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = os.environ.get("REF") or sys.exit("set REF to the path of the RAFTInfer checkout")

from oracle import bindings as ob  # noqa: E402
from raftinfer_b200 import synth  # noqa: E402


def decode_fixture(path):
    raw = open(path, "rb").read()
    assert raw[:8] == b"RIFQ35F1"
    version, endian, length = struct.unpack_from("<IIQ", raw, 8)
    assert version == 1 and endian == 0x01020304 and length == len(raw)
    off = 24
    full_names = ["tokens", "hidden_size", "query_heads", "kv_heads", "head_dim", "rotary_dim", "position_offset"]
    full = dict(zip(full_names, struct.unpack_from("<7I", raw, off)))
    off += 28
    full["rope_base"], full["epsilon"] = struct.unpack_from("<ff", raw, off)
    off += 8
    delta_names = ["tokens", "hidden_size", "key_heads", "value_heads", "key_dim", "value_dim", "conv_width"]
    delta = dict(zip(delta_names, struct.unpack_from("<7I", raw, off)))
    off += 28
    (delta["epsilon"],) = struct.unpack_from("<f", raw, off)
    off += 4
    names = ["full_input", "full_query_norm_weight", "full_key_norm_weight", "full_output_weight",
             "full_expected_output", "delta_input", "delta_conv_weight", "delta_recurrent_a", "delta_dt_bias",
             "delta_output_norm_weight", "delta_initial_convolution", "delta_initial_recurrent",
             "delta_expected_output", "delta_expected_convolution", "delta_expected_recurrent"]
    vectors = {}
    for name in names:
        (count,) = struct.unpack_from("<Q", raw, off)
        off += 8
        vectors[name] = [float(x) for x in np.frombuffer(raw, dtype="<f4", count=count, offset=off)]
        off += 4 * count
    assert off == len(raw)
    return {"source_sha256": hashlib.sha256(raw).hexdigest(), "full": full, "delta": delta, "vectors": vectors}


def lift_known_answers(path):
    """Pull the float lists out of the attention and gated-delta blocks of the reference's test."""
    text = open(path).read()
    number = r"-?\d+\.\d+(?:[eE][-+]?\d+)?F?"

    def named(name, occurrence=0):
        bodies = re.findall(name + r"\s*\{([^{}]*)\}", text)
        return [float(tok.rstrip("Ff")) for tok in re.findall(number, bodies[occurrence])]

    def expected_after(marker, count):
        tail = text[text.index(marker):]
        body = re.search(r"std::array<float,\s*%d>\s*\{([^{}]*)\}" % count, tail).group(1)
        return [float(tok.rstrip("Ff")) for tok in re.findall(number, body)]

    attn = {"args": dict(tokens=2, hidden_size=4, query_heads=2, kv_heads=1, head_dim=2, rotary_dim=2,
                         position_offset=0, rope_base=10000.0, epsilon=1.0e-6),
            "input": named("24> input"), "output_weight": named("output_weight", 0),
            "query_norm_weight": named("query_norm_weight"), "key_norm_weight": named("key_norm_weight"),
            "expected": expected_after("qwen35_gated_full_attention(", 8)}
    delta = {"args": dict(tokens=3, hidden_size=4, key_heads=1, value_heads=2, key_dim=2, value_dim=2,
                          conv_width=4, epsilon=1.0e-6),
             "input": named("48> input"), "conv_weight": named("conv_weight"),
             "recurrent_a": named("recurrent_a"), "dt_bias": named("dt_bias"),
             "output_norm_weight": named("output_norm_weight"),
             "expected": expected_after("qwen35_gated_delta_prefill(", 12)}
    rms = {"input": named("6> input"), "weight": named("3> weight"),
           "expected": expected_after("qwen35_rms_norm(input", 6)}
    return {"attention": attn, "gated_delta": delta, "rms_norm": rms}


def model_shape_reference():
    """The unmodified reference library on seeded model-shape operands."""
    assert ob.ref() is not None, "build oracle/_ref first (make -C oracle)"
    out = {}
    # Full attention, 16 q / 4 kv heads, D=256, identity output projection, T=6, rotary 64.
    T, Hq, Hkv, D = 6, 16, 4, 256
    hidden = Hq * D
    seed = 0xB2000010
    q = synth.round_bf16(synth.normal(seed, 0, (T, Hq * D)))
    k = synth.round_bf16(synth.normal(seed, 1, (T, Hkv * D)))
    v = synth.round_bf16(synth.normal(seed, 2, (T, Hkv * D)))
    g = synth.round_bf16(synth.normal(seed, 3, (T, hidden)))
    qw = 1.0 + 0.1 * synth.normal(seed, 4, (D,))
    kw = 1.0 + 0.1 * synth.normal(seed, 5, (D,))
    inp = np.concatenate([q, k, v, g], axis=1)
    eye = np.eye(hidden, dtype=np.float32)
    out["attn_out"] = ob.ref_full_attention_layer(inp, qw, kw, eye, tokens=T, hidden=hidden, q_heads=Hq,
                                                  kv_heads=Hkv, head_dim=D, rotary=64, pos_offset=3,
                                                  rope_base=1.0e7, eps=1.0e-6)
    out["attn_meta"] = np.array([T, Hq, Hkv, D, 64, 3, seed], dtype=np.int64)
    # Gated delta layer, 16 k / 32 v heads, dk = dv = 128, conv 4, T=5.
    T, Hk, Hv, dk, dv, W = 5, 16, 32, 128, 128, 4
    hidden = Hv * dv
    conv_dim = 2 * Hk * dk + hidden
    stride = conv_dim + 2 * Hv + hidden
    seed = 0xB2000011
    inp = synth.round_bf16(synth.normal(seed, 0, (T, stride)))
    conv_w = (0.3 * synth.normal(seed, 1, (conv_dim, W))).astype(np.float32)
    rec_a = (-np.exp(0.3 * synth.normal(seed, 2, (Hv,)))).astype(np.float32)
    dt_bias = (0.5 * synth.normal(seed, 3, (Hv,))).astype(np.float32)
    norm_w = (1.0 + 0.1 * synth.normal(seed, 4, (dv,))).astype(np.float32)
    cs = (0.5 * synth.normal(seed, 5, (conv_dim, W - 1))).astype(np.float32)
    rs = (0.1 * synth.normal(seed, 6, (Hv, dk, dv))).astype(np.float32)
    o, cs2, rs2 = ob.ref_gated_delta_layer(inp, conv_w, rec_a, dt_bias, norm_w, cs, rs,
                                           (T, hidden, Hk, Hv, dk, dv, W, 1.0e-6))
    out["delta_out"] = o
    out["delta_conv_state"] = cs2
    out["delta_state_sample"] = rs2.reshape(-1)[::61].copy()
    out["delta_state_sum"] = np.array([rs2.astype(np.float64).sum(), np.abs(rs2.astype(np.float64)).sum()])
    out["delta_meta"] = np.array([T, Hk, Hv, dk, dv, W, seed], dtype=np.int64)
    return out


def main():
    fixture = decode_fixture(os.path.join(REF, "tests/fixtures/qwen35/tiny-layer-v1.bin"))
    json.dump(fixture, open(os.path.join(HERE, "hf_tiny_layer.json"), "w"), indent=0)
    known = lift_known_answers(os.path.join(REF, "cpp/tests/qwen35_reference_test.cpp"))
    json.dump(known, open(os.path.join(HERE, "known_answers.json"), "w"), indent=0)
    np.savez_compressed(os.path.join(HERE, "ref_model_shape.npz"), **model_shape_reference())
    print("wrote golden fixtures; fixture sha256", fixture["source_sha256"])


if __name__ == "__main__":
    main()
