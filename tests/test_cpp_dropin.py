"""Compiles and runs the C++ drop-in header check (tests/cpp/dropin_compile_test.cpp) against librib200.so."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_dropin_header_compiles_and_behaves(tmp_path):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    cuda_inc = "/usr/local/cuda/include"
    exe = tmp_path / "dropin_test"
    lib_dir = os.path.join(ROOT, "raftinfer_b200")
    subprocess.run([cxx, "-std=c++20", "-O1", "-I", os.path.join(ROOT, "include"), "-I", cuda_inc,
                    os.path.join(ROOT, "tests", "cpp", "dropin_compile_test.cpp"), "-L", lib_dir, "-lrib200",
                    f"-Wl,-rpath,{lib_dir}", "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True)
    assert "dropin ok" in out.stdout


@pytest.mark.gpu
def test_executor_call_sequences_through_the_cpp_headers(tmp_path):
    """tests/cpp/dropin_gpu_test.cu makes the calls RAFTInfer's executor makes (full-attention layer: split, two
    norm/rope calls, qwen35_causal_attention on a 512-token chunk behind a past, then a decode step with a plan and a
    device position; linear layer: qwen35_gated_delta on a chunk, then on one token), FP32 activations, through the
    C++ drop-in headers only.  Its outputs are compared here with the CPU oracle."""
    import numpy as np

    from oracle import bindings as ob
    from raftinfer_b200 import synth

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    exe = tmp_path / "dropin_gpu_test"
    lib_dir = os.path.join(ROOT, "raftinfer_b200")
    subprocess.run([nvcc, "-std=c++20", "-O1", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "dropin_gpu_test.cu"), "-L", lib_dir, "-lrib200", "-Xlinker",
                    f"-rpath={lib_dir}", "-o", str(exe)], check=True)

    hq, hkv, d, rotary, base, eps = 16, 4, 256, 64, 1.0e7, 1.0e-6
    tokens, past, max_ctx, delta_tokens = 512, 640, 1536, 512
    seed = 0xB2004000
    put = lambda name, a: np.ascontiguousarray(a).tofile(tmp_path / f"{name}.bin")
    get = lambda name, dtype, shape: np.fromfile(tmp_path / f"{name}.bin", dtype=dtype).reshape(shape)

    # ---- full-attention layer ----
    query_gate = synth.normal(seed, 0, (tokens + 1, hq, 2, d)).astype(np.float32)
    key = synth.normal(seed, 1, (tokens + 1, hkv, d)).astype(np.float32)
    value = synth.normal(seed, 2, (tokens + 1, hkv, d)).astype(np.float32)
    qw = (1.0 + 0.1 * synth.normal(seed, 3, (d,))).astype(np.float32)
    kw = (1.0 + 0.1 * synth.normal(seed, 4, (d,))).astype(np.float32)
    cache = np.full((2, hkv, max_ctx, d), 0x7FC1, dtype=np.uint16)  # NaN pattern where nothing may be read
    cache[:, :, :past] = synth.bf16_bits(synth.normal(seed, 5, (2, hkv, past, d)).astype(np.float32))
    put("query_gate", query_gate[:tokens]), put("key", key[:tokens]), put("value", value[:tokens])
    put("decode_query_gate", query_gate[tokens:]), put("decode_key", key[tokens:]), put("decode_value", value[tokens:])
    put("q_norm_weight", qw), put("k_norm_weight", kw), put("kv_cache", cache)

    # ---- linear layer ----
    hk, hv, dk, width = 16, 32, 128, 4
    hidden, conv_dim = hv * dk, 2 * hk * dk + hv * dk
    stride = conv_dim + 2 * hv + hidden
    delta_in = synth.normal(seed, 6, (delta_tokens + 1, stride)).astype(np.float32)
    conv_w = (0.3 * synth.normal(seed, 7, (conv_dim, width))).astype(np.float32)
    rec_a = (-np.exp(0.3 * synth.normal(seed, 8, (hv,)))).astype(np.float32)
    dt_bias = (0.5 * synth.normal(seed, 9, (hv,))).astype(np.float32)
    norm_w = (1.0 + 0.1 * synth.normal(seed, 10, (dk,))).astype(np.float32)
    conv_state = (0.5 * synth.normal(seed, 11, (conv_dim, width - 1))).astype(np.float32)
    rec_state = (0.05 * synth.normal(seed, 12, (hv, dk, dk))).astype(np.float32)
    put("delta_input", delta_in), put("conv_weight", conv_w), put("recurrent_a", rec_a), put("dt_bias", dt_bias)
    put("output_norm_weight", norm_w), put("conv_state", conv_state), put("recurrent_state", rec_state)

    done = subprocess.run([str(exe), str(tmp_path), str(tokens), str(past), str(max_ctx), str(delta_tokens)],
                          capture_output=True, text=True, timeout=300)
    assert done.returncode == 0 and "dropin gpu ok" in done.stdout, done.stdout + done.stderr

    def within_tolerance(got, want):
        m = ob.compare(np.asarray(got, dtype=np.float32), np.asarray(want, dtype=np.float32))
        assert m["nonfinite"] == 0 and m["max_abs"] <= 3.0e-2 and m["rel_l2"] <= 1.0e-2, m

    # the oracle on the same operands, quantised where the kernels quantise: K, V and Q go to BF16
    qn = ob.qk_norm_rope(query_gate[:tokens, :, 0], qw, rotary, past, base, eps)
    kn = ob.qk_norm_rope(key[:tokens], kw, rotary, past, base, eps)
    want_cache = cache.copy()
    want_cache[0, :, past:past + tokens] = synth.bf16_bits(kn).transpose(1, 0, 2)
    want_cache[1, :, past:past + tokens] = synth.bf16_bits(value[:tokens]).transpose(1, 0, 2)
    got_cache = get("kv_cache_after", np.uint16, cache.shape)
    assert np.array_equal(got_cache[:, :, :past], cache[:, :, :past]), "the past rows are untouched"
    assert np.array_equal(got_cache[:, :, past + tokens + 1:], cache[:, :, past + tokens + 1:]), "rows behind the step"
    appended = ob.from_bf16_bits(got_cache[:, :, past:past + tokens])
    expected = ob.from_bf16_bits(want_cache[:, :, past:past + tokens])
    # the GPU's norm/rope agrees with the oracle's to 2e-6, so a rounded row may differ in its last BF16 place
    assert np.all(np.abs(appended - expected) <= np.abs(expected) * 2.0 ** -7 + 1.0e-6)
    want = ob.attention_core_cache(synth.round_bf16(qn), query_gate[:tokens, :, 1], got_cache, max_ctx, past)
    within_tolerance(get("attention_output", np.float32, (tokens, hq, d)), want)

    position = past + tokens
    q1 = ob.qk_norm_rope(query_gate[tokens:, :, 0], qw, rotary, position, base, eps)
    want1 = ob.attention_core_cache(q1, query_gate[tokens:, :, 1], got_cache, max_ctx, position)
    within_tolerance(get("decode_output", np.float32, (1, hq, d)), want1)
    k1 = ob.from_bf16_bits(synth.bf16_bits(ob.qk_norm_rope(key[tokens:], kw, rotary, position, base, eps)))[0]
    assert np.all(np.abs(ob.from_bf16_bits(got_cache[0, :, position]) - k1) <= np.abs(k1) * 2.0 ** -7 + 1.0e-6)
    assert np.array_equal(got_cache[1, :, position], synth.bf16_bits(value[tokens]))

    shape = lambda n: (n, hidden, hk, hv, dk, dk, width, eps)
    want_a, cs, rs = ob.gated_delta_layer(delta_in[:delta_tokens], conv_w, rec_a, dt_bias, norm_w, conv_state, rec_state,
                                          shape(delta_tokens))
    want_b, cs, rs = ob.gated_delta_layer(delta_in[delta_tokens:], conv_w, rec_a, dt_bias, norm_w, cs, rs, shape(1))
    got = get("delta_output", np.float32, (delta_tokens + 1, hidden))
    within_tolerance(got[:delta_tokens], want_a)
    within_tolerance(got[delta_tokens:], want_b)
    assert np.array_equal(get("conv_state_after", np.float32, cs.shape), cs)
    m = ob.compare(get("recurrent_state_after", np.float32, rs.shape).reshape(-1), rs.reshape(-1))
    assert m["nonfinite"] == 0 and m["rel_l2"] <= 1.0e-3, m
