"""Causal GQA prefill attention with sigmoid gate on the GPU against the CPU oracle, through the C ABI.

Cases follow the reference's online-attention tests (cpp/tests/qwen35_cuda_attention_test.cu:638-766: shapes
{17,16,4,256,0}, {128,...,0}, {17,...,past=111}, causality under perturbation of the last token, rescaling under
logits from -80 to +80) at the model shape, extended to N(0,1) operands, ragged tails, past contexts that are not
a multiple of the tile and the 4096-token prefill.  Tolerance: BF16 outputs against the fp32-accumulated oracle,
max abs <= 3e-2 and relative L2 <= 1e-2."""
import numpy as np
import pytest
import torch

from oracle import bindings as ob
from raftinfer_b200 import kernels as K
from raftinfer_b200 import synth

from gpu_util import (D, HKV, HQ, act_tensor, cache_bits_of, cache_to_device, compare, dev, gate_bf16_outputs,
                      make_cache, to_numpy_f32)

pytestmark = pytest.mark.gpu
POLICY = K.Qwen35AttentionLaunchPolicy(K.ONLINE_TILED, K.KV_BF16, K.HEAD_MAJOR)


def operands(seed, tokens, past, q_scale=1.0):
    q = synth.round_bf16(synth.normal(seed, 0, (tokens, HQ, D)) * q_scale)
    gate = synth.round_bf16(synth.normal(seed, 1, (tokens, HQ, D)))
    k = synth.round_bf16(synth.normal(seed, 2, (past + tokens, HKV, D)))
    v = synth.round_bf16(synth.normal(seed, 3, (past + tokens, HKV, D)))
    return q, gate, k, v


def run_prefill(tokens, past, max_ctx, dtype, seed, q_scale=1.0, rows_to_check=None, via_dispatcher=False):
    q, gate, k, v = operands(seed, tokens, past, q_scale)
    cache = cache_to_device(make_cache(k, v, max_ctx, past))
    shape = K.Qwen35AttentionShape(tokens, HQ, HKV, D, max_ctx, past)
    out = torch.full((tokens, HQ, D), 5.0, device=dev(), dtype=torch.float32 if dtype == K.DTYPE_F32 else torch.bfloat16)
    stream = torch.cuda.current_stream()
    args = (act_tensor(q, dtype), act_tensor(k[past:], dtype), act_tensor(v[past:], dtype), act_tensor(gate, dtype), out,
            cache, cache.numel() * 2)
    if via_dispatcher:
        K.qwen35_causal_attention(*args, None, 0, shape, dtype, POLICY, stream)
    else:
        K.qwen35_online_attention_prefill(*args, shape, dtype, K.KV_BF16, K.HEAD_MAJOR, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0
    full = make_cache(k, v, max_ctx, past + tokens)
    assert np.array_equal(cache_bits_of(cache).reshape(full.shape), full), "appended cache rows"
    got = to_numpy_f32(out)
    spans = rows_to_check or [(0, tokens)]
    worst = None
    for lo, hi in spans:
        want = ob.attention_core(q[lo:hi], k[:past + hi], v[:past + hi], gate[lo:hi], past=past + lo)
        metrics = compare(got[lo:hi], want)
        gate_bf16_outputs(metrics)
        worst = metrics if worst is None or metrics["rel_l2"] > worst["rel_l2"] else worst
    return got, worst, (q, gate, k, v)


@pytest.mark.parametrize("tokens,past,max_ctx", [(2, 0, 4), (4, 0, 4), (17, 0, 64), (128, 0, 128), (129, 0, 300),
                                                  (17, 111, 128), (64, 200, 512), (512, 0, 512), (300, 77, 1024),
                                                  # few items with many key blocks: two CTAs split an item's keys
                                                  (17, 511, 1024), (128, 1000, 2048), (300, 640, 1024),
                                                  (512, 1536, 2048), (2, 700, 1024)])
@pytest.mark.parametrize("dtype", [K.DTYPE_BF16, K.DTYPE_F32])
def test_prefill_shapes(tokens, past, max_ctx, dtype):
    run_prefill(tokens, past, max_ctx, dtype, seed=0xB2004000 + tokens + past)


def test_prefill_through_the_dispatcher():
    run_prefill(40, 24, 64, K.DTYPE_BF16, seed=0xB2004100, via_dispatcher=True)


def test_reference_chunk_sequence_matches_one_shot():
    """The executor feeds a long prompt as chunks against a growing cache (cpp/execution/qwen35_executor.cu:727-732).
    Chunks 128 + 17 + 4 + 2 must give the rows a one-shot 151-token prefill gives."""
    total, max_ctx, seed = 151, 256, 0xB2004200
    one_shot, _, (q, gate, k, v) = run_prefill(total, 0, max_ctx, K.DTYPE_BF16, seed)
    cache = cache_to_device(make_cache(k, v, max_ctx, 0))
    stream = torch.cuda.current_stream()
    done = 0
    pieces = []
    for chunk in (128, 17, 4, 2):
        shape = K.Qwen35AttentionShape(chunk, HQ, HKV, D, max_ctx, done)
        out = torch.zeros(chunk, HQ, D, device=dev(), dtype=torch.bfloat16)
        sl = slice(done, done + chunk)
        K.qwen35_online_attention_prefill(act_tensor(q[sl], K.DTYPE_BF16), act_tensor(k[sl], K.DTYPE_BF16),
                                          act_tensor(v[sl], K.DTYPE_BF16), act_tensor(gate[sl], K.DTYPE_BF16), out,
                                          cache, cache.numel() * 2, shape, K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, stream)
        pieces.append(out)
        done += chunk
    torch.cuda.synchronize()
    chunked = np.concatenate([to_numpy_f32(x) for x in pieces])
    metrics = compare(chunked, one_shot)
    assert metrics["max_abs"] <= 2.0e-2 and metrics["rel_l2"] <= 5.0e-3, metrics


def test_causality_under_perturbation_of_the_last_token():
    """Changing the last token's K and V must leave every earlier output row bit-identical
    (cpp/tests/qwen35_cuda_attention_test.cu:688-705)."""
    tokens, past, max_ctx, seed = 200, 56, 256, 0xB2004300
    q, gate, k, v = operands(seed, tokens, past)
    outs = []
    for variant in range(2):
        kk, vv = k.copy(), v.copy()
        if variant:
            kk[-1] = synth.round_bf16(kk[-1] * -3.0 + 1.0)
            vv[-1] = synth.round_bf16(vv[-1] * 5.0 - 2.0)
        cache = cache_to_device(make_cache(kk, vv, max_ctx, past))
        out = torch.zeros(tokens, HQ, D, device=dev(), dtype=torch.bfloat16)
        K.qwen35_online_attention_prefill(act_tensor(q, K.DTYPE_BF16), act_tensor(kk[past:], K.DTYPE_BF16),
                                          act_tensor(vv[past:], K.DTYPE_BF16), act_tensor(gate, K.DTYPE_BF16), out, cache,
                                          cache.numel() * 2, K.Qwen35AttentionShape(tokens, HQ, HKV, D, max_ctx, past),
                                          K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, torch.cuda.current_stream())
        torch.cuda.synchronize()
        outs.append(out.view(torch.int16).cpu().numpy())
    assert np.array_equal(outs[0][:-1], outs[1][:-1])
    assert not np.array_equal(outs[0][-1], outs[1][-1])


def test_large_logits_rescale_correctly():
    # logits of order +-80: the lazily moved reference maximum must neither overflow nor lose the dominant key
    run_prefill(140, 0, 256, K.DTYPE_F32, seed=0xB2004400, q_scale=80.0)
    run_prefill(140, 30, 256, K.DTYPE_BF16, seed=0xB2004401, q_scale=80.0)


def test_unwritten_cache_rows_are_never_read():
    # make_cache leaves NaN patterns beyond the live context; a finite output proves they were not touched
    got, _, _ = run_prefill(70, 10, 1024, K.DTYPE_BF16, seed=0xB2004500)
    assert np.isfinite(got).all()


def test_full_4096_token_prefill_on_sampled_rows():
    spans = [(0, 130), (1000, 1040), (2047, 2050), (4000, 4096)]
    _, worst, _ = run_prefill(4096, 0, 4096, K.DTYPE_BF16, seed=0xB2004600, rows_to_check=spans)
    assert worst["rel_l2"] <= 1.0e-2


def test_drop_in_chunk_512_after_3584_past():
    run_prefill(512, 3584, 4096, K.DTYPE_BF16, seed=0xB2004700, rows_to_check=[(0, 64), (448, 512)])


@pytest.mark.parametrize("hq,hkv", [(8, 2), (2, 1), (3, 3), (12, 4), (4, 1)])
def test_other_head_counts(hq, hkv):
    """The prefill signature takes any query_heads that is a multiple of kv_heads (reference
    cpp/kernels/qwen35_online_attention.cu:33-44); a head-sharded rank passes exactly such a slice."""
    tokens, past, max_ctx, seed = 150, 20, 256, 0xB2004800 + hq * 16 + hkv
    q = synth.round_bf16(synth.normal(seed, 0, (tokens, hq, D)))
    gate = synth.round_bf16(synth.normal(seed, 1, (tokens, hq, D)))
    k = synth.round_bf16(synth.normal(seed, 2, (past + tokens, hkv, D)))
    v = synth.round_bf16(synth.normal(seed, 3, (past + tokens, hkv, D)))
    cache_bits = np.full((2, hkv, max_ctx, D), 0x7FC1, dtype=np.uint16)
    cache_bits[0, :, :past] = synth.bf16_bits(k[:past]).transpose(1, 0, 2)
    cache_bits[1, :, :past] = synth.bf16_bits(v[:past]).transpose(1, 0, 2)
    cache = cache_to_device(cache_bits)
    out = torch.zeros(tokens, hq, D, device=dev(), dtype=torch.bfloat16)
    shape = K.Qwen35AttentionShape(tokens, hq, hkv, D, max_ctx, past)
    assert K.qwen35_online_attention_prefill_supported(shape, K.DTYPE_BF16, POLICY)
    K.qwen35_online_attention_prefill(act_tensor(q, K.DTYPE_BF16), act_tensor(k[past:], K.DTYPE_BF16),
                                      act_tensor(v[past:], K.DTYPE_BF16), act_tensor(gate, K.DTYPE_BF16), out, cache,
                                      cache.numel() * 2, shape, K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR,
                                      torch.cuda.current_stream())
    torch.cuda.synchronize()
    want = ob.attention_core(q, k, v, gate, past=past)
    gate_bf16_outputs(compare(to_numpy_f32(out), want))
    got_cache = cache_bits_of(cache).reshape(cache_bits.shape)
    assert np.array_equal(got_cache[0, :, past:past + tokens], synth.bf16_bits(k[past:]).transpose(1, 0, 2))
    assert np.array_equal(got_cache[:, :, past + tokens:], cache_bits[:, :, past + tokens:])


@pytest.mark.parametrize("hq,hkv,dtype", [(2, 1, K.DTYPE_BF16), (3, 3, K.DTYPE_BF16), (2, 1, K.DTYPE_F32)])
def test_a_ranks_slice_of_a_long_prompt_splits_only_its_long_tiles(hq, hkv, dtype):
    """Two or three heads of a 2688-token prompt (what a rank of eight computes): 21 tiles of 1 .. 21 key blocks, few
    enough items for the split form.  Only the tiles of 20 blocks and more share their keys between two CTAs (or pairs);
    the shorter ones are walked by the first CTA of their cluster alone while the second sits them out.  Rows of both
    kinds, and the appended cache rows, against the oracle."""
    tokens, seed = 2688, 0xB2004900 + hq
    q = synth.round_bf16(synth.normal(seed, 0, (tokens, hq, D)))
    gate = synth.round_bf16(synth.normal(seed, 1, (tokens, hq, D)))
    k = synth.round_bf16(synth.normal(seed, 2, (tokens, hkv, D)))
    v = synth.round_bf16(synth.normal(seed, 3, (tokens, hkv, D)))
    cache = cache_to_device(np.full((2, hkv, tokens, D), 0x7FC1, dtype=np.uint16))
    out = torch.zeros(tokens, hq, D, device=dev(), dtype=torch.float32 if dtype == K.DTYPE_F32 else torch.bfloat16)
    shape = K.Qwen35AttentionShape(tokens, hq, hkv, D, tokens, 0)
    stream = torch.cuda.current_stream()
    K.qwen35_online_attention_prefill(act_tensor(q, dtype), act_tensor(k, dtype), act_tensor(v, dtype),
                                      act_tensor(gate, dtype), out, cache, cache.numel() * 2, shape, dtype, K.KV_BF16,
                                      K.HEAD_MAJOR, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0
    got = to_numpy_f32(out)
    # the first tile, the last unsplit tile and the first split one (rows 2304 .. 2559), the end of the prompt
    for lo, hi in ((0, 64), (2304, 2560), (tokens - 64, tokens)):
        want = ob.attention_core(q[lo:hi], k[:hi], v[:hi], gate[lo:hi], past=lo)
        gate_bf16_outputs(compare(got[lo:hi], want))
    got_cache = cache_bits_of(cache).reshape(2, hkv, tokens, D)
    assert np.array_equal(got_cache[0], synth.bf16_bits(k).transpose(1, 0, 2))
    assert np.array_equal(got_cache[1], synth.bf16_bits(v).transpose(1, 0, 2))
