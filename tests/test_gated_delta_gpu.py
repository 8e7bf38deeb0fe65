"""Gated delta-rule kernels on the GPU against the CPU oracle, through the C ABI.

Cases follow cpp/tests/qwen35_cuda_delta_test.cu (T in {1,2,4,17}, decode after prefill, continued prefill, launches
sharing device state without a sync, saturation edges, mixed weight dtypes, the dk = dv = 128 model shape) with
N(0,1) operands.  Operands are quantised identically on both sides (cpp/tests/qwen35_cuda_delta_test.cu:257-270).
Tolerances: outputs max abs <= 3e-2 and relative L2 <= 1e-2; FP32 state relative L2 <= 1e-3."""
import numpy as np
import pytest
import torch

from oracle import bindings as ob
from raftinfer_b200 import kernels as K
from raftinfer_b200 import synth

from gpu_util import act_tensor, bf16_tensor, compare, dev, to_numpy_f32

pytestmark = pytest.mark.gpu
HK, HV, DK = 16, 32, 128


def core_operands(seed, tokens, hk=HK, hv=HV, quantise=True):
    q = synth.round_bf16(synth.normal(seed, 0, (tokens, hk, DK)))
    k = synth.round_bf16(synth.normal(seed, 1, (tokens, hk, DK)))
    v = synth.round_bf16(synth.normal(seed, 2, (tokens, hv, DK)))
    q = q / np.sqrt((q.astype(np.float64) ** 2).sum(-1, keepdims=True) + 1e-6) / np.sqrt(DK)
    k = k / np.sqrt((k.astype(np.float64) ** 2).sum(-1, keepdims=True) + 1e-6)
    q, k = q.astype(np.float32), k.astype(np.float32)
    if quantise:
        q, k = synth.round_bf16(q), synth.round_bf16(k)
    beta = synth.sigmoid(synth.normal(seed, 3, (tokens, hv)))
    g = (-synth.softplus(synth.normal(seed, 4, (tokens, hv)))).astype(np.float32)
    return q, k, v, beta, g


def run_core(tokens, dtype, seed, hk=HK, hv=HV, state0=None):
    q, k, v, beta, g = core_operands(seed, tokens, hk, hv, quantise=dtype == K.DTYPE_BF16)
    if state0 is None:
        state0 = (0.05 * synth.normal(seed, 5, (hv, DK, DK))).astype(np.float32)
    state = torch.from_numpy(state0.copy()).to(dev())
    out = torch.zeros(tokens, hv, DK, device=dev())
    ws_bytes = K.gdn_core_workspace_bytes(tokens, hk, hv, DK, DK)
    ws = torch.zeros(max(ws_bytes // 4, 4), device=dev())
    K.gdn_core(act_tensor(q, dtype), act_tensor(k, dtype), act_tensor(v, dtype),
               torch.from_numpy(beta).to(dev()), torch.from_numpy(g).to(dev()), state, out, ws, ws_bytes, tokens, hk, hv,
               DK, DK, dtype, torch.cuda.current_stream())
    torch.cuda.synchronize()
    want_out, want_state = ob.gdn_core(q, k, v, beta, np.exp(g), state0)
    m_out = compare(to_numpy_f32(out), want_out)
    m_state = compare(to_numpy_f32(state), want_state)
    return m_out, m_state


@pytest.mark.parametrize("tokens", [1, 2, 4, 17, 63])
@pytest.mark.parametrize("dtype", [K.DTYPE_BF16, K.DTYPE_F32])
def test_recurrent_core(tokens, dtype):
    m_out, m_state = run_core(tokens, dtype, seed=0xB2001000 + tokens)
    assert m_out["nonfinite"] == 0 and m_out["max_abs"] <= 1.0e-4 and m_out["rel_l2"] <= 1.0e-4, m_out
    assert m_state["nonfinite"] == 0 and m_state["rel_l2"] <= 1.0e-5, m_state


@pytest.mark.parametrize("tokens", [64, 65, 100, 128, 257, 1024])
@pytest.mark.parametrize("dtype", [K.DTYPE_BF16, K.DTYPE_F32])
def test_chunked_core_matches_the_sequential_recurrence(tokens, dtype):
    """Runs of 64 tokens or more take the chunk-64 WY-form kernels; the ground truth stays the token-sequential
    recurrence.  Outputs: max abs <= 3e-2, relative L2 <= 1e-2 (held to 2e-3); FP32 state relative L2 <= 1e-3."""
    m_out, m_state = run_core(tokens, dtype, seed=0xB2001300 + tokens)
    assert m_out["nonfinite"] == 0 and m_out["max_abs"] <= 3.0e-2 and m_out["rel_l2"] <= 2.0e-3, m_out
    assert m_state["nonfinite"] == 0 and m_state["rel_l2"] <= 1.0e-3, m_state


@pytest.mark.parametrize("hk,hv", [(16, 32), (4, 8)])
def test_chunked_core_long_run_equals_the_same_run_in_pieces(hk, hv):
    """A run of 9 297 tokens (146 chunks, ragged tail) in one call and the same tokens in three calls that split on
    chunk boundaries walk the same chunks with the same arithmetic: outputs and final state are bit-identical.  It
    also takes the barrier phases and the staging rings of the chunk kernels well past their first wrap-arounds."""
    tokens, cuts = 9297, (0, 4096, 4096 + 64, 9297)
    gen = torch.Generator(device=dev()).manual_seed(0xB2001500 + hv)
    unit = lambda x: x / x.norm(dim=-1, keepdim=True)
    q = (unit(torch.randn(tokens, hk, DK, device=dev(), generator=gen)) / DK ** 0.5).to(torch.bfloat16)
    k = unit(torch.randn(tokens, hk, DK, device=dev(), generator=gen)).to(torch.bfloat16)
    v = torch.randn(tokens, hv, DK, device=dev(), generator=gen).to(torch.bfloat16)
    beta = torch.sigmoid(torch.randn(tokens, hv, device=dev(), generator=gen))
    g = -torch.nn.functional.softplus(torch.randn(tokens, hv, device=dev(), generator=gen))
    state0 = 0.05 * torch.randn(hv, DK, DK, device=dev(), generator=gen)
    stream = torch.cuda.current_stream()

    def run(pieces):
        state = state0.clone()
        out = torch.zeros(tokens, hv, DK, device=dev())
        for lo, hi in pieces:
            n = hi - lo
            ws_bytes = K.gdn_core_workspace_bytes(n, hk, hv, DK, DK)
            ws = torch.zeros(max(ws_bytes // 4, 4), device=dev())
            K.gdn_core(q[lo:hi], k[lo:hi], v[lo:hi], beta[lo:hi], g[lo:hi], state, out[lo:hi], ws, ws_bytes, n, hk, hv,
                       DK, DK, K.DTYPE_BF16, stream)
        torch.cuda.synchronize()
        return out, state

    whole_out, whole_state = run([(0, tokens)])
    parts_out, parts_state = run(list(zip(cuts[:-1], cuts[1:])))
    assert K.device_status(stream) == 0
    assert torch.isfinite(whole_out).all() and torch.isfinite(whole_state).all()
    assert torch.equal(whole_out, parts_out) and torch.equal(whole_state, parts_state)


def test_chunked_prefill_4096_then_128_decode_steps():
    """The benchmark's gated-delta configuration: zero state, 4096-token chunked prefill, then 128 recurrent steps."""
    tokens, steps, seed = 4096, 128, 0xB2001400
    q, k, v, beta, g = core_operands(seed, tokens + steps)
    state0 = np.zeros((HV, DK, DK), dtype=np.float32)
    state = torch.zeros(HV, DK, DK, device=dev())
    out = torch.zeros(tokens + steps, HV, DK, device=dev())
    dq, dk, dv = bf16_tensor(q), bf16_tensor(k), bf16_tensor(v)
    dbeta, dg = torch.from_numpy(beta).to(dev()), torch.from_numpy(g).to(dev())
    ws_bytes = K.gdn_core_workspace_bytes(tokens, HK, HV, DK, DK)
    ws = torch.zeros(ws_bytes // 4, device=dev())
    stream = torch.cuda.current_stream()
    K.gdn_core(dq, dk, dv, dbeta, dg, state, out, ws, ws_bytes, tokens, HK, HV, DK, DK, K.DTYPE_BF16, stream)
    for t in range(tokens, tokens + steps):
        K.gdn_core(dq[t], dk[t], dv[t], dbeta[t], dg[t], state, out[t], None, 0, 1, HK, HV, DK, DK, K.DTYPE_BF16, stream)
    torch.cuda.synchronize()
    want_out, want_state = ob.gdn_core(q, k, v, beta, np.exp(g), state0)
    m_out = compare(to_numpy_f32(out), want_out)
    m_state = compare(to_numpy_f32(state), want_state)
    assert m_out["nonfinite"] == 0 and m_out["max_abs"] <= 3.0e-2 and m_out["rel_l2"] <= 1.0e-2, m_out
    assert m_state["nonfinite"] == 0 and m_state["rel_l2"] <= 1.0e-3, m_state


@pytest.mark.parametrize("hk,hv", [(2, 2), (1, 3), (3, 6)])
@pytest.mark.parametrize("dtype", [K.DTYPE_BF16, K.DTYPE_F32])
def test_chunked_core_other_head_counts(hk, hv, dtype):
    """Key heads equal to value heads, one key head for three value heads, odd counts: fewer (chunk, head) items than
    SMs, a ragged last chunk (200 tokens), the key head of a value head is head % key_heads."""
    m_out, m_state = run_core(200, dtype, seed=0xB2001900 + 16 * hk + hv, hk=hk, hv=hv)
    assert m_out["nonfinite"] == 0 and m_out["max_abs"] <= 3.0e-2 and m_out["rel_l2"] <= 2.0e-3, m_out
    assert m_state["nonfinite"] == 0 and m_state["rel_l2"] <= 1.0e-3, m_state


def test_recurrent_core_small_head_counts():
    m_out, m_state = run_core(3, K.DTYPE_F32, seed=0xB2001100, hk=2, hv=4)
    assert m_out["rel_l2"] <= 1.0e-4 and m_state["rel_l2"] <= 1.0e-5


def test_batched_decode_step():
    batch = 6
    seed = 0xB2001200
    q, k, v, beta, g = core_operands(seed, batch)  # one token per sequence
    states0 = [(0.05 * synth.normal(seed, 10 + i, (HV, DK, DK))).astype(np.float32) for i in range(batch)]
    states = [torch.from_numpy(s.copy()).to(dev()) for s in states0]
    ptrs = torch.tensor([s.data_ptr() for s in states], device=dev(), dtype=torch.int64)
    out = torch.zeros(batch, HV, DK, device=dev())
    K.batched_gdn_decode(bf16_tensor(q), bf16_tensor(k), bf16_tensor(v), torch.from_numpy(beta).to(dev()),
                         torch.from_numpy(g).to(dev()), ptrs, out, batch, HK, HV, torch.cuda.current_stream())
    torch.cuda.synchronize()
    got = to_numpy_f32(out)
    for i in range(batch):
        want_out, want_state = ob.gdn_core(q[i:i + 1], k[i:i + 1], v[i:i + 1], beta[i:i + 1], np.exp(g[i:i + 1]),
                                           states0[i])
        assert compare(got[i], want_out[0])["rel_l2"] <= 1.0e-4
        assert compare(to_numpy_f32(states[i]), want_state)["rel_l2"] <= 1.0e-5


# ---- whole layer (packed input) -------------------------------------------------------------------
def layer_operands(seed, tokens, hk, hv, width, scale=1.0):
    hidden = hv * DK
    conv_dim = 2 * hk * DK + hidden
    stride = conv_dim + 2 * hv + hidden
    inp = synth.round_bf16(scale * synth.normal(seed, 0, (tokens, stride)))
    conv_w = synth.round_bf16(0.3 * synth.normal(seed, 1, (conv_dim, width)))
    rec_a = (-np.exp(0.3 * synth.normal(seed, 2, (hv,)))).astype(np.float32)
    dt_bias = (0.5 * synth.normal(seed, 3, (hv,))).astype(np.float32)
    norm_w = (1.0 + 0.1 * synth.normal(seed, 4, (DK,))).astype(np.float32)
    conv_state = (0.5 * synth.normal(seed, 5, (conv_dim, width - 1))).astype(np.float32)
    rec_state = (0.05 * synth.normal(seed, 6, (hv, DK, DK))).astype(np.float32)
    return inp, conv_w, rec_a, dt_bias, norm_w, conv_state, rec_state


class LayerRun:
    """Device-side layer state carried across calls, with the oracle run in lock step."""

    def __init__(self, seed, hk, hv, width, dtype, wdtype, tokens_total, scale=1.0):
        self.hk, self.hv, self.width, self.dtype, self.wdtype = hk, hv, width, dtype, wdtype
        ops = layer_operands(seed, tokens_total, hk, hv, width, scale)
        self.inp, self.conv_w, self.rec_a, self.dt_bias, self.norm_w, self.cs, self.rs = ops
        if wdtype != K.DTYPE_F32:
            self.rec_a, self.dt_bias, self.norm_w = (synth.round_bf16(x) for x in (self.rec_a, self.dt_bias, self.norm_w))
        self.d_conv_w = act_tensor(self.conv_w, wdtype)
        self.d_rec_a = act_tensor(self.rec_a, wdtype)
        self.d_dt = act_tensor(self.dt_bias, wdtype)
        self.d_norm = act_tensor(self.norm_w, wdtype)
        self.d_cs = torch.from_numpy(self.cs.copy()).to(dev())
        self.d_rs = torch.from_numpy(self.rs.copy()).to(dev())
        self.done = 0

    def step(self, tokens, sync=True):
        hidden = self.hv * DK
        shape = K.GatedDeltaShape(tokens, hidden, self.hk, self.hv, DK, DK, self.width, 1.0e-6)
        chunk = self.inp[self.done:self.done + tokens]
        self.done += tokens
        ws_bytes = K.qwen35_gated_delta_workspace_bytes(shape)
        ws = torch.zeros(ws_bytes // 4, device=dev())
        out = torch.zeros(tokens, hidden, device=dev(),
                          dtype={K.DTYPE_F32: torch.float32, K.DTYPE_F16: torch.float16}.get(self.dtype, torch.bfloat16))
        d_in = act_tensor(chunk, self.dtype)
        K.qwen35_gated_delta(d_in, self.d_conv_w, self.d_rec_a, self.d_dt, self.d_norm, out, self.d_cs, self.d_rs, ws,
                             ws_bytes, shape, self.dtype, self.wdtype, torch.cuda.current_stream())
        if sync:
            torch.cuda.synchronize()
        want, self.cs, self.rs = ob.gated_delta_layer(chunk, self.conv_w, self.rec_a, self.dt_bias, self.norm_w, self.cs,
                                                      self.rs, (tokens, hidden, self.hk, self.hv, DK, DK, self.width,
                                                                1.0e-6))
        return out, want, (d_in, ws)

    def check(self, out, want, chunked=False):
        m = compare(to_numpy_f32(out), want)
        assert m["nonfinite"] == 0 and m["max_abs"] <= 3.0e-2 and m["rel_l2"] <= 1.0e-2, m
        if self.dtype == K.DTYPE_F32 and not chunked:
            assert m["max_abs"] <= 2.0e-3 and m["rel_l2"] <= 2.0e-4, m  # FP32 recurrent path
        if self.dtype == K.DTYPE_F32 and chunked:
            assert m["max_abs"] <= 1.5e-2 and m["rel_l2"] <= 2.0e-3, m  # TF32 tensor-core products
        cs = compare(to_numpy_f32(self.d_cs).reshape(-1), self.cs.reshape(-1))
        assert cs["max_abs"] == 0.0, cs
        rs = compare(to_numpy_f32(self.d_rs).reshape(-1), self.rs.reshape(-1))
        assert rs["nonfinite"] == 0 and rs["rel_l2"] <= 1.0e-3, rs


@pytest.mark.parametrize("tokens", [1, 2, 4, 17])
@pytest.mark.parametrize("dtype,wdtype", [(K.DTYPE_BF16, K.DTYPE_F32), (K.DTYPE_F32, K.DTYPE_F32),
                                          (K.DTYPE_BF16, K.DTYPE_BF16), (K.DTYPE_F32, K.DTYPE_BF16)])
def test_layer_small_heads(tokens, dtype, wdtype):
    run = LayerRun(0xB2002000 + tokens, 2, 4, 3, dtype, wdtype, tokens)
    out, want, _ = run.step(tokens)
    run.check(out, want)


@pytest.mark.parametrize("tokens", [3, 150])
@pytest.mark.parametrize("wdtype", [K.DTYPE_F32, K.DTYPE_F16])
def test_layer_f16_activations(tokens, wdtype):
    """FP16 input and output (the reference's delta launcher takes F32, F16 and BF16, cpp/kernels/qwen35_delta.cu:
    811-897): operands that FP16 holds exactly on both sides, the recurrent kernel (3 tokens) and the chunked one."""
    run = LayerRun(0xB2002600 + tokens, 2, 4, 4, K.DTYPE_F16, wdtype, tokens)
    half = lambda x: x.astype(np.float16).astype(np.float32)
    run.inp = half(run.inp)
    if wdtype == K.DTYPE_F16:
        run.conv_w, run.rec_a, run.dt_bias, run.norm_w = (half(x) for x in (run.conv_w, run.rec_a, run.dt_bias,
                                                                             run.norm_w))
        run.d_conv_w, run.d_rec_a = act_tensor(run.conv_w, wdtype), act_tensor(run.rec_a, wdtype)
        run.d_dt, run.d_norm = act_tensor(run.dt_bias, wdtype), act_tensor(run.norm_w, wdtype)
    out, want, _ = run.step(tokens)
    m = compare(to_numpy_f32(out), want)
    assert m["nonfinite"] == 0 and m["max_abs"] <= 3.0e-2 and m["rel_l2"] <= 1.0e-2, m
    assert compare(to_numpy_f32(run.d_cs).reshape(-1), run.cs.reshape(-1))["max_abs"] == 0.0
    assert compare(to_numpy_f32(run.d_rs).reshape(-1), run.rs.reshape(-1))["rel_l2"] <= 1.0e-3


def test_layer_model_shape_prefill_then_decode_then_continued_prefill():
    run = LayerRun(0xB2002100, HK, HV, 4, K.DTYPE_BF16, K.DTYPE_F32, 3 + 1 + 1 + 5)
    for tokens in (3, 1, 1, 5):
        out, want, _ = run.step(tokens)
        run.check(out, want)


@pytest.mark.parametrize("dtype", [K.DTYPE_BF16, K.DTYPE_F32])
def test_layer_chunked_prefill_then_decode(dtype):
    """A 150-token call takes the chunked kernels inside the layer; a one-token call follows on the same states."""
    run = LayerRun(0xB2002500, 4, 8, 4, dtype, K.DTYPE_F32, 151)
    for tokens in (150, 1):
        out, want, _ = run.step(tokens)
        run.check(out, want, chunked=True)


def test_layer_three_launches_share_device_state_without_a_sync():
    run = LayerRun(0xB2002200, 2, 4, 4, K.DTYPE_F32, K.DTYPE_F32, 6)
    results = [run.step(2, sync=False) for _ in range(3)]
    torch.cuda.synchronize()
    for out, want, _ in results[:-1]:
        m = compare(to_numpy_f32(out), want)
        assert m["max_abs"] <= 2.0e-3 and m["rel_l2"] <= 2.0e-4, m
    run.check(results[-1][0], results[-1][1])


def test_layer_conv_width_one_and_wide():
    for width in (1, 2, 6):
        run = LayerRun(0xB2002300 + width, 2, 4, width, K.DTYPE_F32, K.DTYPE_F32, 5)
        if width == 1:
            run.d_cs = torch.zeros(4, device=dev())
            run.cs = np.zeros((run.cs.shape[0], 0), dtype=np.float32)
        out, want, _ = run.step(5)
        m = compare(to_numpy_f32(out), want)
        assert m["max_abs"] <= 2.0e-3 and m["rel_l2"] <= 2.0e-4, (width, m)


def test_layer_saturation_edges_stay_finite():
    """Extreme gate inputs (cpp/tests/qwen35_cuda_delta_test.cu:568-603): A from -12 to -0.001, dt_bias -25..5,
    b = +-30, z = +-18.  Everything must stay finite and match the oracle."""
    hk, hv, width, tokens = 2, 4, 4, 4
    run = LayerRun(0xB2002400, hk, hv, width, K.DTYPE_F32, K.DTYPE_F32, tokens)
    hidden = hv * DK
    conv_dim = 2 * hk * DK + hidden
    run.rec_a = np.array([-12.0, -1.0, -0.05, -0.001], dtype=np.float32)
    run.dt_bias = np.array([-25.0, -3.0, 0.5, 5.0], dtype=np.float32)
    run.d_rec_a, run.d_dt = act_tensor(run.rec_a, K.DTYPE_F32), act_tensor(run.dt_bias, K.DTYPE_F32)
    run.inp[:, conv_dim:conv_dim + hv] = np.array([30.0, -30.0, 30.0, -30.0], dtype=np.float32)
    run.inp[:, conv_dim + 2 * hv::2] = 18.0
    run.inp[:, conv_dim + 2 * hv + 1::2] = -18.0
    out, want, _ = run.step(tokens)
    assert np.isfinite(to_numpy_f32(out)).all() and np.isfinite(to_numpy_f32(run.d_rs)).all()
    run.check(out, want)


def test_batched_decode_step_64_sequences_at_full_size():
    """The serving configuration's gated-delta half at its full size: one recurrent step on each of 64 sequences'
    FP32 [32][128][128] states in one launch (the kernel that splits the (sequence, head) units evenly over the SMs);
    every sequence's output and new state against the oracle."""
    batch, seed = 64, 0xB2001600
    q, k, v, beta, g = core_operands(seed, batch)  # one token per sequence
    gen = torch.Generator(device=dev()).manual_seed(seed)
    states = [0.05 * torch.randn(HV, DK, DK, device=dev(), generator=gen) for _ in range(batch)]
    states0 = [to_numpy_f32(s) for s in states]
    ptrs = torch.tensor([s.data_ptr() for s in states], device=dev(), dtype=torch.int64)
    out = torch.zeros(batch, HV, DK, device=dev())
    K.batched_gdn_decode(bf16_tensor(q), bf16_tensor(k), bf16_tensor(v), torch.from_numpy(beta).to(dev()),
                         torch.from_numpy(g).to(dev()), ptrs, out, batch, HK, HV, torch.cuda.current_stream())
    torch.cuda.synchronize()
    got = to_numpy_f32(out)
    for i in range(batch):
        want_out, want_state = ob.gdn_core(q[i:i + 1], k[i:i + 1], v[i:i + 1], beta[i:i + 1], np.exp(g[i:i + 1]),
                                           states0[i])
        assert compare(got[i], want_out[0])["rel_l2"] <= 1.0e-4, i
        assert compare(to_numpy_f32(states[i]), want_state)["rel_l2"] <= 1.0e-5, i


@pytest.mark.parametrize("batch", [8, 9, 37, 300])
def test_batched_decode_step_streaming_kernel(batch):
    """The batches the streaming kernel takes (8 sequences and up): unit counts that do not divide by the SM count,
    one or two units a CTA, and more units per CTA (300 x 32 over 148) than state pointers it keeps in shared memory.
    At 300 sequences every seventh one is checked against the oracle."""
    seed = 0xB2001700 + batch
    q, k, v, beta, g = core_operands(seed, batch)
    gen = torch.Generator(device=dev()).manual_seed(seed)
    states = [0.05 * torch.randn(HV, DK, DK, device=dev(), generator=gen) for _ in range(batch)]
    checked = range(batch) if batch <= 64 else range(0, batch, 7)
    states0 = {i: to_numpy_f32(states[i]) for i in checked}
    ptrs = torch.tensor([s.data_ptr() for s in states], device=dev(), dtype=torch.int64)
    out = torch.zeros(batch, HV, DK, device=dev())
    stream = torch.cuda.current_stream()
    K.batched_gdn_decode(bf16_tensor(q), bf16_tensor(k), bf16_tensor(v), torch.from_numpy(beta).to(dev()),
                         torch.from_numpy(g).to(dev()), ptrs, out, batch, HK, HV, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0
    got = to_numpy_f32(out)
    for i in checked:
        want_out, want_state = ob.gdn_core(q[i:i + 1], k[i:i + 1], v[i:i + 1], beta[i:i + 1], np.exp(g[i:i + 1]),
                                           states0[i])
        assert compare(got[i], want_out[0])["rel_l2"] <= 1.0e-4, i
        assert compare(to_numpy_f32(states[i]), want_state)["rel_l2"] <= 1.0e-5, i


def test_batched_decode_step_reports_a_state_pointer_off_its_boundary():
    """The state pointers live in device memory, so the host cannot check them.  The streaming kernel looks at each
    one before it copies from it: a pointer off a 16-byte boundary is not read (the copy would fault); the kernel sets
    RIB200_DEVICE_POINTER_MISALIGNED instead, and the context carries on with the next, well-formed call."""
    batch, seed = 16, 0xB2001800
    q, k, v, beta, g = core_operands(seed, batch)
    gen = torch.Generator(device=dev()).manual_seed(seed)
    pool = 0.05 * torch.randn(batch, HV * DK * DK + 4, device=dev(), generator=gen)
    addresses = [pool[i].data_ptr() for i in range(batch)]
    bad = list(addresses)
    bad[5] += 4
    out = torch.zeros(batch, HV, DK, device=dev())
    stream = torch.cuda.current_stream()
    operands = (bf16_tensor(q), bf16_tensor(k), bf16_tensor(v), torch.from_numpy(beta).to(dev()),
                torch.from_numpy(g).to(dev()))
    assert K.device_status(stream) == 0
    K.batched_gdn_decode(*operands, torch.tensor(bad, device=dev(), dtype=torch.int64), out, batch, HK, HV, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == K.DEVICE_POINTER_MISALIGNED
    assert K.device_status(stream) == 0  # reading cleared it
    fresh = 0.05 * torch.randn(batch, HV * DK * DK + 4, device=dev(), generator=gen)
    before = to_numpy_f32(fresh[3, :HV * DK * DK]).reshape(HV, DK, DK)
    K.batched_gdn_decode(*operands, torch.tensor([fresh[i].data_ptr() for i in range(batch)], device=dev(),
                                                 dtype=torch.int64), out, batch, HK, HV, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0
    want_out, want_state = ob.gdn_core(q[3:4], k[3:4], v[3:4], beta[3:4], np.exp(g[3:4]), before)
    assert compare(to_numpy_f32(out)[3], want_out[0])["rel_l2"] <= 1.0e-4
    assert compare(to_numpy_f32(fresh[3, :HV * DK * DK]).reshape(HV, DK, DK), want_state)["rel_l2"] <= 1.0e-5
