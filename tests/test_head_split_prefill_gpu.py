"""Head-sharded prefill: the epilogue stores its tiles into full-width output buffers (its own and its peers')
and a device-side rendezvous replaces the all-gather.  No counterpart in the reference; the check is that the
heads a rank computes land, bit for bit, where the plain prefill of those heads would put them.

One GPU: a rank's slice (8 of 16 query heads, 2 of 4 KV heads) is scattered into shared buffers it also maps
itself, with a rendezvous of world 1.  Two or more GPUs: child processes under torchrun compare, on every rank, the
assembled result with the CPU oracle and with NCCL all-gather + permute (tests/head_split_worker.py)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from raftinfer_b200 import kernels as K
from raftinfer_b200 import synth
from raftinfer_b200.peer import SharedBuffer

from gpu_util import D, HKV, HQ, act_tensor, cache_to_device, dev, make_cache

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype,torch_dtype", [(K.DTYPE_BF16, torch.bfloat16), (K.DTYPE_F32, torch.float32)])
@pytest.mark.parametrize("tokens,past", [(300, 0), (129, 77)])
def test_slice_lands_in_the_full_width_buffer(tokens, past, dtype, torch_dtype):
    stream = torch.cuda.current_stream()
    hq, hkv, offset = HQ // 2, HKV // 2, HQ // 2  # the second of two ranks
    max_ctx = past + tokens
    q = synth.round_bf16(synth.normal(91, 0, (tokens, hq, D)))
    gate = synth.round_bf16(synth.normal(91, 1, (tokens, hq, D)))
    k = synth.round_bf16(synth.normal(91, 2, (past + tokens, hkv, D)))
    v = synth.round_bf16(synth.normal(91, 3, (past + tokens, hkv, D)))

    def fresh_cache():
        bits = np.full((2, hkv, max_ctx, D), 0x7FC1, dtype=np.uint16)
        bits[0, :, :past] = synth.bf16_bits(k[:past]).transpose(1, 0, 2)
        bits[1, :, :past] = synth.bf16_bits(v[:past]).transpose(1, 0, 2)
        return cache_to_device(bits)

    shape = K.Qwen35AttentionShape(tokens, hq, hkv, D, max_ctx, past)
    operands = (act_tensor(q, dtype), act_tensor(k[past:], dtype), act_tensor(v[past:], dtype), act_tensor(gate, dtype))
    plain = torch.zeros(tokens, hq, D, device=dev(), dtype=torch_dtype)
    cache = fresh_cache()
    K.qwen35_online_attention_prefill(*operands, plain, cache, cache.numel() * 2, shape, dtype, K.KV_BF16, K.HEAD_MAJOR,
                                      stream)

    first = SharedBuffer((tokens, HQ, D), torch_dtype, 0, 1, None, dev())
    second = SharedBuffer((tokens, HQ, D), torch_dtype, 0, 1, None, dev())  # stands in for a peer's buffer
    flags = SharedBuffer((1,), torch.int32, 0, 1, None, dev())
    cache2 = fresh_cache()
    K.online_attention_prefill_scatter(*operands, [first.pointers[0], second.pointers[0]], 0, HQ, offset, cache2,
                                       cache2.numel() * 2, shape, dtype, K.KV_BF16, K.HEAD_MAJOR, stream)
    K.peer_rendezvous(flags.pointers, 0, 7, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0
    assert int(flags.local[0].item()) == 7
    for buffer in (first, second):
        assert torch.equal(buffer.local[:, offset:offset + hq], plain), "this rank's heads"
        assert torch.count_nonzero(buffer.local[:, :offset].float()) == 0, "other ranks' heads are not touched"
    assert torch.equal(cache2, cache), "the cache append does not depend on where the tiles go"
    for buffer in (first, second, flags):
        buffer.close()


def test_scatter_rejects_bad_arguments():
    stream = torch.cuda.current_stream()
    shape = K.Qwen35AttentionShape(4, 8, 2, D, 4, 0)
    t = torch.zeros(4, 8, D, device=dev(), dtype=torch.bfloat16)
    kv = torch.zeros(4, 2, D, device=dev(), dtype=torch.bfloat16)
    out = torch.zeros(4, HQ, D, device=dev(), dtype=torch.bfloat16)
    cache = torch.zeros(2, 2, 4, D, device=dev(), dtype=torch.bfloat16)
    with pytest.raises(K.Qwen35PrimitiveError):  # 8 heads at offset 12 do not fit in 16
        K.online_attention_prefill_scatter(t, kv, kv, t, [out], 0, HQ, 12, cache, cache.numel() * 2, shape, K.DTYPE_BF16,
                                           K.KV_BF16, K.HEAD_MAJOR, stream)
    with pytest.raises(K.Qwen35PrimitiveError):  # more than eight destinations
        K.online_attention_prefill_scatter(t, kv, kv, t, [out] * 9, 0, HQ, 0, cache, cache.numel() * 2, shape, K.DTYPE_BF16,
                                           K.KV_BF16, K.HEAD_MAJOR, stream)


def test_rendezvous_wait_runs_out_and_the_context_stays_usable():
    """A rank that never arrives: world 2 on one GPU with two flag arrays this process owns, rank 0 calls, nothing ever
    writes rank 1's slot.  The wait is bounded (two million cycles, about a millisecond), so the kernel gives up,
    records RIB200_DEVICE_WAIT_TIMED_OUT and returns; the status word reads back, clears, and the next calls on the
    same stream work as usual.  This is what stands where the reference traps
    (cpp/kernels/qwen35_online_attention.cu:714-717): a status the host reads, not a lost context."""
    stream = torch.cuda.current_stream()
    mine = torch.zeros(2, device=dev(), dtype=torch.int32)
    theirs = torch.zeros(2, device=dev(), dtype=torch.int32)
    assert K.device_status(stream) == 0
    K.peer_rendezvous_bounded([mine, theirs], 0, 1, 2_000_000, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == K.DEVICE_WAIT_TIMED_OUT
    assert mine.tolist() == [1, 0] and theirs.tolist() == [1, 0]  # rank 0 published its epoch in both arrays
    assert K.device_status(stream) == 0  # reading cleared it
    # the peer arrives after all (its slot is written by hand): the same epoch now completes within the bound
    mine[1] = 1
    K.peer_rendezvous_bounded([mine, theirs], 0, 1, 2_000_000, stream)
    K.peer_rendezvous([mine], 0, 5, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0 and int(mine[0].item()) == 5
    with pytest.raises(K.Qwen35PrimitiveError):
        K.peer_rendezvous_bounded([mine, theirs], 0, 2, 0, stream)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_against_the_oracle_and_the_all_gather_form():
    """Two child processes, one per GPU: each checks the full-width result it holds after the rendezvous (its own
    heads and the ones the other rank stored over NVLink) against the CPU oracle, and bit for bit against the plain
    prefill of its heads followed by an NCCL all-gather (tests/head_split_worker.py)."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(ROOT, "tests", "head_split_worker.py")]
    done = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    for rank in (0, 1):
        assert f"oracle_and_all_gather_parity rank {rank} of 2" in done.stdout
