"""Child process of tests/test_head_split_prefill_gpu.py (one per GPU, started by torchrun).

Every rank builds the same seeded prompt (16 query heads, 4 KV heads), takes its slice of the heads, and runs the
head-sharded prefill: tiles stored into every rank's full-width buffer, then the device-side rendezvous.  Checked on
every rank: (a) the full-width result against the CPU oracle over all 16 heads, on the first and the last rows of the
prompt (the rows that other ranks wrote arrive over NVLink, so a misplaced or missing tile shows here); (b) the same
result, bit for bit, against the plain prefill of the rank's heads followed by an NCCL all-gather and a permute."""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import numpy as np
import torch
import torch.distributed as dist

from oracle import bindings as ob
from raftinfer_b200 import kernels as K
from raftinfer_b200 import synth
from raftinfer_b200.peer import SharedBuffer

HQ, HKV, D = 16, 4, 256
TOKENS = 384
SEED = 0xB2007000


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    torch.cuda.set_stream(torch.cuda.Stream(device=dev))
    stream = torch.cuda.current_stream()

    def bf16(values):
        bits = synth.bf16_bits(np.ascontiguousarray(values, dtype=np.float32))
        return torch.from_numpy(bits.view(np.int16)).to(dev).view(torch.bfloat16)

    q = synth.round_bf16(synth.normal(SEED, 0, (TOKENS, HQ, D)))
    gate = synth.round_bf16(synth.normal(SEED, 1, (TOKENS, HQ, D)))
    k = synth.round_bf16(synth.normal(SEED, 2, (TOKENS, HKV, D)))
    v = synth.round_bf16(synth.normal(SEED, 3, (TOKENS, HKV, D)))

    hq = HQ // world
    hkv = max(1, HKV // world)
    head0 = rank * hq
    kv0 = head0 // (HQ // HKV)  # the KV heads this rank's query heads read (two ranks may hold the same one)
    mine = (bf16(q[:, head0:head0 + hq]), bf16(k[:, kv0:kv0 + hkv]), bf16(v[:, kv0:kv0 + hkv]),
            bf16(gate[:, head0:head0 + hq]))
    shape = K.Qwen35AttentionShape(TOKENS, hq, hkv, D, TOKENS, 0)

    shared_out = SharedBuffer((TOKENS, HQ, D), torch.bfloat16, rank, world, dist, dev)
    shared_flags = SharedBuffer((world,), torch.int32, rank, world, dist, dev)
    cache = torch.zeros(2, hkv, TOKENS, D, device=dev, dtype=torch.bfloat16)
    K.online_attention_prefill_scatter(*mine, shared_out.pointers, rank, HQ, head0, cache, cache.numel() * 2, shape,
                                       K.DTYPE_BF16, K.KV_BF16, K.HEAD_MAJOR, stream)
    K.peer_rendezvous(shared_flags.pointers, rank, 1, stream)
    torch.cuda.synchronize()
    assert K.device_status(stream) == 0
    got = shared_out.local.float().cpu().numpy()

    # (a) every head, as this rank sees it after the rendezvous, against the oracle
    for lo, hi in ((0, 48), (TOKENS - 48, TOKENS)):
        want = ob.attention_core(q[lo:hi], k[:hi], v[:hi], gate[lo:hi], past=lo)
        metrics = ob.compare(np.asarray(got[lo:hi], dtype=np.float32), np.asarray(want, dtype=np.float32))
        assert metrics["nonfinite"] == 0 and metrics["max_abs"] <= 3.0e-2 and metrics["rel_l2"] <= 1.0e-2, metrics

    # (b) plain prefill of this rank's heads, all-gather, permute: the same bits
    local_out = torch.zeros(TOKENS, hq, D, device=dev, dtype=torch.bfloat16)
    cache2 = torch.zeros_like(cache)
    K.qwen35_online_attention_prefill(*mine, local_out, cache2, cache2.numel() * 2, shape, K.DTYPE_BF16, K.KV_BF16,
                                      K.HEAD_MAJOR, stream)
    torch.cuda.synchronize()
    gathered = torch.zeros(world, TOKENS, hq, D, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(gathered, local_out)
    full = gathered.permute(1, 0, 2, 3).reshape(TOKENS, HQ, D)
    same = bool(torch.equal(shared_out.local, full)) and bool(torch.equal(cache, cache2))
    assert same, "fused head-split prefill differs from all-gather + permute"
    assert K.device_status(stream) == 0

    dist.barrier()  # nobody unmaps a buffer a peer may still be storing into
    shared_flags.close()
    shared_out.close()
    print(f"oracle_and_all_gather_parity rank {rank} of {world}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
