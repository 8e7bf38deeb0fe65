"""Host-side partitioning of the path across the GPUs of one box (one process per GPU).

Batched decode shards by sequence: sequences are independent, every rank owns the KV caches and gated-delta states
of its sequences for their lifetime, and there is no collective on the data path.  Prefill shards by KV-head
group and needs one all-gather of the outputs (see raftinfer_b200.benchmarks.head_split_prefill).
"""
from __future__ import annotations


def assign_sequences(lengths, world):
    """Greedy longest-first assignment of sequences to ranks, balancing context tokens (KV bytes), not counts.
    Returns (owner rank per sequence, tokens per rank)."""
    order = sorted(range(len(lengths)), key=lambda i: (-lengths[i], i))
    load = [0] * world
    owner = [0] * len(lengths)
    for i in order:
        r = min(range(world), key=lambda x: (load[x], x))
        owner[i] = r
        load[r] += lengths[i]
    return owner, load


def head_slice(rank, world, query_heads=16, kv_heads=4):
    """Query heads [begin, end) and the KV heads they read for `rank` of `world` under the head-group split.
    With more ranks than KV heads a KV head is replicated on the ranks that share it."""
    per_rank = query_heads // world
    group = query_heads // kv_heads
    begin = rank * per_rank
    end = begin + per_rank
    kv_begin = begin // group
    kv_end = (end - 1) // group + 1
    return (begin, end), (kv_begin, kv_end)
