"""Host-side sharding logic, run as two gloo ranks on CPU: the sequence assignment used by the sharded serving
decode and the max-over-ranks reduction of step times.  No GPU and no library call is involved."""
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_assign_sequences_balances_bytes():
    sys.path.insert(0, ROOT)
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_assign", os.path.join(ROOT, "raftinfer_b200", "sharding.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    lengths = [32768, 1024, 20000, 20000, 5000, 9000, 31000, 2000]
    for world in (1, 2, 4, 8):
        owner, load = mod.assign_sequences(lengths, world)
        assert sorted(set(owner)) == list(range(min(world, len(lengths))))
        assert sum(load) == sum(lengths)
        assert max(load) - min(load) <= max(lengths)
    owner, load = mod.assign_sequences(lengths, 2)
    assert abs(load[0] - load[1]) <= 2000


def test_two_gloo_ranks_agree_on_assignment_and_reduce_times(tmp_path):
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    sock.close()
    script = textwrap.dedent("""
        import os, sys, importlib.util
        import torch, torch.distributed as dist
        spec = importlib.util.spec_from_file_location("sharding", os.path.join(%r, "raftinfer_b200", "sharding.py"))
        mod = importlib.util.module_from_spec(spec); spec.loader.exec_module(mod)
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        gen = torch.Generator().manual_seed(0xB2000004)
        lengths = torch.randint(1024, 32769, (64,), generator=gen).tolist()
        owner, load = mod.assign_sequences(lengths, world)
        mine = [n for n, r in zip(lengths, owner) if r == rank]
        total = torch.tensor([float(sum(mine))]); dist.all_reduce(total)
        assert int(total.item()) == sum(lengths)
        t = torch.tensor([1.0 + rank], dtype=torch.float64); dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == float(world)
        owners = [None] * world; dist.all_gather_object(owners, owner)
        assert all(o == owners[0] for o in owners)
        dist.barrier(); dist.destroy_process_group()
        print("rank", rank, "ok")
    """ % ROOT)
    path = tmp_path / "rank_script.py"
    path.write_text(script)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), str(path)],
                         env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.count("ok") == 2


def test_head_slices_cover_all_heads():
    sys.path.insert(0, ROOT)
    from raftinfer_b200 import sharding

    for world in (1, 2, 4, 8):
        seen = []
        for rank in range(world):
            (b, e), (kb, ke) = sharding.head_slice(rank, world)
            seen.extend(range(b, e))
            assert e - b == 16 // world and ke - kb == max(1, 4 // world)
            assert all(h // 4 in range(kb, ke) for h in range(b, e))
        assert seen == list(range(16))
