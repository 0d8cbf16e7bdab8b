"""Host-side logic of batch-sharded inference, on CPU ranks (gloo, world size 2)."""
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds(pkg):
    from chainer_compiler_b200.dataparallel import shard_bounds
    for total, world in ((256, 8), (10, 4), (3, 8), (0, 2), (16384, 8)):
        spans = [shard_bounds(total, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %r)
    import torch, torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    from chainer_compiler_b200 import dataparallel as dp
    rank, local_rank, world = dp.init(backend="gloo")
    assert world == 2 and dist.get_backend() == "gloo"
    # even split: every rank contributes its rows, every rank sees the whole batch in rank order
    total, classes = 8, 5
    full = torch.arange(total * classes, dtype=torch.float32).reshape(total, classes)
    b, e = dp.shard_bounds(total, world, rank)
    got = dp.gather_logits(full[b:e].clone(), world)
    assert torch.equal(got, full)
    # ragged split (7 rows over 2 ranks)
    full = torch.arange(7 * classes, dtype=torch.float32).reshape(7, classes)
    b, e = dp.shard_bounds(7, world, rank)
    assert torch.equal(dp.gather_ragged(full[b:e].clone(), 7, world, rank), full)
    # MatMulInteger with the rows of A sharded (B replicated, int32 rows gathered): ragged 7 rows over 2 ranks
    g = torch.Generator().manual_seed(0)
    A = torch.randint(0, 256, (7, 12), generator=g, dtype=torch.int32)
    B = torch.randint(-127, 128, (12, 5), generator=g, dtype=torch.int32)
    za = torch.tensor([128], dtype=torch.int32)
    cpu_mm = lambda a, b, za_, zb_: ((a - za_) @ b).to(torch.int32)   # stand-in for the GPU op: the host logic is what runs here
    b7, e7 = dp.shard_bounds(7, world, rank)
    Y = dp.sharded_matmul_integer(A[b7:e7], B, za, None, total_rows=7, world=world, rank=rank, gather=True, matmul=cpu_mm)
    assert torch.equal(Y, ((A - 128) @ B).to(torch.int32))
    Yl = dp.sharded_matmul_integer(A[b7:e7], B, za, None, total_rows=7, world=world, rank=rank, gather=False, matmul=cpu_mm)
    assert torch.equal(Yl, Y[b7:e7])
    try:
        dp.sharded_matmul_integer(A, B, za, None, total_rows=7, world=world, rank=rank, matmul=cpu_mm)
        raise SystemExit("a shard of the wrong size was accepted")
    except ValueError:
        pass
    # timing rule: the slowest rank's time is what every rank reports
    assert dp.max_over_ranks(1.0 + rank, torch.device("cpu"), world) == 2.0
    dist.barrier()
    dist.destroy_process_group()
    print("rank %%d ok" %% rank)
""") % ROOT


def test_gather_two_cpu_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   CUDA_VISIBLE_DEVICES="")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for rank, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o
        assert "rank %d ok" % rank in o
