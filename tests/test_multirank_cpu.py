"""N > 1 host logic on the CPU: two gloo ranks shard a workload over
(batch x heads) units with no data-path collective, time with a max over
ranks, and gather results only for verification — the same scheme bench.py
uses over NCCL.  The per-unit "kernel" here is the CPU oracle, so the test
needs no GPU."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def shard_units(n_units: int, world: int, rank: int) -> range:
    """Contiguous, balanced split of independent (batch, head) units."""
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    from oracle import oracle as O
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)          # identical full tensors on every rank, then slice
        B, N, H, D = 3, 17, 5, 16
        q = torch.randn(B, N, H, D, generator=g)
        units = shard_units(B * H, world, rank)
        flat = q.permute(0, 2, 1, 3).reshape(B * H, N, D)       # unit-major view
        mine = O.headln_fwd(flat[units.start:units.stop], 1e-5)
        # "timing": every rank reports its own elapsed, the job's time is the max
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == float(world)
        # verification gather (ragged: pad to the largest shard)
        sizes = [len(shard_units(B * H, world, r)) for r in range(world)]
        pad = torch.zeros(max(sizes), N, D)
        pad[: mine.shape[0]] = mine
        bucket = [torch.zeros_like(pad) for _ in range(world)]
        dist.all_gather(bucket, pad)
        if rank == 0:
            full = torch.cat([b[:n] for b, n in zip(bucket, sizes)])
            want = O.headln_fwd(flat, 1e-5)
            assert torch.equal(full, want)
            # dweight-style partial sums: per-rank partials add up to the global reduction
        part = flat[units.start:units.stop].sum(dim=(0, 1))
        dist.all_reduce(part)
        torch.testing.assert_close(part, flat.sum(dim=(0, 1)), rtol=1e-5, atol=1e-5)
        dist.barrier()
        (Path(out_dir) / f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_shard_units_cover_everything_once():
    for n in (1, 7, 64, 65):
        for w in (1, 2, 3, 8):
            seen = [u for r in range(w) for u in shard_units(n, w, r)]
            assert seen == list(range(n))
            sizes = [len(shard_units(n, w, r)) for r in range(w)]
            assert max(sizes) - min(sizes) <= 1


def test_two_gloo_ranks_shard_gather_and_time(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_rank_that_never_joins_times_out(tmp_path):
    """Failure detection on the host: a peer that never joins makes the
    rendezvous fail with an error within the process-group timeout instead of
    hanging."""
    import datetime
    port = _free_port()
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    with pytest.raises(Exception):
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
    if dist.is_initialized():
        dist.destroy_process_group()
