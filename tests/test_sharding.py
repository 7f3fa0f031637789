"""Cloud sharding and the output gather, on CPU ranks (gloo, world size 2)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from minuet_b200 import sharding


def test_assign_clouds_balances_and_is_deterministic():
    sizes = [120, 80, 200, 50, 50, 199, 1, 130]
    shards = sharding.assign_clouds(sizes, 3)
    assert sorted(c for s in shards for c in s) == list(range(8))
    loads = [sum(sizes[c] for c in s) for s in shards]
    assert max(loads) - min(loads) <= max(sizes)
    assert shards == sharding.assign_clouds(sizes, 3)
    assert sharding.assign_clouds([5, 5, 5, 5], 4) == [[0], [1], [2], [3]]
    assert sharding.assign_clouds([7], 2) == [[0], []]


def test_take_clouds():
    coords = np.arange(30).reshape(10, 3).astype(np.int32)
    bd = np.array([0, 3, 3, 7, 10])
    feats = np.arange(10, dtype=np.float32)[:, None]
    c, b, f = sharding.take_clouds(coords, bd, feats, [0, 3])
    assert b.tolist() == [0, 3, 6] and c[:, 0].tolist() == [0, 3, 6, 21, 24, 27]
    assert f[:, 0].tolist() == [0, 1, 2, 7, 8, 9]
    c, b, f = sharding.take_clouds(coords, bd, None, [1])
    assert len(c) == 0 and b.tolist() == [0, 0] and f is None


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, sizes, result_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shards = sharding.assign_clouds(sizes, world)
        # row value = global row index of the original batch, so order is checkable
        starts = np.concatenate([[0], np.cumsum(sizes)])
        mine = [torch.arange(starts[c], starts[c + 1], dtype=torch.float32) for c in shards[rank]]
        local = (torch.cat(mine) if mine else torch.zeros(0))[:, None].repeat(1, 3)
        gathered = sharding.gather_rows(local, dst=0)
        # row counts known from the shard plan: same result, no count exchange
        planned = [sum(sizes[c] for c in shard) for shard in shards]
        again = sharding.gather_rows(local, dst=0, counts=planned)
        if rank == 0:
            assert all(torch.equal(a, b) for a, b in zip(gathered, again))
            full = sharding.reassemble(gathered, shards, sizes)
            torch.save(full, result_path)
        else:
            assert gathered is None
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("sizes", [[5, 9, 2, 7, 7], [4], [3, 0, 6]])
def test_gather_rows_world2(tmp_path, sizes):
    path = str(tmp_path / "out.pt")
    mp.spawn(_worker, args=(2, _free_port(), sizes, path), nprocs=2, join=True)
    full = torch.load(path)
    total = sum(sizes)
    assert full.shape == (total, 3)
    assert torch.equal(full[:, 0], torch.arange(total, dtype=torch.float32))


def _dropout_worker(rank, world, port, result_path):
    """Rank 1 leaves between steps (no collective in flight); rank 0's next gather
    must end with an error after the short process-group timeout instead of hanging."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    local = torch.full((3 + rank, 2), float(rank))
    sharding.gather_rows(local, dst=0)          # step 1: both ranks present
    if rank == 1:
        os._exit(0)                              # the rank disappears between steps
    try:
        sharding.gather_rows(local, dst=0)      # step 2: the peer is gone
        outcome = "no error"
    except Exception as exc:                     # gloo reports a timeout / connection error
        outcome = "error: " + type(exc).__name__
    with open(result_path, "w") as f:
        f.write(outcome)
    os._exit(0)


def test_lost_rank_is_reported_not_waited_for_forever(tmp_path):
    path = str(tmp_path / "outcome.txt")
    ctx = mp.spawn(_dropout_worker, args=(2, _free_port(), path), nprocs=2, join=False)
    deadline = 60
    import time
    t0 = time.time()
    while not os.path.exists(path) and time.time() - t0 < deadline:
        time.sleep(0.2)
    for p in ctx.processes:
        p.join(timeout=5)
        if p.is_alive():
            p.kill()
    assert os.path.exists(path), "rank 0 was still waiting after 60 s"
    assert open(path).read().startswith("error")
