"""Rank logic of the per-GPU sharding layer, on CPU: index assignment and the optional statistics
gather over a real 2-process gloo group."""

import os
import socket
import sys
from pathlib import Path

import pytest

from spdl_b200.sharding import (RankInfo, gather_stats, rank_info, shard_indices, shard_range)

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("total,world", [(64, 8), (2048, 8), (10, 3), (5, 8), (0, 4), (7, 1)])
def test_blocks_partition_everything_once(total, world):
    seen = []
    for r in range(world):
        a, b = shard_range(total, r, world)
        assert 0 <= a <= b <= total
        seen += list(range(a, b))
    assert seen == list(range(total))
    sizes = [len(shard_indices(total, r, world)) for r in range(world)]
    assert max(sizes) - min(sizes) <= 1


def test_workload_splits():
    # 64 clips over 8 GPUs -> 8 each; 2048 images -> 256 each (contiguous blocks)
    assert shard_range(64, 3, 8) == (24, 32)
    assert shard_range(2048, 7, 8) == (1792, 2048)


def test_strided_matches_reference_sampler_rule():
    # src/spdl/source/_sampler.py: range(rank, N, world_size)
    for r in range(3):
        assert list(shard_indices(10, r, 3, "strided")) == list(range(r, 10, 3))
    with pytest.raises(RuntimeError):
        shard_indices(10, 0, 3, "diagonal")
    with pytest.raises(RuntimeError):
        shard_range(10, 3, 3)


def test_rank_info_from_env():
    assert rank_info({}) == RankInfo(0, 0, 1)
    assert rank_info({"RANK": "5", "LOCAL_RANK": "1", "WORLD_SIZE": "8"}) == RankInfo(5, 1, 8)
    with pytest.raises(RuntimeError):
        rank_info({"RANK": "8", "WORLD_SIZE": "8"})


def test_gather_without_group_is_identity():
    assert gather_stats([1.0, 2.5]) == [[1.0, 2.5]]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, q) -> None:
    sys.path.insert(0, str(ROOT))
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist

    from spdl_b200.sharding import gather_stats, rank_info, shard_indices

    info = rank_info()
    dist.init_process_group("gloo", rank=info.rank, world_size=info.world_size)
    mine = shard_indices(2048, info.rank, info.world_size)
    # each rank "processes" its block and reports (items, first index, seconds)
    stats = gather_stats([len(mine), mine[0], 0.5 + info.rank])
    dist.barrier()
    dist.destroy_process_group()
    q.put((rank, stats))


def test_two_rank_gloo_gather():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    results = dict(q.get(timeout=120) for _ in range(2))
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    want = [[1024.0, 0.0, 0.5], [1024.0, 1024.0, 1.5]]
    assert results[0] == want and results[1] == want
    # whole-job throughput = all items / slowest rank
    total = sum(r[0] for r in want)
    assert total / max(r[2] for r in want) == 2048 / 1.5


def _rank_that_may_leave(rank: int, world: int, port: int, q) -> None:
    """Rank 1 leaves between steps without joining the gather; rank 0 must learn of it through
    the collective's error (or the group's short timeout) and keep its own statistics."""
    import datetime

    sys.path.insert(0, str(ROOT))
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist

    from spdl_b200.sharding import gather_stats

    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=10))
    dist.barrier()  # both ranks are up; the data path itself needs no communication
    if rank == 1:
        q.put((rank, "left"))
        q.close()
        q.join_thread()  # the message is on the pipe before the process goes away
        os._exit(0)
    import time

    time.sleep(1.0)
    try:
        gather_stats([1.0], on_failure="raise")
        strict = "no error"
    except Exception as e:
        strict = type(e).__name__
    q.put((rank, strict, gather_stats([7.0, 8.0], on_failure="local")))
    q.close()
    q.join_thread()
    os._exit(0)


def test_gather_survives_a_rank_that_left():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_that_may_leave, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    got = {}
    for _ in range(2):
        item = q.get(timeout=120)
        got[item[0]] = item[1:]
    [p.join(timeout=60) for p in procs]
    assert got[1] == ("left",)
    strict, local = got[0]
    assert strict != "no error"        # the strict mode surfaces the failure
    assert local == [[7.0, 8.0]]       # the tolerant mode keeps this rank's own numbers


def test_numa_helpers_against_a_fake_sysfs(tmp_path):
    import os

    from spdl_b200.sharding import bind_to_gpu_node, gpu_numa_node, node_cpus, parse_cpulist

    assert parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert parse_cpulist("") == []
    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    unknown = tmp_path / "bus/pci/devices/0000:3c:00.0"
    unknown.mkdir(parents=True)
    (unknown / "numa_node").write_text("-1\n")
    allowed = sorted(os.sched_getaffinity(0))
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    # the node owns the first allowed CPU and one that does not exist here
    (node / "cpulist").write_text(f"{allowed[0]},100000\n")
    assert gpu_numa_node("0000:1B:00.0", str(tmp_path)) == 1
    assert gpu_numa_node("0000:3c:00.0", str(tmp_path)) is None
    assert gpu_numa_node("0000:ff:00.0", str(tmp_path)) is None
    assert node_cpus(1, str(tmp_path)) == [allowed[0], 100000]
    # unknown node: nothing changes
    r = bind_to_gpu_node(0, str(tmp_path), pci_bus_id="0000:3c:00.0")
    assert r["bound"] is False and sorted(os.sched_getaffinity(0)) == allowed
    r = bind_to_gpu_node(0, str(tmp_path), pci_bus_id="0000:1b:00.0")
    try:
        assert r["node"] == 1 and r["previous"] == allowed
        if len(allowed) > 1:
            assert r["bound"] is True and sorted(os.sched_getaffinity(0)) == [allowed[0]]
        else:
            assert r["bound"] is False
    finally:
        os.sched_setaffinity(0, allowed)
