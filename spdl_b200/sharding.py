"""Per-GPU sharding of a sample stream: one worker per GPU, no collective on the data path.

Frames, clips and images are independent, so each rank converts its own slice of the stream on
its own device and stream.  Rank selection follows the reference (``LOCAL_RANK`` picks the
device, ``src/spdl/io/_transfer.py:116-121``); index assignment offers the reference sampler's
strided rule ``range(rank, N, world_size)`` (``src/spdl/source/_sampler.py:63-126``) and the
contiguous blocks used when a batch is already packed in memory.  The only communication is an
optional gather of per-rank statistics at the end of a run.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Sequence

__all__ = ["RankInfo", "rank_info", "shard_range", "shard_indices", "ShardWorker", "gather_stats"]


@dataclass(frozen=True)
class RankInfo:
    rank: int
    local_rank: int
    world_size: int


def rank_info(env: dict[str, str] | None = None) -> RankInfo:
    """Rank, local rank and world size from the launcher's environment (defaults 0, 0, 1)."""
    e = os.environ if env is None else env
    rank = int(e.get("RANK", "0"))
    world = int(e.get("WORLD_SIZE", "1"))
    local = int(e.get("LOCAL_RANK", str(rank)))
    if world < 1 or not 0 <= rank < world:
        raise RuntimeError(f"Inconsistent rank/world size: RANK={rank}, WORLD_SIZE={world}")
    return RankInfo(rank, local, world)


def shard_range(total: int, rank: int, world_size: int) -> tuple[int, int]:
    """Contiguous block ``[start, stop)`` of ``total`` items for ``rank``; the first
    ``total % world_size`` ranks get one extra item, every item is assigned exactly once."""
    if total < 0 or world_size < 1 or not 0 <= rank < world_size:
        raise RuntimeError(f"Invalid shard request: total={total}, rank={rank}, world={world_size}")
    base, extra = divmod(total, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_indices(total: int, rank: int, world_size: int, mode: str = "block") -> range:
    """Indices of ``rank``: ``"block"`` = contiguous, ``"strided"`` = ``range(rank, total,
    world_size)`` as the reference's distributed samplers assign them."""
    if mode == "block":
        return range(*shard_range(total, rank, world_size))
    if mode == "strided":
        if total < 0 or world_size < 1 or not 0 <= rank < world_size:
            raise RuntimeError(
                f"Invalid shard request: total={total}, rank={rank}, world={world_size}")
        return range(rank, total, world_size)
    raise RuntimeError(f"Unknown shard mode: {mode}")


class ShardWorker:
    """The device, private stream and ``CUDAConfig`` of one rank."""

    def __init__(self, info: RankInfo | None = None) -> None:
        import torch

        from . import _lib
        from .io import cuda_config

        self.info = info or rank_info()
        if self.info.local_rank >= torch.cuda.device_count():
            raise RuntimeError("The local rank is larger than the number of available GPUs.")
        self.device = torch.device(f"cuda:{self.info.local_rank}")
        torch.cuda.set_device(self.device)
        _lib.check(_lib.lib().b2_init(self.info.local_rank))
        self.stream = torch.cuda.Stream(self.device)
        self.config = cuda_config(self.info.local_rank, stream=self.stream.cuda_stream)

    def my_slice(self, total: int, mode: str = "block") -> range:
        return shard_indices(total, self.info.rank, self.info.world_size, mode)


def gather_stats(stats: Sequence[float], device: Any = None,
                 on_failure: str = "raise") -> list[list[float]]:
    """All ranks' statistics vectors, in rank order.  Uses the initialised ``torch.distributed``
    group (NCCL on GPUs, gloo on CPU); without one it returns ``[stats]``.

    The gather is bookkeeping, not part of the data path: with ``on_failure="local"`` a rank
    whose peers have gone away (the collective raises or runs into the group's timeout) keeps
    its own numbers and returns ``[stats]`` instead of failing the run.
    """
    import torch
    import torch.distributed as dist

    if on_failure not in ("raise", "local"):
        raise RuntimeError(f"Unknown on_failure mode: {on_failure}")
    vec = [float(x) for x in stats]
    if not (dist.is_available() and dist.is_initialized()):
        return [vec]
    on_gpu = dist.get_backend() == "nccl"
    dev = device if device is not None else (torch.device("cuda", torch.cuda.current_device())
                                              if on_gpu else torch.device("cpu"))
    mine = torch.tensor(vec, dtype=torch.float64, device=dev)
    out = [torch.zeros_like(mine) for _ in range(dist.get_world_size())]
    try:
        dist.all_gather(out, mine)
        result = [t.cpu().tolist() for t in out]
    except Exception:
        if on_failure == "raise":
            raise
        return [vec]
    return result
