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

__all__ = ["RankInfo", "rank_info", "shard_range", "shard_indices", "ShardWorker", "gather_stats",
           "parse_cpulist", "gpu_numa_node", "node_cpus", "bind_to_gpu_node"]


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


# ---- host locality: keep a rank's threads and pinned buffers on its GPU's NUMA node ---------------
# Each rank uploads its own frames over its own PCIe link.  On a two-socket host a pinned buffer
# that sits on the other socket makes every upload cross the socket interconnect, which then
# bounds the aggregate upload rate of all ranks.  Binding the rank's process to the CPUs of the
# GPU's node before it allocates pinned memory (pages are placed on the node of the allocating
# thread) keeps uploads local.


def parse_cpulist(text: str) -> list[int]:
    """``"0-3,8,10-11"`` (the kernel's cpulist format) -> ``[0, 1, 2, 3, 8, 10, 11]``."""
    cpus: list[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.extend(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_numa_node(pci_bus_id: str, sysfs: str = "/sys") -> int | None:
    """NUMA node of the PCI device ``"0000:1b:00.0"`` (None when the host does not say)."""
    try:
        with open(os.path.join(sysfs, "bus/pci/devices", pci_bus_id.lower(), "numa_node")) as f:
            node = int(f.read().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def node_cpus(node: int, sysfs: str = "/sys") -> list[int]:
    try:
        with open(os.path.join(sysfs, "devices/system/node", f"node{node}", "cpulist")) as f:
            return parse_cpulist(f.read())
    except (OSError, ValueError):
        return []


def _pci_bus_id(device_index: int) -> str | None:
    import torch

    p = torch.cuda.get_device_properties(device_index)
    try:
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except AttributeError:
        return None


def bind_to_gpu_node(device_index: int, sysfs: str = "/sys", pci_bus_id: str | None = None) -> dict:
    """Restrict this process to the CPUs of the NUMA node of GPU ``device_index`` (those of them
    it is allowed to run on).  Returns ``{"node", "cpus", "bound", "previous"}``; ``previous`` is
    the affinity to hand to ``os.sched_setaffinity`` to undo the binding.  Does nothing when the
    node is unknown or none of its CPUs is available."""
    allowed = sorted(os.sched_getaffinity(0))
    out = {"node": None, "cpus": len(allowed), "bound": False, "previous": allowed}
    bus = pci_bus_id or _pci_bus_id(device_index)
    node = gpu_numa_node(bus, sysfs) if bus else None
    if node is None:
        return out
    out["node"] = node
    local = sorted(set(node_cpus(node, sysfs)) & set(allowed))
    if not local or local == allowed:
        return out
    os.sched_setaffinity(0, local)
    out.update(cpus=len(local), bound=True)
    return out


class ShardWorker:
    """The device, private stream and ``CUDAConfig`` of one rank."""

    def __init__(self, info: RankInfo | None = None, bind_host: bool = False) -> None:
        """``bind_host``: also restrict the process to the CPUs next to the rank's GPU (see
        ``bind_to_gpu_node``); the result is kept in ``self.host_binding``."""
        import torch

        from . import _lib
        from .io import cuda_config

        self.info = info or rank_info()
        if self.info.local_rank >= torch.cuda.device_count():
            raise RuntimeError(f"Local rank {self.info.local_rank} was asked for, but this process "
                               f"sees only {torch.cuda.device_count()} CUDA device(s).")
        self.device = torch.device(f"cuda:{self.info.local_rank}")
        torch.cuda.set_device(self.device)
        _lib.check(_lib.lib().b2_init(self.info.local_rank))
        self.stream = torch.cuda.Stream(self.device)
        self.config = cuda_config(self.info.local_rank, stream=self.stream.cuda_stream)
        self.host_binding = bind_to_gpu_node(self.info.local_rank) if bind_host else None

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
