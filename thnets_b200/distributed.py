"""Multi-rank plumbing of the benchmark: one process per GPU, nothing exchanged on the data path.

A batch-sharded forward needs no collective (every operator treats images independently, so each rank
runs the whole network on its own images); `torch.distributed` is used only to line the ranks up around
the timed region and to take the slowest rank's time.  Backend "nccl" on GPUs, "gloo" in CPU tests.
"""
from __future__ import annotations

import os


class Ranks:
    def __init__(self, backend: str | None = None):
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.dist = None
        self.device = "cpu"
        if self.world > 1:
            import torch
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
            if backend == "nccl":
                torch.cuda.set_device(self.local_rank)
                self.device = "cuda"
                dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            else:
                dist.init_process_group(backend)
            self.dist = dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def max(self, value: float) -> float:
        """the slowest rank's value (times are reported as the maximum over ranks)"""
        if self.dist is None:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum(self, value: float) -> float:
        if self.dist is None:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def host_signal(self, key: str):
        """Set a key in the rendezvous store: a message to ranks blocked in host_wait.  No GPU work is involved, so a
        rank can wait for another one while its GPU stays idle (a collective would park a kernel on it)."""
        if self.dist is not None:
            self._store().set(key, "1")

    def host_wait(self, key: str, timeout_s: float = 900.0):
        """Block on the host until some rank has set `key`."""
        if self.dist is not None:
            import datetime
            self._store().wait([key], datetime.timedelta(seconds=timeout_s))

    def _store(self):
        from torch.distributed import distributed_c10d
        return distributed_c10d._get_default_store()

    def shard(self, total: int):
        """contiguous slice [offset, offset+count) of `total` units for this rank; remainder to the lowest ranks"""
        base, extra = divmod(total, self.world)
        count = base + (1 if self.rank < extra else 0)
        offset = self.rank * base + min(self.rank, extra)
        return offset, count

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()
            self.dist = None
