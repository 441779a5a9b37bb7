"""Rank plumbing for multi-GPU replica runs: one process per GPU, rendezvous through torch.distributed (NCCL on GPUs,
gloo on CPU for tests).  The data path has no collective; the only reductions are of timings, outside timed regions."""
from __future__ import annotations

import os


def env_ranks() -> tuple[int, int, int]:
    """(rank, local_rank, world_size) from the launcher's environment (torchrun); a plain run is rank 0 of 1."""
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


class Ranks:
    def __init__(self, backend: str | None = None):
        import torch
        self.torch = torch
        self.rank, self.local_rank, self.world = env_ranks()
        self.backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        self.active = self.world > 1
        if self.active:
            import torch.distributed as dist
            self.dist = dist
            kw = {}
            if self.backend == "nccl":
                kw["device_id"] = torch.device("cuda", self.local_rank)
            dist.init_process_group(self.backend, **kw)

    def _tensor(self, v: float):
        dev = "cuda" if self.backend == "nccl" else "cpu"
        return self.torch.tensor([float(v)], dtype=self.torch.float64, device=dev)

    def barrier(self) -> None:
        if self.active:
            self.dist.barrier()

    def max(self, v: float) -> float:
        if not self.active:
            return float(v)
        t = self._tensor(v)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum(self, v: float) -> float:
        if not self.active:
            return float(v)
        t = self._tensor(v)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def close(self) -> None:
        if self.active:
            self.dist.barrier()
            self.dist.destroy_process_group()
            self.active = False
