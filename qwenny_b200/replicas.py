"""Multi-GPU for this path is replicas only: every GPU runs a full model on its own request slots and no data crosses
between them. What ranks share is the measurement: a barrier around the timed region and the slowest rank's time."""
from __future__ import annotations

import torch
import torch.distributed as dist


def slowest_ms(ms_local: float, device: torch.device | str = "cpu") -> float:
    """The timed region's duration as the job sees it: the maximum over ranks (1 rank: itself)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(ms_local)
    t = torch.tensor([ms_local], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def job_throughput(units_per_rank_step: int, ms_per_step: float, world: int) -> float:
    """Units per second of the whole job: every rank does the same fixed work per step (weak scaling)."""
    return world * units_per_rank_step / ms_per_step * 1e3


def rank_slots(total_slots: int, rank: int, world: int) -> range:
    """The request slots rank `rank` serves when `total_slots` independent sequences are dealt to `world` replicas."""
    per, extra = divmod(total_slots, world)
    lo = rank * per + min(rank, extra)
    return range(lo, lo + per + (1 if rank < extra else 0))
