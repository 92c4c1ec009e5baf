"""Data-parallel plumbing: which observation a rank runs, and the max-over-ranks reduction of timings.

The chunk has no cross-observation dependency, so N GPUs run N independent observations with replicated
weights and no collective in the data path; torch.distributed is only used to line the ranks up and to report
the slowest one.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def observation_seed(base_seed: int, rank: int, index: int = 0) -> int:
    """Seed of observation `index` of GPU `rank` (every GPU and every slot gets its own prefix K/V and noise)."""
    return base_seed + 1000 * rank + index


def max_over_ranks(values: list[float], device: torch.device | str = "cpu") -> list[float]:
    """Element-wise maximum over all ranks (identity without an initialised process group)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(values)
    t = torch.tensor(values, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


def chunks_per_second(world_size: int, ms_per_chunk_slowest: float, per_gpu_batch: int = 1) -> float:
    """Whole-job throughput when every rank finishes `per_gpu_batch` chunks per step."""
    return world_size * per_gpu_batch * 1e3 / ms_per_chunk_slowest
