"""Request sharding across the GPUs of one box: whole requests, full weight replica per GPU, no collective on the data path.

The reference scales out the same way on paper ("one process per GPU ... a worker owns its weights", docs/RUNNER.md:896-907; the engine
takes a `device` ordinal, runner/src/capi/c_api.cpp:110-113). A request's result is a pure function of that request
(runner/cuda/src/device.hpp:21-24), so the only decision is who takes which request.
"""
from __future__ import annotations

from typing import List, Sequence


def deal_requests(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Longest-processing-time-first: requests sorted by length (ties by index), each given to the rank with the least tokens so far
    (ties to the lowest rank). Deterministic, so every rank computes the same plan without talking to the others.
    Returns, per rank, the indices of its requests in the order it should run them (longest first)."""
    if world < 1:
        raise ValueError("world must be at least 1")
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    load = [0] * world
    plan: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        if lengths[i] <= 0:
            raise ValueError("a request needs at least one token")
        r = min(range(world), key=lambda g: (load[g], g))
        load[r] += int(lengths[i])
        plan[r].append(i)
    return plan


def ideal_speedup(lengths: Sequence[int], world: int) -> float:
    """Upper bound of the speed-up over one GPU when requests are not split: limited by the longest request and by the mean load."""
    total = float(sum(lengths))
    return total / max(max(lengths), total / world)
