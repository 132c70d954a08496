"""Multi-GPU partition of the attention path: by (batch, kv-head group), no data-path collective.

Every quantisation statistic of the path is local to one (batch, head) slice (the NVFP4 global
scale is ``amax/2688`` of that slice), and a kv head is only ever combined with the query heads of
its own group, so a rank that owns a set of (batch, kv-head) units computes exactly the rows of
O, LSE, dQ, dK and dV that belong to them.  The reference runs data-parallel replicas only
(``torchtitan/experiments/fa4/exact_lowp_attention.py:4123-4136``); this module is what a caller
uses to split one global problem instead.  ``torch.distributed`` appears only in the helpers that
time or check a run, never between the kernels.
"""

from __future__ import annotations

import torch


def unit_range(n_units: int, world: int, rank: int) -> range:
    """Contiguous, balanced share of ``n_units`` for ``rank`` (the first ``n_units % world`` ranks get one more)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def shard_units(B: int, Hkv: int, world: int, rank: int) -> list[tuple[int, int]]:
    """The (batch, kv head) units of ``rank``, batch-major."""
    return [(u // Hkv, u % Hkv) for u in unit_range(B * Hkv, world, rank)]


def shard_attention_inputs(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rank: int, world: int, *more_q_like: torch.Tensor):
    """This rank's units as a batch of single-kv-head problems.

    ``q [B,Hq,S,D]``, ``k, v [B,Hkv,S,D]`` -> ``q' [U,G,S,D]``, ``k', v' [U,1,S,D]`` with ``U`` the number of
    units and ``G = Hq/Hkv``; tensors shaped like ``q`` (``dout``, ``o``) given in ``more_q_like`` are
    sharded the same way.  Contiguous unit ranges of a contiguous tensor come back as views.
    """
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    if Hq % Hkv:
        raise ValueError(f"Hq={Hq} is not a multiple of Hkv={Hkv}")
    G = Hq // Hkv
    units = unit_range(B * Hkv, world, rank)
    sl = slice(units.start, units.stop)

    def q_like(t):
        return t.reshape(B * Hkv, G, S, D)[sl]

    def kv_like(t):
        return t.reshape(B * Hkv, 1, S, D)[sl]

    return (q_like(q), kv_like(k), kv_like(v), *[q_like(t) for t in more_q_like])


def unshard_q_like(parts: list[torch.Tensor], B: int, Hq: int) -> torch.Tensor:
    """Inverse of the ``q``-shaped sharding, given every rank's ``[U_r,G,S,D]`` (or ``[U_r,G,S]``) in rank order."""
    cat = torch.cat(parts, dim=0)
    return cat.reshape(B, Hq, *cat.shape[2:])


def unshard_kv_like(parts: list[torch.Tensor], B: int, Hkv: int) -> torch.Tensor:
    cat = torch.cat(parts, dim=0)
    return cat.reshape(B, Hkv, *cat.shape[2:])


def max_over_ranks(value: float, device: torch.device | str = "cpu") -> float:
    """A device time reduced the way multi-GPU numbers are reported: the slowest rank's."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
