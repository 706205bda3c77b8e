"""Tensor-parallel partition of the linear hot path on one node (one process per GPU).

Column-parallel layers (qkv, gate_up) split the weight's N; every rank quantises the full activation
and no collective is needed (an all-gather only when the caller wants the unsharded output).
Row-parallel layers (o, down) split K: rank r quantises x[:, r*K/tp:(r+1)*K/tp] -- block scales are
local to 16/32-element blocks and the NVFP4 global scale is a per-layer constant, so its codes equal the
corresponding slice of the unsharded run -- and the BF16 partial outputs are summed with one
all-reduce.  K-extended (KEXT) weights are cut with ``ResidueShardPlan``.  The reference leaves these
collectives to vLLM's RowParallelLinear (its own code only holds the partition rule,
quant/vllm_integration/residue_tp.py).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .vllm_integration.residue_tp import ResidueShardPlan


def shard_bounds(size: int, tp: int, rank: int, align: int = 1) -> tuple[int, int]:
    if size % tp or (size // tp) % align:
        raise ValueError(f"size {size} does not split into {tp} shards aligned to {align}")
    w = size // tp
    return rank * w, (rank + 1) * w


def shard_weight(w: torch.Tensor, parallel: str, tp: int, rank: int) -> torch.Tensor:
    """Dense [N, K] weight -> this rank's shard ("col": rows of N, "row": columns of K, 128-aligned)."""
    if parallel == "col":
        lo, hi = shard_bounds(w.shape[0], tp, rank, 32)
        return w[lo:hi]
    if parallel == "row":
        lo, hi = shard_bounds(w.shape[1], tp, rank, 128)
        return w[:, lo:hi]
    raise ValueError(f"unknown parallel mode {parallel!r}")


def shard_activation(x: torch.Tensor, parallel: str, tp: int, rank: int) -> torch.Tensor:
    if parallel == "col":
        return x
    lo, hi = shard_bounds(x.shape[-1], tp, rank, 128)
    return x[..., lo:hi]


def shard_extended_weight(w_ext: torch.Tensor, k_base: int, num_salient: int, tp: int, rank: int,
                          channels_per_element: int = 1, **plan_kw) -> torch.Tensor:
    """[W | W[:, sel]] (last dim, in elements of ``channels_per_element`` channels) -> this rank's
    [W_r | W[:, sel_r]] for a row-parallel KEXT layer; raises ResidueTPError for cuts the rule forbids."""
    plan = ResidueShardPlan(k_base, num_salient, tp, rank, **plan_kw)
    plan.validate()
    return plan.gather(w_ext, channels_per_element)


def finish_output(y: torch.Tensor, parallel: str, group=None, gather: bool = False) -> torch.Tensor:
    """Row-parallel: sum the partial outputs over ranks (in place).  Column-parallel: optionally
    all-gather the N shards."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return y
    if parallel == "row":
        dist.all_reduce(y, group=group)
        return y
    if gather:
        parts = [torch.empty_like(y) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, y.contiguous(), group=group)
        return torch.cat(parts, dim=-1)
    return y
