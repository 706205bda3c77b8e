"""Tensor-parallel shard plan for K-extended (``[base | salient]``) NVFP4 / MXFP4 tensors.

Pure index arithmetic on CPU tensors, no process group: the rule of the reference's
quant/vllm_integration/residue_tp.py:29-278 with the same class / function names, properties and
error type.  A row-parallel rank r owns base channels [r*K/tp, (r+1)*K/tp) and the salient channels
that fall into that range; the extended tensor is cut in two ranges per rank and may be re-ordered
once (``interleave_extended_for_tp``) so that an ordinary contiguous narrow per rank lands on them.

Alignment rules (``validate``): K/tp must be a multiple of 8 (whole salient blocks), of 128 (a residue
scale group spans up to 128 base channels, so a cut inside one would change that rank's residue
amax), and both K/tp and S/tp must be multiples of scale_vec_size * scale_swizzle_blocks (64 for
NVFP4's swizzled scales, 32 for MXFP4's raw scales).
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import torch

SALIENT_BLOCK = 8                  # salient channels are chosen per block of eight
SF_VEC_SIZE = 16                   # channels per NVFP4 scale
SF_SWIZZLE_BLOCKS = 4              # scale blocks per swizzled tile along K
RESIDUE_SF_GROUP_CHANNELS = 128    # base channels one residue scale can span (ratio 0.125)


class ResidueTPError(ValueError):
    """A shape the residue TP sharding rule cannot honour."""


def _round_up(v: int, a: int) -> int:
    return -(-v // a) * a


@dataclass(frozen=True)
class ResidueShardPlan:
    """How to cut one extended tensor for one rank (widths in logical channels)."""

    k_base: int
    num_salient: int
    tp_size: int
    tp_rank: int
    scale_vec_size: int = SF_VEC_SIZE
    scale_swizzle_blocks: int = SF_SWIZZLE_BLOCKS
    residue_sf_group_channels: int = RESIDUE_SF_GROUP_CHANNELS
    k_alignment: int = 1

    k_ext = property(lambda self: self.k_base + self.num_salient)
    base_shard = property(lambda self: self.k_base // self.tp_size)
    salient_shard = property(lambda self: self.num_salient // self.tp_size)
    k_ext_shard = property(lambda self: self.base_shard + self.salient_shard)
    k_padded = property(lambda self: _round_up(self.k_ext, self.k_alignment))
    k_shard_padded = property(lambda self: _round_up(self.k_ext_shard, self.k_alignment))

    def validate(self) -> None:
        """Raise ResidueTPError for shapes the two-range rule cannot serve."""
        tp = self.tp_size
        if (self.scale_vec_size not in (16, 32) or self.scale_swizzle_blocks <= 0
                or self.residue_sf_group_channels <= 0 or self.k_alignment <= 0):
            raise ResidueTPError("invalid FP4 scale or K alignment")
        if tp <= 0 or not 0 <= self.tp_rank < tp:
            raise ResidueTPError(f"bad tp_rank={self.tp_rank} for tp_size={tp}")
        if self.k_base % tp:
            raise ResidueTPError(f"K_base={self.k_base} not divisible by tp_size={tp}")
        if self.num_salient % tp:
            raise ResidueTPError(f"num_salient={self.num_salient} not divisible by tp_size={tp}; "
                                 "the salient split would be ragged")
        if self.base_shard % SALIENT_BLOCK:
            raise ResidueTPError(f"K_base/tp={self.base_shard} is not a multiple of {SALIENT_BLOCK}: "
                                 "ranks would get different salient counts")
        if self.base_shard % self.residue_sf_group_channels:
            raise ResidueTPError(
                f"K_base/tp={self.base_shard} is not a multiple of {self.residue_sf_group_channels}: the "
                "boundary would split a residue scale-factor group, so this rank would compute a different "
                "residue amax than the unsharded model")
        grid = self.scale_vec_size * self.scale_swizzle_blocks
        for name, width in (("K_base/tp", self.base_shard), ("S/tp", self.salient_shard)):
            if width % grid:
                raise ResidueTPError(f"{name}={width} is not a multiple of {grid}; the block-scale group "
                                     "cannot be split there")
        if self.k_ext_shard * tp != self.k_ext:
            raise ResidueTPError("K_ext must split evenly")
        if self.k_padded % self.scale_vec_size or self.k_shard_padded % self.scale_vec_size:
            raise ResidueTPError("padded K must align with scale groups")

    def ranges(self, channels_per_element: int = 1):
        """((base offset, base length), (salient offset, salient length)) in storage elements:
        1 channel per element for logical indices, 2 for packed FP4, scale_vec_size for scales."""
        c = channels_per_element
        if c <= 0:
            raise ResidueTPError("channels_per_element must be positive")
        for name, v in (("k_base", self.k_base), ("base_shard", self.base_shard),
                        ("salient_shard", self.salient_shard)):
            if v % c:
                raise ResidueTPError(f"{name}={v} not divisible by channels_per_element={c}")
        return ((self.tp_rank * self.base_shard // c, self.base_shard // c),
                ((self.k_base + self.tp_rank * self.salient_shard) // c, self.salient_shard // c))

    def gather(self, full: torch.Tensor, channels_per_element: int = 1, dim: int = -1) -> torch.Tensor:
        """This rank's ``[base_r | salient_r | zero pad]`` slice of ``full`` (a local slice + concat,
        not a collective)."""
        c = channels_per_element
        (b_off, b_len), (s_off, s_len) = self.ranges(c)
        if self.k_padded % c or self.k_shard_padded % c:
            raise ResidueTPError("padded K is not divisible by channels_per_element")
        if full.shape[dim] != self.k_padded // c:
            raise ResidueTPError(f"expected extended dim {self.k_padded // c} along dim {dim}, got {full.shape[dim]}")
        parts = [full.narrow(dim, b_off, b_len), full.narrow(dim, s_off, s_len)]
        pad = (self.k_shard_padded - self.k_ext_shard) // c
        if pad:                                      # FP4 code 0 and E8M0 code 0 both mean zero
            shape = list(parts[0].shape)
            shape[dim] = pad
            parts.append(full.new_zeros(shape))
        return torch.cat(parts, dim=dim)

    def local_salient_indices(self, full_indices: torch.Tensor) -> torch.Tensor:
        """Salient indices owned by this rank, rebased to its first channel.  The indices must be
        globally sorted so that the rank's share is the r-th contiguous run (checked)."""
        lo = self.tp_rank * self.base_shard
        mine = full_indices[(full_indices >= lo) & (full_indices < lo + self.base_shard)]
        if mine.numel() != self.salient_shard:
            raise ResidueTPError(
                f"rank {self.tp_rank} owns {mine.numel()} salient channels, expected {self.salient_shard}: "
                "the export's per-block uniformity no longer holds, so TP sharding is unsafe")
        run = full_indices.narrow(0, self.tp_rank * self.salient_shard, self.salient_shard)
        if not torch.equal(mine, run):
            raise ResidueTPError("salient indices are not globally sorted; the contiguous-run assumption "
                                 "behind TP sharding is broken")
        return mine - lo


def interleave_extended_for_tp(full: torch.Tensor, plan: ResidueShardPlan, channels_per_element: int = 1,
                               dim: int = -1) -> torch.Tensor:
    """Reorder ``[base | salient]`` into ``[base_0 | sal_0 | base_1 | sal_1 | ...]`` so that rank r's
    contiguous range [r*K_shard_padded, (r+1)*K_shard_padded) is its two-range gather.  A pure function
    of the full tensor (identical on every rank)."""
    return torch.cat([replace(plan, tp_rank=r).gather(full, channels_per_element, dim)
                      for r in range(plan.tp_size)], dim=dim).contiguous()


def plan_from_partition(*, extended_dim: int, input_size_per_partition: int, input_size: int, num_salient: int,
                        tp_rank: int = 0, scale_vec_size: int = SF_VEC_SIZE,
                        scale_swizzle_blocks: int = SF_SWIZZLE_BLOCKS,
                        residue_sf_group_channels: int = RESIDUE_SF_GROUP_CHANNELS,
                        k_alignment: int = 1) -> ResidueShardPlan | None:
    """Plan from what a row-parallel layer knows at weight-creation time.  Returns None when the input
    is not sharded (column-parallel: every rank holds the whole extended K)."""
    if input_size_per_partition >= input_size:
        return None
    if input_size % input_size_per_partition:
        raise ResidueTPError(f"input_size={input_size} is not a whole multiple of "
                             f"input_size_per_partition={input_size_per_partition}")
    k_base = extended_dim - num_salient
    if k_base != input_size:
        raise ResidueTPError(f"extended_dim={extended_dim} minus num_salient={num_salient} is {k_base}, "
                             f"which does not match input_size={input_size}")
    plan = ResidueShardPlan(k_base, num_salient, input_size // input_size_per_partition, tp_rank,
                            scale_vec_size, scale_swizzle_blocks, residue_sf_group_channels, k_alignment)
    plan.validate()
    return plan


def current_tp_rank() -> int:
    """Rank inside ``torch.distributed``'s default group (0 when not initialised)."""
    import torch.distributed as dist
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
