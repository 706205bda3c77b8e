"""Static launch selection for ResAttn decode: KV split count and reducer.

Keeps the reference's selection interface and policy names (csrc/resattn/plan.py:21-93):
``(splits, reducer)`` with reducer in {"none", "kernel", "cga_sharded", "gmem_fused"} and the
RESIDUE_ATTN_REDUCTION policy {"legacy", "auto", "deterministic"}.  Both reducers of this library are fused
into the decode launch and combine the partials in split order, so they give the same bits:

* "kernel" (and "gmem_fused", which runs the same way): every CTA of a (sequence, KV head) takes a ticket and the
  one that draws the last ticket sums the partials from a global workspace (the counterpart of the reference's
  "gmem_fused" reducer, csrc/resattn/kernel_paged_decode.py:2365-2431, without its spin wait);
* "cga_sharded": the splits of a (sequence, KV head) are one thread-block cluster and combine through distributed
  shared memory, each CTA a share of the output.  Chosen for BF16 output when the whole grid is a handful of
  clusters and the context is not very long (measured on B200, one sequence, 8 KV heads: 14.6 against 18.7 us
  at 2.5 K tokens, 15.9 against 20.6 us at 4 K; with 16 clusters or more the cluster launch loses to the ticket
  form, which spreads its CTAs over the SMs freely).  Unlike the reference, head_dim 256 takes it too.

The split count itself is chosen for this library's kernel (128-token tiles): enough CTAs to cover the SMs while
leaving every split at least a few tiles.
"""
from __future__ import annotations

import os

_REDUCERS = ("none", "kernel", "cga_sharded", "gmem_fused")


def _reduction_policy(value=None):
    value = os.environ.get("RESIDUE_ATTN_REDUCTION", "legacy") if value is None else value
    if value not in ("legacy", "auto", "deterministic"):
        raise ValueError(f"unknown ResAttn reduction policy: {value}")
    return value


def _check_output_dimension(head_dim, output_nvfp4):
    if head_dim not in (128, 256):
        raise NotImplementedError("ResAttn supports head_dim=128 or 256")
    if head_dim == 256 and output_nvfp4:
        raise NotImplementedError("D256 supports BF16 output only")


def _pow2_floor(v: int) -> int:
    return 1 << (max(1, v).bit_length() - 1)


def _select_splits(batch: int, heads: int, length: int, sms: int, min_tiles_per_split: int = 4,
                   ctas_per_sm: int = 1) -> int:
    """`ctas_per_sm` CTAs per SM at a time (two for head_dim 128, one for 256), 128-token tiles, and every
    split covers the same number of tiles
    (ceil(tiles(length) / splits)) whatever the sequence: short sequences simply use fewer splits and
    the CTAs of their unused splits leave at once.  Measured on B200, the best piece size is the one
    that lets the working CTAs of the whole batch fit the SMs in one wave (a CTA costs about 5 us of
    set-up and merge, a tile about 1 us), so the piece is the expected tile count of the batch divided
    by the SM count, with 15 % head room; a batch of several sequences is assumed to average half of
    the longest length."""
    grid = max(1, batch * heads)
    tiles = max(1, (length + 127) // 128)
    total = grid * tiles * (0.5 if batch > 1 else 1.0)      # expected tiles of the whole batch
    slots = sms * ctas_per_sm
    piece = max(min_tiles_per_split, -(-int(total * 1.15) // slots))
    splits = -(-tiles // piece)
    # a few waves of unequal sequences: pieces of at most a third of the longest context even out the
    # tail (with very many CTAs the tail is short anyway and every extra CTA costs its set-up)
    if grid <= 8 * slots:
        splits = max(splits, min(3, tiles // 64))
    return max(1, min(splits, 64))


def _working_ctas(seq_lens, heads: int, splits: int, tiles_max: int) -> int:
    """CTAs of a ticket launch that have tiles to read: every sequence is cut into pieces of
    ceil(tiles_max / splits) tiles, the CTAs of the splits beyond its end leave at once."""
    piece = -(-tiles_max // splits)
    return heads * sum(-(-((max(int(n), 0) + 127) // 128) // piece) for n in seq_lens)


def _select_splits_exact(seq_lens, heads: int, tiles_max: int, slots: int) -> int:
    """With the lengths known on the host and a grid well below the device: the largest split count whose working
    CTAs still run in one wave.  Measured on B200 over batches of 2 to 16 sequences, equal and unequal lengths,
    both head dimensions, that count is the fastest or within a few percent of it (equal lengths of 32 K tokens,
    head_dim 128: 16 / 12 / 8 / 6 / 4 splits for 2 / 3 / 4 / 6 / 8 sequences); one more wave costs 15 to 40 %."""
    best = 1
    for s in range(2, min(64, tiles_max) + 1):
        if _working_ctas(seq_lens, heads, s, tiles_max) <= slots:
            best = s
    piece = -(-tiles_max // best)
    return -(-tiles_max // piece)                     # no CTAs beyond the last piece of the longest sequence


def select_decode_plan(batch, num_kv_heads, max_kv_len, sm_count, *, output_nvfp4=False,
                       grouped_head_tile=16, residue_fold=True, reduction_policy=None, head_dim=128, seq_lens=None):
    """Select the static split/reducer, then apply the caller's reduction policy.  ``seq_lens`` (optional; this
    library's addition): the sequences' lengths as host integers, when the caller has them without a device
    synchronisation -- small grids are then planned on the real tile counts instead of an assumed distribution."""
    _check_output_dimension(head_dim, output_nvfp4)
    if not residue_fold or grouped_head_tile not in (8, 16):
        raise NotImplementedError("production ResAttn requires residue Q8/Q16")
    policy = _reduction_policy(reduction_policy)
    if not output_nvfp4 and policy != "deterministic":
        cga = _cluster_splits(batch, num_kv_heads, max_kv_len, sm_count)
        if cga >= 2:
            return cga, "cga_sharded"
    ctas_per_sm = 2 if head_dim == 128 else 1
    slots = sm_count * ctas_per_sm
    if seq_lens is not None and len(seq_lens) == batch and 2 * batch * num_kv_heads <= slots:
        splits = _select_splits_exact(seq_lens, num_kv_heads, max(1, (max_kv_len + 127) // 128), slots)
    else:
        splits = _select_splits(batch, num_kv_heads, max_kv_len, sm_count, ctas_per_sm=ctas_per_sm)
    return (1, "none") if splits == 1 else (splits, "kernel")


_MAX_CLUSTERS = 8            # (sequence, KV head) pairs up to which the cluster reducer wins
_CLUSTER_MAX_TILES = 160     # ... and the context (128-token tiles) up to which: beyond it 16 ticket splits are faster
CLUSTER_SIZES = (2, 3, 4, 5, 6, 7, 8, 16)


def _cluster_splits(batch: int, heads: int, length: int, sms: int) -> int:
    """Cluster size for the "cga_sharded" reducer, 0 when the ticket reducer is the better choice: at most
    `_MAX_CLUSTERS` clusters of at most eight CTAs, one CTA per SM, one split per 128-token tile at most.  Measured
    for one sequence and 8 KV heads: eight clustered CTAs beat every ticket plan up to 16 K tokens (29.9 against
    31.7 us there) and lose to sixteen ticket splits from 24 K on (38.8 against 35.2 us); a cluster of sixteen, which
    the kernel accepts, is slower than either (the device places few of them at a time)."""
    clusters = max(1, batch * heads)
    tiles = max(1, (length + 127) // 128)
    if clusters > _MAX_CLUSTERS or tiles < 2:
        return 0
    if tiles > _CLUSTER_MAX_TILES:
        return 0
    return min(8, sms // clusters, tiles)


def static_compile_plans(*, output_nvfp4=False, grouped_head_tile=16, residue_fold=True, head_dim=128):
    """Enumerate decode kernel variants (nothing is compiled at run time here; kept for callers that
    warm up one launch per plan)."""
    if not residue_fold or grouped_head_tile not in (8, 16):
        raise NotImplementedError("production ResAttn requires residue Q8/Q16")
    _check_output_dimension(head_dim, output_nvfp4)
    plans = ((1, "none"), (2, "kernel"), (4, "kernel"))
    return plans if output_nvfp4 else plans + ((4, "cga_sharded"),)


def validate_decode_plan(plan, *, output_nvfp4=False, head_dim=128):
    """Check launch constraints before workspace allocation."""
    _check_output_dimension(head_dim, output_nvfp4)
    splits, reducer = plan
    if type(splits) is not int or splits < 1:
        raise ValueError(f"decode plan splits must be a positive integer, got {splits!r}")
    if reducer not in _REDUCERS:
        raise ValueError(f"unsupported decode reducer: {reducer!r}")
    if head_dim == 256 and reducer == "gmem_fused":
        raise NotImplementedError("D256 supports none/kernel/cga_sharded reduction only")
    if output_nvfp4 and reducer == "cga_sharded":
        raise NotImplementedError("cga_sharded does not support output_nvfp4=True")
    if reducer == "cga_sharded" and splits not in (1,) + CLUSTER_SIZES:
        raise ValueError(f"cga_sharded requires splits in {(1,) + CLUSTER_SIZES}")
    if reducer == "none" and splits != 1:
        raise ValueError("none reduction requires splits=1")
    if splits > 256:
        raise ValueError("at most 256 KV splits are supported")
