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


class PeerAllReduce:
    """One-shot all-reduce of small BF16 partials over peer memory (``ri_peer_allreduce_bf16``).

    Every rank allocates ``slots`` partial buffers of ``max_numel`` BF16 values and a flag array in one
    device allocation, exports it to the other ranks of the node through CUDA IPC (handles travel over the
    process group as Python objects) and maps theirs.  ``partial(shape)`` hands out the next buffer as a
    tensor for the GEMM to write into; ``reduce(partial, out)`` sums the same slot of every rank into
    ``out``.  Buffers are used round-robin; with two or more slots a buffer is only written again after
    this rank's next reduce has completed, which is what the kernel's contract asks for.

    ``ops.fp4_gemm(..., allreduce=self)`` is the GEMM whose epilogue does the reduction itself: it stores its
    tiles into every rank's inbox (``slots`` inboxes with one area per source rank, in the same exported
    allocation) and uses per-tile flags (``max_tiles`` of them; a call needs ``ri_fp4_gemm_allreduce_tiles(M, N)``).

    All ranks must call ``partial`` / ``reduce`` (or the fused GEMM) in the same order.  Raises RuntimeError if peer mapping is
    not possible (ranks on different nodes, IPC disabled); callers then stay with NCCL."""

    def __init__(self, max_numel: int, group=None, slots: int = 2, device=None, enable_pdl: bool = True,
                 max_tiles: int = 4096):
        from .. import _cabi
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("PeerAllReduce needs an initialised process group")
        if slots < 2:
            raise ValueError("at least two partial buffers are needed (a buffer must outlive the next reduce)")
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if not 2 <= self.world <= 8:
            raise RuntimeError(f"PeerAllReduce supports 2..8 ranks, got {self.world}")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.lib = _cabi.load()
        self.max_numel = (int(max_numel) + 7) // 8 * 8
        self.slots = slots
        self.enable_pdl = enable_pdl
        self.slot_bytes = (2 * self.max_numel + 255) // 256 * 256
        flag_bytes = int(self.lib.ri_peer_allreduce_flag_bytes())
        self.flag_off = self.slots * self.slot_bytes
        # behind the flags of the stand-alone kernel: the per-tile flags of the GEMM with the fused reduction
        self.max_tiles = int(max_tiles)
        self.tile_flag_off = self.flag_off + (flag_bytes + 255) // 256 * 256
        # ... and its inboxes: per slot one area of max_numel values for every source rank
        self.inbox_off = self.tile_flag_off + (int(self.lib.ri_fp4_gemm_allreduce_flag_bytes(self.max_tiles)) + 255) // 256 * 256
        total = self.inbox_off + self.slots * self.world * 2 * self.slot_bytes       # 4 bytes per element (pair format)
        # Every step that can fail on one rank only is followed by an exchange of the outcome, so that all
        # ranks raise together and none is left waiting in a collective the others never enter.
        handle, err = None, None
        try:
            # a private allocation (not a slice of a cached block that other tensors share)
            self.local = torch.zeros(total, dtype=torch.uint8, device=self.device)
            self.state = torch.zeros(int(self.lib.ri_peer_allreduce_state_bytes()), dtype=torch.uint8, device=self.device)
            self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.tile_calls = torch.zeros(int(self.lib.ri_fp4_gemm_allreduce_call_bytes(self.max_tiles)),
                                          dtype=torch.uint8, device=self.device)
            torch.cuda.synchronize(self.device)
            handle = self.local.untyped_storage()._share_cuda_()
        except Exception as e:                                # IPC disabled, out of memory
            err = f"rank {self.rank} cannot export its buffer: {type(e).__name__}: {e}"
        handles = [None] * self.world
        dist.all_gather_object(handles, (handle, err), group=group)
        errs = [e for _, e in handles if e]
        if errs:
            raise RuntimeError("; ".join(errs))
        self._peer_storages = []
        self.bases = []
        err = None
        for r, (h, _) in enumerate(handles):
            if r == self.rank:
                self.bases.append(self.local.data_ptr())
                continue
            try:
                with torch.cuda.device(self.device):
                    st = torch.UntypedStorage._new_shared_cuda(self.device.index, *h[1:])
            except Exception as e:                            # not on this node, no peer access, IPC refused
                err = f"rank {self.rank} cannot map the buffer of rank {r}: {type(e).__name__}: {e}"
                break
            self._peer_storages.append(st)
            self.bases.append(st.data_ptr())
        outcomes = [None] * self.world
        dist.all_gather_object(outcomes, err, group=group)   # also: every rank has mapped every buffer
        errs = [e for e in outcomes if e]
        if errs:
            raise RuntimeError("; ".join(errs))
        import ctypes
        self._ct = ctypes
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*[b + self.flag_off for b in self.bases])
        self._data_ptrs = [(ctypes.c_void_p * self.world)(*[b + s * self.slot_bytes for b in self.bases])
                           for s in range(self.slots)]
        self.tile_flag_ptrs = (ctypes.c_void_p * self.world)(*[b + self.tile_flag_off for b in self.bases])
        self._inbox_ptrs = [(ctypes.c_void_p * self.world)(*[b + self.inbox_off + s * self.world * 2 * self.slot_bytes
                                                             for b in self.bases]) for s in range(self.slots)]
        self._next = 0
        self._next_inbox = 0

    def partial(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
        """The next partial buffer of this rank as a tensor of ``shape`` (row-major, BF16)."""
        if dtype != torch.bfloat16:
            raise ValueError("PeerAllReduce sums BF16 partials")
        n = 1
        for s in shape:
            n *= int(s)
        if n > self.max_numel or n % 8:
            raise ValueError(f"{n} elements: at most {self.max_numel}, a multiple of 8")
        slot = self._next
        self._next = (self._next + 1) % self.slots
        off = slot * self.slot_bytes
        t = self.local[off:off + 2 * n].view(torch.bfloat16).view(*shape)
        t._ri_slot = slot
        return t

    def next_inbox(self, numel: int):
        """The next inbox for a GEMM with the reduction in its epilogue: (C array of every rank's mapping of
        it, elements per source rank's area -- an area is four bytes per element).  Inboxes alternate like partials."""
        if numel > self.max_numel:
            raise ValueError(f"{numel} elements: at most {self.max_numel}")
        slot = self._next_inbox
        self._next_inbox = (self._next_inbox + 1) % self.slots
        return self._inbox_ptrs[slot], self.slot_bytes // 2

    def reduce(self, partial: torch.Tensor, out: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
        """Sum ``partial`` (a tensor from ``partial()``) over the ranks into ``out`` (local BF16, same shape).

        The kernel waits for the peers for about ten seconds at most.  If a peer never announces its partial
        the kernel writes THIS rank's partial to ``out`` (a defined value, not the sum) and stores
        ``0x40000000 | missing_rank << 8 | rank`` in the status word: ``status`` if given, else this object's
        own word, which ``check()`` reads.  Callers that cannot tolerate a silent local-only result call
        ``check()`` at a point where a device synchronisation is acceptable (end of a step)."""
        from .. import _cabi
        slot = getattr(partial, "_ri_slot", None)
        if slot is None:
            raise ValueError("reduce() takes a tensor handed out by partial()")
        if out is None:
            out = torch.empty(partial.shape, dtype=torch.bfloat16, device=self.device)
        if out.dtype != torch.bfloat16 or out.numel() != partial.numel() or not out.is_contiguous():
            raise ValueError("out must be a contiguous BF16 tensor of the partial's size")
        word = self.status if status is None else status
        st = self.lib.ri_peer_allreduce_bf16(self._data_ptrs[slot], self._flag_ptrs, self.rank, self.world,
                                             partial.numel(), out.data_ptr(), self.state.data_ptr(),
                                             word.data_ptr(), _cabi.current_stream(self.device),
                                             int(self.enable_pdl))
        _cabi.check(st, "peer all-reduce")
        return out

    def check(self) -> None:
        """Synchronising read of this object's status word; raises RuntimeError (and clears the word) when a
        reduce gave up waiting for a peer since the last check."""
        v = int(self.status.item())
        if v:
            self.status.zero_()
            raise RuntimeError(f"peer all-reduce: rank {v & 0xFF} gave up waiting for rank {(v >> 8) & 0xFF} "
                               f"(status 0x{v & 0xFFFFFFFF:08x}); the output of that call is the local partial")
