"""The GEMM whose epilogue sums the partial outputs over the ranks (``ri_fp4_gemm_allreduce``), on ONE GPU.

No second rank runs here (kernels that wait for one another never share a GPU): the "peers" are buffers of this
process.  Their partials are written into this rank's inbox BEFORE the launch the way their kernels would write
them -- as (value, call number) pairs for small partials, as plain BF16 tiles plus per-tile flags for large ones
-- so the kernel finds everything in place and never waits; its own stores into the "peers'" inboxes are read
back.  Checked bit for bit against ``ri_fp4_gemm`` followed by the rank-ordered FP32 sum, for plans that finish a
tile in one CTA, that split K over CTAs (both finishing paths) and that use two-CTA tiles, in both protocols; the
kernel's own announcements and call counters are read back.  The two-GPU run is ``tests/peer_allreduce_worker.py``.

The bounded wait, both protocols: with nothing in place and the limit shortened, the kernel gives up, names the
missing rank in the status word and writes its own partial; the next call works once the peer is back in step."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


class LocalRanks:
    """Stands in for ``resinfer_b200.quant.tp.PeerAllReduce`` with every rank's inboxes and flags in this process."""

    def __init__(self, world, rank, max_numel, dev, max_tiles=1024):
        from resinfer_b200 import _cabi
        self.lib = lib = _cabi.load()
        self.world, self.rank, self.max_tiles, self.dev = world, rank, max_tiles, dev
        self.area = (max_numel + 127) // 128 * 128
        # inbox[slot][owner rank]: `world` areas of 4 bytes per element, area s receives rank s's partial
        self.inbox = [[torch.zeros(world * self.area, dtype=torch.int32, device=dev) for _ in range(world)] for _ in range(2)]
        self.flags = [torch.zeros(lib.ri_fp4_gemm_allreduce_flag_bytes(max_tiles) // 4, dtype=torch.int32, device=dev)
                      for _ in range(world)]
        self.tile_calls = torch.zeros(lib.ri_fp4_gemm_allreduce_call_bytes(max_tiles) // 4, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.tile_flag_ptrs = (ctypes.c_void_p * world)(*[f.data_ptr() for f in self.flags])
        self._ptrs = [(ctypes.c_void_p * world)(*[t.data_ptr() for t in self.inbox[s]]) for s in range(2)]
        self._next = 0

    def next_inbox(self, numel):
        s = self._next
        self._next ^= 1
        return self._ptrs[s], self.area

    def pairs(self, m, n):
        """True if a partial of this shape travels as (value, call number) pairs."""
        return bool(self.lib.ri_fp4_gemm_allreduce_uses_pairs(m, n, self.world))

    def _area(self, owner, source, slot):
        return self.inbox[slot][owner][source * self.area:(source + 1) * self.area]

    def put(self, owner, source, slot, partial, call):
        """Write rank `source`'s partial into rank `owner`'s inbox the way the kernel of `source` would."""
        m, n = partial.shape
        words = partial.contiguous().view(torch.int32).reshape(-1)              # two BF16 values per word
        if self.pairs(m, n):
            a = self._area(owner, source, slot)[:2 * words.numel()].view(-1, 2)
            a[:, 0] = words
            a[:, 1] = call
        else:
            self._area(owner, source, slot)[:words.numel()].copy_(words)

    def get(self, owner, source, slot, shape, call):
        """Rank `source`'s partial as it lies in rank `owner`'s inbox (pairs: also checks the call numbers)."""
        m, n = shape
        nw = m * n // 2
        if self.pairs(m, n):
            a = self._area(owner, source, slot)[:2 * nw].view(-1, 2)
            assert bool((a[:, 1] == call).all())
            words = a[:, 0].contiguous()
        else:
            words = self._area(owner, source, slot)[:nw].contiguous()
        return words.view(torch.bfloat16).view(m, n)

    def announce_all(self, call):
        """What the peers' kernels would have stored with the flag protocol: call number `call` for every tile,
        from every peer."""
        f = self.flags[self.rank].view(self.max_tiles, 8)
        for r in range(self.world):
            if r != self.rank:
                f[:, r] = call


def _operands(m, n, k, dev, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    codes = torch.randint(0, 256, (2 * m, k // 2), generator=g, dtype=torch.uint8).to(dev)
    sf = torch.randint(0x30, 0x40, (((2 * m + 127) // 128) * (k // 64) * 512,), generator=g, dtype=torch.uint8).to(dev)
    w = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8).to(dev)
    w_sf = torch.randint(0x30, 0x40, (((n + 127) // 128) * (k // 64) * 512,), generator=g, dtype=torch.uint8).to(dev)
    alpha = torch.tensor([2.0 ** -8], dtype=torch.float32, device=dev)
    return codes, sf, w, w_sf, alpha


@pytest.mark.parametrize("m,n,k,splits,world,rank", [
    (1, 512, 1024, 1, 2, 0),          # complete tiles, one CTA each
    (16, 5120, 8192, 0, 2, 1),        # K split over CTAs, ragged ranges (both finishing paths)
    (5, 1000, 4096, 4, 3, 1),         # three ranks: the order of the sum matters; N not a multiple of 128
    (128, 5120, 4096, 0, 4, 2),
    (300, 640, 2048, 1, 2, 0),        # several token tiles
    (1024, 1152, 2048, -2, 2, 0),     # two-CTA tiles, nine weight tiles: the last pair is half empty
    (64, 5120, 25600, 0, 8, 7),
])
def test_fused_reduction_equals_gemm_then_rank_ordered_sum(cuda_device, m, n, k, splits, world, rank):
    from resinfer_b200 import ops
    dev = cuda_device
    codes, sf, w, w_sf, alpha = _operands(m, n, k, dev, seed=m + n)
    mine = ops.fp4_gemm(codes, sf, w, w_sf, alpha, m=m, layout="row_pair", splits=splits)
    ranks = LocalRanks(world, rank, m * n, dev, max_tiles=4096)
    for call in (1, 2, 3):                                    # both inboxes, and the first one again
        slot = (call - 1) & 1
        g = torch.Generator(device="cpu").manual_seed(100 * call + rank)
        want = torch.zeros(m, n, dtype=torch.float32, device=dev)
        for r in range(world):
            if r == rank:
                want += mine.float()
            else:
                peer = (torch.randn(m, n, generator=g) * 40).to(torch.bfloat16).to(dev)
                ranks.put(rank, r, slot, peer, call)
                want += peer.float()
        ranks.announce_all(call)
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize()
        ops.fp4_gemm(codes, sf, w, w_sf, alpha, m=m, layout="row_pair", splits=splits, out=out, allreduce=ranks)
        torch.cuda.synchronize()
        ops.check_status(dev)
        assert int(ranks.status.item()) == 0
        for r in range(world):                                 # every peer's inbox received the plain GEMM of this rank
            if r != rank:
                assert torch.equal(ranks.get(r, rank, slot, (m, n), call), mine), (call, r)
        assert torch.equal(out, want.to(torch.bfloat16)), call
        if ranks.pairs(m, n):                                  # launches counted, ticket back at zero
            assert ranks.tile_calls[ranks.max_tiles:].tolist() == [call, 0]
        else:
            calls = ranks.tile_calls[:ranks.max_tiles]
            used = calls != 0
            assert int(used.sum().item()) > 0 and bool((calls[used] == call).all())
            for r in range(world):                             # announced to every peer, for the used tiles
                if r != rank:
                    got = ranks.flags[r].view(-1, 8)[:, rank]
                    assert torch.equal(got != 0, used) and bool((got[used] == call).all())


@pytest.mark.parametrize("m,n,k", [(16, 512, 2048), (1100, 512, 1024)])     # pair protocol; flag protocol
def test_fused_reduction_gives_up_on_a_missing_peer_and_recovers(cuda_device, m, n, k):
    from resinfer_b200 import _cabi, ops
    lib = _cabi.load()
    dev = cuda_device
    codes, sf, w, w_sf, alpha = _operands(m, n, k, dev, seed=9)
    mine = ops.fp4_gemm(codes, sf, w, w_sf, alpha, m=m, layout="row_pair")
    ranks = LocalRanks(2, 0, m * n, dev)
    peer = torch.randn(m, n, device=dev).to(torch.bfloat16)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
    lib.ri_peer_allreduce_set_wait_ms(100)
    try:
        ops.fp4_gemm(codes, sf, w, w_sf, alpha, m=m, layout="row_pair", out=out, allreduce=ranks)   # nothing has arrived
        torch.cuda.synchronize()
        assert int(ranks.status.item()) == (0x40000000 | (1 << 8) | 0)
        assert torch.equal(out, mine)                          # a defined value: this rank's own partial
        ops.check_status(dev)                                  # the GEMM itself had no expired wait
        # back in step: the peer's partial of call 2 arrives (second inbox)
        ranks.status.zero_()
        ranks.put(0, 1, 1, peer, 2)
        ranks.announce_all(2)
        ops.fp4_gemm(codes, sf, w, w_sf, alpha, m=m, layout="row_pair", out=out, allreduce=ranks)
        torch.cuda.synchronize()
        assert int(ranks.status.item()) == 0
        assert torch.equal(out, (mine.float() + peer.float()).to(torch.bfloat16))
    finally:
        lib.ri_peer_allreduce_set_wait_ms(10000)


def test_fused_reduction_rejects_bad_arguments(cuda_device):
    from resinfer_b200 import ops
    dev = cuda_device
    m, n, k = 16, 512, 1024
    codes, sf, w, w_sf, alpha = _operands(m, n, k, dev, seed=3)
    ranks = LocalRanks(2, 0, m * n, dev, max_tiles=2)           # 4 weight tiles need 4 flag entries
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError, match="tile flags"):
        ops.fp4_gemm(codes, sf, w, w_sf, alpha, m=m, layout="row_pair", out=out, allreduce=ranks)
    with pytest.raises(ValueError):
        ops.fp4_gemm(codes, sf, w, w_sf, alpha, m=m, layout="row_pair", out=out.float(), allreduce=LocalRanks(2, 0, m * n, dev))
