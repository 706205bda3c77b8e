"""Worker of tests/test_gpu_peer_allreduce.py: one process per GPU under torchrun (gloo for the
rendezvous and the handle exchange; the reduction itself runs over peer memory)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def data(rank, it, shape, dev):
    g = torch.Generator(device="cpu").manual_seed(1000 * it + rank)
    return torch.randn(shape, generator=g, dtype=torch.float32).to(torch.bfloat16).to(dev)


def fused_gemm(rank, world, dev, ar):
    """The GEMM with the reduction in its epilogue against the plain GEMM of every rank + rank-ordered FP32 sum,
    eagerly and under graph replay, for plans with whole tiles, split K and two-CTA tiles."""
    from resinfer_b200 import ops

    def operands(r, m, n, k):
        g = torch.Generator(device="cpu").manual_seed(77 * r + m + n)
        codes = torch.randint(0, 256, (2 * m, k // 2), generator=g, dtype=torch.uint8).to(dev)
        sf = torch.randint(0x30, 0x40, (((2 * m + 127) // 128) * (k // 64) * 512,), generator=g, dtype=torch.uint8).to(dev)
        w = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8).to(dev)
        w_sf = torch.randint(0x30, 0x40, (((n + 127) // 128) * (k // 64) * 512,), generator=g, dtype=torch.uint8).to(dev)
        return codes, sf, w, w_sf

    alpha = torch.tensor([2.0 ** -8], dtype=torch.float32, device=dev)
    cases = [(1, 5120, 4096, 0), (16, 5120, 12800, 0), (128, 5120, 4096, 0), (40, 1000, 2048, 1), (1024, 1152, 2048, -2)]
    for m, n, k, splits in cases:
        want = torch.zeros(m, n, dtype=torch.float32, device=dev)
        for r in range(world):                                  # every rank computes every rank's plain partial
            c, s, w, ws = operands(r, m, n, k)
            want += ops.fp4_gemm(c, s, w, ws, alpha, m=m, layout="row_pair", splits=splits).float()
        want = want.to(torch.bfloat16)
        c, s, w, ws = operands(rank, m, n, k)
        outs = [torch.zeros(m, n, dtype=torch.bfloat16, device=dev) for _ in range(4)]
        for o in outs[:2]:
            ops.fp4_gemm(c, s, w, ws, alpha, m=m, layout="row_pair", splits=splits, out=o, allreduce=ar)
        torch.cuda.synchronize()
        ar.check()
        ops.check_status(dev)
        assert torch.equal(outs[0], want) and torch.equal(outs[1], want), (rank, m, n, k)

        # the same sum through the two-kernel form that the context manager selects for the registered ops
        with ops.row_parallel_reduction(ar, epilogue=False):
            two = [ops.fp4_gemm(c, s, w, ws, alpha, m=m, layout="row_pair", splits=splits) for _ in range(2)]
        torch.cuda.synchronize()
        ar.check()
        assert torch.equal(two[0], want) and torch.equal(two[1], want), (rank, m, n, k, "two kernels")

        def body():
            for o in outs:
                ops.fp4_gemm(c, s, w, ws, alpha, m=m, layout="row_pair", splits=splits, out=o, allreduce=ar)

        st = torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            body()
        torch.cuda.current_stream().wait_stream(st)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            body()
        for _ in range(3):
            for o in outs:
                o.zero_()
            g.replay()
            torch.cuda.synchronize()
            ar.check()
            for o in outs:
                assert torch.equal(o, want), (rank, m, n, k, "graph")
        dist.barrier()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from resinfer_b200.quant.tp import PeerAllReduce
    ar = PeerAllReduce(1024 * 1280, slots=2)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    shapes = [(1, 5120), (16, 5120), (128, 5120), (3, 8), (64, 4096)]
    it = 0
    for rep in range(3):
        for shape in shapes:
            p = ar.partial(shape)
            p.copy_(data(rank, it, shape, dev))
            out = ar.reduce(p, status=status)
            acc = torch.zeros(shape, dtype=torch.float32, device=dev)
            for r in range(world):
                acc += data(r, it, shape, dev).float()
            torch.cuda.synchronize()
            assert int(status.item()) == 0, hex(int(status.item()))
            assert torch.equal(out, acc.to(torch.bfloat16)), (rank, it, shape)
            it += 1
    # the same under CUDA-graph replay: four reduces per graph (both slots twice), replayed
    shape = (16, 5120)
    xs = [data(rank, 500 + j, shape, dev) for j in range(4)]
    outs = [torch.empty(shape, dtype=torch.bfloat16, device=dev) for _ in range(4)]

    def body():
        for j in range(4):
            p = ar.partial(shape)
            p.copy_(xs[j])
            ar.reduce(p, outs[j], status=status)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        body()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        body()
    for _ in range(5):
        for o in outs:
            o.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for j in range(4):
            acc = torch.zeros(shape, dtype=torch.float32, device=dev)
            for r in range(world):
                acc += data(r, 500 + j, shape, dev).float()
            assert torch.equal(outs[j], acc.to(torch.bfloat16)), (rank, j)
    fused_gemm(rank, world, dev, ar)
    dist.barrier()
    if rank == 0:
        print("PEER_ALLREDUCE_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
