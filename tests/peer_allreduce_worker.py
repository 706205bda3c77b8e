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


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from resinfer_b200.quant.tp import PeerAllReduce
    ar = PeerAllReduce(128 * 5120, slots=2)
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
    dist.barrier()
    if rank == 0:
        print("PEER_ALLREDUCE_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
