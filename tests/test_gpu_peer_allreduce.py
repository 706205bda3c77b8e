"""One-shot peer-memory all-reduce (ri_peer_allreduce_bf16).

Two GPUs of one node: bit-exact against the rank-ordered FP32 sum, eager and under CUDA-graph replay (skipped
with fewer than two GPUs).  One GPU: the bounded wait.  Rank 0 of a two-rank group is launched alone, with both
ranks' buffers in this process's memory; nothing ever sets rank 1's flag, so the wait runs out after the
(shortened) limit, the status word names the missing rank, the output holds rank 0's own partial, and the next
call works normally once the missing announcement is written by hand -- the context stays usable."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_allreduce_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533",
                        os.path.join(here, "peer_allreduce_worker.py")],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "PEER_ALLREDUCE_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_wait_for_a_missing_peer_runs_out_and_reports(cuda_device):
    import ctypes

    from resinfer_b200 import _cabi
    lib = _cabi.load()
    dev = cuda_device
    n = 4096
    parts = [torch.randn(n, device=dev).to(torch.bfloat16) for _ in range(2)]
    flags = [torch.zeros(lib.ri_peer_allreduce_flag_bytes() // 4, dtype=torch.int32, device=dev) for _ in range(2)]
    state = torch.zeros(lib.ri_peer_allreduce_state_bytes(), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    data_ptrs = (ctypes.c_void_p * 2)(*[p.data_ptr() for p in parts])
    flag_ptrs = (ctypes.c_void_p * 2)(*[f.data_ptr() for f in flags])
    call = lambda: lib.ri_peer_allreduce_bf16(data_ptrs, flag_ptrs, 0, 2, n, out.data_ptr(), state.data_ptr(),   # noqa: E731
                                              status.data_ptr(), _cabi.current_stream(dev), 0)
    lib.ri_peer_allreduce_set_wait_ms(200)
    try:
        assert call() == 0
        torch.cuda.synchronize()
        assert int(status.item()) == (0x40000000 | (1 << 8) | 0)
        assert torch.equal(out, parts[0])                     # a defined value: the local partial
        # rank 0 announced call 1 to both flag arrays
        assert int(flags[0][0].item()) == 1 and int(flags[1][0].item()) == 1
        # the second call: write rank 1's announcement of call 2 by hand; the sum now comes out
        status.zero_()
        flags[0][1] = 2
        assert call() == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(out, (parts[0].float() + parts[1].float()).to(torch.bfloat16))
    finally:
        lib.ri_peer_allreduce_set_wait_ms(10000)


def test_slice_exchange_of_large_partials_on_many_ranks(cuda_device):
    """More than 4 MB of peer reads per rank on more than two ranks: the kernel sums only its own slice of the
    vectors, puts the sums back into its own partial buffer and fetches the other slices from their owners.  Rank 1
    of four is launched alone with every buffer in this process and both announcements of every "peer" written by
    hand, so nothing waits: its own slice must come out as the rank-ordered FP32 sum, the other slices as whatever
    their owners' buffers hold (stand-ins for their sums), and its own buffer must hold its slice's sums."""
    import ctypes

    from resinfer_b200 import _cabi
    lib = _cabi.load()
    dev = cuda_device
    world, rank, n = 4, 1, 128 * 8192
    g = torch.Generator(device="cpu").manual_seed(4)
    parts = [torch.randn(n, generator=g).to(torch.bfloat16).to(dev) for _ in range(world)]
    before = [p.clone() for p in parts]
    flags = [torch.zeros(lib.ri_peer_allreduce_flag_bytes() // 4, dtype=torch.int32, device=dev) for _ in range(world)]
    flags[rank].fill_(1)                                       # every rank has announced call 1, both times
    state = torch.zeros(lib.ri_peer_allreduce_state_bytes(), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    data_ptrs = (ctypes.c_void_p * world)(*[p.data_ptr() for p in parts])
    flag_ptrs = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
    torch.cuda.synchronize()
    assert lib.ri_peer_allreduce_bf16(data_ptrs, flag_ptrs, rank, world, n, out.data_ptr(), state.data_ptr(),
                                      status.data_ptr(), _cabi.current_stream(dev), 0) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    length = (n // 8 + world - 1) // world * 8                 # elements per slice (whole 16-byte vectors)
    want = torch.empty_like(out)
    for q in range(world):
        lo, hi = q * length, min((q + 1) * length, n)
        if q == rank:
            acc = torch.zeros(hi - lo, dtype=torch.float32, device=dev)
            for r in range(world):
                acc += before[r][lo:hi].float()
            want[lo:hi] = acc.to(torch.bfloat16)
        else:
            want[lo:hi] = before[q][lo:hi]
    assert torch.equal(out, want)
    lo, hi = rank * length, min((rank + 1) * length, n)
    assert torch.equal(parts[rank][lo:hi], want[lo:hi])        # the sums are where the peers will fetch them
    assert torch.equal(parts[rank][:lo], before[rank][:lo]) and torch.equal(parts[rank][hi:], before[rank][hi:])
    # both announcements went out to every peer
    for r in range(world):
        if r != rank:
            assert int(flags[r][rank].item()) == 1 and int(flags[r][8 + rank].item()) == 1


def test_status_check_raises_and_clears(cuda_device):
    from resinfer_b200 import ops
    st = ops.status_word(cuda_device)
    st.fill_(7)
    with pytest.raises(RuntimeError, match="status 7"):
        ops.check_status(cuda_device)
    ops.check_status(cuda_device)                            # cleared by the failed check
