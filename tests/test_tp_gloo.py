"""World-size-2 test of the tensor-parallel partition on CPU ranks (gloo): sharded quantise +
dequantised product + collective equals the unsharded run."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _linear_oracle(x, w, sel=None):
    """deq(quantiser(x)) . deq(q(W))^T with the oracle (MEXT when sel is None, KEXT otherwise)."""
    import oracle as O
    gi = np.float32(64.0)                                  # per-layer constant shared by all ranks
    if sel is None:
        codes, sf, _ = O.nvfp4_quant_mext(x, gi, O.LAYOUT_ROW_PAIR)
        a = O.dequant_operand(codes, sf, "nvfp4")
        a = a[0::2] + a[1::2]
        w_use = w
    else:
        mask = np.zeros(x.shape[1] // 8, np.uint8)
        np.bitwise_or.at(mask, sel // 8, (1 << (sel % 8)).astype(np.uint8))
        per8 = sel.size * 8 // x.shape[1]
        codes, sf, _ = O.nvfp4_quant_kext(x, gi, mask, per8)
        a = O.dequant_operand(codes, sf, "nvfp4")
        w_use = np.concatenate([w, w[:, sel]], axis=1)
    wc, wsf = O.nvfp4_quant_plain(w_use, np.float32(1000.0))
    return O.fp4_linear_reference(a, O.dequant_operand(wc, wsf, "nvfp4"), 1.0, round_bf16=False)


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle as O
        from resinfer_b200.quant import tp
        from resinfer_b200.quant.vllm_integration.residue_tp import ResidueShardPlan
        m, k, n = 4, 512, 64
        x, w = O.make_activation(m, k, seed=0), O.make_weight(n, k, seed=1)
        full = _linear_oracle(x, w)
        # row-parallel MEXT: K split, all-reduce of the partial outputs
        xr = tp.shard_activation(torch.from_numpy(x), "row", world, rank).numpy()
        wr = tp.shard_weight(torch.from_numpy(w), "row", world, rank).numpy()
        part = torch.from_numpy(_linear_oracle(np.ascontiguousarray(xr), np.ascontiguousarray(wr)))
        tot = tp.finish_output(part, "row")
        # weight block scales are local, so the sharded weight codes equal the slice of the full ones
        err_row = float(np.linalg.norm(tot.numpy() - full) / np.linalg.norm(full))
        # column-parallel: N split, all-gather
        wc = tp.shard_weight(torch.from_numpy(w), "col", world, rank).numpy()
        yc = tp.finish_output(torch.from_numpy(_linear_oracle(x, np.ascontiguousarray(wc))), "col", gather=True)
        err_col = float(np.abs(yc.numpy() - full).max())
        # row-parallel KEXT: two-range gather of the extended weight, rank-local salient indices
        sel = O.mask_to_indices(O.make_kext_mask(k, 2, seed=4))
        plan = ResidueShardPlan(k, sel.size, world, rank)
        plan.validate()
        loc = plan.local_salient_indices(torch.from_numpy(sel)).numpy()
        w_ext = torch.from_numpy(np.concatenate([w, w[:, sel]], axis=1))
        w_loc = tp.shard_extended_weight(w_ext, k, sel.size, world, rank).numpy()
        assert np.array_equal(w_loc, np.concatenate([wr, wr[:, loc]], axis=1))
        part = torch.from_numpy(_linear_oracle(np.ascontiguousarray(xr), np.ascontiguousarray(wr), loc))
        tot_k = tp.finish_output(part, "row")
        full_k = _linear_oracle(x, w, sel)
        err_kext = float(np.linalg.norm(tot_k.numpy() - full_k) / np.linalg.norm(full_k))
        if rank == 0:
            q.put((err_row, err_col, err_kext))
    finally:
        dist.destroy_process_group()


def test_row_and_column_parallel_match_unsharded():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    err_row, err_col, err_kext = q.get(timeout=10)
    # the weight's per-tensor global scale is a constant here, so shards reproduce the full run up to
    # the summation order of the all-reduce
    assert err_row < 1e-6 and err_col == 0.0 and err_kext < 1e-6


def test_shard_bounds_errors():
    from resinfer_b200.quant import tp
    assert tp.shard_bounds(1024, 4, 3, 128) == (768, 1024)
    with pytest.raises(ValueError):
        tp.shard_bounds(1000, 3, 0)
    with pytest.raises(ValueError):
        tp.shard_bounds(25600 // 2, 8, 0, 128 * 16)
